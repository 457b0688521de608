// Attention of a decode step on the fifth-generation tensor cores, for models whose K/V heads serve many
// query heads (33 to 128 of them, head size 64: Falcon-7B's multi-query attention has 71 on one K/V
// head). Every sequence brings one token; the rows of the tile are the query heads of a K/V group, so
// one read of the group's keys and values serves all of them, and 71 heads fill more than half of
// the 128-row matrix instruction where the mma.sync kernel of attention_decode.cu needs five warps of
// 16 rows each, every one a chain of dependent work per page.
//
// One block = one sequence x one K/V head x one share of the sequence's pages. Roles as in
// attention_tc.cu: 128 softmax threads (thread t = query head t of the group = tensor-memory lane t),
// one warp whose first lane issues the matrix instructions, one warp whose first lane asks the tensor
// memory accelerator for the pages (TMA, 128-byte swizzle, a ring of stages with "landed" and "free"
// mbarriers). S = Q K^T and O += P V are tcgen05.mma with S (two buffers), O and P (two buffers, written
// back with tcgen05.st and read as the A operand) in tensor memory.
//
// Before the loop the block stages the token's row of the fused projection in shared memory, rotates
// queries and key there (float32 angles from the step's table, rounded to bfloat16 as the stored
// queries and keys of the other paths are), lays the queries out as the swizzled Q tile, and, if it is
// the block that covers the token's page, writes key and value into the cache and only then lets the
// copy thread ask for that page, so that the page arrives with the token's row in it.
//
// The blocks that share a (sequence, K/V head) form one thread-block cluster (1 to 8 blocks). Each
// leaves (maximum, sum, unnormalised output) of its rows in its own shared memory; after a cluster
// barrier every block joins a share of the rows from all blocks' shared memory (distributed shared
// memory) and writes them out: no workspace in global memory, no second launch.
//
// A long sequence in a small batch needs more blocks than a cluster holds: then `n_teams` clusters (teams)
// share the sequence's pages. Each team leaves its joined rows (maximum, sum, unnormalised output) in a
// workspace in global memory and takes a ticket; the block that draws the last ticket for its share of
// the rows joins the teams, always in the order of the teams, and leaves the ticket counter at zero.
//
// Every wait on an mbarrier is bounded; when one runs out the block raises the error flag in global
// memory and goes on to its end without waiting again (tensor memory is freed, the cluster barriers
// are passed, copies in flight are waited for): a fault shows as an error, never as a hang.
#include <cooperative_groups.h>

#include "mma_common.cuh"
#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int ROWS = 128;        // rows of the tile = query heads of a K/V group, padded
constexpr int DD = 64;           // head size
constexpr int STAGES_D = 4;
constexpr int TILE_Q = ROWS * DD * 2;      // 16 KB
constexpr int TILE_KV = KEYS * DD * 2;     // 8 KB
constexpr int SOFTMAX_T = ROWS;
constexpr int BLOCK_T = SOFTMAX_T + 64;

template <int RS> __device__ __forceinline__ uint32_t swz_blk(int row, int c) {
  return uint32_t((c >> 3) * (RS * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}

struct DecodeTcParams {
  int heads, kv_heads, n_splits, n_teams, rot_pairs, write_cache, interleaved;
  float scale;
};
constexpr int PART = DD + 2;     // floats of a row in the teams' workspace: output, maximum, sum

__global__ void __launch_bounds__(BLOCK_T, 2)
attention_decode_tc_kernel(const __nv_bfloat16* __restrict__ fused, __nv_bfloat16* __restrict__ k_pool,
                           __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out, StepBatch sb,
                           const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, DecodeTcParams p,
                           const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                           float* __restrict__ team_parts, int* __restrict__ tickets, int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* q_tile = smem;
  unsigned char* k_ring = q_tile + TILE_Q;
  unsigned char* v_ring = k_ring + STAGES_D * TILE_KV;
  // the token's row: query heads of the group, key, value (bfloat16), then cos and sin (float32)
  __nv_bfloat16* rowbuf = reinterpret_cast<__nv_bfloat16*>(v_ring + STAGES_D * TILE_KV);
  float* cs = reinterpret_cast<float*>(rowbuf + (ROWS + 2) * DD);
  // barriers: S written [2], O updated [2], P written [2] (even / odd pages), per stage landed and free,
  // "the token's key and value are in the cache", "the Q tile is written"
  uint64_t* bars = reinterpret_cast<uint64_t*>(cs + DD);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8 + 2 * STAGES_D);
  // partial results for the join reuse the page ring once the loop is over: po [ROWS][DD], pml [ROWS][2]
  float* po = reinterpret_cast<float*>(k_ring);
  float* pml = po + ROWS * DD;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool mma_warp = warp == SOFTMAX_T / 32, copy_warp = warp == SOFTMAX_T / 32 + 1;
  const int seq = blockIdx.x, g = blockIdx.y;
  const int split = blockIdx.z % p.n_splits, team = blockIdx.z / p.n_splits;   // a cluster = consecutive z
  const int qpk = p.heads / p.kv_heads;
  const int pos = sb.seq_past[seq];            // position of the new token
  const int tok = sb.seq_start[seq];           // its row in the step
  const int fused_width = p.kv_heads * (qpk + 2) * DD;
  const __nv_bfloat16* frow = fused + size_t(tok) * fused_width + size_t(g) * (qpk + 2) * DD;
  const int P = rope_cos ? p.rot_pairs : 0;
  const int* pages = sb.pages + size_t(seq) * sb.pages_stride;

  // pages of this block
  const int kb_last = pos / KEYS;
  const int n_pages = kb_last + 1;
  const int n_sharers = p.n_splits * p.n_teams;
  const int kb_begin = int((long long)blockIdx.z * n_pages / n_sharers);
  const int kb_end = int((long long)(blockIdx.z + 1) * n_pages / n_sharers);
  const int n_mine = kb_end - kb_begin;
  const bool covers_new = n_mine > 0 && kb_end == n_pages;

  const uint32_t bar_s = smem_u32(&bars[0]), bar_o = smem_u32(&bars[2]), bar_p = smem_u32(&bars[4]);
  const uint32_t bar_k = smem_u32(&bars[6]), bar_free = smem_u32(&bars[6 + STAGES_D]);
  const uint32_t bar_new = smem_u32(&bars[6 + 2 * STAGES_D]), bar_q = smem_u32(&bars[7 + 2 * STAGES_D]);
  // Warps whose 32 rows all lie past the group's heads take no part in the softmax: they would spend a
  // quarter or half of the exponential unit's time on rows that nobody reads. Their rows of P and O in
  // tensor memory hold whatever was there; a row of the products depends on its own row of P only.
  const int active_warps = (qpk + 31) / 32;
  // The usual rotation (the halves of the head, or none) is done in registers, a thread per head; any
  // other number of rotated pairs goes the general way through shared memory.
  const bool in_registers = (P == DD / 2 && !p.interleaved) || P == 0;
  // The copy warp's first lane sets the barriers up and asks for this block's first pages at once (their
  // numbers read by the warp's lanes, one each): they travel while tensor memory is allocated and the token's
  // row is staged. Nobody else touches a barrier before the block-wide barrier below. The token's own
  // page waits for the token's key and value and is asked for after that barrier.
  auto ask_page = [&](int b, int page) {
    const int st = b % STAGES_D;
    const int y = (page * p.kv_heads + g) * KEYS;
    const uint32_t full = bar_k + 8 * st;
    mbar_expect_tx(full, 2 * TILE_KV);
    tma_load_2d(smem_u32(k_ring + st * TILE_KV), &k_map, 0, y, full);
    tma_load_2d(smem_u32(v_ring + st * TILE_KV), &v_map, 0, y, full);
  };
  int my_page = 0, early = 0;   // copy warp: page number of page kb_begin + lane; pages asked for before the barrier
  if (copy_warp) {
    my_page = lane < n_mine ? pages[kb_begin + lane] : 0;
    if (lane == 0) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(bar_s + 8 * b, 1);
        mbar_init(bar_o + 8 * b, 1);
        mbar_init(bar_p + 8 * b, uint32_t(active_warps) * 32);
      }
      for (int s = 0; s < STAGES_D; ++s) {
        mbar_init(bar_k + 8 * s, 1);
        mbar_init(bar_free + 8 * s, 1);
      }
      mbar_init(bar_new, in_registers ? 1 : SOFTMAX_T);
      mbar_init(bar_q, SOFTMAX_T);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    early = min(n_mine, STAGES_D);
    if (p.write_cache && covers_new) early = min(early, n_mine - 1);
    for (int b = 0; b < early; ++b) {
      const int page = __shfl_sync(0xffffffffu, my_page, b);
      if (lane == 0) ask_page(b, page);
    }
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(256));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  tc_fence_before();
  __syncthreads();        // barriers and tensor memory are ready; from here the three roles go their own ways
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128;     // S at [0, 64) and [64, 128), O at [128, 192), P at [192, 224), [224, 256)
  constexpr uint32_t TMEM_P = 192;
  bool alive = true;
  auto softmax_sync = [] { asm volatile("bar.sync 1, %0;\n" ::"n"(SOFTMAX_T) : "memory"); };   // the 128 softmax threads

  if (!copy_warp && !mma_warp && in_registers) {
    // thread t = query head t: its 64 values come straight from the fused projection into registers,
    // are rotated there (pairs (e, e + 32), the angles from the step's table) and go into the swizzled Q
    // tile; rows past the group's heads are zero
    uint4 raw[DD / 8];
#pragma unroll
    for (int c = 0; c < DD / 8; ++c)
      raw[c] = tid < qpk ? *reinterpret_cast<const uint4*>(frow + size_t(tid) * DD + c * 8) : make_uint4(0, 0, 0, 0);
    if (P > 0 && tid < qpk) {
      const float* cosr = rope_cos + size_t(tok) * p.rot_pairs;
      const float* sinr = rope_sin + size_t(tok) * p.rot_pairs;
#pragma unroll
      for (int c = 0; c < DD / 16; ++c) {
        float a[8], b[8], cv[8], sv[8];
        unpack_bf16x8(raw[c], a);
        unpack_bf16x8(raw[c + DD / 16], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          cv[j] = __ldg(cosr + c * 8 + j);
          sv[j] = __ldg(sinr + c * 8 + j);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) rotate_pair(a[j], b[j], cv[j], sv[j], a[j], b[j]);
        raw[c] = pack_bf16x8(a);
        raw[c + DD / 16] = pack_bf16x8(b);
      }
    }
#pragma unroll
    for (int c = 0; c < DD / 8; ++c) *reinterpret_cast<uint4*>(q_tile + swz_blk<ROWS>(tid, c)) = raw[c];
    proxy_fence_async();
    mbar_arrive(bar_q);
  } else if (mma_warp && in_registers && covers_new && p.write_cache) {
    // the token's key (rotated) and value go to the cache from the block that covers the token's page:
    // lanes 0..3 take the key's pairs of 16-byte chunks, lanes 4..11 the value's chunks; the copy thread
    // asks for that page only after these writes (made visible to the TMA's proxy)
    const __nv_bfloat16* krow = frow + size_t(qpk) * DD;
    const size_t off = kv_offset(pages[kb_last], g, pos % KEYS, p.kv_heads, DD);
    if (lane < DD / 16) {
      float a[8], b[8];
      unpack_bf16x8(*reinterpret_cast<const uint4*>(krow + lane * 8), a);
      unpack_bf16x8(*reinterpret_cast<const uint4*>(krow + DD / 2 + lane * 8), b);
      if (P > 0) {
        const float* cosr = rope_cos + size_t(tok) * p.rot_pairs;
        const float* sinr = rope_sin + size_t(tok) * p.rot_pairs;
#pragma unroll
        for (int j = 0; j < 8; ++j) rotate_pair(a[j], b[j], __ldg(cosr + lane * 8 + j), __ldg(sinr + lane * 8 + j), a[j], b[j]);
      }
      *reinterpret_cast<uint4*>(k_pool + off + lane * 8) = pack_bf16x8(a);
      *reinterpret_cast<uint4*>(k_pool + off + DD / 2 + lane * 8) = pack_bf16x8(b);
    } else if (lane < DD / 16 + DD / 8) {
      const int c = lane - DD / 16;
      *reinterpret_cast<uint4*>(v_pool + off + c * 8) = *reinterpret_cast<const uint4*>(krow + DD + c * 8);
    }
    __threadfence();
    asm volatile("fence.proxy.async;\n" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_new);
  }
  if (!copy_warp && !mma_warp && !in_registers) {
    // stage the token's row: 16-byte copies of the group's queries, key, value; the rotation's cos / sin
    const uint4* src = reinterpret_cast<const uint4*>(frow);
    uint4* dst = reinterpret_cast<uint4*>(rowbuf);
    for (int i = tid; i < qpk * (DD / 8); i += SOFTMAX_T) dst[i] = src[i];
    const uint4* src_kv = reinterpret_cast<const uint4*>(frow + size_t(qpk) * DD);
    uint4* dst_kv = reinterpret_cast<uint4*>(rowbuf + ROWS * DD);
    for (int i = tid; i < 2 * (DD / 8); i += SOFTMAX_T) dst_kv[i] = src_kv[i];
    for (int e = tid; e < P; e += SOFTMAX_T) {
      cs[e] = rope_cos[size_t(tok) * p.rot_pairs + e];
      cs[P + e] = rope_sin[size_t(tok) * p.rot_pairs + e];
    }
    softmax_sync();
    for (int idx = tid; idx < (qpk + 1) * P; idx += SOFTMAX_T) {
      const int r = idx / P, e = idx % P;
      __nv_bfloat16* row = rowbuf + size_t(r < qpk ? r : ROWS) * DD;
      float ra, rb;
      const int ia = p.interleaved ? 2 * e : e, ib = p.interleaved ? 2 * e + 1 : e + P;   // the pair's two dims
      rotate_pair(__bfloat162float(row[ia]), __bfloat162float(row[ib]), cs[e], cs[P + e], ra, rb);
      row[ia] = __float2bfloat16_rn(ra);
      row[ib] = __float2bfloat16_rn(rb);
    }
    softmax_sync();
    const __nv_bfloat16* krow = rowbuf + size_t(ROWS) * DD;   // rotated key, then the value
    // the token's key and value go to the cache from the block that covers the token's page; the copy
    // thread asks for that page only after all of these writes (made visible to the TMA's proxy)
    if (covers_new && p.write_cache && tid < 2 * (DD / 8)) {
      const size_t off = kv_offset(pages[kb_last], g, pos % KEYS, p.kv_heads, DD);
      __nv_bfloat16* dstkv = (tid < DD / 8 ? k_pool : v_pool) + off + (tid % (DD / 8)) * 8;
      *reinterpret_cast<uint4*>(dstkv) = *reinterpret_cast<const uint4*>(krow + tid * 8);
      __threadfence();
      asm volatile("fence.proxy.async;\n" ::: "memory");
    }
    mbar_arrive(bar_new);
    // the Q tile: row t = query head t (zero past the group's heads), 128-byte swizzle
#pragma unroll
    for (int c = 0; c < DD / 8; ++c) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (tid < qpk) v = *reinterpret_cast<const uint4*>(rowbuf + size_t(tid) * DD + c * 8);
      *reinterpret_cast<uint4*>(q_tile + swz_blk<ROWS>(tid, c)) = v;
    }
    proxy_fence_async();
    mbar_arrive(bar_q);
  }

  if (copy_warp) {
    // The rest is the first lane's alone. (All lanes walking the loop, with the page numbers read 32 at a
    // time and handed round by shuffles, made long walks 7 % slower.)
    if (lane == 0) {
      int issued = early;
      for (int b = early; b < n_mine; ++b) {
        if (b >= STAGES_D && !mbar_wait(bar_free + 8 * (b % STAGES_D), ((b / STAGES_D) - 1) & 1, error_flag, 6)) break;
        // the token's page waits for the token's key and value
        if (kb_begin + b == kb_last && p.write_cache && !mbar_wait(bar_new, 0, error_flag, 7)) break;
        ask_page(b, pages[kb_begin + b]);
        issued = b + 1;
      }
      if (issued < n_mine)
        for (int b = max(0, issued - STAGES_D); b < issued; ++b)
          mbar_wait(bar_k + 8 * (b % STAGES_D), (b / STAGES_D) & 1, error_flag, 6);
    }
  } else if (mma_warp) {
    if (lane == 0 && n_mine > 0) {
      constexpr uint32_t IDESC_S = idesc_bf16(ROWS, KEYS, false);
      constexpr uint32_t IDESC_PV = idesc_bf16(ROWS, 64, true);
      const uint64_t desc_q = smem_desc(smem_u32(q_tile), 16, 1024);
      const uint64_t desc_k0 = smem_desc(smem_u32(k_ring), 16, 1024);
      const uint64_t desc_v0 = smem_desc(smem_u32(v_ring), 16, 1024);
      constexpr uint64_t STAGE_UNITS = TILE_KV >> 4;
      auto issue_s = [&](int b, int st) {
        tc_mma4<2, 2>(tmem_base + (b & 1) * 64, desc_q, desc_k0 + st * STAGE_UNITS, IDESC_S, 0u);
        tc_commit(bar_s + (b & 1) * 8);
      };
      alive = mbar_wait(bar_q, 0, error_flag, 8) && mbar_wait(bar_k, 0, error_flag, 4);
      tc_fence_after();
      if (alive) issue_s(0, 0);
      int st = 0, st_next = 1 % STAGES_D;
      for (int i = 0; i < n_mine && alive; ++i) {
        if (i + 1 < n_mine) {
          alive = mbar_wait(bar_k + 8 * st_next, ((i + 1) / STAGES_D) & 1, error_flag, 4);
          tc_fence_after();
          issue_s(i + 1, st_next);
        }
        if (alive) alive = mbar_wait(bar_p + (i & 1) * 8, (i >> 1) & 1, error_flag, 5);
        tc_fence_after();
        tc_mma4_ts<128>(tmem_o, tmem_base + TMEM_P + (i & 1) * 32, desc_v0 + st * STAGE_UNITS, IDESC_PV, i > 0 ? 1u : 0u);
        tc_commit(bar_o + (i & 1) * 8);
        tc_commit(bar_free + 8 * st);
        st = st_next;
        st_next = (st_next + 1 == STAGES_D) ? 0 : st_next + 1;
      }
    }
  } else if (warp < active_warps) {
    // ------------------------------------------------------------ softmax threads: row = query head
    const int row = tid;
    const uint32_t lane_base = tmem_base + (uint32_t(warp * 32) << 16);
    float m_run = -INFINITY, l_run = 0.f;
    const float sl2 = p.scale * 1.4426950408889634f;
    for (int i = 0; i < n_mine; ++i) {
      const int kb = kb_begin + i;
      if (alive) alive = mbar_wait(bar_s + (i & 1) * 8, (i >> 1) & 1, error_flag, 1);
      tc_fence_after();
      float s[KEYS];
      tmem_ld<KEYS>(lane_base + (i & 1) * 64, s);
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (kb == kb_last) {
        const int visible = pos - kb * KEYS;   // columns j <= visible are keys up to the token's own
#pragma unroll
        for (int j = 0; j < KEYS; ++j) {
          s[j] = (j <= visible) ? s[j] : -INFINITY;
          mx[j & 3] = fmaxf(mx[j & 3], s[j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < KEYS; ++j) mx[j & 3] = fmaxf(mx[j & 3], s[j]);
      }
      const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      float m_new = fmaxf(m_run, m_blk);
      if ((m_new - m_run) * sl2 <= RESCALE_LOG2) m_new = m_run;   // (false from -inf: the first scores set it)
      const float corr = (m_run == -INFINITY) ? 0.f : fast_exp2((m_run - m_new) * sl2);
      const bool moved = (m_new != m_run) && (m_run != -INFINITY);
      m_run = m_new;
      const float m_off = (m_run == -INFINITY) ? 0.f : m_run * sl2;
      if (i > 0 && __any_sync(0xffffffffu, moved)) {
        if (alive) alive = mbar_wait(bar_o + ((i - 1) & 1) * 8, ((i - 1) >> 1) & 1, error_flag, 2);
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < DD; c0 += 32) {
          float o[32];
          tmem_ld32(lane_base + 128 + c0, o);
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] *= corr;
          tmem_st32(lane_base + 128 + c0, o);
        }
        tmem_st_wait();
      }
      l_run *= corr;
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t w[KEYS / 2];
#pragma unroll
      for (int e = 0; e < KEYS / 2; ++e) {
        const float a = fast_exp2(fmaf(s[2 * e], sl2, -m_off));
        const float b = fast_exp2(fmaf(s[2 * e + 1], sl2, -m_off));
        ls[e & 3] += a + b;
        w[e] = pack_bf16(a, b);
      }
      tmem_st_u32<KEYS / 2>(lane_base + TMEM_P + (i & 1) * 32, w);
      tmem_st_wait();
      l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tc_fence_before();
      mbar_arrive(bar_p + (i & 1) * 8);
    }
    // this block's result for its row: straight to the output (one block per sequence and K/V head), or
    // as a partial result (maximum in units of raw scores, sum, unnormalised output) for the join
    if (n_mine > 0) {
      if (alive) alive = mbar_wait(bar_o + ((n_mine - 1) & 1) * 8, ((n_mine - 1) >> 1) & 1, error_flag, 3);
      tc_fence_after();
    }
    __nv_bfloat16* out_row = out + (size_t(tok) * p.heads + size_t(g) * qpk + row) * DD;
#pragma unroll
    for (int c0 = 0; c0 < DD; c0 += 32) {
      float o[32];
      if (n_mine > 0) tmem_ld32(lane_base + 128 + c0, o);
      else {
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = 0.f;
      }
      if (p.n_splits == 1 && p.n_teams > 1) {
        // a team of one block: its rows go to the workspace as they are
        if (row < qpk) {
          float* dst = team_parts + ((size_t(seq) * p.kv_heads + g) * p.n_teams + team) * qpk * PART + size_t(row) * PART;
#pragma unroll
          for (int j = 0; j < 32; j += 2) *reinterpret_cast<float2*>(dst + c0 + j) = make_float2(o[j], o[j + 1]);
          if (c0 == 0) *reinterpret_cast<float2*>(dst + DD) = make_float2(m_run, l_run);
        }
      } else if (p.n_splits == 1) {
        if (row < qpk) {
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t wv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) wv[e] = pack_bf16(o[c * 8 + 2 * e] * inv, o[c * 8 + 2 * e + 1] * inv);
            *reinterpret_cast<uint4*>(out_row + c0 + c * 8) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
          }
        }
      } else {
        // every landed page has been consumed (the last O += P V is complete): the ring is free
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(po + size_t(row) * DD + c0 + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
      }
    }
    if (p.n_splits > 1) {
      pml[row * 2 + 0] = m_run;
      pml[row * 2 + 1] = l_run;
    }
  }

  if (p.n_splits > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();   // every block of the cluster has left its partial results
    const float sl2 = p.scale * 1.4426950408889634f;
    const int n_splits = p.n_splits;
    // rows r with r % n_splits == split are joined by this block: thread -> (row, 4 dims)
    const int per_row = DD / 4;
    const int my_rows = (qpk - split + n_splits - 1) / n_splits;
    for (int idx = tid; idx < my_rows * per_row; idx += BLOCK_T) {
      const int r = split + (idx / per_row) * n_splits;
      const int d0 = (idx % per_row) * 4;
      // all blocks' values first (the loads from the other blocks' shared memory are in flight together),
      // then the sums, always in the order of the blocks
      float2 ml[8];
      float4 vs[8];
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        if (s < n_splits) {
          ml[s] = *reinterpret_cast<const float2*>(cluster.map_shared_rank(pml, s) + r * 2);
          vs[s] = *reinterpret_cast<const float4*>(cluster.map_shared_rank(po, s) + size_t(r) * DD + d0);
        } else {
          ml[s] = make_float2(-INFINITY, 0.f);
          vs[s] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      float m = -INFINITY;
#pragma unroll
      for (int s = 0; s < 8; ++s) m = fmaxf(m, ml[s].x);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      float l = 0.f;
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        if (s < n_splits) {
          const float wgt = (ml[s].x == -INFINITY) ? 0.f : exp2f((ml[s].x - m) * sl2);
          l += ml[s].y * wgt;
          acc[0] += vs[s].x * wgt; acc[1] += vs[s].y * wgt; acc[2] += vs[s].z * wgt; acc[3] += vs[s].w * wgt;
        }
      }
      if (p.n_teams > 1) {
        float* dst = team_parts + ((size_t(seq) * p.kv_heads + g) * p.n_teams + team) * qpk * PART + size_t(r) * PART;
        *reinterpret_cast<float2*>(dst + d0) = make_float2(acc[0], acc[1]);
        *reinterpret_cast<float2*>(dst + d0 + 2) = make_float2(acc[2], acc[3]);
        if (d0 == 0) *reinterpret_cast<float2*>(dst + DD) = make_float2(m, l);
        continue;
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = out + (size_t(tok) * p.heads + size_t(g) * qpk + r) * DD + d0;
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc[0] * inv, acc[1] * inv), pack_bf16(acc[2] * inv, acc[3] * inv));
    }
    cluster.sync();   // no block leaves while another still reads its shared memory
  }
  if (p.n_teams > 1) {
    // the teams' join: the block with the last ticket for its share of the rows (r % n_splits == split)
    __threadfence();
    __syncthreads();
    int* ticket = tickets + (size_t(seq) * p.kv_heads + g) * p.n_splits + split;
    if (tid == 0) tmem_slot[1] = (atomicAdd(ticket, 1) == p.n_teams - 1) ? 1u : 0u;
    __syncthreads();
    if (tmem_slot[1]) {
      __threadfence();
      const float sl2 = p.scale * 1.4426950408889634f;
      const float* parts = team_parts + (size_t(seq) * p.kv_heads + g) * p.n_teams * qpk * PART;
      const int per_row = DD / 4;
      const int my_rows = (qpk - split + p.n_splits - 1) / p.n_splits;
      for (int idx = tid; idx < my_rows * per_row; idx += BLOCK_T) {
        const int r = split + (idx / per_row) * p.n_splits;
        const int d0 = (idx % per_row) * 4;
        // eight teams' loads in flight at a time: this block alone reads what all teams left
        float m = -INFINITY;
        for (int t0 = 0; t0 < p.n_teams; t0 += 8) {
          float mt[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            mt[u] = (t0 + u < p.n_teams) ? __ldcg(parts + (size_t(t0 + u) * qpk + r) * PART + DD) : -INFINITY;
#pragma unroll
          for (int u = 0; u < 8; ++u) m = fmaxf(m, mt[u]);
        }
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        float l = 0.f;
        for (int t0 = 0; t0 < p.n_teams; t0 += 8) {
          float2 ml[8], v0[8], v1[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const float* pr = parts + (size_t(min(t0 + u, p.n_teams - 1)) * qpk + r) * PART;
            ml[u] = __ldcg(reinterpret_cast<const float2*>(pr + DD));
            v0[u] = __ldcg(reinterpret_cast<const float2*>(pr + d0));
            v1[u] = __ldcg(reinterpret_cast<const float2*>(pr + d0 + 2));
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {   // always in the order of the teams
            const float wgt = (t0 + u >= p.n_teams || ml[u].x == -INFINITY) ? 0.f : exp2f((ml[u].x - m) * sl2);
            l += ml[u].y * wgt;
            acc[0] += v0[u].x * wgt; acc[1] += v0[u].y * wgt; acc[2] += v1[u].x * wgt; acc[3] += v1[u].y * wgt;
          }
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = out + (size_t(tok) * p.heads + size_t(g) * qpk + r) * DD + d0;
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc[0] * inv, acc[1] * inv), pack_bf16(acc[2] * inv, acc[3] * inv));
      }
      if (tid == 0) *ticket = 0;   // for the next launch
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(256));
}

}  // namespace

// heads per K/V head that this kernel takes (fewer: the rows of the 128-row tile would be mostly empty)
PTB_API int ptb_attention_decode_tc_supports(int head_dim, int q_per_kv) {
  return (head_dim == DD && q_per_kv > 32 && q_per_kv <= ROWS) ? 1 : 0;
}

static size_t decode_tc_smem() {
  // Q tile, page ring, the token's row and its cos / sin, barriers; the join's partial results
  // (ROWS x (DD + 2) float32) reuse the ring
  return 1024 + TILE_Q + 2 * STAGES_D * TILE_KV + size_t(ROWS + 2) * DD * 2 + DD * sizeof(float) + 256;
}
static bool decode_tc_configure() {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(decode_tc_smem())) != cudaSuccess)
      return false;
    configured = true;
  }
  return true;
}

// Every sequence of the step brings exactly one token. fused [n_seqs, kv_heads * (q_per_kv + 2) * 64]
// bfloat16; k_pool / v_pool: the pools of one cache entry, [pool_pages][kv_heads][64][64]; out
// [n_seqs, heads * 64]. n_teams clusters of n_splits (1 to 8) blocks share a sequence's pages; more than
// one team needs `team_parts` (n_seqs * kv_heads * n_teams * q_per_kv * 66 floats) and `tickets`
// (n_seqs * kv_heads * n_splits ints, zero before the launch and after it). rope_cos / rope_sin:
// [n_seqs, rot_pairs] float32 tables for the step's tokens, or null for no rotation (pairs (e, e + rot_pairs),
// or with `interleaved` (2 e, 2 e + 1)). No score bias, no window. `error_flag`: a device int that stays 0 unless a bounded wait inside the kernel ran out.
PTB_API int ptb_attention_decode_tc(const void* fused, void* k_pool, void* v_pool, int pool_pages, void* out,
                                    const StepBatch* sb, const float* rope_cos, const float* rope_sin, int rot_pairs,
                                    int interleaved, int heads, int kv_heads, int head_dim, int n_splits, int n_teams, float scale,
                                    int write_cache, float* team_parts, size_t team_floats, int* tickets, int n_tickets,
                                    int* error_flag, cudaStream_t stream) {
  if (sb->n_seqs <= 0) return PTB_OK;
  if (sb->n_tokens != sb->n_seqs) return PTB_ERR_SIZE;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || kv_heads > 65535 || error_flag == nullptr)
    return PTB_ERR_SIZE;
  if (!ptb_attention_decode_tc_supports(head_dim, heads / kv_heads)) return PTB_ERR_SIZE;
  if (n_splits < 1 || n_splits > 8 || rot_pairs < 0 || 2 * rot_pairs > head_dim) return PTB_ERR_SIZE;
  if (n_teams < 1 || n_splits * n_teams > 65535) return PTB_ERR_SIZE;
  if (n_teams > 1) {
    const size_t need = size_t(sb->n_seqs) * kv_heads * n_teams * (heads / kv_heads) * PART;
    if (team_parts == nullptr || tickets == nullptr || team_floats < need ||
        size_t(n_tickets) < size_t(sb->n_seqs) * kv_heads * n_splits || (reinterpret_cast<uintptr_t>(team_parts) & 7))
      return PTB_ERR_SIZE;
  }
  if ((rope_cos == nullptr) != (rope_sin == nullptr)) return PTB_ERR_SIZE;
  if (pool_pages <= 0 || ((reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool) |
                           reinterpret_cast<uintptr_t>(fused)) & 15))
    return PTB_ERR_ALIGN;
  const CUtensorMap* km = pool_map(k_pool, pool_pages, kv_heads, DD);
  const CUtensorMap* vm = pool_map(v_pool, pool_pages, kv_heads, DD);
  if (km == nullptr || vm == nullptr) return PTB_ERR_LAUNCH;
  DecodeTcParams p;
  p.heads = heads; p.kv_heads = kv_heads; p.n_splits = n_splits; p.n_teams = n_teams; p.rot_pairs = rot_pairs;
  p.write_cache = write_cache; p.scale = scale; p.interleaved = interleaved ? 1 : 0;
  const size_t smem = decode_tc_smem();
  if (!decode_tc_configure()) return PTB_ERR_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sb->n_seqs, kv_heads, n_splits * n_teams);
  cfg.blockDim = dim3(BLOCK_T);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = n_splits;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, attention_decode_tc_kernel, (const __nv_bfloat16*)fused, (__nv_bfloat16*)k_pool,
                         (__nv_bfloat16*)v_pool, (__nv_bfloat16*)out, *sb, rope_cos, rope_sin, p, *km, *vm,
                         team_parts, tickets, error_flag) != cudaSuccess) {
    (void)cudaGetLastError();
    return PTB_ERR_LAUNCH;
  }
  return launch_status();
}
