// Prompt attention on the fifth-generation tensor cores (tcgen05) with the accumulators in tensor
// memory, for head sizes 64 and 128, bfloat16, causal, with or without per-head score slopes (ALiBi),
// over the paged cache. The description below
// is for head size 64; with 128 the tiles of Q, K and V are two blocks of 64 dims, S takes two groups
// of matrix instructions, O two (one per 64 dims of the output), and one block fits on an SM.
//
// One block = 128 consecutive new tokens of one sequence x one query head. 128 softmax threads, one per
// query row (tensor-memory lane t = row t). One more warp's first lane issues every matrix
// instruction, another warp's first lane asks the tensor memory accelerator for the pages. The roles
// meet only at mbarriers (page landed, stage free, S written, P written, O updated): there is no
// block-wide barrier in the loop. Keys are walked one cache page (64 keys) at a time:
//
//   S = Q K^T      tcgen05.mma  M=128 N=64 K=64   A = Q  (shared, K-major, 128-byte swizzle)
//                                                 B = K page (shared, K-major, 128-byte swizzle)
//                                                 D = S in tensor memory, three buffers of 64 columns:
//                                                 the products of the next two pages run under this
//                                                 page's softmax
//   softmax        each thread reads its row of S with tcgen05.ld, masks, keeps the running maximum and
//                  sum in float32, rescales its row of O in tensor memory when the maximum moved (only
//                  then it waits for the previous page's O += P V), and writes P = exp2(S - max) as
//                  bfloat16 pairs back into tensor memory with tcgen05.st, in place of its row of S
//   O += P V       tcgen05.mma  M=128 N=64 K=64   A = P read from tensor memory, B = V page (shared,
//                                                 MN-major: head dims are contiguous), D = O in tensor
//                                                 memory, columns [192, 256)
//
// The page tiles [64 keys][64 dims] bfloat16 come by TMA (cp.async.bulk.tensor.2d over the cache pool
// seen as rows of D values, 128-byte swizzle) into a four-stage ring: exactly the canonical layout that
// the matrix descriptors name (K-major for Q and K; MN-major for V); a stage's mbarrier counts the
// bytes, and tcgen05.commit after the O += P V that read a stage gives it back to the copy thread. The
// softmax threads neither copy nor wait for copies. Completion of the matrix instructions is signalled
// through tcgen05.commit on mbarriers. Every wait on a barrier is bounded: if it runs out, a flag in
// global memory is raised and the block carries on to its end (tensor memory is freed on every path,
// copies in flight are waited for), so a fault in the pipeline shows as an error, never as a hang.
//
// Two blocks fit on an SM (81 KB of shared memory and 256 columns of tensor memory each): while one
// block's threads do softmax, the other's matrix instructions run. Warps of a block may be up to three
// pages apart (S runs that far ahead), which is why "P written" has a barrier per S buffer and "O
// updated" four that take turns (page % 4): a wait names a barrier's phase by its parity, and an
// arrival for a later or an earlier page must not count for page i.
//
// The copy warp sets the barriers up and asks for the first four pages before the block-wide barrier:
// they travel while the other warps fetch Q and tensor memory is allocated.
//
// Decisions that rest on measurements (2,048 tokens, 71 heads on one K/V head; the profile of this kernel
// has the series): one softmax thread per row; O is rescaled only when a row's maximum has grown by more
// than 2^8; three S buffers with P in place of S; P in tensor memory rather than in shared memory; no cap
// on registers; both halves of a row of S asked for before one wait, three-input maxima and packed
// two-value multiply-adds and adds in the softmax (3 %); four page stages. A block is one chain of
// dependent steps per page (about 1,500 clocks with two chains an SM, of which the exponential unit is
// busy 1,024) plus 6 us of set-up and drain; blocks that stay and draw one tile after another from a
// counter saved the set-up but ran their pages 10 to 25 % slower, and were taken out again.
#include "mma_common.cuh"
#include "tc_common.cuh"

namespace {

__device__ __forceinline__ float max3(float a, float b, float c) {
  float m;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(m) : "f"(a), "f"(b), "f"(c));
  return m;
}
// two float32 values in one 64-bit register for the packed multiply-add and add instructions
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

constexpr int TQ = 128;          // query rows per block
constexpr int STAGES_TC = 4;      // page stages (three are 15 to 30 % slower, five bring nothing)
// Tiles of D = 64 or 128 dims are kept as D / 64 blocks of [rows][64 dims], one after another, each
// block with the 128-byte swizzle: the layout that the matrix descriptors name for K-major operands
// (Q, K: a block per 64 values of the contraction) and for the MN-major V (a block per 64 dims of
// the output). Byte offset of 16-byte chunk `c` of row `row`:
template <int ROWS> __device__ __forceinline__ uint32_t swz_tc(int row, int c) {
  return uint32_t((c >> 3) * (ROWS * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}
struct TcParams {
  int heads, kv_heads;
  float scale;
  const float* slopes;   // per-head score slopes (ALiBi), or null
};

constexpr int SOFTMAX_THREADS = TQ;                 // one thread per query row
// one more warp whose first lane issues the matrix instructions, and one whose first lane asks the
// tensor memory accelerator for the pages
constexpr int BLOCK_THREADS = SOFTMAX_THREADS + 64;

// BIAS: a per-head slope times the key's position is added to the raw scores, formed in bfloat16 as
// the reference forms it.
template <int D, bool BIAS>
__global__ void __launch_bounds__(BLOCK_THREADS, D == 64 ? 2 : 1)
attention_tc_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                    const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out, StepBatch sb,
                    const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, TcParams p,
                    const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                    int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment: the swizzle pattern is a function of address bits 4..9
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  constexpr int TILE_Q_BYTES = TQ * D * 2;       // 16 or 32 KB
  constexpr int TILE_KV_BYTES = KEYS * D * 2;    // 8 or 16 KB
  // tensor memory: three S buffers of 64 columns (page i uses buffer i % 3), O at [192, 192 + D). P of a
  // page (64 keys as bfloat16 pairs, 32 columns) takes the place of its S: a thread has its row of S in
  // registers before it writes its row of P, nobody else touches that row, and the S of three pages later
  // is issued after the O += P V that reads this P (the tensor pipe runs in order). With three buffers S
  // runs two pages ahead of the softmax, so the softmax does not wait for a matrix product that was
  // issued only when the slowest warp finished the page before.
  constexpr uint32_t TMEM_O = 192, TMEM_COLS = (D == 64) ? 256 : 512;
  unsigned char* q_tile = smem;
  unsigned char* k_ring = q_tile + TILE_Q_BYTES;                      // STAGES_TC pages
  unsigned char* v_ring = k_ring + STAGES_TC * TILE_KV_BYTES;         // STAGES_TC pages
  // barriers: [0..2] S buffer written; [3..6] O updated (page % 4); [7..9] P written (page % 3);
  // then per stage: page landed, stage free again
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_ring + STAGES_TC * TILE_KV_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10 + 2 * STAGES_TC);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool mma_warp = warp == SOFTMAX_THREADS / 32;
  const bool copy_warp = warp == SOFTMAX_THREADS / 32 + 1;
  const int row = tid & (TQ - 1);        // query row of a softmax thread (= its tensor-memory lane)
  // heads are the fast index of the grid: the blocks of one tile start together (they read the same
  // pages), and tiles come in the order of the list, which the caller sorts by falling key count so that
  // the longest chains start first and the short ones fill the end
  const int tile = blockIdx.y, h = blockIdx.x;
  const int qpk = p.heads / p.kv_heads;
  const int g = h / qpk;
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int n_new = sb.seq_new[seq], past = sb.seq_past[seq], start = sb.seq_start[seq];
  const int tok_valid = min(TQ, n_new - q0);
  const bool row_ok = row < tok_valid;
  const int row_pos = row_ok ? past + q0 + row : -1;
  const int last_pos = past + q0 + tok_valid - 1;
  const int n_blocks = last_pos / KEYS + 1;
  const int* pages = sb.pages + size_t(seq) * sb.pages_stride;

  // A warp may be up to three pages ahead of another one (S of page i + 2 is issued before P of page i is
  // complete, S of page i + 3 only after it): arrivals for pages i + 1 and i + 2 must not count for page
  // i, hence a "P written" barrier per S buffer. A wait names a barrier's phase by its parity, which is
  // only right if the completion before the awaited one has happened already. A thread that has read S of
  // page i knows that O += P V of page i - 3 has completed (the tensor pipe runs in order), and so the one
  // of page i - 4: hence four "O updated" barriers that take turns. With two, a warp that reached the end
  // of its walk pages ahead of the others could take the completion of page i - 2 for that of page i and
  // read O before the last products were in it.
  const uint32_t bar_s = smem_u32(&bars[0]), bar_o = smem_u32(&bars[3]);
  const uint32_t bar_p = smem_u32(&bars[7]);
  const uint32_t bar_k = smem_u32(&bars[10]), bar_free = smem_u32(&bars[10 + STAGES_TC]);
  // The copy warp's first lane sets the barriers up and asks for the first pages at once (their numbers
  // read by the warp's lanes, one each): they are on their way while the other warps fetch Q and tensor
  // memory is allocated. Nobody else touches a barrier before the block-wide barrier below.
  constexpr uint32_t PAGE_BYTES = 2 * TILE_KV_BYTES;
  auto ask_page = [&](int b, int page) {
    const int st = b % STAGES_TC;
    const int y = (page * p.kv_heads + g) * KEYS;   // first row of the page in the pool seen as [rows][D]
    const uint32_t full = bar_k + 8 * st;
    mbar_expect_tx(full, PAGE_BYTES);
#pragma unroll
    for (int blk = 0; blk < D / 64; ++blk) {
      tma_load_2d(smem_u32(k_ring + st * TILE_KV_BYTES + blk * (KEYS * 128)), &k_map, blk * 64, y, full);
      tma_load_2d(smem_u32(v_ring + st * TILE_KV_BYTES + blk * (KEYS * 128)), &v_map, blk * 64, y, full);
    }
  };
  int first_pages = 0;   // the copy warp's lanes: the number of page b = lane
  if (copy_warp) {
    first_pages = lane < n_blocks ? pages[lane] : 0;
    if (lane == 0) {
      for (int b = 0; b < 3; ++b) {
        mbar_init(bar_s + 8 * b, 1);
        mbar_init(bar_p + 8 * b, SOFTMAX_THREADS);
      }
      for (int b = 0; b < 4; ++b) mbar_init(bar_o + 8 * b, 1);
      for (int s = 0; s < STAGES_TC; ++s) {
        mbar_init(bar_k + 8 * s, 1);      // the copy thread's expect_tx; the bytes complete it
        mbar_init(bar_free + 8 * s, 1);   // tcgen05.commit after the stage's O += P V
      }
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    for (int b = 0; b < STAGES_TC && b < n_blocks; ++b) {
      const int page = __shfl_sync(0xffffffffu, first_pages, b);
      if (lane == 0) ask_page(b, page);
    }
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  if (!mma_warp && !copy_warp) {
    // Q tile: rows of the tile, zero beyond the valid tokens
    const uint32_t qs = smem_u32(q_tile);
    for (int i = tid; i < TQ * (D / 8); i += SOFTMAX_THREADS) {
      const int r = i / (D / 8), c = i % (D / 8);
      if (r < tok_valid)
        cp_async16(qs + swz_tc<TQ>(r, c), q + (size_t(start + q0 + r) * p.heads + h) * D + c * 8);
      else
        *reinterpret_cast<uint4*>(q_tile + swz_tc<TQ>(r, c)) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    proxy_fence_async();
  }
  tc_fence_before();
  __syncthreads();        // barriers, tensor memory and Q are ready for everyone
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + TMEM_O;
  bool alive = true;  // false after a wait ran out: keep going without waiting, results are void

  if (copy_warp) {
    // ------------------------------------------------------------ the thread that asks for the pages
    // Page b goes into stage b % STAGES_TC as D / 64 boxes [64 keys x 64 dims] for K and for V, in
    // the swizzled layout; the stage's barrier counts the bytes. A stage is free again when the
    // O += P V that read it has completed (S of that page completed before it).
    // The first pages were asked for above; the rest is the first lane's alone.
    if (lane == 0) {
      int issued = min(n_blocks, STAGES_TC);
      for (int b = STAGES_TC; b < n_blocks; ++b) {
        if (!mbar_wait(bar_free + 8 * (b % STAGES_TC), ((b / STAGES_TC) - 1) & 1, error_flag, 6)) break;
        ask_page(b, pages[b]);
        issued = b + 1;
      }
      if (issued < n_blocks) {
        // a wait ran out: what is in flight lands before the block ends (bounded waits again)
        for (int b = max(0, issued - STAGES_TC); b < issued; ++b)
          mbar_wait(bar_k + 8 * (b % STAGES_TC), (b / STAGES_TC) & 1, error_flag, 6);
      }
    }
  } else if (mma_warp) {
    // ------------------------------------------------------------ the thread that issues matrix instructions
    if (lane == 0) {
      constexpr uint32_t IDESC_S = idesc_bf16(TQ, KEYS, false);
      // all D dims of the output in one instruction: an instruction of M = 128, K = 16 takes 51 clocks at
      // least whatever its N (N / 2 clocks from N = 128 on), so their number is what a page costs
      constexpr uint32_t IDESC_PV = idesc_bf16(TQ, D, true);
      const uint64_t desc_q = smem_desc(smem_u32(q_tile), 16, 1024);
      const uint64_t desc_k0 = smem_desc(smem_u32(k_ring), 16, 1024);
      // V is MN-major: blocks of 64 dims lie KEYS * 128 bytes apart (the leading offset), groups of 8 keys
      // 1024 bytes (the stride offset)
      const uint64_t desc_v0 = smem_desc(smem_u32(v_ring), KEYS * 128, 1024);
      constexpr uint64_t STAGE_UNITS = TILE_KV_BYTES >> 4;   // the address field counts 16-byte units
      constexpr uint64_t Q_BLOCK = (TQ * 128) >> 4, KV_BLOCK = (KEYS * 128) >> 4;   // blocks of 64 dims
      // S_b = Q K_b^T into S buffer `buf`; the page sits in stage b % STAGES_TC
      auto issue_s = [&](int b, int buf) {
        const int st = b % STAGES_TC;
#pragma unroll
        for (int blk = 0; blk < D / 64; ++blk)
          tc_mma4<2, 2>(tmem_base + buf * 64, desc_q + blk * Q_BLOCK, desc_k0 + st * STAGE_UNITS + blk * KV_BLOCK,
                        IDESC_S, blk > 0 ? 1u : 0u);
        tc_commit(bar_s + buf * 8);
      };
      // S of the first two pages
      for (int b = 0; b < 2 && b < n_blocks && alive; ++b) {
        alive = mbar_wait(bar_k + 8 * b, 0, error_flag, 4);
        tc_fence_after();
        if (alive) issue_s(b, b);
      }
      int buf = 0, phase = 0;   // S buffer of page i (i % 3) and the parity of its barriers ((i / 3) & 1)
      for (int i = 0; i < n_blocks && alive; ++i) {
        if (i + 2 < n_blocks) {
          // page i + 2 landed; S_{i+2} goes where S_{i-1} and P_{i-1} were: every thread had read that S
          // before it reported P_{i-1}, and the O += P_{i-1} V_{i-1} that reads the P was issued before
          alive = mbar_wait(bar_k + 8 * ((i + 2) % STAGES_TC), ((i + 2) / STAGES_TC) & 1, error_flag, 4);
          tc_fence_after();
          issue_s(i + 2, buf == 0 ? 2 : buf - 1);
        }
        // P_i is written and O is rescaled: O += P_i V_i (16 keys: 32 bytes along P's rows, 2048 bytes
        // down V's rows)
        if (alive) alive = mbar_wait(bar_p + buf * 8, phase, error_flag, 5);
        tc_fence_after();
        const int st = i % STAGES_TC;
        tc_mma4_ts<128>(tmem_o, tmem_base + buf * 64, desc_v0 + st * STAGE_UNITS, IDESC_PV, i > 0 ? 1u : 0u);
        tc_commit(bar_o + 8 * (i & 3));
        tc_commit(bar_free + 8 * st);   // the copy thread may refill this stage
        if (++buf == 3) { buf = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax threads
    const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16);   // this warp's lanes
    const uint32_t o_addr = lane_addr + TMEM_O;
    int buf = 0, phase = 0;   // S buffer of page i (i % 3) and the parity of its barriers ((i / 3) & 1)
    float m_run = -INFINITY, l_run = 0.f;   // running maximum of the raw scores, the row's sum
    const float slope = BIAS ? p.slopes[h] : 0.f;
    const float sl2 = p.scale * 1.4426950408889634f;
    const uint64_t sl2_2 = pack2(sl2, sl2);
    for (int i = 0; i < n_blocks; ++i) {
      // (1) this thread's row of S_i: both halves asked for, one wait
      if (alive) alive = mbar_wait(bar_s + buf * 8, phase, error_flag, 1);
      tc_fence_after();
      float s[KEYS];
      tmem_ld64_once(lane_addr + buf * 64, s);
      if (BIAS) {
#pragma unroll
        for (int j = 0; j < KEYS; ++j) s[j] += alibi_bias(slope, i * KEYS + j);
      }
      // (2) maximum of the visible scores; only pages that reach past some row's position need the test
      if (i * KEYS + KEYS - 1 > past + q0 || !row_ok) {   // first part is uniform over the block
        const int visible = row_pos - i * KEYS;   // columns j <= visible are seen by this row
#pragma unroll
        for (int j = 0; j < KEYS; ++j) s[j] = (j <= visible) ? s[j] : -INFINITY;
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < KEYS; j += 8) {
        mx[0] = max3(mx[0], s[j], s[j + 1]);
        mx[1] = max3(mx[1], s[j + 2], s[j + 3]);
        mx[2] = max3(mx[2], s[j + 4], s[j + 5]);
        mx[3] = max3(mx[3], s[j + 6], s[j + 7]);
      }
      float m_new = fmaxf(m_run, fmaxf(max3(mx[0], mx[1], mx[2]), mx[3]));
      if ((m_new - m_run) * sl2 <= RESCALE_LOG2) m_new = m_run;   // (false from -inf: the first scores set it)
      const float corr = (m_run == -INFINITY) ? 0.f : fast_exp2((m_run - m_new) * sl2);
      const bool moved = (m_new != m_run) && (m_run != -INFINITY);
      m_run = m_new;
      const float m_off = (m_run == -INFINITY) ? 0.f : m_run * sl2;   // exp2(s * sl2 - m_off); exp2(-inf) = 0
      // (3) rescale this thread's row of O if any row of the warp moved its maximum; only then this warp
      // waits for the previous page's O += P V
      if (i > 0 && __any_sync(0xffffffffu, moved)) {
        if (alive) alive = mbar_wait(bar_o + 8 * ((i - 1) & 3), ((i - 1) >> 2) & 1, error_flag, 2);
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          float o[32];
          tmem_ld32(o_addr + c0, o);
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] *= corr;
          tmem_st32(o_addr + c0, o);
        }
        tmem_st_wait();
      }
      // (4) P = exp2(S - max) as bfloat16 pairs, two values per packed multiply-add
      const uint64_t moff_2 = pack2(-m_off, -m_off);
      uint64_t acc2[4] = {0ull, 0ull, 0ull, 0ull};
      uint32_t w[KEYS / 2];
#pragma unroll
      for (int e = 0; e < KEYS / 2; ++e) {
        float x0, x1;
        unpack2(fma2(pack2(s[2 * e], s[2 * e + 1]), sl2_2, moff_2), x0, x1);
        const float a = fast_exp2(x0), b = fast_exp2(x1);
        acc2[e & 3] = add2(acc2[e & 3], pack2(a, b));
        w[e] = pack_bf16(a, b);
      }
      // P in place of this page's S: keys 2c, 2c + 1 in column c of the buffer (this thread's row of S is in
      // registers since the load above)
      tmem_st_u32<KEYS / 2>(lane_addr + buf * 64, w);
      tmem_st_wait();
      float l0, l1, l2, l3;
      unpack2(add2(acc2[0], acc2[1]), l0, l1);
      unpack2(add2(acc2[2], acc2[3]), l2, l3);
      l_run = l_run * corr + ((l0 + l1) + (l2 + l3));
      tc_fence_before();
      mbar_arrive(bar_p + buf * 8);   // (5) the issuing thread starts O += P V when all rows have arrived
      if (++buf == 3) { buf = 0; phase ^= 1; }
    }
    // the walk's last O += P V
    if (alive) alive = mbar_wait(bar_o + 8 * ((n_blocks - 1) & 3), ((n_blocks - 1) >> 2) & 1, error_flag, 3);
    tc_fence_after();
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* dst = out + (size_t(start + q0 + row) * p.heads + h) * D;
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 32) {
      float o[32];
      tmem_ld32(o_addr + c0, o);
      if (row_ok) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) w[e] = pack_bf16(o[c * 8 + 2 * e] * inv, o[c * 8 + 2 * e + 1] * inv);
          *reinterpret_cast<uint4*>(dst + c0 + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS));
}


// ------------------------------------------------------------------------------------------------
// Two query heads of one K/V group in a block ("pair"), keys in steps of two pages.
//
// A tcgen05.mma of M = 128, K = 16 takes 51 clocks at least whatever its N, N / 2 clocks from N = 128 on,
// and no less than its operands take to come from shared memory at 128 bytes a clock (4 KB of A, 32 N
// bytes of B); measured by issuing them back to back. With N = 64 half of the pipe's time is that floor,
// and what a page costs is the number of instructions issued for it (one O += P V group with N = 128
// instead of two with N = 64 took a seventh off the kernel above at head size 128). Here S = Q K^T is
// formed for 128 keys at once (N = 128: half the instructions a key) and O += P V with N = D.
//
// A block = 128 tokens x heads (h, h + 1) of one K/V group: two chains that share every K/V stage. 256
// softmax threads (threads 0..127 the first head, 128..255 the second; both groups sit on tensor-memory
// lanes 0..127, the second on columns 256..511), one issuing thread, one copy warp. A group with an odd
// number of heads ends in a block whose second chain is idle. Per chain, in tensor memory: S [128 x 128]
// in columns 0..127, P (128 keys as bfloat16 pairs, 64 columns) in place of it, O in columns 128..128+D.
// S has one buffer: S of step j + 1 is issued right after O += P V of step j (the pipe runs in order),
// and while a chain waits for it the other chain's softmax has the SM. It follows that a thread that has
// read S of step j finds O += P V of step j - 1 completed: rescaling O needs no wait, only the walk's
// last product is waited for.
//
// Stages hold 128 keys: two pages side by side (rows 0..63 and 64..127 of the K-major K tile and of the
// MN-major V tile; with head size 128 two blocks of 64 dims each). K and V stages are given back
// separately (K after both chains' S, V after both chains' O += P V). A walk with an odd number of pages
// takes its last page twice: the second copy's keys lie past every row's position and are masked.
//
// The issuing thread never blocks on one chain while the other could move: it polls (mbarrier.test_wait)
// "stage landed" and "P written" of both chains in turn, parks for a fraction of a microsecond when
// nothing can be issued, and gives up like every wait when that goes on for seconds.
constexpr int PAIR_SOFTMAX = 2 * TQ;
constexpr int PAIR_THREADS = PAIR_SOFTMAX + 64;
constexpr int STEP_KEYS = 2 * KEYS;
constexpr uint32_t POLL_LIMIT = 1u << 24;

__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// one try with a time hint: parks the thread for `ns` at most (the result is not used)
__device__ __forceinline__ void mbar_park(uint32_t bar, uint32_t parity, uint32_t ns) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1, %2;\n\t}\n"
      ::"r"(bar), "r"(parity), "r"(ns) : "memory");
}

template <int D> struct PairShape {
  static constexpr int STAGES = D == 64 ? 4 : 2;           // stages of 128 keys, for K and for V
  static constexpr int TILE_Q_BYTES = TQ * D * 2;
  static constexpr int STAGE_BYTES = STEP_KEYS * D * 2;     // 16 or 32 KB
  static constexpr int N_BARS = 8 + 4 * STAGES;
  static constexpr size_t SMEM = 1024 + 2 * size_t(TILE_Q_BYTES) + 2 * size_t(STAGES) * STAGE_BYTES + N_BARS * 8 + 16;
};

template <int D, bool BIAS>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
attention_tc_pair_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, StepBatch sb,
                         const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, TcParams p,
                         const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                         int* __restrict__ error_flag) {
  using Shape = PairShape<D>;
  constexpr int STAGES = Shape::STAGES, TILE_Q_BYTES = Shape::TILE_Q_BYTES, STAGE_BYTES = Shape::STAGE_BYTES;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  constexpr uint32_t CHAIN_COLS = 256, TMEM_O = 128;
  unsigned char* q_tiles = smem;
  unsigned char* k_ring = q_tiles + 2 * TILE_Q_BYTES;
  unsigned char* v_ring = k_ring + STAGES * STAGE_BYTES;
  // barriers: per chain c at 3 c: S written, P written, the walk's last O += P V; [6], [7] unused; then
  // per stage: K landed, V landed, K free, V free
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_ring + STAGES * STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Shape::N_BARS);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool mma_warp = warp == PAIR_SOFTMAX / 32;
  const bool copy_warp = warp == PAIR_SOFTMAX / 32 + 1;
  const int chain = (tid >> 7) & 1;
  const int row = tid & (TQ - 1);
  const int tile = blockIdx.y;
  const int qpk = p.heads / p.kv_heads;
  const int pairs = (qpk + 1) / 2;                 // blocks a K/V group
  const int g = blockIdx.x / pairs;
  const int h0 = g * qpk + 2 * (blockIdx.x % pairs);
  const bool two = h0 + 1 < (g + 1) * qpk;          // the second chain has a head
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int n_new = sb.seq_new[seq], past = sb.seq_past[seq], start = sb.seq_start[seq];
  const int tok_valid = min(TQ, n_new - q0);
  const bool row_ok = row < tok_valid;
  const int row_pos = row_ok ? past + q0 + row : -1;
  const int last_pos = past + q0 + tok_valid - 1;
  const int n_pages = last_pos / KEYS + 1;
  const int n_steps = (n_pages + 1) / 2;
  const int* pages = sb.pages + size_t(seq) * sb.pages_stride;

  const uint32_t bar0 = smem_u32(bars);
  auto bar_s = [&](int c) { return bar0 + 8u * uint32_t(3 * c); };
  auto bar_p = [&](int c) { return bar0 + 8u * uint32_t(3 * c + 1); };
  auto bar_end = [&](int c) { return bar0 + 8u * uint32_t(3 * c + 2); };
  const uint32_t bar_k = bar0 + 8u * 8, bar_v = bar_k + 8u * STAGES, bar_kfree = bar_v + 8u * STAGES,
                 bar_vfree = bar_kfree + 8u * STAGES;
  // step j: pages 2j and 2j + 1 (or 2j again) into stage j % STAGES, per block of 64 dims rows 0..63 and 64..127
  auto ask = [&](unsigned char* ring, const CUtensorMap* map, uint32_t full, int j, int page_a, int page_b) {
    unsigned char* stage = ring + (j % STAGES) * STAGE_BYTES;
    mbar_expect_tx(full, STAGE_BYTES);
#pragma unroll
    for (int blk = 0; blk < D / 64; ++blk) {
      tma_load_2d(smem_u32(stage + blk * (STEP_KEYS * 128)), map, blk * 64, (page_a * p.kv_heads + g) * KEYS, full);
      tma_load_2d(smem_u32(stage + blk * (STEP_KEYS * 128) + KEYS * 128), map, blk * 64, (page_b * p.kv_heads + g) * KEYS, full);
    }
  };
  // page i of the walk; past its end the last page again (an odd number of pages: its keys are masked)
  auto page_of = [&](int i) { return pages[min(i, n_pages - 1)]; };
  if (copy_warp && lane == 0) {
    for (int c = 0; c < 2; ++c) {
      mbar_init(bar_s(c), 1);
      mbar_init(bar_p(c), TQ);
      mbar_init(bar_end(c), 1);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_k + 8 * s, 1);
      mbar_init(bar_v + 8 * s, 1);
      mbar_init(bar_kfree + 8 * s, 1);
      mbar_init(bar_vfree + 8 * s, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    // the first stages are asked for at once: they travel while Q is fetched and tensor memory allocated
    for (int j = 0; j < STAGES && j < n_steps; ++j) {
      const int pa = page_of(2 * j), pb = page_of(2 * j + 1);
      ask(k_ring, &k_map, bar_k + 8 * (j % STAGES), j, pa, pb);
      ask(v_ring, &v_map, bar_v + 8 * (j % STAGES), j, pa, pb);
    }
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  const bool chain_on = chain == 0 || two;
  if (!mma_warp && !copy_warp && chain_on) {
    unsigned char* q_tile = q_tiles + chain * TILE_Q_BYTES;
    const uint32_t qs = smem_u32(q_tile);
    const int h = h0 + chain;
    for (int i = row; i < TQ * (D / 8); i += TQ) {
      const int r = i / (D / 8), c = i % (D / 8);
      if (r < tok_valid)
        cp_async16(qs + swz_tc<TQ>(r, c), q + (size_t(start + q0 + r) * p.heads + h) * D + c * 8);
      else
        *reinterpret_cast<uint4*>(q_tile + swz_tc<TQ>(r, c)) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    proxy_fence_async();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool alive = true;

  if (copy_warp) {
    if (lane == 0) {
      int k_asked = min(n_steps, STAGES), v_asked = k_asked;
      for (int j = STAGES; j < n_steps && alive; ++j) {
        const int pa = page_of(2 * j), pb = page_of(2 * j + 1);
        const uint32_t before = ((j / STAGES) - 1) & 1;
        alive = mbar_wait(bar_kfree + 8 * (j % STAGES), before, error_flag, 6);
        if (!alive) break;
        ask(k_ring, &k_map, bar_k + 8 * (j % STAGES), j, pa, pb);
        k_asked = j + 1;
        alive = mbar_wait(bar_vfree + 8 * (j % STAGES), before, error_flag, 6);
        if (!alive) break;
        ask(v_ring, &v_map, bar_v + 8 * (j % STAGES), j, pa, pb);
        v_asked = j + 1;
      }
      if (!alive) {
        // a wait ran out: what is in flight lands before the block ends (bounded waits again)
        for (int j = max(0, k_asked - STAGES); j < k_asked; ++j) mbar_wait(bar_k + 8 * (j % STAGES), (j / STAGES) & 1, error_flag, 6);
        for (int j = max(0, v_asked - STAGES); j < v_asked; ++j) mbar_wait(bar_v + 8 * (j % STAGES), (j / STAGES) & 1, error_flag, 6);
      }
    }
  } else if (mma_warp) {
    if (lane == 0) {
      constexpr uint32_t IDESC_S = idesc_bf16(TQ, STEP_KEYS, false);
      constexpr uint32_t IDESC_PV = idesc_bf16(TQ, D, true);
      const uint64_t desc_q0 = smem_desc(smem_u32(q_tiles), 16, 1024);
      const uint64_t desc_k0 = smem_desc(smem_u32(k_ring), 16, 1024);
      // V is MN-major: blocks of 64 dims lie STEP_KEYS * 128 bytes apart (the leading offset), groups of 8
      // keys 1024 bytes (the stride offset)
      const uint64_t desc_v0 = smem_desc(smem_u32(v_ring), STEP_KEYS * 128, 1024);
      constexpr uint64_t STAGE_UNITS = STAGE_BYTES >> 4, Q_UNITS = TILE_Q_BYTES >> 4;
      constexpr uint64_t Q_BLOCK = (TQ * 128) >> 4, K_BLOCK = (STEP_KEYS * 128) >> 4;
      const int n_chains = two ? 2 : 1;
      int s_next[2] = {0, 0};   // next step whose S is to be issued, per chain
      int p_next[2] = {0, 0};   // next step whose O += P V is to be issued
      int k_freed = 0, v_freed = 0;
      uint32_t idle = 0;
      auto behind = [&](const int* v) { return n_chains == 2 ? min(v[0], v[1]) : v[0]; };
      while (behind(p_next) < n_steps && alive) {
        bool moved = false;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (c >= n_chains) continue;
          // O += P V of step i when its P is written (O rescaled) and its V has landed
          const int i = p_next[c];
          if (i < s_next[c] && mbar_test(bar_p(c), i & 1) && mbar_test(bar_v + 8 * (i % STAGES), (i / STAGES) & 1)) {
            tc_fence_after();
            const uint32_t o = tmem_base + c * CHAIN_COLS + TMEM_O, pp = tmem_base + c * CHAIN_COLS;
            const uint64_t dv = desc_v0 + (i % STAGES) * STAGE_UNITS;
            tc_mma4_ts<128>(o, pp, dv, IDESC_PV, i > 0 ? 1u : 0u);                       // keys 0..63 of the step
            tc_mma4_ts<128>(o, pp + 32, dv + ((KEYS * 128) >> 4), IDESC_PV, 1u);          // keys 64..127
            if (i + 1 == n_steps) tc_commit(bar_end(c));
            p_next[c] = i + 1;
            moved = true;
            while (v_freed < behind(p_next)) {   // both chains' products of the step have been issued
              tc_commit(bar_vfree + 8 * (v_freed % STAGES));
              ++v_freed;
            }
          }
          // S of step j: the buffer held S and P of step j - 1, whose O += P V must have been issued
          const int j = s_next[c];
          if (j < n_steps && j == p_next[c] && mbar_test(bar_k + 8 * (j % STAGES), (j / STAGES) & 1)) {
            tc_fence_after();
#pragma unroll
            for (int blk = 0; blk < D / 64; ++blk)
              tc_mma4<2, 2>(tmem_base + c * CHAIN_COLS, desc_q0 + c * Q_UNITS + blk * Q_BLOCK,
                            desc_k0 + (j % STAGES) * STAGE_UNITS + blk * K_BLOCK, IDESC_S, blk > 0 ? 1u : 0u);
            tc_commit(bar_s(c));
            s_next[c] = j + 1;
            moved = true;
            while (k_freed < behind(s_next)) {
              tc_commit(bar_kfree + 8 * (k_freed % STAGES));
              ++k_freed;
            }
          }
        }
        if (moved) idle = 0;
        else if (++idle > POLL_LIMIT) {
          atomicExch(error_flag, 13);
          alive = false;
        } else {
          // nothing to issue: park on what the chain further behind waits for (a spinning thread would take
          // issue slots from the softmax warps of its quarter of the SM)
          const bool second = n_chains == 2 && p_next[1] < p_next[0];
          const int i = second ? p_next[1] : p_next[0], sn = second ? s_next[1] : s_next[0];
          if (i < sn) mbar_park(bar_p(second ? 1 : 0), i & 1, 200);
          else mbar_park(bar_k + 8 * (i % STAGES), (i / STAGES) & 1, 200);
        }
      }
    }
  } else if (chain_on) {
    // ------------------------------------------------------------ softmax threads of chain `chain`
    const int h = h0 + chain;
    const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16) + chain * CHAIN_COLS;
    const uint32_t o_addr = lane_addr + TMEM_O;
    float m_run = -INFINITY, l_run = 0.f;
    const float slope = BIAS ? p.slopes[h] : 0.f;
    const float sl2 = p.scale * 1.4426950408889634f;
    const uint64_t sl2_2 = pack2(sl2, sl2);
    for (int j = 0; j < n_steps; ++j) {
      if (alive) alive = mbar_wait(bar_s(chain), j & 1, error_flag, 1);
      tc_fence_after();
      const int key0 = j * STEP_KEYS;
      const bool masked = key0 + STEP_KEYS - 1 > past + q0 || !row_ok;   // first part is uniform over the block
      // (1) the row's maximum over the step's 128 scores, a half of 64 at a time
      float m_new = m_run;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float s[KEYS];
        tmem_ld64_once(lane_addr + half * KEYS, s);
        if (BIAS) {
#pragma unroll
          for (int e = 0; e < KEYS; ++e) s[e] += alibi_bias(slope, key0 + half * KEYS + e);
        }
        if (masked) {
          const int visible = row_pos - key0 - half * KEYS;
#pragma unroll
          for (int e = 0; e < KEYS; ++e) s[e] = (e <= visible) ? s[e] : -INFINITY;
        }
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < KEYS; e += 8) {
          mx[0] = max3(mx[0], s[e], s[e + 1]);
          mx[1] = max3(mx[1], s[e + 2], s[e + 3]);
          mx[2] = max3(mx[2], s[e + 4], s[e + 5]);
          mx[3] = max3(mx[3], s[e + 6], s[e + 7]);
        }
        m_new = fmaxf(m_new, fmaxf(max3(mx[0], mx[1], mx[2]), mx[3]));
      }
      if ((m_new - m_run) * sl2 <= RESCALE_LOG2) m_new = m_run;   // (false from -inf: the first scores set it)
      const float corr = (m_run == -INFINITY) ? 0.f : fast_exp2((m_run - m_new) * sl2);
      const bool moved = (m_new != m_run) && (m_run != -INFINITY);
      m_run = m_new;
      const float m_off = (m_run == -INFINITY) ? 0.f : m_run * sl2;
      // (2) O rescaled if any row of the warp moved its maximum: O += P V of the step before has completed
      // (S of this step was issued after it)
      if (j > 0 && __any_sync(0xffffffffu, moved)) {
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          float o[32];
          tmem_ld32(o_addr + c0, o);
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] *= corr;
          tmem_st32(o_addr + c0, o);
        }
        tmem_st_wait();
      }
      // (3) P = exp2(S - max), a half at a time: the first half's P goes over the first half's S (read for
      // the last time just before), the second half's P over the rest of the first half's S
      const uint64_t moff_2 = pack2(-m_off, -m_off);
      uint64_t acc2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float s[KEYS];
        tmem_ld64_once(lane_addr + half * KEYS, s);
        if (BIAS) {
#pragma unroll
          for (int e = 0; e < KEYS; ++e) s[e] += alibi_bias(slope, key0 + half * KEYS + e);
        }
        if (masked) {
          const int visible = row_pos - key0 - half * KEYS;
#pragma unroll
          for (int e = 0; e < KEYS; ++e) s[e] = (e <= visible) ? s[e] : -INFINITY;
        }
        uint32_t w[KEYS / 2];
#pragma unroll
        for (int e = 0; e < KEYS / 2; ++e) {
          float x0, x1;
          unpack2(fma2(pack2(s[2 * e], s[2 * e + 1]), sl2_2, moff_2), x0, x1);
          const float a = fast_exp2(x0), b = fast_exp2(x1);
          acc2[e & 3] = add2(acc2[e & 3], pack2(a, b));
          w[e] = pack_bf16(a, b);
        }
        tmem_st_u32<KEYS / 2>(lane_addr + half * (KEYS / 2), w);
      }
      tmem_st_wait();
      float l0, l1, l2, l3;
      unpack2(add2(acc2[0], acc2[1]), l0, l1);
      unpack2(add2(acc2[2], acc2[3]), l2, l3);
      l_run = l_run * corr + ((l0 + l1) + (l2 + l3));
      tc_fence_before();
      mbar_arrive(bar_p(chain));
    }
    if (alive) alive = mbar_wait(bar_end(chain), 0, error_flag, 3);
    tc_fence_after();
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* dst = out + (size_t(start + q0 + row) * p.heads + h) * D;
#pragma unroll
    for (int c0 = 0; c0 < D; c0 += 32) {
      float o[32];
      tmem_ld32(o_addr + c0, o);
      if (row_ok) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) w[e] = pack_bf16(o[c * 8 + 2 * e] * inv, o[c * 8 + 2 * e + 1] * inv);
          *reinterpret_cast<uint4*>(dst + c0 + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
}

template <int D, bool BIAS>
int launch_tc_pair(const void* q, const void* k_pool, const void* v_pool, int pool_pages, void* out, const StepBatch& sb,
                   const int* tile_seq, const int* tile_q0, int n_tiles, const TcParams& p, int* error_flag,
                   cudaStream_t stream) {
  const CUtensorMap* km = pool_map(k_pool, pool_pages, p.kv_heads, D);
  const CUtensorMap* vm = pool_map(v_pool, pool_pages, p.kv_heads, D);
  if (km == nullptr || vm == nullptr) return PTB_ERR_LAUNCH;
  constexpr size_t smem = PairShape<D>::SMEM;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_tc_pair_kernel<D, BIAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = true;
  }
  const int qpk = p.heads / p.kv_heads;
  dim3 grid(p.kv_heads * ((qpk + 1) / 2), n_tiles);
  attention_tc_pair_kernel<D, BIAS><<<grid, PAIR_THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, (__nv_bfloat16*)out, sb, tile_seq, tile_q0, p, *km, *vm, error_flag);
  return launch_status();
}
}  // namespace

static int g_pair_mode = 1;
// for measurements and tests: 0 = every head a block of its own also where pairs would do, 1 = pairs where
// they fill the device (the default), 2 = pairs wherever a K/V group has two heads or more
PTB_API void ptb_attention_tc_pairs(int mode) { g_pair_mode = mode; }
PTB_API int ptb_attention_tc_supports(int head_dim) { return (head_dim == 64 || head_dim == 128) ? 1 : 0; }
PTB_API int ptb_attention_tc_tile_tokens() { return TQ; }

namespace {
template <int D, bool BIAS>
int launch_tc(const void* q, const void* k_pool, const void* v_pool, int pool_pages, void* out, const StepBatch& sb,
              const int* tile_seq, const int* tile_q0, int n_tiles, const TcParams& p, int* error_flag,
              cudaStream_t stream) {
  const CUtensorMap* km = pool_map(k_pool, pool_pages, p.kv_heads, D);
  const CUtensorMap* vm = pool_map(v_pool, pool_pages, p.kv_heads, D);
  if (km == nullptr || vm == nullptr) return PTB_ERR_LAUNCH;
  const size_t smem = 1024 + TQ * D * 2 + 2 * STAGES_TC * KEYS * D * 2 + 192;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_tc_kernel<D, BIAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = true;
  }
  dim3 grid(p.heads, n_tiles);
  attention_tc_kernel<D, BIAS><<<grid, BLOCK_THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, sb,
      tile_seq, tile_q0, p, *km, *vm, error_flag);
  return launch_status();
}
}  // namespace

// Causal attention of prompt tiles of 128 tokens (tile_seq / tile_q0 as for the other attention
// kernels, 128 tokens per tile), bfloat16, head size 64 or 128, no window. k_pool / v_pool: the pools of
// one cache entry, [pool_pages][kv_heads][64][head_dim]. `slopes`: per-head score
// slopes [heads] float32 (already rounded to bfloat16 values), or null. `error_flag` is a device int
// that stays 0 unless a bounded wait inside the kernel ran out.
PTB_API int ptb_attention_tc(const void* q, const void* k_pool, const void* v_pool, int pool_pages, void* out,
                             const StepBatch* sb,
                             const int* tile_seq, const int* tile_q0, int n_tiles, const float* slopes, int heads,
                             int kv_heads, int head_dim, float scale, int* error_flag, cudaStream_t stream) {
  if (n_tiles <= 0) return PTB_OK;
  if (pool_pages <= 0 || (reinterpret_cast<uintptr_t>(k_pool) | reinterpret_cast<uintptr_t>(v_pool)) & 15) return PTB_ERR_ALIGN;
  if ((head_dim != 64 && head_dim != 128) || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || n_tiles > 65535 ||
      error_flag == nullptr)
    return PTB_ERR_SIZE;
  TcParams p;
  p.heads = heads; p.kv_heads = kv_heads; p.scale = scale; p.slopes = slopes;
  if (head_dim == 64)
    return slopes ? launch_tc<64, true>(q, k_pool, v_pool, pool_pages, out, *sb, tile_seq, tile_q0, n_tiles, p, error_flag, stream)
                  : launch_tc<64, false>(q, k_pool, v_pool, pool_pages, out, *sb, tile_seq, tile_q0, n_tiles, p, error_flag, stream);
  // Head size 128 leaves room for one block an SM: two heads of a K/V group share a block, with keys in
  // steps of two pages, where a group has two heads or more and the pairs fill the device. (With head size
  // 64 two blocks of the kernel above share an SM, each with three S buffers, and are a quarter faster than
  // the pairs with their one S buffer a chain: 833 against 1,067 us at 8,192 tokens and 71 heads.)
  const int qpk = heads / kv_heads;
  const long long pair_blocks = (long long)kv_heads * ((qpk + 1) / 2) * n_tiles;
  if (qpk >= 2 && g_pair_mode != 0 && (pair_blocks >= sm_count() || g_pair_mode == 2))
    return slopes ? launch_tc_pair<128, true>(q, k_pool, v_pool, pool_pages, out, *sb, tile_seq, tile_q0, n_tiles, p, error_flag, stream)
                  : launch_tc_pair<128, false>(q, k_pool, v_pool, pool_pages, out, *sb, tile_seq, tile_q0, n_tiles, p, error_flag, stream);
  return slopes ? launch_tc<128, true>(q, k_pool, v_pool, pool_pages, out, *sb, tile_seq, tile_q0, n_tiles, p, error_flag, stream)
                : launch_tc<128, false>(q, k_pool, v_pool, pool_pages, out, *sb, tile_seq, tile_q0, n_tiles, p, error_flag, stream);
}
