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
      // all D dims of the output in one instruction: the tensor pipe takes a matrix instruction about every
      // hundred clocks whatever its N, so their number is what a page costs
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
// Two query heads of one K/V group in a block ("pair"): for shapes whose tiles leave room for one block
// an SM only (head size 128: 32 KB of Q and 32 KB a page), a block of one head is one chain of dependent
// steps per page and the SM idles between them. Here a block holds two chains that share every page
// stage: 128 tokens x heads (2j, 2j + 1), 256 softmax threads (threads 0..127 head 2j, 128..255 head
// 2j + 1; both groups sit on tensor-memory lanes 0..127, the second on columns 256..511), one issuing
// thread that serves whichever chain is ready, one copy warp. Per chain: two S buffers (S one page ahead
// of the softmax, the third buffer's column space goes to the second chain), P in place of S, O.
//
// The issuing thread never blocks on one chain while the other could move: it polls (mbarrier.test_wait)
// "P written" and "page landed" of both chains in turn; a page's stage goes back to the copy thread when
// both chains' O += P V of that page have been issued. Its polling is bounded like every wait.
// "O updated" has two barriers a chain: with S two pages ahead of O += P V at most, a thread that has read S
// of page i knows that the product of page i - 2 has completed, the one before page i on its barrier.
constexpr int PAIR_SOFTMAX = 2 * TQ;
constexpr int PAIR_THREADS = PAIR_SOFTMAX + 64;
constexpr uint32_t POLL_LIMIT = 1u << 26;
#ifndef PTB_PARK_NS
#define PTB_PARK_NS 200
#endif

__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

template <int D, bool BIAS>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
attention_tc_pair_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, StepBatch sb,
                         const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, TcParams p,
                         const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                         int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  constexpr int TILE_Q_BYTES = TQ * D * 2;
  constexpr int TILE_KV_BYTES = KEYS * D * 2;
  // tensor memory of chain c: columns [256 c, 256 c + 256): S buffers at +0 and +64, O at +128
  constexpr uint32_t CHAIN_COLS = 256, TMEM_O = 128;
  unsigned char* q_tiles = smem;                                       // two Q tiles
  unsigned char* k_ring = q_tiles + 2 * TILE_Q_BYTES;
  unsigned char* v_ring = k_ring + STAGES_TC * TILE_KV_BYTES;
  // barriers: per chain c at 6 c: [0..1] S written, [2..3] O updated, [4..5] P written (page % 2); then per
  // stage: page landed, stage free again
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_ring + STAGES_TC * TILE_KV_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12 + 2 * STAGES_TC);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool mma_warp = warp == PAIR_SOFTMAX / 32;
  const bool copy_warp = warp == PAIR_SOFTMAX / 32 + 1;
  const int chain = (tid >> 7) & 1;      // softmax threads: which head of the pair
  const int row = tid & (TQ - 1);        // query row = tensor-memory lane
  const int tile = blockIdx.y;
  const int qpk = p.heads / p.kv_heads;
  const int h0 = 2 * blockIdx.x;         // heads h0 and h0 + 1: the same K/V group (qpk is even)
  const int g = h0 / qpk;
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int n_new = sb.seq_new[seq], past = sb.seq_past[seq], start = sb.seq_start[seq];
  const int tok_valid = min(TQ, n_new - q0);
  const bool row_ok = row < tok_valid;
  const int row_pos = row_ok ? past + q0 + row : -1;
  const int last_pos = past + q0 + tok_valid - 1;
  const int n_blocks = last_pos / KEYS + 1;
  const int* pages = sb.pages + size_t(seq) * sb.pages_stride;

  const uint32_t bar0 = smem_u32(bars);
  auto bar_s = [&](int c, int b) { return bar0 + 8u * uint32_t(6 * c + b); };
  auto bar_o = [&](int c, int b) { return bar0 + 8u * uint32_t(6 * c + 2 + b); };
  auto bar_p = [&](int c, int b) { return bar0 + 8u * uint32_t(6 * c + 4 + b); };
  const uint32_t bar_k = bar0 + 8u * 12, bar_free = bar_k + 8u * STAGES_TC;
  constexpr uint32_t PAGE_BYTES = 2 * TILE_KV_BYTES;
  auto ask_page = [&](int b, int page) {
    const int st = b % STAGES_TC;
    const int y = (page * p.kv_heads + g) * KEYS;
    const uint32_t full = bar_k + 8 * st;
    mbar_expect_tx(full, PAGE_BYTES);
#pragma unroll
    for (int blk = 0; blk < D / 64; ++blk) {
      tma_load_2d(smem_u32(k_ring + st * TILE_KV_BYTES + blk * (KEYS * 128)), &k_map, blk * 64, y, full);
      tma_load_2d(smem_u32(v_ring + st * TILE_KV_BYTES + blk * (KEYS * 128)), &v_map, blk * 64, y, full);
    }
  };
  int first_pages = 0;
  if (copy_warp) {
    // barriers set up and the first pages asked for before the block-wide barrier, as in the kernel above
    first_pages = lane < n_blocks ? pages[lane] : 0;
    if (lane == 0) {
      for (int c = 0; c < 2; ++c)
        for (int b = 0; b < 2; ++b) {
          mbar_init(bar_s(c, b), 1);
          mbar_init(bar_o(c, b), 1);
          mbar_init(bar_p(c, b), TQ);
        }
      for (int s = 0; s < STAGES_TC; ++s) {
        mbar_init(bar_k + 8 * s, 1);
        mbar_init(bar_free + 8 * s, 1);
      }
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    for (int b = 0; b < STAGES_TC && b < n_blocks; ++b) {
      const int page = __shfl_sync(0xffffffffu, first_pages, b);
      if (lane == 0) ask_page(b, page);
    }
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  if (!mma_warp && !copy_warp) {
    // Q tile of this thread's head: rows of the tile, zero beyond the valid tokens
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
      int issued = min(n_blocks, STAGES_TC);
      for (int b = STAGES_TC; b < n_blocks; ++b) {
        if (!mbar_wait(bar_free + 8 * (b % STAGES_TC), ((b / STAGES_TC) - 1) & 1, error_flag, 6)) break;
        ask_page(b, pages[b]);
        issued = b + 1;
      }
      if (issued < n_blocks)
        for (int b = max(0, issued - STAGES_TC); b < issued; ++b)
          mbar_wait(bar_k + 8 * (b % STAGES_TC), (b / STAGES_TC) & 1, error_flag, 6);
    }
  } else if (mma_warp) {
    if (lane == 0) {
      constexpr uint32_t IDESC_S = idesc_bf16(TQ, KEYS, false);
      constexpr uint32_t IDESC_PV = idesc_bf16(TQ, D, true);   // all D dims of the output in one instruction
      const uint64_t desc_q0 = smem_desc(smem_u32(q_tiles), 16, 1024);
      const uint64_t desc_k0 = smem_desc(smem_u32(k_ring), 16, 1024);
      const uint64_t desc_v0 = smem_desc(smem_u32(v_ring), KEYS * 128, 1024);
      constexpr uint64_t STAGE_UNITS = TILE_KV_BYTES >> 4, Q_UNITS = TILE_Q_BYTES >> 4;
      constexpr uint64_t Q_BLOCK = (TQ * 128) >> 4, KV_BLOCK = (KEYS * 128) >> 4;
      int s_next[2] = {0, 0};   // next page whose S is to be issued, per chain
      int p_next[2] = {0, 0};   // next page whose O += P V is to be issued, per chain
      int freed = 0;            // pages whose stage has been given back
      uint32_t idle = 0;
      while ((p_next[0] < n_blocks || p_next[1] < n_blocks) && alive) {
        bool moved = false;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          // S of page j: its buffer (j % 2) held S and P of page j - 2, whose O += P V must have been
          // issued (the tensor pipe runs in order); the page must have landed
          const int j = s_next[c];
          if (j < n_blocks && j <= p_next[c] + 1 && mbar_test(bar_k + 8 * (j % STAGES_TC), (j / STAGES_TC) & 1)) {
            tc_fence_after();
            const int st = j % STAGES_TC;
#pragma unroll
            for (int blk = 0; blk < D / 64; ++blk)
              tc_mma4<2, 2>(tmem_base + c * CHAIN_COLS + (j & 1) * 64, desc_q0 + c * Q_UNITS + blk * Q_BLOCK,
                            desc_k0 + st * STAGE_UNITS + blk * KV_BLOCK, IDESC_S, blk > 0 ? 1u : 0u);
            tc_commit(bar_s(c, j & 1));
            s_next[c] = j + 1;
            moved = true;
          }
          // O += P V of page i when its P is written (and O rescaled)
          const int i = p_next[c];
          if (i < n_blocks && i < s_next[c] && mbar_test(bar_p(c, i & 1), (i >> 1) & 1)) {
            tc_fence_after();
            const int st = i % STAGES_TC;
            tc_mma4_ts<128>(tmem_base + c * CHAIN_COLS + TMEM_O, tmem_base + c * CHAIN_COLS + (i & 1) * 64,
                            desc_v0 + st * STAGE_UNITS, IDESC_PV, i > 0 ? 1u : 0u);
            tc_commit(bar_o(c, i & 1));
            p_next[c] = i + 1;
            moved = true;
            // a stage is free when both chains' products of its page have completed
            while (freed < min(p_next[0], p_next[1])) {
              tc_commit(bar_free + 8 * (freed % STAGES_TC));
              ++freed;
            }
          }
        }
        if (moved) idle = 0;
        else if (++idle > POLL_LIMIT) {
          atomicExch(error_flag, 13);
          alive = false;
        } else {
          // nothing to issue: park on the barrier that the chain further behind waits for, for a fraction of
          // a microsecond at most (a spinning thread would take issue slots from the softmax warps of its
          // quarter of the SM); the tests above then look at every barrier again
          const int c = p_next[0] <= p_next[1] ? 0 : 1;
          const int i = p_next[c];
          const uint32_t parked = (i < s_next[c]) ? bar_p(c, i & 1) : bar_k + 8 * (s_next[c] % STAGES_TC);
          const uint32_t parity = (i < s_next[c]) ? uint32_t((i >> 1) & 1) : uint32_t((s_next[c] / STAGES_TC) & 1);
          uint32_t ok;
          asm volatile(
              "{\n\t.reg .pred p;\n\t"
              "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
              "selp.u32 %0, 1, 0, p;\n\t}\n"
              : "=r"(ok) : "r"(parked), "r"(parity), "r"(PTB_PARK_NS) : "memory");
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax threads of chain `chain`
    const int h = h0 + chain;
    const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16) + chain * CHAIN_COLS;
    const uint32_t o_addr = lane_addr + TMEM_O;
    float m_run = -INFINITY, l_run = 0.f;
    const float slope = BIAS ? p.slopes[h] : 0.f;
    const float sl2 = p.scale * 1.4426950408889634f;
    const uint64_t sl2_2 = pack2(sl2, sl2);
    for (int i = 0; i < n_blocks; ++i) {
      const int buf = i & 1, phase = (i >> 1) & 1;
      if (alive) alive = mbar_wait(bar_s(chain, buf), phase, error_flag, 1);
      tc_fence_after();
      float s[KEYS];
      tmem_ld64_once(lane_addr + buf * 64, s);
      if (BIAS) {
#pragma unroll
        for (int j = 0; j < KEYS; ++j) s[j] += alibi_bias(slope, i * KEYS + j);
      }
      if (i * KEYS + KEYS - 1 > past + q0 || !row_ok) {
        const int visible = row_pos - i * KEYS;
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
      if ((m_new - m_run) * sl2 <= RESCALE_LOG2) m_new = m_run;
      const float corr = (m_run == -INFINITY) ? 0.f : fast_exp2((m_run - m_new) * sl2);
      const bool moved = (m_new != m_run) && (m_run != -INFINITY);
      m_run = m_new;
      const float m_off = (m_run == -INFINITY) ? 0.f : m_run * sl2;
      if (i > 0 && __any_sync(0xffffffffu, moved)) {
        if (alive) alive = mbar_wait(bar_o(chain, (i - 1) & 1), ((i - 1) >> 1) & 1, error_flag, 2);
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
      tmem_st_u32<KEYS / 2>(lane_addr + buf * 64, w);
      tmem_st_wait();
      float l0, l1, l2, l3;
      unpack2(add2(acc2[0], acc2[1]), l0, l1);
      unpack2(add2(acc2[2], acc2[3]), l2, l3);
      l_run = l_run * corr + ((l0 + l1) + (l2 + l3));
      tc_fence_before();
      mbar_arrive(bar_p(chain, buf));
    }
    if (alive) alive = mbar_wait(bar_o(chain, (n_blocks - 1) & 1), ((n_blocks - 1) >> 1) & 1, error_flag, 3);
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

}  // namespace

static bool g_no_pair = false;
// for measurements: 0 = every head its own block also where pairs would do
PTB_API void ptb_attention_tc_pairs(int on) { g_no_pair = on == 0; }
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
template <int D, bool BIAS>
int launch_tc_pair(const void* q, const void* k_pool, const void* v_pool, int pool_pages, void* out, const StepBatch& sb,
                   const int* tile_seq, const int* tile_q0, int n_tiles, const TcParams& p, int* error_flag,
                   cudaStream_t stream) {
  const CUtensorMap* km = pool_map(k_pool, pool_pages, p.kv_heads, D);
  const CUtensorMap* vm = pool_map(v_pool, pool_pages, p.kv_heads, D);
  if (km == nullptr || vm == nullptr) return PTB_ERR_LAUNCH;
  const size_t smem = 1024 + 2 * TQ * D * 2 + 2 * STAGES_TC * KEYS * D * 2 + 256;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_tc_pair_kernel<D, BIAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = true;
  }
  dim3 grid(p.heads / 2, n_tiles);
  attention_tc_pair_kernel<D, BIAS><<<grid, PAIR_THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, (__nv_bfloat16*)out, sb, tile_seq, tile_q0, p, *km, *vm, error_flag);
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
  // head size 128 leaves room for one block an SM: two heads of a K/V group share a block where the group
  // has an even number of heads
  if ((heads / kv_heads) % 2 == 0 && !g_no_pair)
    return slopes ? launch_tc_pair<128, true>(q, k_pool, v_pool, pool_pages, out, *sb, tile_seq, tile_q0, n_tiles, p, error_flag, stream)
                  : launch_tc_pair<128, false>(q, k_pool, v_pool, pool_pages, out, *sb, tile_seq, tile_q0, n_tiles, p, error_flag, stream);
  return slopes ? launch_tc<128, true>(q, k_pool, v_pool, pool_pages, out, *sb, tile_seq, tile_q0, n_tiles, p, error_flag, stream)
                : launch_tc<128, false>(q, k_pool, v_pool, pool_pages, out, *sb, tile_seq, tile_q0, n_tiles, p, error_flag, stream);
}
