// Linear layer for a few rows (decode steps): y[m, n] = act(sum_k x[m, k] w[n, k] + bias[n]) + add[m, n]
// for m < 16 or 32, bfloat16 operands, float32 accumulation and epilogue. The work is the read of
// the weight matrix, once, at memory speed: the kernel is built around that stream.
//
// A block owns 16 * MT consecutive weight rows (output columns) and all of K; its 8 warps take
// 32-wide chunks of K in turn and join their partial sums through shared memory. Weights go from
// global memory straight into tensor-core fragments: the weight tile is the A operand (16 rows x 16
// k) and the few activation rows are the B operand (16 k x 8 rows) of mma.m16n8k16. A dot product
// does not care in which order k is visited, so each thread loads 16 contiguous bytes (8 values of
// k) of a weight row and of an activation row and feeds them to two mma instructions; both operands
// use the same permutation of k, and every 32-byte sector that is fetched is used in full.
#include "common.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int KC = 32;  // k values per chunk (one 16-byte load per thread and operand row)

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// steps c0 = first, first + stride, ... below `limit`; a step has the UNROLL chunks c0, c0 + apart,
// c0 + 2 apart, ... in flight together (those past the last chunk are skipped)
template <int MT, int NT, int UNROLL>
__device__ __forceinline__ void sweep(float (&acc)[MT][NT][4], const __nv_bfloat16* const (&wrow)[MT][2],
                                      const __nv_bfloat16* const (&xrow)[NT], const bool (&xok)[NT], int first,
                                      int limit, int stride, int apart, int chunks) {
  for (int c0 = first; c0 < limit; c0 += stride) {
    uint4 wa[UNROLL][MT][2];
    uint4 xb[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int c = c0 + u * apart;
      if (c < chunks) {
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          wa[u][i][0] = ld_stream16(wrow[i][0] + size_t(c) * KC);
          wa[u][i][1] = ld_stream16(wrow[i][1] + size_t(c) * KC);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int c = c0 + u * apart;
      if (c < chunks) {
#pragma unroll
        for (int j = 0; j < NT; ++j)
          xb[u][j] = xok[j] ? *reinterpret_cast<const uint4*>(xrow[j] + size_t(c) * KC) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      if (c0 + u * apart < chunks) {
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            // the thread's 8 k values: .x .y feed the first mma (as k pairs 2t and 2t + 8), .z .w the second
            mma16816(acc[i][j], wa[u][i][0].x, wa[u][i][1].x, wa[u][i][0].y, wa[u][i][1].y, xb[u][j].x, xb[u][j].y);
            mma16816(acc[i][j], wa[u][i][0].z, wa[u][i][1].z, wa[u][i][0].w, wa[u][i][1].w, xb[u][j].z, xb[u][j].w);
          }
      }
    }
  }
}

// MT: 16-row weight tiles per block; NT: 8-row activation tiles (M <= 8 * NT)
template <int MT, int NT, int UNROLL>
__global__ void __launch_bounds__(WARPS * 32)
skinny_linear_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                     const float* __restrict__ bias, const __nv_bfloat16* __restrict__ add,
                     __nv_bfloat16* __restrict__ y_bf16, float* __restrict__ y_f32, int M, int N, int K, int act,
                     int ksplit, float* __restrict__ scratch, int* __restrict__ tickets) {
  __shared__ float red[WARPS][MT * 16][NT * 8 + 1];
  __shared__ int is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  // ksplit blocks share a tile of weight rows, each with a share of K
  const int rank = blockIdx.x % ksplit, tile = blockIdx.x / ksplit;
  const int n0 = tile * (16 * MT);
  float acc[MT][NT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

  // rows of w this thread reads (clamped at the matrix edge; those results are never stored)
  const __nv_bfloat16* wrow[MT][2];
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    wrow[i][0] = w + size_t(min(n0 + i * 16 + g, N - 1)) * K + t * 8;
    wrow[i][1] = w + size_t(min(n0 + i * 16 + g + 8, N - 1)) * K + t * 8;
  }
  const __nv_bfloat16* xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    xok[j] = (j * 8 + g) < M;
    xrow[j] = x + size_t(xok[j] ? j * 8 + g : 0) * K + t * 8;
  }

  // The warps take the 32-wide chunks of K in turn, UNROLL chunks at a time: at any moment the block
  // reads WARPS * UNROLL consecutive chunks of every weight row (one stretch of a DRAM page). What
  // is left after the last full round is dealt round the warps chunk by chunk, in one more step, so
  // that no warp idles.
  const int chunks_all = K / KC;
  const int per_block = (chunks_all + ksplit - 1) / ksplit;
  const int c_begin = min(chunks_all, rank * per_block), chunks = min(chunks_all, c_begin + per_block);
  const int full = (chunks - c_begin) / (WARPS * UNROLL) * (WARPS * UNROLL);
  sweep<MT, NT, UNROLL>(acc, wrow, xrow, xok, c_begin + warp * UNROLL, c_begin + full, WARPS * UNROLL, 1, chunks);
  sweep<MT, NT, UNROLL>(acc, wrow, xrow, xok, c_begin + full + warp, c_begin + full + WARPS, WARPS, WARPS, chunks);
  // partial sums of the 8 warps -> shared memory: red[warp][weight row][activation row]
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      red[warp][i * 16 + g][j * 8 + 2 * t] = acc[i][j][0];
      red[warp][i * 16 + g][j * 8 + 2 * t + 1] = acc[i][j][1];
      red[warp][i * 16 + g + 8][j * 8 + 2 * t] = acc[i][j][2];
      red[warp][i * 16 + g + 8][j * 8 + 2 * t + 1] = acc[i][j][3];
    }
  __syncthreads();
  constexpr int TILE_ELEMS = MT * 16 * NT * 8;
  if (ksplit > 1) {
    // This block's partial sums go to its slot of the scratch buffer; the block of the tile that
    // arrives last (a ticket per tile, put back to zero by that block) sums the slots in the order
    // of the blocks and runs the epilogue. No atomics on values: the result does not depend on who
    // arrives when.
    float* mine = scratch + (size_t(tile) * ksplit + rank) * TILE_ELEMS;
    for (int idx = threadIdx.x; idx < TILE_ELEMS; idx += WARPS * 32) {
      const int r = idx % (MT * 16), m = idx / (MT * 16);
      float v = 0.f;
#pragma unroll
      for (int wi = 0; wi < WARPS; ++wi) v += red[wi][r][m];
      mine[idx] = v;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int arrived = atomicAdd(&tickets[tile], 1);
      is_last = (arrived == ksplit - 1) ? 1 : 0;
      if (is_last) tickets[tile] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
  }
  // epilogue: thread -> (activation row m, weight row r); consecutive threads take consecutive r,
  // which are consecutive addresses of y
  for (int idx = threadIdx.x; idx < MT * 16 * NT * 8; idx += WARPS * 32) {
    const int r = idx % (MT * 16), m = idx / (MT * 16);
    const int n = n0 + r;
    if (m >= M || n >= N) continue;
    float v = 0.f;
    if (ksplit > 1) {
      for (int b = 0; b < ksplit; ++b) v += __ldcg(scratch + (size_t(tile) * ksplit + b) * TILE_ELEMS + idx);
    } else {
#pragma unroll
      for (int wi = 0; wi < WARPS; ++wi) v += red[wi][r][m];
    }
    if (bias) v += bias[n];
    v = apply_activation(v, act);
    if (add) v += __bfloat162float(add[size_t(m) * N + n]);
    if (y_f32) y_f32[size_t(m) * N + n] = v;
    else y_bf16[size_t(m) * N + n] = __float2bfloat16_rn(v);
  }
}

// Blocks per tile of weight rows, each with a share of K. The blocks of a launch are all resident at
// once and share the SMs' memory bandwidth, so the launch takes as long as the SM with the most blocks:
// 512 tiles on 148 SMs are 3.46 a piece, some SMs get 4, and the launch takes 16 % longer than its share
// of the bandwidth. Dividing K by 2, 3 or 4 changes the count to one that divides better. Taken when it
// saves more than 3 %, every block keeps at least 16 full rounds of its warps (blocks with a short K are
// slower per byte: K = 16384 in 4 shares 30.8 us against 24.6 us undivided; K = 32768 in 2 shares 95
// against 111 us), and the caller has given scratch memory and tickets.
int k_split(int tiles, int chunks, int round) {
  const int sms = sm_count();
  auto excess = [&](int blocks) { return double((blocks + sms - 1) / sms) * sms / blocks; };
  int best = 1;
  double best_excess = excess(tiles);
  for (int s = 2; s <= 4; ++s) {
    if (chunks / s < 16 * round) break;
    const double e = excess(tiles * s);
    if (e < best_excess - 0.03) {
      best = s;
      best_excess = e;
    }
  }
  return best;
}

template <int MT, int NT, int U>
int launch_skinny(const void* x, const void* w, const float* bias, const void* add, void* y_bf16, float* y_f32,
                  int M, int N, int K, int act, float* scratch, size_t scratch_floats, int* tickets, int n_tickets,
                  size_t* need_floats, cudaStream_t stream) {
  const int tiles = (N + 16 * MT - 1) / (16 * MT);
  int ksplit = k_split(tiles, K / KC, WARPS * U);
  const size_t need = ksplit > 1 ? size_t(tiles) * ksplit * (MT * 16 * NT * 8) : 0;
  if (need_floats != nullptr) {   // a question, not a launch
    *need_floats = need;
    return PTB_OK;
  }
  if (scratch == nullptr || tickets == nullptr || scratch_floats < need || n_tickets < tiles) ksplit = 1;
  skinny_linear_kernel<MT, NT, U><<<tiles * ksplit, WARPS * 32, 0, stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, (const __nv_bfloat16*)add, (__nv_bfloat16*)y_bf16,
      y_f32, M, N, K, act, ksplit, scratch, tickets);
  return launch_status();
}

int dispatch_skinny(const void* x, const void* w, const float* bias, const void* add, void* y_bf16, float* y_f32, int M,
                    int N, int K, int act, float* scratch, size_t scratch_floats, int* tickets, int n_tickets,
                    size_t* need_floats, cudaStream_t stream) {
  // Tile height and chunks in flight per warp, from a sweep over matrices of 4,096 to 65,024 rows (each
  // alone, from HBM): matrices with four tiles or more per SM (many rows, short K) want 32 rows per
  // block and four chunks in flight at up to 8 activation rows, 16 rows and two chunks at up to 16;
  // the others 16 rows and four chunks.
  const bool wide = N >= 16 * sm_count() * 4;   // four 16-row tiles or more per SM
#define PTB_SKINNY(MT, NT, U) \
  return launch_skinny<MT, NT, U>(x, w, bias, add, y_bf16, y_f32, M, N, K, act, scratch, scratch_floats, tickets, \
                                  n_tickets, need_floats, stream)
  if (M <= 8) {
    if (wide) PTB_SKINNY(2, 1, 4);
    PTB_SKINNY(1, 1, 4);
  }
  if (M <= 16) {
    if (wide) PTB_SKINNY(1, 2, 2);
    PTB_SKINNY(1, 2, 4);
  }
  if (wide) PTB_SKINNY(2, 4, 2);
  PTB_SKINNY(1, 4, 4);
#undef PTB_SKINNY
}

}  // namespace

// rows that the kernel takes at most, and the multiple that K must be of
PTB_API int ptb_skinny_linear_max_rows() { return 32; }
PTB_API int ptb_skinny_linear_k_multiple() { return KC; }

// y = act(x w^T + bias) + add. x [M, K], w [N, K], add [M, N] bfloat16; bias float32 [N];
// exactly one of y_bf16, y_f32 is given. M <= 32, K a multiple of 32, 16-byte aligned x and w.
// scratch (float32, scratch_floats of them) and tickets (int32, n_tickets of them, all zero between
// launches: the kernel puts them back) let the kernel divide K among several blocks per tile where that
// balances the SMs; without them it does not divide. ptb_skinny_linear_scratch says how many floats a
// launch would use.
PTB_API int ptb_skinny_linear(const void* x, const void* w, const float* bias, const void* add, void* y_bf16,
                              float* y_f32, int M, int N, int K, int act, float* scratch, size_t scratch_floats,
                              int* tickets, int n_tickets, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return PTB_OK;
  if (M > 32 || K <= 0 || K % KC != 0 || !activation_known(act)) return PTB_ERR_SIZE;
  if ((y_bf16 == nullptr) == (y_f32 == nullptr)) return PTB_ERR_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return PTB_ERR_ALIGN;
  return dispatch_skinny(x, w, bias, add, y_bf16, y_f32, M, N, K, act, scratch, scratch_floats, tickets, n_tickets,
                         nullptr, stream);
}

PTB_API long long ptb_skinny_linear_scratch(int M, int N, int K) {
  if (M <= 0 || N <= 0 || M > 32 || K <= 0 || K % KC != 0) return 0;
  size_t need = 0;
  dispatch_skinny(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, M, N, K, 0, nullptr, 0, nullptr, 0, &need, nullptr);
  return (long long)need;
}
