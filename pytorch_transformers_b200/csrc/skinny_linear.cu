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
__device__ __forceinline__ float act_f(float v, int act) {
  switch (act) {
    case 1: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
    case 2: return 0.5f * v * (1.0f + tanhf(0.79788456080286535588f * (v + 0.044715f * v * v * v)));
    case 3: return fmaxf(v, 0.f);
    default: return v;
  }
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
                     __nv_bfloat16* __restrict__ y_bf16, float* __restrict__ y_f32, int M, int N, int K, int act) {
  __shared__ float red[WARPS][MT * 16][NT * 8 + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * (16 * MT);
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
  const int chunks = K / KC;
  const int full = chunks / (WARPS * UNROLL) * (WARPS * UNROLL);
  sweep<MT, NT, UNROLL>(acc, wrow, xrow, xok, warp * UNROLL, full, WARPS * UNROLL, 1, chunks);
  sweep<MT, NT, UNROLL>(acc, wrow, xrow, xok, full + warp, full + WARPS, WARPS, WARPS, chunks);
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
  // epilogue: thread -> (activation row m, weight row r); consecutive threads take consecutive r,
  // which are consecutive addresses of y
  for (int idx = threadIdx.x; idx < MT * 16 * NT * 8; idx += WARPS * 32) {
    const int r = idx % (MT * 16), m = idx / (MT * 16);
    const int n = n0 + r;
    if (m >= M || n >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int wi = 0; wi < WARPS; ++wi) v += red[wi][r][m];
    if (bias) v += bias[n];
    v = act_f(v, act);
    if (add) v += __bfloat162float(add[size_t(m) * N + n]);
    if (y_f32) y_f32[size_t(m) * N + n] = v;
    else y_bf16[size_t(m) * N + n] = __float2bfloat16_rn(v);
  }
}

template <int MT, int NT, int U>
int launch_skinny(const void* x, const void* w, const float* bias, const void* add, void* y_bf16, float* y_f32,
                  int M, int N, int K, int act, cudaStream_t stream) {
  const int grid = (N + 16 * MT - 1) / (16 * MT);
  skinny_linear_kernel<MT, NT, U><<<grid, WARPS * 32, 0, stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, (const __nv_bfloat16*)add, (__nv_bfloat16*)y_bf16,
      y_f32, M, N, K, act);
  return launch_status();
}

}  // namespace

// rows that the kernel takes at most, and the multiple that K must be of
PTB_API int ptb_skinny_linear_max_rows() { return 32; }
PTB_API int ptb_skinny_linear_k_multiple() { return KC; }

// y = act(x w^T + bias) + add. x [M, K], w [N, K], add [M, N] bfloat16; bias float32 [N];
// exactly one of y_bf16, y_f32 is given. M <= 32, K a multiple of 32, 16-byte aligned x and w.
PTB_API int ptb_skinny_linear(const void* x, const void* w, const float* bias, const void* add, void* y_bf16,
                              float* y_f32, int M, int N, int K, int act, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return PTB_OK;
  if (M > 32 || K <= 0 || K % KC != 0 || act < 0 || act > 3) return PTB_ERR_SIZE;
  if ((y_bf16 == nullptr) == (y_f32 == nullptr)) return PTB_ERR_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return PTB_ERR_ALIGN;
  // Tile height and chunks in flight per warp, from a sweep over the projections of Falcon-7B, 11B and
  // 40B (each matrix alone, from HBM): wide matrices (many rows, short K) want 32 rows per block and
  // four chunks in flight at up to 8 activation rows, 16 rows and two chunks at up to 16; the others
  // 16 rows and four chunks.
  const bool wide = N >= 16 * 148 * 4;
  if (M <= 8) return wide ? launch_skinny<2, 1, 4>(x, w, bias, add, y_bf16, y_f32, M, N, K, act, stream)
                          : launch_skinny<1, 1, 4>(x, w, bias, add, y_bf16, y_f32, M, N, K, act, stream);
  if (M <= 16) return wide ? launch_skinny<1, 2, 2>(x, w, bias, add, y_bf16, y_f32, M, N, K, act, stream)
                           : launch_skinny<1, 2, 4>(x, w, bias, add, y_bf16, y_f32, M, N, K, act, stream);
  return wide ? launch_skinny<2, 4, 2>(x, w, bias, add, y_bf16, y_f32, M, N, K, act, stream)
              : launch_skinny<1, 4, 4>(x, w, bias, add, y_bf16, y_f32, M, N, K, act, stream);
}
