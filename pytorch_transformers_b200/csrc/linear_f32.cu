// True float32 linear layer on the CUDA cores: y[m, n] = act(sum_k x[m, k] * w[n, k] + bias[n]).
// No tensor cores and no reduced-precision mode: every product and sum is an IEEE float32 FMA.
// Each output element is accumulated by one thread over k in ascending order (16 products at a
// time, then into the total), so a row's result does not depend on how many other rows are in the
// launch or on the tiling, and the rounding error stays small for K in the tens of thousands.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;  // tile of the output and step along K
constexpr int TM = 4, TN = 4;             // outputs per thread; 256 threads


__global__ void __launch_bounds__(256) linear_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                         const float* __restrict__ bias, float* __restrict__ y, int M,
                                                         int N, int K, int act) {
  // k-major tiles: xs[k][m], ws[k][n]; +4 padding keeps the transposing stores off one bank
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * TM, tn = (tid % 16) * TN;
  // loader mapping: 256 threads fetch 64 rows x 16 k: thread -> (row = tid / 4, k = (tid % 4) * 4 .. +3)
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int k = k0 + lk + q;
      const int gm = m0 + lrow, gn = n0 + lrow;
      xs[lk + q][lrow] = (gm < M && k < K) ? x[size_t(gm) * K + k] : 0.f;
      ws[lk + q][lrow] = (gn < N && k < K) ? w[size_t(gn) * K + k] : 0.f;
    }
    __syncthreads();
    // two levels of summation: the 16 products of this step are summed on their own and then added
    // to the total, so the rounding error grows with K / 16 + 16 instead of with K
    float part[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) part[i][j] = 0.f;
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[k][tm + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[k][tn + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] += part[i][j];
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      y[size_t(gm) * N + gn] = apply_activation(v, act);
    }
  }
}

}  // namespace

PTB_API int ptb_linear_f32(const float* x, const float* w, const float* bias, float* y, int M, int N, int K, int act,
                           cudaStream_t stream) {
  if (M <= 0 || N <= 0) return PTB_OK;
  if (K <= 0 || !activation_known(act)) return PTB_ERR_SIZE;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return PTB_ERR_SIZE;
  linear_f32_kernel<<<grid, 256, 0, stream>>>(x, w, bias, y, M, N, K, act);
  return launch_status();
}
