// Row-wise and elementwise kernels: embedding gather, row gather, LayerNorm / RMSNorm with one
// or two affine outputs, bias + activation, residual sums. All arithmetic is float32; tensors of
// activations are float32 or bfloat16 (template T); gains, biases are float32 vectors.
#include "common.cuh"

// blocks of a grid-stride launch: enough to cover `total`, at most 16 per SM
static int grid_for(size_t total, int threads) {
  const size_t want = (total + threads - 1) / threads, most = size_t(sm_count()) * 16;
  return int(want < most ? want : most);
}

// ------------------------------------------------------------------------------------------------
// rows of a table: out[t, :] = table[ids[t], :]. An id outside [0, rows) raises bit 0 of *status
// and reads row 0.
template <typename T>
__global__ void gather_rows_kernel(const int* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                   int width, int rows, int* status) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= rows) {
    if (threadIdx.x == 0 && status) atomicOr(status, 1);
    id = 0;
  }
  const T* src = table + size_t(id) * width;
  T* dst = out + size_t(t) * width;
  const size_t row_bytes = size_t(width) * sizeof(T);
  if (row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(table) % 16 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0)) {
    const int4* s4 = reinterpret_cast<const int4*>(src);
    int4* d4 = reinterpret_cast<int4*>(dst);
    const int n4 = int(row_bytes / 16);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
  }
}

PTB_API int ptb_gather_rows(int dtype, const int* ids, const void* table, void* out, int n, int width, int rows,
                            int* status, cudaStream_t stream) {
  if (n <= 0) return PTB_OK;
  if (width <= 0 || rows <= 0) return PTB_ERR_SIZE;
  if (dtype == PTB_F32)
    gather_rows_kernel<float><<<n, 256, 0, stream>>>(ids, (const float*)table, (float*)out, width, rows, status);
  else if (dtype == PTB_BF16)
    gather_rows_kernel<__nv_bfloat16><<<n, 256, 0, stream>>>(ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out,
                                                             width, rows, status);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

// ------------------------------------------------------------------------------------------------
// Normalisation of rows. kind 0: LayerNorm, y = (x - mean) / sqrt(var + eps) * gain + bias with the
// biased variance; kind 1: RMSNorm, y = x / sqrt(mean(x^2) + eps) * gain (+ bias if given).
// With gain2 != nullptr a second output with its own gain and bias is written from the same
// statistics (two norms of one input share the read and the reductions).
// With addend != nullptr the input is the sum x + addend (formed in float32, rounded once to T);
// the rounded sum is written to sum_out and is what gets normalised: two branches of a residual
// stream are joined and normed in one pass.
// The row is held in shared memory as float32: 4 * width bytes of dynamic shared memory.
template <typename T>
__global__ void norm_kernel(const T* __restrict__ x, const T* __restrict__ addend, T* __restrict__ sum_out,
                            const float* __restrict__ gain1, const float* __restrict__ bias1,
                            T* __restrict__ y1, const float* __restrict__ gain2, const float* __restrict__ bias2,
                            T* __restrict__ y2, int width, float eps, int kind) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  const size_t base = size_t(blockIdx.x) * width;
  float s = 0.f;
  // bfloat16 rows whose width is a multiple of 8 move in 16-byte words (row starts are then aligned)
  const bool vec = sizeof(T) == 2 && width % 8 == 0 && aligned16(x) && aligned16(y1) &&
                   (!addend || (aligned16(addend) && aligned16(sum_out))) && (!gain2 || aligned16(y2));
  if (vec) {
    const uint4* xv = reinterpret_cast<const uint4*>(x + base);
    const uint4* av = addend ? reinterpret_cast<const uint4*>(addend + base) : nullptr;
    uint4* sv = addend ? reinterpret_cast<uint4*>(sum_out + base) : nullptr;
    for (int i = threadIdx.x; i < width / 8; i += blockDim.x) {
      float f[8];
      unpack_bf16x8(xv[i], f);
      if (av) {
        float g[8];
        unpack_bf16x8(av[i], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += g[e];
        const uint4 r = pack_bf16x8(f);
        sv[i] = r;
        unpack_bf16x8(r, f);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        row[i * 8 + e] = f[e];
        s += f[e];
      }
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float v = to_f(x[base + i]);
      if (addend) {
        const T r = from_f<T>(v + to_f(addend[base + i]));
        sum_out[base + i] = r;
        v = to_f(r);
      }
      row[i] = v;
      s += v;
    }
  }
  float mean = 0.f;
  if (kind == 0) mean = block_sum(s, scratch) / float(width);
  float q = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float c = row[i] - mean;
    q += c * c;
  }
  const float var = block_sum(q, scratch) / float(width);
  const float rstd = 1.0f / sqrtf(var + eps);
  if (vec) {
    uint4* o1 = reinterpret_cast<uint4*>(y1 + base);
    uint4* o2 = gain2 ? reinterpret_cast<uint4*>(y2 + base) : nullptr;
    for (int i = threadIdx.x; i < width / 8; i += blockDim.x) {
      float n[8], a[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        n[e] = (row[i * 8 + e] - mean) * rstd;
        a[e] = n[e] * gain1[i * 8 + e];
        if (bias1) a[e] += bias1[i * 8 + e];
      }
      o1[i] = pack_bf16x8(a);
      if (o2) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          a[e] = n[e] * gain2[i * 8 + e];
          if (bias2) a[e] += bias2[i * 8 + e];
        }
        o2[i] = pack_bf16x8(a);
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float n = (row[i] - mean) * rstd;
    float a = n * gain1[i];
    if (bias1) a += bias1[i];
    y1[base + i] = from_f<T>(a);
    if (gain2) {
      float b = n * gain2[i];
      if (bias2) b += bias2[i];
      y2[base + i] = from_f<T>(b);
    }
  }
}

// The same for bfloat16 rows that move in 16-byte words, with the row in registers: thread t holds
// the words t, t + 256, ... (VPT of them), so there is no pass through shared memory and a block
// needs only the two reductions. 256 threads: rows up to 2048 * VPT values.
constexpr int NORM_REG_THREADS = 256;
__device__ __forceinline__ void load_f32x8(const float* __restrict__ p, float (&v)[8]) {   // p 16-byte aligned
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <int VPT>
__global__ void __launch_bounds__(NORM_REG_THREADS)
norm_bf16_reg_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ addend,
                     __nv_bfloat16* __restrict__ sum_out, const float* __restrict__ gain1,
                     const float* __restrict__ bias1, __nv_bfloat16* __restrict__ y1,
                     const float* __restrict__ gain2, const float* __restrict__ bias2,
                     __nv_bfloat16* __restrict__ y2, int width, float eps, int kind) {
  __shared__ float scratch[32];
  const size_t base = size_t(blockIdx.x) * width;
  const int nvec = width / 8;
  const uint4* xv = reinterpret_cast<const uint4*>(x + base);
  const uint4* av = addend ? reinterpret_cast<const uint4*>(addend + base) : nullptr;
  uint4* sv = addend ? reinterpret_cast<uint4*>(sum_out + base) : nullptr;
  float f[VPT][8];
  uint4 raw[VPT], rawa[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {   // all loads first: they are in flight together
    const int i = threadIdx.x + v * NORM_REG_THREADS;
    raw[v] = i < nvec ? xv[i] : make_uint4(0, 0, 0, 0);
    rawa[v] = (av && i < nvec) ? av[i] : make_uint4(0, 0, 0, 0);
  }
  float s = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * NORM_REG_THREADS;
    unpack_bf16x8(raw[v], f[v]);
    if (av) {
      float g[8];
      unpack_bf16x8(rawa[v], g);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[v][e] += g[e];
      const uint4 r = pack_bf16x8(f[v]);
      if (i < nvec) sv[i] = r;
      unpack_bf16x8(r, f[v]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) s += f[v][e];
  }
  float mean = 0.f;
  if (kind == 0) mean = block_sum(s, scratch) / float(width);
  float q = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    if (threadIdx.x + v * NORM_REG_THREADS < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float c = f[v][e] - mean;
        q += c * c;
      }
    }
  }
  const float var = block_sum(q, scratch) / float(width);
  const float rstd = 1.0f / sqrtf(var + eps);
  uint4* o1 = reinterpret_cast<uint4*>(y1 + base);
  uint4* o2 = gain2 ? reinterpret_cast<uint4*>(y2 + base) : nullptr;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * NORM_REG_THREADS;
    if (i >= nvec) continue;
    float n[8], a[8], gb[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) n[e] = (f[v][e] - mean) * rstd;
    load_f32x8(gain1 + i * 8, gb);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = n[e] * gb[e];
    if (bias1) {
      load_f32x8(bias1 + i * 8, gb);
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] += gb[e];
    }
    o1[i] = pack_bf16x8(a);
    if (o2) {
      load_f32x8(gain2 + i * 8, gb);
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] = n[e] * gb[e];
      if (bias2) {
        load_f32x8(bias2 + i * 8, gb);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] += gb[e];
      }
      o2[i] = pack_bf16x8(a);
    }
  }
}

template <int VPT>
void launch_norm_reg(const void* x, const void* addend, void* sum_out, const float* gain1, const float* bias1, void* y1,
                     const float* gain2, const float* bias2, void* y2, int n, int width, float eps, int kind,
                     cudaStream_t stream) {
  norm_bf16_reg_kernel<VPT><<<n, NORM_REG_THREADS, 0, stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)addend, (__nv_bfloat16*)sum_out, gain1, bias1,
      (__nv_bfloat16*)y1, gain2, bias2, (__nv_bfloat16*)y2, width, eps, kind);
}

PTB_API int ptb_norm(int dtype, const void* x, const void* addend, void* sum_out, const float* gain1,
                     const float* bias1, void* y1, const float* gain2, const float* bias2, void* y2, int n, int width,
                     float eps, int kind, cudaStream_t stream) {
  if (n <= 0) return PTB_OK;
  if (width <= 0 || kind < 0 || kind > 1) return PTB_ERR_SIZE;
  if ((addend == nullptr) != (sum_out == nullptr)) return PTB_ERR_SIZE;
  const bool all16 = aligned16(x) && aligned16(y1) && aligned16(gain1) && (!bias1 || aligned16(bias1)) &&
                     (!addend || (aligned16(addend) && aligned16(sum_out))) &&
                     (!gain2 || (aligned16(y2) && aligned16(gain2) && (!bias2 || aligned16(bias2))));
  if (dtype == PTB_BF16 && width % 8 == 0 && width <= 2048 * 8 && all16) {
    const int vpt = (width / 8 + NORM_REG_THREADS - 1) / NORM_REG_THREADS;
    if (vpt <= 1) launch_norm_reg<1>(x, addend, sum_out, gain1, bias1, y1, gain2, bias2, y2, n, width, eps, kind, stream);
    else if (vpt <= 2) launch_norm_reg<2>(x, addend, sum_out, gain1, bias1, y1, gain2, bias2, y2, n, width, eps, kind, stream);
    else if (vpt <= 4) launch_norm_reg<4>(x, addend, sum_out, gain1, bias1, y1, gain2, bias2, y2, n, width, eps, kind, stream);
    else launch_norm_reg<8>(x, addend, sum_out, gain1, bias1, y1, gain2, bias2, y2, n, width, eps, kind, stream);
    return launch_status();
  }
  const size_t smem = size_t(width) * sizeof(float);
  if (smem > 200 * 1024) return PTB_ERR_SIZE;
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  cudaError_t e = cudaSuccess;
  static size_t configured_f32 = 48 * 1024, configured_bf16 = 48 * 1024;
  if (dtype == PTB_F32) {
    if (smem > configured_f32) {
      e = cudaFuncSetAttribute(norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      configured_f32 = smem;
    }
    if (e != cudaSuccess) return PTB_ERR_LAUNCH;
    norm_kernel<float><<<n, threads, smem, stream>>>((const float*)x, (const float*)addend, (float*)sum_out, gain1,
                                                     bias1, (float*)y1, gain2, bias2, (float*)y2, width, eps, kind);
  } else if (dtype == PTB_BF16) {
    if (smem > configured_bf16) {
      e = cudaFuncSetAttribute(norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      configured_bf16 = smem;
    }
    if (e != cudaSuccess) return PTB_ERR_LAUNCH;
    norm_kernel<__nv_bfloat16><<<n, threads, smem, stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)addend, (__nv_bfloat16*)sum_out, gain1, bias1,
        (__nv_bfloat16*)y1, gain2, bias2, (__nv_bfloat16*)y2, width, eps, kind);
  } else {
    return PTB_ERR_DTYPE;
  }
  return launch_status();
}

// ------------------------------------------------------------------------------------------------
// Bias and activation (codes and formulas: apply_activation in common.cuh).

// y[r, c] = act(y[r, c] + bias[c]) in place (bias may be null).
template <typename T>
__global__ void bias_act_kernel(T* __restrict__ y, const float* __restrict__ bias, size_t total, int width, int act) {
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    float v = to_f(y[i]);
    if (bias) v += bias[i % width];
    y[i] = from_f<T>(apply_activation(v, act));
  }
}

// GELU (erf form) for values that are rounded to bfloat16 afterwards: erf by the rational
// approximation 7.1.26 of Abramowitz and Stegun (absolute error below 1.5e-7, three orders of
// magnitude under bfloat16's resolution), one reciprocal and one exp2 instead of erff's long
// polynomial. The float32 kernels keep erff.
//   t = 1 / (1 + 0.3275911 z), z = |v| / sqrt 2;  erf z = 1 - (a1 t + ... + a5 t^5) exp(-z^2)
// Two values go through it in one 64-bit register (fma.rn.f32x2 / mul.rn.f32x2: half the instructions on
// the multiply-add pipe; 38.0 -> 29.9 us on 2,048 x 18,176 values). log2(e) is folded into the argument
// (z' = |v| sqrt(log2 e / 2), the rational's constant divided accordingly), the sign into
// 0.5 v + 0.5 |v| erf(|v| / sqrt 2), and the reciprocal is the approximate one (an error of one unit in
// the last place of float32).
__device__ __forceinline__ uint64_t f2_pack(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;\n" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_const(float c) { return f2_pack(c, c); }
__device__ __forceinline__ void gelu_erf_for_bf16_x2(float& v0, float& v1) {
  constexpr uint64_t ABS = 0x7fffffff7fffffffull, SIGN = 0x8000000080000000ull;
  const uint64_t v = f2_pack(v0, v1);
  const uint64_t hv = f2_mul(v, f2_const(0.5f));
  const uint64_t z = f2_mul(v & ABS, f2_const(0.84932180028801904272f));        // |v| sqrt(log2(e) / 2)
  float d0, d1;
  f2_unpack(f2_fma(f2_const(0.27273748f), z, f2_const(1.0f)), d0, d1);          // 1 + 0.3275911 |v| / sqrt 2
  float t0, t1;
  asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(t0) : "f"(d0));
  asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(t1) : "f"(d1));
  const uint64_t t = f2_pack(t0, t1);
  uint64_t poly = f2_fma(f2_const(1.061405429f), t, f2_const(-1.453152027f));
  poly = f2_fma(poly, t, f2_const(1.421413741f));
  poly = f2_fma(poly, t, f2_const(-0.284496736f));
  poly = f2_fma(poly, t, f2_const(0.254829592f));
  float x0, x1, e0, e1;
  f2_unpack(f2_mul(z ^ SIGN, z), x0, x1);                                       // -(v^2 / 2) log2(e)
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e0) : "f"(x0));
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e1) : "f"(x1));
  const uint64_t erf_abs = f2_fma(f2_mul(poly, t) ^ SIGN, f2_pack(e0, e1), f2_const(1.0f));
  f2_unpack(f2_fma(hv & ABS, erf_abs, hv), v0, v1);                             // 0.5 v + 0.5 |v| erf
}

// eight bfloat16 values per 16-byte word (width a multiple of 8, 16-byte aligned rows); a
// thread takes two words per step, both loads in flight before the arithmetic of either. The
// presence of a bias is compile-time (without one the loop holds no division for the column), and
// so is the erf GELU with its cheaper form (FAST_GELU); every other activation goes by its code.
template <bool FAST_GELU, bool BIAS>
__device__ __forceinline__ uint4 bias_act_word(uint4 word, const float* __restrict__ bias, size_t i, unsigned words_per_row,
                                               int act) {
  float f[8];
  unpack_bf16x8(word, f);
  if (BIAS) {
    float b[8];
    load_f32x8(bias + size_t(unsigned(i % words_per_row)) * 8, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] += b[e];
  }
  if constexpr (FAST_GELU) {
#pragma unroll
    for (int e = 0; e < 8; e += 2) gelu_erf_for_bf16_x2(f[e], f[e + 1]);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = apply_activation(f[e], act);
  }
  return pack_bf16x8(f);
}
template <bool FAST_GELU, bool BIAS>
__global__ void __launch_bounds__(256)
bias_act_bf16x8_kernel(uint4* __restrict__ y, const float* __restrict__ bias, size_t total8, unsigned words_per_row,
                       int act) {
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + stride < total8; i += 2 * stride) {
    const uint4 a = y[i], b = y[i + stride];
    y[i] = bias_act_word<FAST_GELU, BIAS>(a, bias, i, words_per_row, act);
    y[i + stride] = bias_act_word<FAST_GELU, BIAS>(b, bias, i + stride, words_per_row, act);
  }
  if (i < total8) y[i] = bias_act_word<FAST_GELU, BIAS>(y[i], bias, i, words_per_row, act);
}
template <bool FAST_GELU>
void launch_bias_act_x8(void* y, const float* bias, size_t total8, int width, int act, cudaStream_t stream) {
  const int grid = grid_for(total8, 256);
  const unsigned words = unsigned(width / 8);
  if (bias) bias_act_bf16x8_kernel<FAST_GELU, true><<<grid, 256, 0, stream>>>((uint4*)y, bias, total8, words, act);
  else bias_act_bf16x8_kernel<FAST_GELU, false><<<grid, 256, 0, stream>>>((uint4*)y, bias, total8, words, act);
}

PTB_API int ptb_bias_act(int dtype, void* y, const float* bias, int rows, int width, int act, cudaStream_t stream) {
  const size_t total = size_t(rows) * width;
  if (total == 0) return PTB_OK;
  if (!activation_known(act)) return PTB_ERR_SIZE;
  if (dtype == PTB_BF16 && width % 8 == 0 && aligned16(y) && (!bias || aligned16(bias))) {
    if (act == PTB_ACT_GELU_ERF) launch_bias_act_x8<true>(y, bias, total / 8, width, act, stream);
    else launch_bias_act_x8<false>(y, bias, total / 8, width, act, stream);
    return launch_status();
  }
  const int threads = 256;
  const int blocks = grid_for(total, threads);
  if (dtype == PTB_F32)
    bias_act_kernel<float><<<blocks, threads, 0, stream>>>((float*)y, bias, total, width, act);
  else if (dtype == PTB_BF16)
    bias_act_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)y, bias, total, width, act);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

// out = x + (a + b), or x + a when b is null: the residual sum, formed in float32 and rounded once.
template <typename T>
__global__ void residual_kernel(const T* __restrict__ x, const T* __restrict__ a, const T* __restrict__ b,
                                T* __restrict__ out, size_t total) {
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    float s = to_f(a[i]);
    if (b) s += to_f(b[i]);
    out[i] = from_f<T>(to_f(x[i]) + s);
  }
}

__global__ void residual_bf16x8_kernel(const uint4* __restrict__ x, const uint4* __restrict__ a,
                                       const uint4* __restrict__ b, uint4* __restrict__ out, size_t total8) {
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total8; i += stride) {
    float fx[8], fa[8], fb[8];
    unpack_bf16x8(x[i], fx);
    unpack_bf16x8(a[i], fa);
    if (b) {
      unpack_bf16x8(b[i], fb);
#pragma unroll
      for (int e = 0; e < 8; ++e) fa[e] += fb[e];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) fx[e] += fa[e];
    out[i] = pack_bf16x8(fx);
  }
}

PTB_API int ptb_residual(int dtype, const void* x, const void* a, const void* b, void* out, long long total,
                         cudaStream_t stream) {
  if (total <= 0) return PTB_OK;
  if (dtype == PTB_BF16 && total % 8 == 0 && aligned16(x) && aligned16(a) && aligned16(b) && aligned16(out)) {
    residual_bf16x8_kernel<<<grid_for(size_t(total) / 8, 256), 256, 0, stream>>>(
        (const uint4*)x, (const uint4*)a, (const uint4*)b, (uint4*)out, size_t(total) / 8);
    return launch_status();
  }
  const int threads = 256;
  const int blocks = grid_for(size_t(total), threads);
  if (dtype == PTB_F32)
    residual_kernel<float><<<blocks, threads, 0, stream>>>((const float*)x, (const float*)a, (const float*)b,
                                                           (float*)out, size_t(total));
  else if (dtype == PTB_BF16)
    residual_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)a,
                                                                   (const __nv_bfloat16*)b, (__nv_bfloat16*)out,
                                                                   size_t(total));
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

// x *= factor in place, the product formed in float32 and rounded once (a scale on the embeddings or on
// the logits, where an architecture has one)
template <typename T>
__global__ void scale_kernel(T* __restrict__ x, float factor, size_t total) {
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
    x[i] = from_f<T>(__fmul_rn(to_f(x[i]), factor));
}

PTB_API int ptb_scale(int dtype, void* x, float factor, long long total, cudaStream_t stream) {
  if (total <= 0) return PTB_OK;
  const int threads = 256;
  const int blocks = grid_for(size_t(total), threads);
  if (dtype == PTB_F32) scale_kernel<float><<<blocks, threads, 0, stream>>>((float*)x, factor, size_t(total));
  else if (dtype == PTB_BF16)
    scale_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)x, factor, size_t(total));
  else return PTB_ERR_DTYPE;
  return launch_status();
}

// float32 copy of rows of any dtype: out[r, :] = float(x[r, :]) (logits of a bfloat16 head)
template <typename T>
__global__ void to_float_kernel(const T* __restrict__ x, float* __restrict__ out, size_t total) {
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) out[i] = to_f(x[i]);
}

PTB_API int ptb_to_float(int dtype, const void* x, float* out, long long total, cudaStream_t stream) {
  if (total <= 0) return PTB_OK;
  const int threads = 256;
  const int blocks = grid_for(size_t(total), threads);
  if (dtype == PTB_F32)
    to_float_kernel<float><<<blocks, threads, 0, stream>>>((const float*)x, out, size_t(total));
  else if (dtype == PTB_BF16)
    to_float_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)x, out, size_t(total));
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}
