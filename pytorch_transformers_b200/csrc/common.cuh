// Shared helpers of the sm_100a kernels: element access in float32 and bfloat16, reductions,
// the step's batch description and the paged cache's addressing.
#pragma once
#include <cstdio>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define PTB_API extern "C" __attribute__((visibility("default")))

// dtype codes used by every entry point
enum { PTB_F32 = 0, PTB_BF16 = 1 };

// error codes returned by entry points (0 = launched)
enum {
  PTB_OK = 0,
  PTB_ERR_DTYPE = 1,      // unknown dtype code
  PTB_ERR_SIZE = 2,       // a size that the kernel does not take
  PTB_ERR_LAUNCH = 3,     // the launch itself failed (cudaGetLastError)
  PTB_ERR_ALIGN = 4,      // a pointer or a row size that is not aligned as the kernel needs
};

// Activations, by the codes that every entry point with an `act` argument takes. This is the one table:
// a new activation is an entry here, a case in apply_activation and a name in kernels.ACTIVATIONS.
enum { PTB_ACT_NONE = 0, PTB_ACT_GELU_ERF = 1, PTB_ACT_GELU_TANH = 2, PTB_ACT_RELU = 3, PTB_ACT_COUNT = 4 };
inline bool activation_known(int act) { return act >= 0 && act < PTB_ACT_COUNT; }
__device__ __forceinline__ float apply_activation(float v, int act) {
  switch (act) {
    case PTB_ACT_GELU_ERF: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
    case PTB_ACT_GELU_TANH: return 0.5f * v * (1.0f + tanhf(0.79788456080286535588f * (v + 0.044715f * v * v * v)));
    case PTB_ACT_RELU: return fmaxf(v, 0.f);
    default: return v;
  }
}

// multiprocessors of the current device (asked once per process and device)
inline int sm_count() {
  static int sms[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms[dev] = n;
  }
  return sms[dev];
}

// tokens of a cache page; a sequence holds whole pages
constexpr int PTB_PAGE = 64;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// eight bfloat16 values in one 16-byte word <-> eight floats
__device__ __forceinline__ void unpack_bf16x8(const uint4& w, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
  uint4 w;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return w;
}
__host__ __device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// round a float to the nearest bfloat16 value (ties to even), kept as float
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block; every thread gets the result. `scratch` holds at least 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarp) ? scratch[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarp) ? scratch[lane] : -INFINITY;
  return warp_max(r);
}

// The ragged batch of one step, as device arrays of int32 (built on the host).
//   tok_seq[t], tok_pos[t]   sequence index in the batch and absolute position of token t
//   seq_start[b]             index of sequence b's first token among the step's tokens
//   seq_new[b], seq_past[b]  tokens of b in this step, tokens of b already in the cache
//   pages[b * pages_stride + i]  cache page that holds positions [64 i, 64 i + 63] of sequence b
struct StepBatch {
  const int* tok_seq;
  const int* tok_pos;
  const int* seq_start;
  const int* seq_new;
  const int* seq_past;
  const int* pages;
  int pages_stride;
  int n_tokens;
  int n_seqs;
};

// Element offset of (page, kv head, slot in page, 0) in a layer's K or V pool laid out as
// [pages][kv_heads][PTB_PAGE][head_dim].
__device__ __forceinline__ size_t kv_offset(int page, int kv_head, int in_page, int kv_heads, int head_dim) {
  return ((size_t(page) * kv_heads + kv_head) * PTB_PAGE + in_page) * size_t(head_dim);
}

// ALiBi bias of a key position as the reference forms it: bfloat16(slope) * bfloat16(position),
// the product rounded to bfloat16. `slope_bf16` is the slope already rounded.
__device__ __forceinline__ float alibi_bias(float slope_bf16, int key_pos) {
  return round_bf16(slope_bf16 * round_bf16(float(key_pos)));
}

// Rotation of one pair (a, b) by an angle given as (cos, sin): every kernel that rotates uses this
// one form, so that a key written by one kernel equals the key another would have written.
__device__ __forceinline__ void rotate_pair(float a, float b, float c, float s, float& out_a, float& out_b) {
  out_a = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
  out_b = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
}

// the status of the launch just made; a failure is said on stderr with the runtime's own words
inline int launch_status() {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return PTB_OK;
  fprintf(stderr, "[pytorch_transformers_b200] a CUDA launch failed: %s (%s)\n", cudaGetErrorName(e), cudaGetErrorString(e));
  return PTB_ERR_LAUNCH;
}
