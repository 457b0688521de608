// Random weights on the device: out[i] = offset + std * z_i, z_i standard normal, a pure function of
// (key, i). The host twin (weights/generator.py) computes the same bits: every float64 operation
// here is an explicitly rounded intrinsic (no fused multiply-add), and logarithm, sine and cosine
// are the series written out below, not the math library's.
//
//   pair j (elements 2j, 2j+1): r = mix(key + (j + 1) * GAMMA)        (the splitmix64 sequence)
//   radius: u = (2 hi + 1) / 2^33, m = 2 hi + 1 = f * 2^e with f in (sqrt(1/2), sqrt(2)],
//           -ln u = (33 - e) ln 2 - 2 atanh((f - 1) / (f + 1)),  radius = sqrt(2 * -ln u)
//   angle:  2 pi lo / 2^32 = (pi / 4) (octant + x), x = (frac + 1/2) / 2^29 the middle of the cell;
//           odd octants use 1 - x; sine and cosine of the reduced angle by Taylor series
//   z = radius * (cos, sin); value rounded to float32, and from there to bfloat16 where asked.
#include "common.cuh"

namespace {

constexpr uint64_t GAMMA = 0x9E3779B97F4A7C15ull;
constexpr double LN2 = 0x1.62e42fefa39efp-1;
constexpr double SQRT2 = 0x1.6a09e667f3bcdp+0;
constexpr double QUARTER_PI = 0x1.921fb54442d18p-1;
__constant__ double ATANH_COEF[11] = {0x1.0000000000000p+0, 0x1.5555555555555p-2, 0x1.999999999999ap-3,
                                      0x1.2492492492492p-3, 0x1.c71c71c71c71cp-4, 0x1.745d1745d1746p-4,
                                      0x1.3b13b13b13b14p-4, 0x1.1111111111111p-4, 0x1.e1e1e1e1e1e1ep-5,
                                      0x1.af286bca1af28p-5, 0x1.8618618618618p-5};
__constant__ double SIN_COEF[8] = {0x1.0000000000000p+0,  -0x1.5555555555555p-3, 0x1.1111111111111p-7,
                                   -0x1.a01a01a01a01ap-13, 0x1.71de3a556c734p-19, -0x1.ae64567f544e4p-26,
                                   0x1.6124613a86d09p-33,  -0x1.ae7f3e733b81fp-41};
__constant__ double COS_COEF[9] = {0x1.0000000000000p+0,  -0x1.0000000000000p-1, 0x1.5555555555555p-5,
                                   -0x1.6c16c16c16c17p-10, 0x1.a01a01a01a01ap-16, -0x1.27e4fb7789f5cp-22,
                                   0x1.1eed8eff8d898p-29,  -0x1.93974a8c07c9dp-37, 0x1.ae7f3e733b81fp-45};

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// the two standard normal values of pair j
__device__ __forceinline__ void normal_pair(uint64_t key, uint64_t j, double& z0, double& z1) {
  const uint64_t r = mix64(key + (j + 1) * GAMMA);
  const uint32_t hi = uint32_t(r >> 32), lo = uint32_t(r);

  const uint64_t m = 2ull * hi + 1ull;                 // odd, below 2^33
  int e = 63 - __clzll((long long)m);
  double f = __dmul_rn(double(m), __longlong_as_double((long long)(1023 - e) << 52));   // m / 2^e, exact
  if (f > SQRT2) {
    f = __dmul_rn(f, 0.5);
    e += 1;
  }
  const double s = __ddiv_rn(__dadd_rn(f, -1.0), __dadd_rn(f, 1.0));
  const double s2 = __dmul_rn(s, s);
  double p = ATANH_COEF[10];
#pragma unroll
  for (int k = 9; k >= 0; --k) p = __dadd_rn(__dmul_rn(p, s2), ATANH_COEF[k]);
  const double ln_f = __dmul_rn(__dmul_rn(s, p), 2.0);
  const double t = __dsub_rn(__dmul_rn(double(33 - e), LN2), ln_f);
  const double radius = __dsqrt_rn(__dmul_rn(t, 2.0));

  const int octant = int(lo >> 29);
  const double frac = double(lo & ((1u << 29) - 1));
  double x = __dmul_rn(__dadd_rn(frac, 0.5), 0x1p-29);
  if (octant & 1) x = __dsub_rn(1.0, x);
  const double a = __dmul_rn(x, QUARTER_PI);
  const double a2 = __dmul_rn(a, a);
  double ps = SIN_COEF[7];
#pragma unroll
  for (int k = 6; k >= 0; --k) ps = __dadd_rn(__dmul_rn(ps, a2), SIN_COEF[k]);
  const double sin_a = __dmul_rn(ps, a);
  double pc = COS_COEF[8];
#pragma unroll
  for (int k = 7; k >= 0; --k) pc = __dadd_rn(__dmul_rn(pc, a2), COS_COEF[k]);
  const double cos_a = pc;
  const bool swap = ((octant + 1) >> 1) & 1;
  double c = swap ? sin_a : cos_a, sn = swap ? cos_a : sin_a;
  if (((octant + 2) >> 2) & 1) c = -c;
  if (octant >> 2) sn = -sn;
  z0 = __dmul_rn(radius, c);
  z1 = __dmul_rn(radius, sn);
}

__device__ __forceinline__ float finish(double z, double std, double offset, int round_bf16_first) {
  const float v = __double2float_rn(__dadd_rn(__dmul_rn(z, std), offset));
  return round_bf16_first ? round_bf16(v) : v;
}

// One thread per pair. `first` is the index of out[0] within the tensor's stream of elements.
template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, size_t count, size_t first, uint64_t key, double std,
                                   double offset, int round_bf16_first) {
  const size_t p0 = first / 2, lead = first - 2 * p0;        // out[i] is element first + i of pair (first + i) / 2
  const size_t n_pairs = (first + count + 1) / 2 - p0;
  const bool pair_stores = lead == 0 && reinterpret_cast<uintptr_t>(out) % (2 * sizeof(T)) == 0;
  for (size_t q = size_t(blockIdx.x) * blockDim.x + threadIdx.x; q < n_pairs; q += size_t(gridDim.x) * blockDim.x) {
    double z0, z1;
    normal_pair(key, p0 + q, z0, z1);
    const size_t e0 = 2 * q;                                   // element index relative to pair p0
    const T v0 = from_f<T>(finish(z0, std, offset, round_bf16_first));
    const T v1 = from_f<T>(finish(z1, std, offset, round_bf16_first));
    if (pair_stores && e0 + 1 < count) {                       // both elements in one store
      if constexpr (sizeof(T) == 2) {
        __nv_bfloat162 two;
        two.x = v0;
        two.y = v1;
        *reinterpret_cast<__nv_bfloat162*>(out + e0) = two;
      } else {
        *reinterpret_cast<float2*>(out + e0) = make_float2(v0, v1);
      }
      continue;
    }
    if (e0 >= lead && e0 - lead < count) out[e0 - lead] = v0;
    if (e0 + 1 >= lead && e0 + 1 - lead < count) out[e0 + 1 - lead] = v1;
  }
}

}  // namespace

// Fill `count` elements of `out` (float32 or bfloat16, by `dtype`) with elements first .. first+count-1
// of the stream of `key`. `round_bf16_first`: round the float32 value to bfloat16 before storing it
// (a float32 tensor that holds what a bfloat16 file would hold).
PTB_API int ptb_fill_normal(int dtype, void* out, unsigned long long count, unsigned long long first,
                            unsigned long long key, double std, double offset, int round_bf16_first,
                            cudaStream_t stream) {
  if (count == 0) return PTB_OK;
  const size_t pairs = (size_t(count) + 2) / 2;
  const int threads = 256;
  const size_t want = (pairs + threads - 1) / threads;
  const size_t most = size_t(sm_count()) * 32;
  const int blocks = int(want < most ? want : most);
  if (dtype == PTB_F32)
    fill_normal_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, count, first, key, std, offset,
                                                              round_bf16_first);
  else if (dtype == PTB_BF16)
    fill_normal_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, count, first, key, std,
                                                                      offset, round_bf16_first);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}
