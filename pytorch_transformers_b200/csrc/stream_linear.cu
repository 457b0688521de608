// Linear layer for a few rows (decode steps), second form: the weight matrix is streamed through a
// ring of shared-memory stages by the tensor memory accelerator (cp.async.bulk.tensor.2d: one request
// brings a box of 32 weight rows x 256 k) that signals mbarriers, so that the number of bytes in flight
// does not depend on registers or occupancy.
//
//   y[m, n] = act(sum_k x[m, k] w[n, k] + bias[n]) + add[m, n],   m <= 16, bfloat16 in, float32 math
//
// Persistent blocks: block b owns the 32-row weight tiles b, b + grid, ... A stage of the ring holds
// 256 values of k for the tile's 32 weight rows and for the activation rows (40 or 48 rows of 512
// bytes). One producer thread refills stages with two TMA requests (weights, activations; columns
// past K and activation rows past M are filled with zeros by the hardware) and the stage's "full"
// barrier counts the bytes (complete_tx). Eight consumer warps each take one 32-wide chunk
// of every stage, build mma.m16n8k16 fragments straight from 16-byte shared loads (the k permutation
// of skinny_linear.cu: both operands take the same 8 consecutive k per thread), and release the
// stage through its "empty" barrier. The ring keeps running across tiles. Partial sums of the
// eight warps meet in shared memory; the epilogue adds bias, applies the activation, adds the
// residual and writes bfloat16 or float32.
//
// Every wait on a barrier is bounded; when one runs out the block raises the error flag and
// leaves its loops, so a fault shows as an error and never as a hang.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

constexpr int CW = 8;                 // consumer warps
constexpr int KS = 256;               // k values per stage
constexpr int ROW_BYTES = KS * 2;     // dense rows: the layout a TMA box lands in
constexpr int WROWS = 32;             // weight rows per tile
constexpr uint32_t SPIN_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code) {
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i)
    if (bar_try(bar, parity)) return true;
  atomicExch(error_flag, code);
  return false;
}
// TMA: the box of `map` whose first element is (x = k offset, y = row) -> shared memory; completion is
// counted in bytes on `bar`. x * 2 bytes must be a multiple of 16 (it is a multiple of 512 here).
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma16816s(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float act_s(float v, int act) {
  switch (act) {
    case 1: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
    case 2: return 0.5f * v * (1.0f + tanhf(0.79788456080286535588f * (v + 0.044715f * v * v * v)));
    case 3: return fmaxf(v, 0.f);
    default: return v;
  }
}

// NT: 8-row activation tiles (M <= 8 NT)
template <int NT>
__global__ void __launch_bounds__((CW + 1) * 32)
stream_linear_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                     const float* __restrict__ bias, const __nv_bfloat16* __restrict__ add,
                     __nv_bfloat16* __restrict__ y_bf16, float* __restrict__ y_f32, int M, int N, int K, int act,
                     int stages, int* __restrict__ error_flag) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int XROWS = 8 * NT;
  constexpr int STAGE_ROWS = WROWS + XROWS;
  constexpr int STAGE_BYTES = STAGE_ROWS * ROW_BYTES;
  unsigned char* ring = smem;
  float* red = reinterpret_cast<float*>(ring + size_t(stages) * STAGE_BYTES);  // [CW][WROWS][XROWS + 1]
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + CW * WROWS * (XROWS + 1));  // full[stages], empty[stages]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t full0 = s_u32(bars), empty0 = s_u32(bars + stages);

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      bar_init(full0 + 8 * s, 1);
      bar_init(empty0 + 8 * s, CW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  const int n_tiles = (N + WROWS - 1) / WROWS;
  const int k_stages = (K + KS - 1) / KS;

  if (warp == CW) {
    // ---------------------------------------------------------------- producer
    int it = 0;  // stages issued so far (over all tiles of this block)
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      const int n0 = tile * WROWS;
      for (int ks = 0; ks < k_stages; ++ks, ++it) {
        const int st = it % stages;
        const uint32_t round = it / stages;
        if (round > 0) {  // the consumers have released this stage `round` times by then
          if (!bar_wait(empty0 + 8 * st, (round - 1) & 1, error_flag, 11)) return;
        }
        if (lane == 0) {
          const uint32_t full = full0 + 8 * st;
          const uint32_t base = s_u32(ring + size_t(st) * STAGE_BYTES);
          bar_expect_tx(full, STAGE_BYTES);   // a box always delivers all its bytes, zeros where out of range
          tma_2d(base, &w_map, ks * KS, n0, full);
          tma_2d(base + WROWS * ROW_BYTES, &x_map, ks * KS, 0, full);
        }
        __syncwarp();
      }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  const int g = lane >> 2, t = lane & 3;
  int it = 0;
  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int n0 = tile * WROWS;
    float acc[2][NT][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
    for (int ks = 0; ks < k_stages; ++ks, ++it) {
      const int st = it % stages;
      if (!bar_wait(full0 + 8 * st, (it / stages) & 1, error_flag, 12)) return;
      if (ks * KS + warp * 32 < K) {  // chunks past K hold zeros: skip them
        const unsigned char* base = ring + size_t(st) * STAGE_BYTES + warp * 64 + t * 16;
        uint4 wa[2][2], xb[NT];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          wa[i][0] = *reinterpret_cast<const uint4*>(base + (i * 16 + g) * ROW_BYTES);
          wa[i][1] = *reinterpret_cast<const uint4*>(base + (i * 16 + g + 8) * ROW_BYTES);
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) xb[j] = *reinterpret_cast<const uint4*>(base + (WROWS + j * 8 + g) * ROW_BYTES);
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            mma16816s(acc[i][j], wa[i][0].x, wa[i][1].x, wa[i][0].y, wa[i][1].y, xb[j].x, xb[j].y);
            mma16816s(acc[i][j], wa[i][0].z, wa[i][1].z, wa[i][0].w, wa[i][1].w, xb[j].z, xb[j].w);
          }
      }
      __syncwarp();
      if (lane == 0) bar_arrive(empty0 + 8 * st);
    }
    // partial sums of the 8 warps: red[warp][weight row][activation row]
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        float* r0 = red + (size_t(warp) * WROWS + i * 16 + g) * (XROWS + 1) + j * 8 + 2 * t;
        float* r1 = r0 + 8 * (XROWS + 1);
        r0[0] = acc[i][j][0];
        r0[1] = acc[i][j][1];
        r1[0] = acc[i][j][2];
        r1[1] = acc[i][j][3];
      }
    asm volatile("bar.sync 1, %0;\n" ::"n"(CW * 32) : "memory");  // the consumer warps only
    for (int idx = tid; idx < WROWS * XROWS; idx += CW * 32) {
      const int r = idx % WROWS, m = idx / WROWS;
      const int n = n0 + r;
      if (m >= M || n >= N) continue;
      float v = 0.f;
#pragma unroll
      for (int wi = 0; wi < CW; ++wi) v += red[(size_t(wi) * WROWS + r) * (XROWS + 1) + m];
      if (bias) v += bias[n];
      v = act_s(v, act);
      if (add) v += __bfloat162float(add[size_t(m) * N + n]);
      if (y_f32) y_f32[size_t(m) * N + n] = v;
      else y_bf16[size_t(m) * N + n] = __float2bfloat16_rn(v);
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(CW * 32) : "memory");  // red is free for the next tile
  }
}

// ---- tensor maps (host). cuTensorMapEncodeTiled comes from the driver through the runtime's
// entry-point query, so the library does not link against libcuda.
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// a [rows, K] bfloat16 row-major matrix, boxes of box_rows x KS
bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  auto fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(K) * 2};
  const cuuint32_t box[2] = {cuuint32_t(KS), cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapKey {
  const void* p; int rows, k, box;
  bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && k == o.k && box == o.box; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.p) ^ (size_t(k.rows) * 1000003u) ^ (size_t(k.k) << 20) ^ size_t(k.box);
  }
};
// weight maps are made once per matrix and kept (weights do not move)
const CUtensorMap* weight_map(const void* w, int N, int K) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const MapKey key{w, N, K, WROWS};
  auto it = cache.find(key);
  if (it != cache.end()) return &it->second;
  CUtensorMap m;
  if (!make_map(&m, w, N, K, WROWS)) return nullptr;
  return &cache.emplace(key, m).first->second;
}

template <int NT>
int launch_stream(const void* x, const void* w, const float* bias, const void* add, void* y_bf16, float* y_f32,
                  int M, int N, int K, int act, int* error_flag, int sms, cudaStream_t stream) {
  constexpr int XROWS = 8 * NT;
  constexpr int STAGE_BYTES = (WROWS + XROWS) * ROW_BYTES;
  const size_t fixed = size_t(CW) * WROWS * (XROWS + 1) * sizeof(float);
  int stages = int((200 * 1024 - fixed - 256) / STAGE_BYTES);
  if (stages > 12) stages = 12;
  if (stages < 2) return PTB_ERR_SIZE;
  const size_t smem = size_t(stages) * STAGE_BYTES + fixed + size_t(2 * stages) * 8 + 128;
  static size_t configured[3] = {0, 0, 0};
  if (smem > configured[NT]) {
    if (cudaFuncSetAttribute(stream_linear_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
        cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured[NT] = smem;
  }
  const CUtensorMap* wm = weight_map(w, N, K);
  CUtensorMap xm;
  if (wm == nullptr || !make_map(&xm, x, M, K, XROWS)) return PTB_ERR_LAUNCH;
  const int n_tiles = (N + WROWS - 1) / WROWS;
  const int grid = n_tiles < sms ? n_tiles : sms;
  stream_linear_kernel<NT><<<grid, (CW + 1) * 32, smem, stream>>>(
      xm, *wm, bias, (const __nv_bfloat16*)add, (__nv_bfloat16*)y_bf16, y_f32, M, N, K, act, stages, error_flag);
  return launch_status();
}

}  // namespace

PTB_API int ptb_stream_linear_max_rows() { return 16; }

// y = act(x w^T + bias) + add for M <= 16 rows; K a multiple of 32; x and w 16-byte aligned. `sms`: blocks to
// launch at most (the SM count of the device). `error_flag` as for the attention kernels.
PTB_API int ptb_stream_linear(const void* x, const void* w, const float* bias, const void* add, void* y_bf16,
                              float* y_f32, int M, int N, int K, int act, int sms, int* error_flag,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return PTB_OK;
  if (M > 16 || K <= 0 || K % 32 != 0 || N < 1 || act < 0 || act > 3 || sms < 1 || error_flag == nullptr) return PTB_ERR_SIZE;
  if ((y_bf16 == nullptr) == (y_f32 == nullptr)) return PTB_ERR_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return PTB_ERR_ALIGN;
  if (M <= 8) return launch_stream<1>(x, w, bias, add, y_bf16, y_f32, M, N, K, act, error_flag, sms, stream);
  return launch_stream<2>(x, w, bias, add, y_bf16, y_f32, M, N, K, act, error_flag, sms, stream);
}
