// Linear layer for up to 128 rows (steps of single tokens at larger batches) on the fifth-generation
// tensor cores, bound by the one read of the weight matrix:
//
//   y[t, n] = act(sum_k x[t, k] w[n, k] + bias[n]) + add[t, n],   bfloat16 in, float32 accumulation
//
// The product is formed transposed: a block owns 128 weight rows, which are the M side of
// tcgen05.mma (M = 128 is the tensor core's full shape), and the tokens are the N side (padded to a
// multiple of 16, or of 32). The accumulator [128 weight rows x tokens] lives in tensor memory.
//
//   producer   one thread: per 64 values of k, two TMA requests (cp.async.bulk.tensor.2d) bring the
//              box [128 weight rows x 64 k] and the box [tokens x 64 k] into a ring of shared-memory
//              stages, in the 128-byte-swizzle layout that the matrix descriptors name; rows past the
//              matrix and columns past K arrive as zeros. A stage's "full" mbarrier counts the bytes.
//   issuer     one thread: per stage four tcgen05.mma (K = 16 each), then tcgen05.commit on the stage's
//              "empty" mbarrier, which the producer waits for before it refills the stage.
//   epilogue   all four warps: a thread owns one weight row (one lane of tensor memory), reads its
//              sums with tcgen05.ld, adds bias, applies the activation, adds the residual and writes
//              y[t, n] for its tokens (a warp writes 32 consecutive n).
//
// Matrices with few rows (the projections back to the model width) would fill a quarter of the
// device. For them the K range is divided over a cluster of 2 or 4 blocks; each block then owns a
// share of the token columns: it receives the other blocks' partial sums for its columns through
// distributed shared memory (one hardware cluster barrier), sums them in rank order and runs the
// epilogue for its share.
//
// Every wait on an mbarrier is bounded; when one runs out, the block raises the error flag in global
// memory and carries on to its end without waiting again (tensor memory is freed and the cluster
// barriers are passed on every path), so a fault shows as an error and never as a hang.
#include <cudaTypedefs.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int WROWS_TC = 128;             // weight rows per block = M of the matrix instruction
constexpr int KC_TC = 64;                 // k per stage: 128 bytes, one swizzle row
constexpr int W_STAGE_BYTES = WROWS_TC * KC_TC * 2;   // 16 KB
constexpr int MAX_STAGES_TC = 4;
constexpr int MAX_TOKENS_TC = 128;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
// the address of `local` (a shared-memory address of this block) in block `rank` of the cluster
__device__ __forceinline__ uint32_t peer_smem(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_peer(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}

struct TcLinearParams {
  int M, N, K;        // tokens, output features, input features
  int n_tok;          // tokens padded: the N of the matrix instruction
  int act;
  int stages;
  int split;          // blocks per cluster, each with a share of K
  int tmem_cols;
};

__global__ void __launch_bounds__(128)
tc_linear_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                 const float* __restrict__ bias, const __nv_bfloat16* __restrict__ add,
                 __nv_bfloat16* __restrict__ y_bf16, float* __restrict__ y_f32, TcLinearParams p,
                 int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment: the swizzle pattern is a function of address bits 4..9
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  const int x_stage_bytes = p.n_tok * KC_TC * 2;
  const int stage_bytes = W_STAGE_BYTES + x_stage_bytes;   // a multiple of 1024
  unsigned char* ring = smem;
  float* recv = reinterpret_cast<float*>(ring);   // [split - 1][share][128], in the ring once every block's main loop is over
  const int share = p.n_tok / p.split;   // token columns that a block of the cluster finishes
  __shared__ uint64_t bars[2 * MAX_STAGES_TC + 1];   // full[stages], empty[stages], accumulator complete
  __shared__ uint32_t tmem_slot;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = p.split > 1 ? cluster_rank() : 0u;
  const int n0 = blockIdx.x * WROWS_TC;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[MAX_STAGES_TC]);
  const uint32_t bar_done = smem_u32(&bars[2 * MAX_STAGES_TC]);

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(bar_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)), "r"(p.tmem_cols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  // this block's share of the k chunks
  const int chunks = (p.K + KC_TC - 1) / KC_TC;
  const int per = (chunks + p.split - 1) / p.split;
  const int c0 = min(chunks, int(rank) * per), c1 = min(chunks, c0 + per);
  const int n_iter = c1 - c0;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const uint32_t ring0 = smem_u32(ring);
      uint32_t st = 0, base = ring0, full = full0, empty = empty0, parity = 1;   // parity of the round before
      int kx = c0 * KC_TC;
      for (int i = 0; i < n_iter; ++i) {
        if (i >= p.stages) {   // the matrix instructions that read this stage have completed
          if (!mbar_wait(empty, parity, error_flag, 21)) {
            // no further copies; the ones in flight land before the block ends (bounded waits again)
            for (int j = max(0, i - p.stages); j < i; ++j)
              mbar_wait(full0 + 8 * (j % p.stages), (j / p.stages) & 1, error_flag, 21);
            break;
          }
        }
        mbar_expect_tx(full, uint32_t(stage_bytes));   // a box delivers all its bytes, zeros where out of range
        tma_load_2d(base, &w_map, kx, n0, full);
        tma_load_2d(base + W_STAGE_BYTES, &x_map, kx, 0, full);
        kx += KC_TC;
        base += stage_bytes; full += 8; empty += 8;
        if (++st == uint32_t(p.stages)) { st = 0; base = ring0; full = full0; empty = empty0; parity ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer
    if (lane == 0) {
      const uint32_t idesc = idesc_bf16(WROWS_TC, p.n_tok, false);
      const uint64_t desc_w0 = smem_desc(smem_u32(ring), 16, 1024);
      const uint64_t desc_step = uint64_t(stage_bytes >> 4);   // the address field counts 16-byte units
      uint64_t desc_w = desc_w0;
      uint32_t st = 0, full = full0, empty = empty0, parity = 0;
      bool alive = true;
      for (int i = 0; i < n_iter; ++i) {
        alive = mbar_wait(full, parity, error_flag, 22);
        if (!alive) break;
        tc_fence_after();
        // four steps of 16 k: 32 bytes = 2 descriptor units along a swizzled row
        tc_mma4(tmem_base, desc_w, desc_w + (W_STAGE_BYTES >> 4), idesc, i > 0 ? 1u : 0u);
        tc_commit(empty);
        desc_w += desc_step; full += 8; empty += 8;
        if (++st == uint32_t(p.stages)) { st = 0; desc_w = desc_w0; full = full0; empty = empty0; parity ^= 1; }
      }
      if (alive && n_iter > 0) {
        tc_commit(bar_done);
        mbar_wait(bar_done, 0, error_flag, 23);   // every matrix instruction of this block has completed
      }
    }
    __syncwarp();
  }
  __syncthreads();
  tc_fence_after();

  // -------------------------------------------------------------------- epilogue
  const int row = warp * 32 + lane;                 // weight row within the tile = lane of tensor memory
  const int n = n0 + row;
  const uint32_t lane_addr = tmem_base + (uint32_t(warp * 32) << 16);
  const bool have = n_iter > 0;                     // a block without k chunks contributes zeros

  if (p.split > 1) {
    // every block of the cluster is past its main loop: the rings are free to receive partial sums
    cluster_arrive();
    cluster_wait();
    // partial sums of the other blocks' columns go to their owners: recv[sender slot][column][row]
    for (int g = 0; g < p.n_tok / 8; ++g) {
      const uint32_t owner = uint32_t(g * 8 / share);
      if (owner == rank) continue;
      float v[8];
      if (have) tmem_ld8(lane_addr + g * 8, v);
      else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
      }
      const uint32_t slot = rank < owner ? rank : rank - 1;
      const uint32_t dst0 = peer_smem(smem_u32(recv + (size_t(slot) * share + (g * 8 - owner * share)) * WROWS_TC + row), owner);
#pragma unroll
      for (int j = 0; j < 8; ++j) st_peer(dst0 + j * WROWS_TC * 4, v[j]);
    }
    cluster_arrive();
    cluster_wait();   // all partial sums for this block's columns have arrived
  }
  const int t0 = int(rank) * share;
  for (int g = 0; g < share / 8; ++g) {
    float v[8];
    if (have) tmem_ld8(lane_addr + t0 + g * 8, v);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    if (p.split > 1) {
      // ranks in ascending order, this block's own sums in their place: one order for every element
      float total[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) total[j] = 0.f;
      for (uint32_t r = 0; r < uint32_t(p.split); ++r) {
        if (r == rank) {
#pragma unroll
          for (int j = 0; j < 8; ++j) total[j] += v[j];
        } else {
          const uint32_t slot = r < rank ? r : r - 1;
          const float* src = recv + (size_t(slot) * share + g * 8) * WROWS_TC + row;
#pragma unroll
          for (int j = 0; j < 8; ++j) total[j] += src[j * WROWS_TC];
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = total[j];
    }
    if (n < p.N) {
      const float b = bias ? bias[n] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = t0 + g * 8 + j;
        if (t >= p.M) continue;
        float o = apply_activation(v[j] + b, p.act);
        const size_t at = size_t(t) * p.N + n;
        if (add) o += __bfloat162float(add[at]);
        if (y_f32) y_f32[at] = o;
        else y_bf16[at] = __float2bfloat16_rn(o);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(p.tmem_cols));
}

// ---- tensor maps (host). cuTensorMapEncodeTiled comes from the driver through the runtime's
// entry-point query, so the library does not link against libcuda.
PFN_cuTensorMapEncodeTiled_v12000 encode_tiled() {
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

// a [rows, K] bfloat16 row-major matrix in boxes of box_rows x 64 k, written with the 128-byte swizzle
bool make_map_sw128(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  auto fn = encode_tiled();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(K) * 2};
  const cuuint32_t box[2] = {cuuint32_t(KC_TC), cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct WKey {
  const void* p; int rows, k;
  bool operator==(const WKey& o) const { return p == o.p && rows == o.rows && k == o.k; }
};
struct WKeyHash {
  size_t operator()(const WKey& k) const {
    return std::hash<const void*>()(k.p) ^ (size_t(k.rows) * 1000003u) ^ (size_t(k.k) << 20);
  }
};
// weight maps are made once per matrix and kept (weights do not move)
const CUtensorMap* weight_map_sw128(const void* w, int N, int K) {
  static std::unordered_map<WKey, CUtensorMap, WKeyHash> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const WKey key{w, N, K};
  auto it = cache.find(key);
  if (it != cache.end()) return &it->second;
  CUtensorMap m;
  if (!make_map_sw128(&m, w, N, K, WROWS_TC)) return nullptr;
  return &cache.emplace(key, m).first->second;
}

}  // namespace

PTB_API int ptb_tc_linear_max_rows() { return MAX_TOKENS_TC; }
PTB_API int ptb_tc_linear_k_multiple() { return 8; }

// y = act(x w^T + bias) + add for M <= 128 rows of x; K a multiple of 8 (a row of x and of w must
// start on a 16-byte boundary); x and w 16-byte aligned. `sms`: the SM count of the device.
// `error_flag`: a device int that stays 0 unless a bounded wait inside the kernel ran out.
PTB_API int ptb_tc_linear(const void* x, const void* w, const float* bias, const void* add, void* y_bf16, float* y_f32,
                          int M, int N, int K, int act, int sms, int* error_flag, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return PTB_OK;
  if (M > MAX_TOKENS_TC || K <= 0 || K % 8 != 0 || !activation_known(act) || sms < 1 || error_flag == nullptr)
    return PTB_ERR_SIZE;
  if ((y_bf16 == nullptr) == (y_f32 == nullptr)) return PTB_ERR_SIZE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return PTB_ERR_ALIGN;

  TcLinearParams p;
  p.M = M; p.N = N; p.K = K; p.act = act;
  const int tiles = (N + WROWS_TC - 1) / WROWS_TC;
  const int chunks = (K + KC_TC - 1) / KC_TC;
  // blocks per cluster: fill the device when the matrix has few rows, with at least 8 chunks per block
  int split = 1;
  while (split < 4 && tiles * split * 2 <= sms && chunks / (split * 2) >= 8) split *= 2;
  p.split = split;
  const int pad = split == 4 ? 32 : 16;   // every block of the cluster owns a multiple of 8 columns
  p.n_tok = (M + pad - 1) / pad * pad;
  p.tmem_cols = 32;
  while (p.tmem_cols < p.n_tok) p.tmem_cols *= 2;
  const int stage_bytes = W_STAGE_BYTES + p.n_tok * KC_TC * 2;
  const size_t recv_bytes = split > 1 ? size_t(split - 1) * (p.n_tok / split) * WROWS_TC * sizeof(float) : 0;
  // An SM's TMA requests in flight are bounded near 64 KB (measured: deeper rings bring nothing), so
  // the ring stays under half of an SM's shared memory: two blocks fit on an SM, which lets every
  // cluster of 4 be resident at once (with one block per SM only 33 clusters of 4 fit on 148 SMs)
  // and lets one block's epilogue and first loads run under another's main loop.
  int stages = int((110 * 1024 - 1024) / stage_bytes);
  if (stages > 4) stages = 4;
  if (stages < 2 || size_t(stages) * stage_bytes < recv_bytes) return PTB_ERR_SIZE;
  p.stages = stages;
  const size_t smem = 1024 + size_t(stages) * stage_bytes;
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(tc_linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = smem;
  }
  const CUtensorMap* wm = weight_map_sw128(w, N, K);
  CUtensorMap xm;
  if (wm == nullptr || !make_map_sw128(&xm, x, M, K, p.n_tok)) return PTB_ERR_LAUNCH;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, split, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = split;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, tc_linear_kernel, *wm, xm, bias, (const __nv_bfloat16*)add, (__nv_bfloat16*)y_bf16, y_f32,
                         p, error_flag) != cudaSuccess)
    return PTB_ERR_LAUNCH;
  return launch_status();
}
