// Pieces shared by the kernels that drive the fifth-generation tensor cores (tcgen05): matrix and
// instruction descriptors, mbarriers with bounded waits, tensor-memory loads and stores, and the
// tensor memory accelerator's tiled copies.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>

#include <map>
#include <mutex>
#include <tuple>

#include "mma_common.cuh"

// Online softmax keeps each row's exponentials relative to a reference score. The reference follows the
// row's maximum only when the maximum has grown by more than this many powers of two: until then P holds
// values up to 2^8 (no loss in bfloat16, whose exponent carries them, nor in the float32 sums), and the
// rescaling of O in tensor memory, which has to wait for the previous page's O += P V, is skipped.
constexpr float RESCALE_LOG2 = 8.0f;
constexpr uint32_t WAIT_LIMIT = 1u << 20;
// Time hint for one try_wait: the hardware may park the thread this long instead of returning "not
// yet" at once, so waiting threads leave the issue slots to the working ones. A wait gives up after
// WAIT_LIMIT tries: some seconds at most.
constexpr uint32_t WAIT_SUSPEND_NS = 2000;

// ---- shared-memory matrix descriptor (sm_100): start address, leading and stride byte offsets in
// 16-byte units, version 1, layout type 2 = 128-byte swizzle
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return uint64_t((addr & 0x3FFFFu) >> 4) | (uint64_t(lbo_bytes >> 4) << 16) | (uint64_t(sbo_bytes >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// ---- instruction descriptor for kind::f16: D float32, A and B bfloat16, N / 8 at bit 17, M / 16 at bit 24
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(WAIT_SUSPEND_NS) : "memory");
  return ok != 0;
}
// bounded wait: false (and the error flag raised) if the barrier did not complete within `limit` tries
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code,
                                          uint32_t limit = WAIT_LIMIT) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  atomicExch(error_flag, code);
  return false;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void proxy_fence_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// 32 consecutive columns of this thread's lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
        "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
        "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
        "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
        "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
        "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// TMA: the box of `map` whose first element is (x = innermost offset, y = row) -> shared memory;
// completion is counted in bytes on `bar`. x times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// 8 consecutive columns of this thread's lane
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
// D (+)= A B over 64 values of k: four matrix instructions of 16 k each, the first one overwriting D
// when `accumulate` is 0. From one instruction to the next the A descriptor advances by A_STEP and
// the B descriptor by B_STEP units of 16 bytes: 2 along a 128-byte-swizzled K-major row (16 k = 32
// bytes), 128 down the rows of an MN-major tile (16 rows of 128 bytes). One asm block: the issuing
// thread's instruction count per tile matters, it is the one thread that feeds the tensor core.
template <int A_STEP = 2, int B_STEP = 2>
__device__ __forceinline__ void tc_mma4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 a, b;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 q, %3, %3;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "add.u64 a, %1, %5;\n\tadd.u64 b, %2, %6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n\t"
      "add.u64 a, a, %5;\n\tadd.u64 b, b, %6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n\t"
      "add.u64 a, a, %5;\n\tadd.u64 b, b, %6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "n"(A_STEP), "n"(B_STEP) : "memory");
}

// 64 consecutive columns of this thread's lane: both loads in flight, one wait
__device__ __forceinline__ void tmem_ld64_once(uint32_t taddr, float (&v)[64]) {
  uint32_t r[64];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t* q = r + 32 * h;
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7]),
          "=r"(q[8]), "=r"(q[9]), "=r"(q[10]), "=r"(q[11]), "=r"(q[12]), "=r"(q[13]), "=r"(q[14]), "=r"(q[15]),
          "=r"(q[16]), "=r"(q[17]), "=r"(q[18]), "=r"(q[19]), "=r"(q[20]), "=r"(q[21]), "=r"(q[22]), "=r"(q[23]),
          "=r"(q[24]), "=r"(q[25]), "=r"(q[26]), "=r"(q[27]), "=r"(q[28]), "=r"(q[29]), "=r"(q[30]), "=r"(q[31])
        : "r"(taddr + 32 * h));
  }
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}

// N consecutive columns of this thread's lane, N = 32 or 64
template <int N> __device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&v)[N]);
template <> __device__ __forceinline__ void tmem_ld<32>(uint32_t taddr, float (&v)[32]) { tmem_ld32(taddr, v); }
template <> __device__ __forceinline__ void tmem_ld<64>(uint32_t taddr, float (&v)[64]) {
  float a[32], b[32];
  tmem_ld32(taddr, a);
  tmem_ld32(taddr + 32, b);
#pragma unroll
  for (int i = 0; i < 32; ++i) { v[i] = a[i]; v[32 + i] = b[i]; }
}

// The same with A read from tensor memory (bfloat16 pairs packed into 32-bit columns, row = lane): from
// one instruction to the next A advances by 8 columns (16 k), the B descriptor by B_STEP units.
template <int B_STEP>
__device__ __forceinline__ void tc_mma4_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 q, %3, %3;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "add.u32 a, %1, 8;\n\tadd.u64 b, %2, %5;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, q;\n\t"
      "add.u32 a, a, 8;\n\tadd.u64 b, b, %5;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, q;\n\t"
      "add.u32 a, a, 8;\n\tadd.u64 b, b, %5;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, q;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "n"(B_STEP) : "memory");
}
// 16 consecutive columns of this thread's lane from 16 registers
__device__ __forceinline__ void tmem_st16_u32(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st32_u32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
template <int N> __device__ __forceinline__ void tmem_st_u32(uint32_t taddr, const uint32_t (&v)[N]);
template <> __device__ __forceinline__ void tmem_st_u32<16>(uint32_t taddr, const uint32_t (&v)[16]) { tmem_st16_u32(taddr, v); }
template <> __device__ __forceinline__ void tmem_st_u32<32>(uint32_t taddr, const uint32_t (&v)[32]) { tmem_st32_u32(taddr, v); }

// ---- host side
// a pool of one cache entry, [pages][kv_heads][64 keys][D], seen as rows of D values: boxes of 64 keys x
// 64 dims land in the 128-byte-swizzle layout. Pools do not move: a map per pool is made once and kept.
inline const CUtensorMap* pool_map(const void* pool, int pool_pages, int kv_heads, int d) {
  struct Key {
    const void* p; long long rows; int d;
    bool operator<(const Key& o) const { return std::tie(p, rows, d) < std::tie(o.p, o.rows, o.d); }
  };
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) != cudaSuccess ||
        qr != cudaDriverEntryPointSuccess)
      return nullptr;
    encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
  const Key key{pool, (long long)pool_pages * kv_heads * KEYS, d};
  auto it = cache.find(key);
  if (it != cache.end()) return &it->second;
  CUtensorMap m;
  const cuuint64_t dims[2] = {cuuint64_t(d), cuuint64_t(key.rows)};
  const cuuint64_t strides[1] = {cuuint64_t(d) * 2};
  const cuuint32_t box[2] = {64, cuuint32_t(KEYS)};
  const cuuint32_t elem[2] = {1, 1};
  if (encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return nullptr;
  return &cache.emplace(key, m).first->second;
}

