// Self-test of the bounded wait that every tcgen05 kernel of this library uses on its mbarriers.
// One warp waits, with a limit of `tries`, on a barrier at which nobody ever arrives; the wait runs
// out, raises the error flag with code PTB_SELFTEST_WAIT_CODE and the kernel returns. Nothing faults
// and nothing hangs: this is the path a kernel takes when a copy or a tensor-core commit that it
// waits for never completes, and the host side of it (check_device_errors) is what the test reads.
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int PTB_SELFTEST_WAIT_CODE = 99;

__global__ void bounded_wait_kernel(int* error_flag, uint32_t tries, int* gave_up) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(&bar);
  if (threadIdx.x == 0) mbar_init(addr, 1);
  __syncthreads();
  const bool done = mbar_wait(addr, 0, error_flag, PTB_SELFTEST_WAIT_CODE, tries);
  if (!done && threadIdx.x == 0 && gave_up) *gave_up = 1;
}

}  // namespace

// tries: 1 .. 100,000 (each try may park the thread for up to two microseconds)
PTB_API int ptb_selftest_bounded_wait(int tries, int* error_flag, int* gave_up, cudaStream_t stream) {
  if (tries < 1 || tries > 100000 || error_flag == nullptr) return PTB_ERR_SIZE;
  bounded_wait_kernel<<<1, 32, 0, stream>>>(error_flag, uint32_t(tries), gave_up);
  return launch_status();
}

// ------------------------------------------------------------------------------------------------
// How often does the tensor pipe take a matrix instruction? One thread of every block issues `reps`
// groups of four tcgen05.mma (M = 128, K = 16 each, N = `n`; A from shared memory, or from tensor memory
// with `a_in_tmem`) on operands that sit in shared memory (zeros), commits, and waits; block 0 writes
// the clocks from the first issue to the completion. With `blocks` = 2 x SMs two blocks share an SM.
namespace {

__global__ void __launch_bounds__(128)
mma_cadence_kernel(int n, int reps, int a_in_tmem, long long* clocks, int* error_flag) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* a_tile = smem;                 // [128 rows][64 k] bfloat16, 128-byte swizzle (zeros)
  unsigned char* b_tile = smem + 128 * 128;     // [256 rows][64 k]
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < (128 + 256) * 128 / 16; i += 128) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  const uint32_t bar_a = smem_u32(&bar);
  if (tid == 0) {
    mbar_init(bar_a, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)), "r"(256));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  proxy_fence_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (tid == 32) {
    const uint32_t idesc = idesc_bf16(128, n, false);
    const uint64_t desc_a = smem_desc(smem_u32(a_tile), 16, 1024), desc_b = smem_desc(smem_u32(b_tile), 16, 1024);
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
      if (a_in_tmem) tc_mma4_ts<2>(tmem_base, tmem_base + 128, desc_b, idesc, r > 0 ? 1u : 0u);   // D cols [0, n), A cols [128, 160)
      else tc_mma4<2, 2>(tmem_base, desc_a, desc_b, idesc, r > 0 ? 1u : 0u);
    }
    tc_commit(bar_a);
    mbar_wait(bar_a, 0, error_flag, 98);
    const long long t1 = clock64();
    if (blockIdx.x == 0) clocks[0] = t1 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(256));
}

}  // namespace

// n: 16 .. 256 in steps of 16 (with A in tensor memory at most 128: D and A share 256 columns); reps: 1 .. 100,000
PTB_API int ptb_selftest_mma_cadence(int n, int reps, int a_in_tmem, int blocks, long long* clocks, int* error_flag,
                                     cudaStream_t stream) {
  if (n < 16 || n > 256 || n % 16 || reps < 1 || reps > 100000 || blocks < 1 || clocks == nullptr || error_flag == nullptr ||
      (a_in_tmem && n > 128))
    return PTB_ERR_SIZE;
  const int smem = 1024 + (128 + 256) * 128;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(mma_cadence_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = true;
  }
  mma_cadence_kernel<<<blocks, 128, smem, stream>>>(n, reps, a_in_tmem, clocks, error_flag);
  return launch_status();
}
