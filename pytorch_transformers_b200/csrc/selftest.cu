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
