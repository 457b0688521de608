// Entry point that allocates nothing. It has no counterpart in the reference (huggingface/
// pytorch-transformers leaves all memory management to PyTorch); it exists for callers of this
// library's C interface that must not, or cannot, obtain device memory at call time:
//
//   * hosts that embed the library through its C symbols without PyTorch's caching allocator and
//     run with a fixed device-memory budget that was handed out completely at start-up, so that a
//     cudaMalloc in the middle of serving would fail or evict somebody;
//   * latency-critical loops that may not take the driver's allocation lock (a cudaMalloc can stall
//     behind another thread's context-wide operation for milliseconds).
//
// ptb_attention_mma_fixed_scratch is ptb_attention_mma (csrc/attention_mma.cu) with the workspace for
// the partial results of split decode attention taken from an array that is part of the library
// image instead of from the caller. Inputs and outputs are still the caller's.
//
// Limits and rules
//   * The workspace holds PTB_FIXED_SCRATCH_FLOATS float32 values (16 MiB). Every GPU that loads the
//     library carries these 16 MiB until the process exits, used or not. A call whose partial results
//     need more (see ptb_attention_mma_scratch_floats) is refused with PTB_ERR_FIXED_SCRATCH_TOO_SMALL
//     and launches nothing; ptb_attention_mma_fixed_scratch_strerror gives the text.
//   * Set-up happens inside the first call on a device: it looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and remembers it per device, and the first
//     call on a device for a head size (64, 128) raises the kernel's shared-memory limit
//     (cudaFuncSetAttribute). Both are guarded by mutexes. Make these first calls, one per device
//     and head size, before any stream capture.
//   * All calls on a device share the one array and find the previous call's contents in it. The
//     kernels write every partial result they later read, so nothing needs clearing; but two calls
//     whose kernels may run at the same time on one GPU (different streams, or graphs replayed
//     concurrently) would overwrite each other's partial results: order them on one stream.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on any path.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PTB_FIXED_SCRATCH_FLOATS (4 * 1024 * 1024)
#define PTB_ERR_FIXED_SCRATCH_TOO_SMALL 5
#define PTB_ERR_FIXED_SCRATCH_SETUP 6

struct StepBatch;

// Same arguments as ptb_attention_mma without `scratch`. Returns 0 when the kernels were launched.
int ptb_attention_mma_fixed_scratch(const void* q, const void* k_pool, const void* v_pool, void* out,
                                    const struct StepBatch* sb, const int* tile_seq, const int* tile_q0, int n_tiles,
                                    const float* alibi_slopes, int heads, int kv_heads, int head_dim, int hpk,
                                    int tokens_per_tile, int n_splits, int warps, float scale, int window,
                                    cudaStream_t stream);

// Capacity of the built-in workspace in float32 values.
long long ptb_attention_mma_fixed_scratch_capacity(void);

// Text for a return code of ptb_attention_mma_fixed_scratch.
const char* ptb_attention_mma_fixed_scratch_strerror(int code);

#ifdef __cplusplus
}
#endif
