// Pieces shared by the tensor-core attention kernels: cp.async, ldmatrix, mma.m16n8k16 wrappers and
// the swizzled shared-memory layout of a cache page.
#pragma once
#include "common.cuh"

constexpr int KEYS = PTB_PAGE;  // keys per step of the main loop

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 2^x by the hardware's approximation unit (relative error about 2^-22, far below bfloat16's): used
// for softmax weights that are rounded to bfloat16 before they meet the tensor cores.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// byte offset of 16-byte chunk `c` of row `row` in a [KEYS][D] bfloat16 tile with the XOR swizzle
template <int D> __device__ __forceinline__ uint32_t swz(int row, int c) {
  return uint32_t(row * (D * 2) + ((c ^ (row & 7)) << 4));
}

// copy one page [KEYS][D] (contiguous in global memory) into a swizzled shared tile
template <int D>
__device__ __forceinline__ void load_page(uint32_t smem_tile, const __nv_bfloat16* page, int tid, int nthreads) {
  constexpr int CHUNKS = D / 8;  // 16-byte chunks per row
  for (int i = tid; i < KEYS * CHUNKS; i += nthreads) {
    const int row = i / CHUNKS, c = i % CHUNKS;
    cp_async16(smem_tile + swz<D>(row, c), page + size_t(row) * D + c * 8);
  }
}

