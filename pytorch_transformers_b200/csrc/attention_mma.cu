// Attention over the paged cache on the tensor cores (bfloat16 operands, float32 accumulation and
// softmax), for prompts and for single tokens, with query heads that share a K/V head packed into
// one tile so that the cache is read once for all of them.
//
// A tile has 16 rows per warp. Row r of a tile stands for (token q0 + r / hpk, head h0 + r % hpk) of
// one K/V head's group: decode packs all heads of the group for the one new token (hpk = heads per
// group), prompts use hpk = 1 and consecutive tokens. Keys are walked in pages of 64 (one cache
// page), double-buffered through shared memory with cp.async into a 16-byte XOR swizzle that makes
// the ldmatrix reads conflict-free. With n_splits > 1 the pages of a sequence are divided among
// gridDim.z blocks which write unnormalised partial results; attention_mma_reduce joins them.
#include <mutex>
#include "mma_common.cuh"

namespace {

struct MmaParams {
  int heads, kv_heads, hpk, tokens_per_tile, n_splits;
  float scale;
  int window;
};

// q [n_tokens, heads, D]; out [n_tokens, heads * D] when part_o == nullptr, else partials:
//   part_o [(tile, group chunk, split)][rows][D] float32 unnormalised, part_ml [...][rows][2] = (max, sum)
template <int D>
__global__ void __launch_bounds__(256)
attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                     const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out,
                     float* __restrict__ part_o, float* __restrict__ part_ml, StepBatch sb,
                     const int* __restrict__ tile_seq, const int* __restrict__ tile_q0,
                     const float* __restrict__ alibi_slopes, MmaParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int TILE_BYTES = KEYS * D * 2;
  const uint32_t smem_base = smem_u32(smem_raw);  // stage s: K at s * 2 * TILE_BYTES, V right after
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
  const int rows_total = 16 * (nthreads >> 5);
  const int g4 = lane >> 2, t4 = lane & 3;

  const int tile = blockIdx.x;
  const int qpk = p.heads / p.kv_heads;
  const int chunks = (qpk + p.hpk - 1) / p.hpk;
  const int g = blockIdx.y / chunks;           // K/V head
  const int h0 = (blockIdx.y % chunks) * p.hpk;  // first head of the chunk within the group
  const int split = blockIdx.z;
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int n_new = sb.seq_new[seq], past = sb.seq_past[seq], start = sb.seq_start[seq];
  const int tok_valid = min(p.tokens_per_tile, n_new - q0);
  const int head_valid = min(p.hpk, qpk - h0);

  // the two rows this thread owns in the warp's 16: r_lo = warp * 16 + g4, r_hi = r_lo + 8
  int row_tok[2], row_head[2], row_pos[2];
  bool row_ok[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = warp * 16 + g4 + 8 * i;
    row_tok[i] = r / p.hpk;
    row_head[i] = r % p.hpk;
    row_ok[i] = row_tok[i] < tok_valid && row_head[i] < head_valid;
    row_pos[i] = row_ok[i] ? past + q0 + row_tok[i] : -1;
  }
  float slope[2] = {0.f, 0.f};
  if (alibi_slopes) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (row_ok[i]) slope[i] = alibi_slopes[g * qpk + h0 + row_head[i]];
  }
  // block-uniform facts about the tile's rows (every row of the tile, not only this thread's)
  const bool all_rows_ok = tok_valid * p.hpk >= rows_total && head_valid == p.hpk;
  const int min_row_pos = past + q0;

  // Q fragments straight from global memory: a[kk][0..3] for k-step kk (16 dims)
  uint32_t qa[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t lo = 0u, hi = 0u;
      if (row_ok[i]) {
        const __nv_bfloat16* qr =
            q + (size_t(start + q0 + row_tok[i]) * p.heads + (g * qpk + h0 + row_head[i])) * D + kk * 16 + t4 * 2;
        lo = *reinterpret_cast<const uint32_t*>(qr);
        hi = *reinterpret_cast<const uint32_t*>(qr + 8);
      }
      qa[kk][i] = lo;       // (row g4 + 8 i, cols t4*2..)    -> a0 / a1
      qa[kk][2 + i] = hi;   // (row g4 + 8 i, cols t4*2 + 8..) -> a2 / a3
    }
  }

  // key pages of this block: the causal (and window) range of the tile, divided among the splits
  const int last_pos = past + q0 + tok_valid - 1;
  int kb_first = 0;
  if (p.window > 0) kb_first = max(0, past + q0 - p.window + 1) / KEYS;
  const int kb_end_all = last_pos / KEYS + 1;
  const int n_pages = kb_end_all - kb_first;
  const int per_split = (n_pages + p.n_splits - 1) / p.n_splits;
  const int kb_begin = kb_first + split * per_split;
  const int kb_end = min(kb_end_all, kb_begin + per_split);
  const int* pages = sb.pages + size_t(seq) * sb.pages_stride;

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl2 = p.scale * 1.4426950408889634f;  // scores are kept in log2 units

  if (kb_begin < kb_end) {
    {
      const int page = pages[kb_begin];
      load_page<D>(smem_base, k_pool + kv_offset(page, g, 0, p.kv_heads, D), tid, nthreads);
      load_page<D>(smem_base + TILE_BYTES, v_pool + kv_offset(page, g, 0, p.kv_heads, D), tid, nthreads);
      cp_async_commit();
    }
    for (int kb = kb_begin; kb < kb_end; ++kb) {
      const int stage = (kb - kb_begin) & 1;
      if (kb + 1 < kb_end) {
        const int page = pages[kb + 1];
        const uint32_t dst = smem_base + (stage ^ 1) * 2 * TILE_BYTES;
        load_page<D>(dst, k_pool + kv_offset(page, g, 0, p.kv_heads, D), tid, nthreads);
        load_page<D>(dst + TILE_BYTES, v_pool + kv_offset(page, g, 0, p.kv_heads, D), tid, nthreads);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const uint32_t ks = smem_base + stage * 2 * TILE_BYTES, vs = ks + TILE_BYTES;

      // S = Q K^T for 64 keys: 8 n-tiles of 8 keys
      float s[KEYS / 8][4];
#pragma unroll
      for (int j = 0; j < KEYS / 8; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; kk += 2) {
          // four 8x8 matrices: keys 8j..8j+7, dim chunks 2kk .. 2kk+3
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, ks + swz<D>(j * 8 + (lane & 7), 2 * kk + (lane >> 3)));
          mma_bf16(s[j], qa[kk], b0, b1);
          mma_bf16(s[j], qa[kk + 1], b2, b3);
        }
      }
      // mask, bias, scale; block maximum per row
      float m_blk[2] = {-INFINITY, -INFINITY};
      // a page whose last key every row of the tile sees (and no window, no bias, no invalid row)
      // needs no per-element test: that is all pages of a long prompt but the diagonal ones
      const bool plain_page = all_rows_ok && p.window <= 0 && alibi_slopes == nullptr &&
                              (kb * KEYS + KEYS - 1) <= min_row_pos;
      if (plain_page) {
#pragma unroll
        for (int j = 0; j < KEYS / 8; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float v = s[j][e] * sl2;
            s[j][e] = v;
            m_blk[e >> 1] = fmaxf(m_blk[e >> 1], v);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < KEYS / 8; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = e >> 1;
            const int key_pos = kb * KEYS + j * 8 + t4 * 2 + (e & 1);
            bool visible = key_pos <= row_pos[i];
            if (p.window > 0) visible = visible && key_pos > row_pos[i] - p.window;
            float v = s[j][e];
            if (alibi_slopes) v += alibi_bias(slope[i], key_pos);
            v = visible ? v * sl2 : -INFINITY;
            s[j][e] = v;
            m_blk[i] = fmaxf(m_blk[i], v);
          }
        }
      }
      float corr[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        m_blk[i] = fmaxf(m_blk[i], __shfl_xor_sync(0xffffffffu, m_blk[i], 1));
        m_blk[i] = fmaxf(m_blk[i], __shfl_xor_sync(0xffffffffu, m_blk[i], 2));
        const float m_new = fmaxf(m_run[i], m_blk[i]);
        corr[i] = (m_run[i] == -INFINITY) ? 0.f : fast_exp2(m_run[i] - m_new);
        m_run[i] = m_new;
      }
      // P = exp2(S - m), row sums, and P as A fragments for the second product
      uint32_t pa[KEYS / 16][4];
      float l_blk[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < KEYS / 8; ++j) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          pv[e] = (s[j][e] == -INFINITY) ? 0.f : fast_exp2(s[j][e] - m_run[i]);
          l_blk[i] += pv[e];
        }
        pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(pv[0], pv[1]);
        pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * corr[i] + l_blk[i];
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        o[j][0] *= corr[0]; o[j][1] *= corr[0];
        o[j][2] *= corr[1]; o[j][3] *= corr[1];
      }
      // O += P V: k-steps of 16 keys, n-tiles of 8 dims, two n-tiles per ldmatrix
#pragma unroll
      for (int kk = 0; kk < KEYS / 16; ++kk) {
#pragma unroll
        for (int j = 0; j < D / 8; j += 2) {
          uint32_t b0, b1, b2, b3;
          const int m = lane >> 3;  // matrix: (m & 1) picks the key half, (m >> 1) the dim chunk
          ldmatrix_x4_trans(b0, b1, b2, b3, vs + swz<D>(kk * 16 + (m & 1) * 8 + (lane & 7), j + (m >> 1)));
          mma_bf16(o[j], pa[kk], b0, b1);
          mma_bf16(o[j + 1], pa[kk], b2, b3);
        }
      }
      __syncthreads();  // the stage is free for the copy after next
    }
  }
  // row sums live in the 4 lanes of a row
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }

  if (part_o == nullptr) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (!row_ok[i]) continue;
      const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
      __nv_bfloat16* dst =
          out + (size_t(start + q0 + row_tok[i]) * p.heads + (g * qpk + h0 + row_head[i])) * D + t4 * 2;
#pragma unroll
      for (int j = 0; j < D / 8; ++j)
        *reinterpret_cast<uint32_t*>(dst + j * 8) = pack_bf16(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
    }
  } else {
    const size_t slot = (size_t(tile) * gridDim.y + blockIdx.y) * p.n_splits + split;
    float* po = part_o + slot * rows_total * D;
    float* pml = part_ml + slot * rows_total * 2;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = warp * 16 + g4 + 8 * i;
#pragma unroll
      for (int j = 0; j < D / 8; ++j)
        *reinterpret_cast<float2*>(po + size_t(r) * D + j * 8 + t4 * 2) = make_float2(o[j][2 * i], o[j][2 * i + 1]);
      if (t4 == 0) {
        pml[r * 2 + 0] = m_run[i];
        pml[r * 2 + 1] = l_run[i];
      }
    }
  }
}

// Joins the partial results of the splits: one warp per row of a tile, a lane per group of D / 32
// dims; blockIdx.z walks the tile's rows four at a time. Every read of a split's row is one
// coalesced line.
template <int D>
__global__ void __launch_bounds__(128)
attention_mma_reduce_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                            __nv_bfloat16* __restrict__ out, StepBatch sb, const int* __restrict__ tile_seq,
                            const int* __restrict__ tile_q0, MmaParams p, int rows_total) {
  constexpr int PER = D / 32;  // dims per lane
  const int tile = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.z * 4 + (threadIdx.x >> 5);
  if (r >= rows_total) return;
  const int qpk = p.heads / p.kv_heads;
  const int chunks = (qpk + p.hpk - 1) / p.hpk;
  const int g = blockIdx.y / chunks, h0 = (blockIdx.y % chunks) * p.hpk;
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int tok = r / p.hpk, hh = r % p.hpk;
  if (tok >= min(p.tokens_per_tile, sb.seq_new[seq] - q0) || hh >= min(p.hpk, qpk - h0)) return;
  const size_t slot0 = (size_t(tile) * gridDim.y + blockIdx.y) * p.n_splits;
  // lanes read the splits' (max, sum) pairs in parallel, 32 splits at a time
  float m = -INFINITY;
  for (int s = lane; s < p.n_splits; s += 32) m = fmaxf(m, part_ml[((slot0 + s) * rows_total + r) * 2]);
  m = warp_max(m);
  float acc[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) acc[e] = 0.f;
  float l = 0.f;
  if (m != -INFINITY) {
    for (int s = 0; s < p.n_splits; ++s) {
      const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((slot0 + s) * rows_total + r) * 2);
      if (ml.x == -INFINITY) continue;
      const float w = exp2f(ml.x - m);
      l += ml.y * w;
      const float* po = part_o + ((slot0 + s) * rows_total + r) * D + lane * PER;
#pragma unroll
      for (int e = 0; e < PER; ++e) acc[e] += po[e] * w;
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* dst = out + (size_t(sb.seq_start[seq] + q0 + tok) * p.heads + (g * qpk + h0 + hh)) * D + lane * PER;
#pragma unroll
  for (int e = 0; e < PER; ++e) dst[e] = __float2bfloat16_rn(acc[e] * inv);
}

template <int D>
int launch_mma(const void* q, const void* k_pool, const void* v_pool, void* out, float* part_o, float* part_ml,
               const StepBatch& sb, const int* tile_seq, const int* tile_q0, int n_tiles, const float* slopes,
               const MmaParams& p, int warps, cudaStream_t stream) {
  const int qpk = p.heads / p.kv_heads;
  const int chunks = (qpk + p.hpk - 1) / p.hpk;
  const size_t smem = size_t(2) * 2 * KEYS * D * 2;  // two stages of (K, V)
  // the kernel's limit of dynamic shared memory is raised once per device and head size (a function
  // attribute belongs to the device's context), by whichever thread comes first
  {
    static std::mutex mutex;
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return PTB_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(mutex);
    if (smem > 48 * 1024 && !configured[dev]) {
      if (cudaFuncSetAttribute(attention_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
          cudaSuccess)
        return PTB_ERR_LAUNCH;
      configured[dev] = true;
    }
  }
  dim3 grid(n_tiles, p.kv_heads * chunks, p.n_splits);
  const bool partial = p.n_splits > 1;
  attention_mma_kernel<D><<<grid, warps * 32, smem, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out,
      partial ? part_o : nullptr, partial ? part_ml : nullptr, sb, tile_seq, tile_q0, slopes, p);
  if (cudaGetLastError() != cudaSuccess) return PTB_ERR_LAUNCH;
  if (partial) {
    dim3 rgrid(n_tiles, p.kv_heads * chunks, (warps * 16 + 3) / 4);
    attention_mma_reduce_kernel<D><<<rgrid, 128, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, sb, tile_seq,
                                                             tile_q0, p, warps * 16);
  }
  return launch_status();
}

}  // namespace

// Head sizes that this kernel takes (others go to the general kernel).
PTB_API int ptb_attention_mma_supports(int head_dim) { return (head_dim == 64 || head_dim == 128) ? 1 : 0; }

// Bytes of float32 scratch that a launch with these sizes needs for the partial results
// (0 when n_splits == 1): part_o then part_ml, each counted in floats.
PTB_API long long ptb_attention_mma_scratch_floats(int n_tiles, int heads, int kv_heads, int hpk, int n_splits,
                                                   int warps, int head_dim) {
  if (n_splits <= 1) return 0;
  const int qpk = heads / kv_heads;
  const int chunks = (qpk + hpk - 1) / hpk;
  return (long long)n_tiles * kv_heads * chunks * n_splits * (warps * 16) * (head_dim + 2);
}

// bfloat16 only. `warps` x 16 rows per tile; hpk * tokens_per_tile must equal warps * 16 or less.
PTB_API int ptb_attention_mma(const void* q, const void* k_pool, const void* v_pool, void* out, float* scratch,
                              const StepBatch* sb, const int* tile_seq, const int* tile_q0, int n_tiles,
                              const float* alibi_slopes, int heads, int kv_heads, int head_dim, int hpk,
                              int tokens_per_tile, int n_splits, int warps, float scale, int window,
                              cudaStream_t stream) {
  if (n_tiles <= 0) return PTB_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || warps < 1 || warps > 8 || hpk < 1 ||
      tokens_per_tile < 1 || hpk * tokens_per_tile > warps * 16 || n_splits < 1 || n_splits > 65535)
    return PTB_ERR_SIZE;
  const int qpk = heads / kv_heads;
  const int chunks = (qpk + hpk - 1) / hpk;
  if (kv_heads * chunks > 65535) return PTB_ERR_SIZE;
  if (n_splits > 1 && scratch == nullptr) return PTB_ERR_SIZE;
  MmaParams p;
  p.heads = heads; p.kv_heads = kv_heads; p.hpk = hpk; p.tokens_per_tile = tokens_per_tile; p.n_splits = n_splits;
  p.scale = scale; p.window = window;
  const long long o_floats = (long long)n_tiles * kv_heads * chunks * n_splits * (warps * 16) * head_dim;
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + o_floats : nullptr;
  switch (head_dim) {
    case 64:
      return launch_mma<64>(q, k_pool, v_pool, out, part_o, part_ml, *sb, tile_seq, tile_q0, n_tiles, alibi_slopes, p,
                            warps, stream);
    case 128:
      return launch_mma<128>(q, k_pool, v_pool, out, part_o, part_ml, *sb, tile_seq, tile_q0, n_tiles, alibi_slopes,
                             p, warps, stream);
    default:
      return PTB_ERR_SIZE;
  }
}

// ------------------------------------------------------------------------------------------------
// The variant that allocates nothing (declared and explained in no_alloc.h).
#include "no_alloc.h"

#include <mutex>

namespace {

// Workspace for the partial results, part of the library image on every device that loads it.
// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_fixed_scratch[PTB_FIXED_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_fixed_scratch_addr[kMaxDevices] = {};
std::mutex g_fixed_scratch_mutex;

// Device address of the workspace on the current device; looked up once per device.
int fixed_scratch_address(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return PTB_ERR_FIXED_SCRATCH_SETUP;
  std::lock_guard<std::mutex> lock(g_fixed_scratch_mutex);
  if (g_fixed_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_fixed_scratch) != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();  // leave no sticky error behind for the caller's next call
      return PTB_ERR_FIXED_SCRATCH_SETUP;
    }
    g_fixed_scratch_addr[dev] = static_cast<float*>(p);
  }
  *out = g_fixed_scratch_addr[dev];
  return PTB_OK;
}

}  // namespace

PTB_API long long ptb_attention_mma_fixed_scratch_capacity(void) { return PTB_FIXED_SCRATCH_FLOATS; }

PTB_API const char* ptb_attention_mma_fixed_scratch_strerror(int code) {
  switch (code) {
    case PTB_OK: return "launched";
    case PTB_ERR_SIZE: return "a size that the kernel does not take";
    case PTB_ERR_LAUNCH: return "the CUDA launch failed";
    case PTB_ERR_FIXED_SCRATCH_TOO_SMALL:
      return "the partial results of this call need more than the built-in workspace of 4194304 float32 values "
             "(16 MiB): use fewer splits or tiles, or call ptb_attention_mma with a workspace of your own";
    case PTB_ERR_FIXED_SCRATCH_SETUP:
      return "the built-in workspace's device address could not be looked up on the current device";
    default: return "unknown error code";
  }
}

PTB_API int ptb_attention_mma_fixed_scratch(const void* q, const void* k_pool, const void* v_pool, void* out,
                                            const StepBatch* sb, const int* tile_seq, const int* tile_q0,
                                            int n_tiles, const float* alibi_slopes, int heads, int kv_heads,
                                            int head_dim, int hpk, int tokens_per_tile, int n_splits, int warps,
                                            float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return PTB_OK;
  // every size is checked before the workspace is counted, so that the count cannot overflow
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || hpk < 1 || warps < 1 || warps > 8 || n_splits < 1 ||
      n_splits > 65535 || tokens_per_tile < 1 || hpk * tokens_per_tile > warps * 16 ||
      !ptb_attention_mma_supports(head_dim))
    return PTB_ERR_SIZE;
  const long long need =
      ptb_attention_mma_scratch_floats(n_tiles, heads, kv_heads, hpk, n_splits, warps, head_dim);
  if (need > (long long)PTB_FIXED_SCRATCH_FLOATS) return PTB_ERR_FIXED_SCRATCH_TOO_SMALL;
  float* scratch = nullptr;
  if (need > 0) {
    const int rc = fixed_scratch_address(&scratch);
    if (rc != PTB_OK) return rc;
  }
  return ptb_attention_mma(q, k_pool, v_pool, out, scratch, sb, tile_seq, tile_q0, n_tiles, alibi_slopes, heads,
                           kv_heads, head_dim, hpk, tokens_per_tile, n_splits, warps, scale, window, stream);
}
