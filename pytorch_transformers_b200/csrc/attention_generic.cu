// Attention over the paged cache, general form (CUDA cores, float32 arithmetic), and the kernel
// that splits a fused projection into rotated queries and cache entries.
//
// The general attention kernel takes every head size up to 256, any number of heads and groups,
// float32 or bfloat16 tensors, rotary or ALiBi models, an optional window, prompts and single
// tokens alike. It is the kernel of the float32 path and the fallback of the bfloat16 path for
// sizes that the tensor-core kernels refuse. Every query row is reduced over its keys in blocks
// of 64 aligned to absolute positions, in ascending order, whatever else is in the launch: the
// result of a position does not depend on how tokens were cut into steps or batched.
#include "common.cuh"

namespace {

constexpr int BQ = 16;        // query rows of a tile
constexpr int THREADS = 128;  // 8 threads per query row
constexpr int MAX_D = 256;    // head sizes up to this
constexpr int DPT = MAX_D / 8;

// ------------------------------------------------------------------------------------------------
// Fused projection [n_tokens, kv_heads * (q_per_kv + 2) * head_dim], rows grouped per K/V head as
// (q_per_kv query heads, K, V), to: q_out [n_tokens, heads, head_dim] (query head = group *
// q_per_kv + index in group) and the K and V pools of one layer. With inv_freq != nullptr the
// first 2 * rot_pairs dims of every query and key head are rotated: pairs (i, i + rot_pairs), or with
// `interleaved` pairs (2 i, 2 i + 1);
// angle = position * inv_freq[i] in float32, x' = x cos - y sin, y' = y cos + x sin. With a table
// (rope_cos, rope_sin: [n_tokens, rot_pairs], made by rope_table_kernel from the same product) the
// cosines and sines are read instead of computed. One block per token.
template <typename T>
__global__ void split_rotate_store_kernel(const T* __restrict__ fused, T* __restrict__ q_out, T* __restrict__ k_pool,
                                          T* __restrict__ v_pool, StepBatch sb, const float* __restrict__ inv_freq,
                                          const float* __restrict__ rope_cos, const float* __restrict__ rope_sin,
                                          int rot_pairs, int kv_heads, int q_per_kv, int head_dim, int write_cache,
                                          int interleaved) {
  const int t = blockIdx.x;
  const int pos = sb.tok_pos[t];
  const int seq = sb.tok_seq[t];
  const int page = sb.pages[size_t(seq) * sb.pages_stride + pos / PTB_PAGE];
  const int in_page = pos % PTB_PAGE;
  const int rows = q_per_kv + 2;
  const int fused_width = kv_heads * rows * head_dim;
  const T* src_tok = fused + size_t(t) * fused_width;
  const int heads = kv_heads * q_per_kv;
  // work items: (group g, row r in group, pair or plain element)
  const int rot_dims = 2 * rot_pairs;
  // bfloat16 with head sizes and rotation widths in multiples of 8 and a table of cosines: 16-byte words
  if (sizeof(T) == 2 && head_dim % 8 == 0 && rot_pairs % 8 == 0 && (rot_pairs == 0 || (rope_cos != nullptr && !interleaved)) &&
      aligned16(fused) && aligned16(q_out) && (!write_cache || (aligned16(k_pool) && aligned16(v_pool)))) {
    const int chunks = head_dim / 8, rot_chunks = rot_pairs / 8;
    const int total_v = kv_heads * rows * chunks;
    for (int w = threadIdx.x; w < total_v; w += blockDim.x) {
      const int c = w % chunks;
      const int gr = w / chunks;
      const int r = gr % rows, g = gr / rows;
      const T* src = src_tok + size_t(g * rows + r) * head_dim;
      T* dst;
      if (r < q_per_kv) {
        dst = q_out + (size_t(t) * heads + (g * q_per_kv + r)) * head_dim;
      } else {
        if (!write_cache) continue;
        dst = ((r == q_per_kv) ? k_pool : v_pool) + kv_offset(page, g, in_page, kv_heads, head_dim);
      }
      const bool rotated_row = (r <= q_per_kv) && rot_chunks > 0;
      if (rotated_row && c < rot_chunks) {
        float a[8], b[8], cs[8], sn[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(src + c * 8), a);
        unpack_bf16x8(*reinterpret_cast<const uint4*>(src + rot_pairs + c * 8), b);
        const float4* cp = reinterpret_cast<const float4*>(rope_cos + size_t(t) * rot_pairs + c * 8);
        const float4* sp = reinterpret_cast<const float4*>(rope_sin + size_t(t) * rot_pairs + c * 8);
        *reinterpret_cast<float4*>(cs) = cp[0];
        *reinterpret_cast<float4*>(cs + 4) = cp[1];
        *reinterpret_cast<float4*>(sn) = sp[0];
        *reinterpret_cast<float4*>(sn + 4) = sp[1];
#pragma unroll
        for (int e = 0; e < 8; ++e) rotate_pair(a[e], b[e], cs[e], sn[e], a[e], b[e]);
        *reinterpret_cast<uint4*>(dst + c * 8) = pack_bf16x8(a);
        *reinterpret_cast<uint4*>(dst + rot_pairs + c * 8) = pack_bf16x8(b);
      } else if (rotated_row && c < 2 * rot_chunks) {
        // the upper half of a rotated pair: written by the thread that holds the lower half
      } else {
        *reinterpret_cast<uint4*>(dst + c * 8) = *reinterpret_cast<const uint4*>(src + c * 8);
      }
    }
    return;
  }
  const int per_row = rot_pairs + (head_dim - rot_dims);  // rotated pairs, then untouched dims
  const int total = kv_heads * rows * per_row;
  for (int w = threadIdx.x; w < total; w += blockDim.x) {
    const int e = w % per_row;
    const int gr = w / per_row;
    const int r = gr % rows;
    const int g = gr / rows;
    const T* src = src_tok + size_t(g * rows + r) * head_dim;
    T* dst;
    if (r < q_per_kv) {
      dst = q_out + (size_t(t) * heads + (g * q_per_kv + r)) * head_dim;
    } else {
      if (!write_cache) continue;
      T* pool = (r == q_per_kv) ? k_pool : v_pool;
      dst = pool + kv_offset(page, g, in_page, kv_heads, head_dim);
    }
    const bool rotated_row = (r <= q_per_kv) && (inv_freq != nullptr || rope_cos != nullptr);  // queries and K, not V
    if (e < rot_pairs) {
      const int ia = interleaved ? 2 * e : e, ib = interleaved ? 2 * e + 1 : e + rot_pairs;   // the pair's two dims
      const float a = to_f(src[ia]);
      const float b = to_f(src[ib]);
      if (rotated_row) {
        float s, c, ra, rb;
        if (rope_cos) {
          c = rope_cos[size_t(t) * rot_pairs + e];
          s = rope_sin[size_t(t) * rot_pairs + e];
        } else {
          sincosf(float(pos) * inv_freq[e], &s, &c);
        }
        rotate_pair(a, b, c, s, ra, rb);
        dst[ia] = from_f<T>(ra);
        dst[ib] = from_f<T>(rb);
      } else {
        dst[ia] = src[ia];
        dst[ib] = src[ib];
      }
    } else {
      const int i = rot_dims + (e - rot_pairs);
      dst[i] = src[i];
    }
  }
}

// ------------------------------------------------------------------------------------------------
// One block = one tile of BQ consecutive new tokens of one sequence x one query head.
//   tile_seq[i], tile_q0[i]: sequence index and first token (within the sequence's new tokens)
// q [n_tokens, heads, head_dim]; out [n_tokens, heads * head_dim].
// score(q at position p, key at position j) = (q . k_j + alibi_h(j)) * scale for j <= p
// (and j > p - window when window > 0); softmax over those keys in float32; out = sum p_j v_j.
template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         T* __restrict__ out, StepBatch sb, const int* __restrict__ tile_seq,
                         const int* __restrict__ tile_q0, const float* __restrict__ alibi_slopes, int heads,
                         int kv_heads, int head_dim, float scale, int window) {
  extern __shared__ float smem[];
  float* qs = smem;                                 // [BQ][head_dim]
  float* kv = qs + BQ * head_dim;                   // [PTB_PAGE][head_dim + 1], K then V
  float* ps = kv + PTB_PAGE * (head_dim + 1);       // [BQ][PTB_PAGE]
  const int kstride = head_dim + 1;

  const int tile = blockIdx.x, h = blockIdx.y;
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int n_new = sb.seq_new[seq], past = sb.seq_past[seq], start = sb.seq_start[seq];
  const int rows = min(BQ, n_new - q0);
  const int g = h / (heads / kv_heads);
  const int tid = threadIdx.x;
  const int r = tid / 8, c = tid % 8;
  const int my_pos = (r < rows) ? past + q0 + r : -1;  // -1: no key is visible, nothing is stored
  const float slope = alibi_slopes ? alibi_slopes[h] : 0.f;

  for (int i = tid; i < BQ * head_dim; i += THREADS) {
    const int rr = i / head_dim, e = i % head_dim;
    qs[i] = (rr < rows) ? to_f(q[(size_t(start + q0 + rr) * heads + h) * head_dim + e]) : 0.f;
  }
  float acc[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  const int last_pos = past + q0 + rows - 1;
  const int first_pos = past + q0;
  int kb_lo = 0;
  if (window > 0) kb_lo = max(0, first_pos - window + 1) / PTB_PAGE;
  const int kb_hi = last_pos / PTB_PAGE;
  const int* pages = sb.pages + size_t(seq) * sb.pages_stride;

  for (int kb = kb_lo; kb <= kb_hi; ++kb) {
    const int page = pages[kb];
    const int valid = min(PTB_PAGE, last_pos + 1 - kb * PTB_PAGE);  // keys of this block that exist
    const T* kp = k_pool + kv_offset(page, g, 0, kv_heads, head_dim);
    const T* vp = v_pool + kv_offset(page, g, 0, kv_heads, head_dim);
    __syncthreads();  // previous block's V and ps are no longer read
    for (int i = tid; i < PTB_PAGE * head_dim; i += THREADS) {
      const int j = i / head_dim, e = i % head_dim;
      kv[j * kstride + e] = (j < valid) ? to_f(kp[i]) : 0.f;
    }
    __syncthreads();
    // scores: this thread owns keys j = c + 8 jj of row r
    float s[8];
    float m_blk = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int j = c + 8 * jj;
      const int key_pos = kb * PTB_PAGE + j;
      float dot = 0.f;
      const float* qr = qs + r * head_dim;
      const float* kr = kv + j * kstride;
      for (int e = 0; e < head_dim; ++e) dot = fmaf(qr[e], kr[e], dot);
      bool visible = key_pos <= my_pos;
      if (window > 0) visible = visible && (key_pos > my_pos - window);
      float sc = -INFINITY;
      if (visible) {
        if (alibi_slopes) dot += alibi_bias(slope, key_pos);
        sc = dot * scale;
      }
      s[jj] = sc;
      m_blk = fmaxf(m_blk, sc);
    }
    // row maximum and sum over the 8 threads of the row (lanes 8 r' .. 8 r' + 7 of a warp)
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) m_blk = fmaxf(m_blk, __shfl_xor_sync(0xffffffffu, m_blk, o));
    const float m_new = fmaxf(m_run, m_blk);
    float corr = 1.f, l_blk = 0.f;
    if (m_new == -INFINITY) {
      // nothing visible so far (rows beyond the tile, or keys left of a window)
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) ps[r * PTB_PAGE + c + 8 * jj] = 0.f;
    } else {
      corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const float p = (s[jj] == -INFINITY) ? 0.f : expf(s[jj] - m_new);
        ps[r * PTB_PAGE + c + 8 * jj] = p;
        l_blk += p;
      }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) l_blk += __shfl_xor_sync(0xffffffffu, l_blk, o);
    l_run = l_run * corr + l_blk;
    m_run = m_new;
    __syncthreads();  // all scores of this block are written, K is no longer read
    for (int i = tid; i < PTB_PAGE * head_dim; i += THREADS) {
      const int j = i / head_dim, e = i % head_dim;
      kv[j * kstride + e] = (j < valid) ? to_f(vp[i]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < DPT; ++i) acc[i] *= corr;
    for (int j = 0; j < PTB_PAGE; ++j) {
      const float p = ps[r * PTB_PAGE + j];
      const float* vr = kv + j * kstride;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const int e = c + 8 * i;
        if (e < head_dim) acc[i] = fmaf(p, vr[e], acc[i]);
      }
    }
  }
  if (r < rows) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    T* o = out + (size_t(start + q0 + r) * heads + h) * head_dim;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int e = c + 8 * i;
      if (e < head_dim) o[e] = from_f<T>(acc[i] * inv);
    }
  }
}

template <typename T>
int launch_attention(const void* q, const void* k_pool, const void* v_pool, void* out, const StepBatch& sb,
                     const int* tile_seq, const int* tile_q0, int n_tiles, const float* slopes, int heads,
                     int kv_heads, int head_dim, float scale, int window, cudaStream_t stream) {
  const size_t smem = sizeof(float) * (size_t(BQ) * head_dim + size_t(PTB_PAGE) * (head_dim + 1) + BQ * PTB_PAGE);
  static size_t configured = 48 * 1024;  // per element type: raised when a larger head size first comes
  if (smem > configured) {
    if (cudaFuncSetAttribute(attention_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
        cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = smem;
  }
  dim3 grid(n_tiles, heads);
  attention_generic_kernel<T><<<grid, THREADS, smem, stream>>>((const T*)q, (const T*)k_pool, (const T*)v_pool,
                                                               (T*)out, sb, tile_seq, tile_q0, slopes, heads, kv_heads,
                                                               head_dim, scale, window);
  return launch_status();
}

}  // namespace

// cos and sin of position * inv_freq[i] for every token of the step: [n_tokens, pairs] each, float32.
__global__ void rope_table_kernel(const int* __restrict__ tok_pos, const float* __restrict__ inv_freq,
                                  float* __restrict__ cos_out, float* __restrict__ sin_out, int n_tokens, int pairs) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * pairs) return;
  float s, c;
  sincosf(float(tok_pos[i / pairs]) * inv_freq[i % pairs], &s, &c);
  cos_out[i] = c;
  sin_out[i] = s;
}

PTB_API int ptb_rope_table(const int* tok_pos, const float* inv_freq, float* cos_out, float* sin_out, int n_tokens,
                           int pairs, cudaStream_t stream) {
  if (n_tokens <= 0 || pairs <= 0) return PTB_OK;
  const int total = n_tokens * pairs;
  rope_table_kernel<<<(total + 255) / 256, 256, 0, stream>>>(tok_pos, inv_freq, cos_out, sin_out, n_tokens, pairs);
  return launch_status();
}

PTB_API int ptb_split_rotate_store(int dtype, const void* fused, void* q_out, void* k_pool, void* v_pool,
                                   const StepBatch* sb, const float* inv_freq, const float* rope_cos,
                                   const float* rope_sin, int rot_pairs, int kv_heads, int q_per_kv, int head_dim,
                                   int write_cache, int interleaved, cudaStream_t stream) {
  if (sb->n_tokens <= 0) return PTB_OK;
  if (kv_heads <= 0 || q_per_kv <= 0 || head_dim <= 0 || rot_pairs < 0 || 2 * rot_pairs > head_dim)
    return PTB_ERR_SIZE;
  if (inv_freq == nullptr && rope_cos == nullptr) rot_pairs = 0;
  if ((rope_cos == nullptr) != (rope_sin == nullptr)) return PTB_ERR_SIZE;
  const int threads = 256;
  if (dtype == PTB_F32)
    split_rotate_store_kernel<float><<<sb->n_tokens, threads, 0, stream>>>(
        (const float*)fused, (float*)q_out, (float*)k_pool, (float*)v_pool, *sb, inv_freq, rope_cos, rope_sin,
        rot_pairs, kv_heads, q_per_kv, head_dim, write_cache, interleaved);
  else if (dtype == PTB_BF16)
    split_rotate_store_kernel<__nv_bfloat16><<<sb->n_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)fused, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, *sb,
        inv_freq, rope_cos, rope_sin, rot_pairs, kv_heads, q_per_kv, head_dim, write_cache, interleaved);
  else
    return PTB_ERR_DTYPE;
  return launch_status();
}

PTB_API int ptb_attention_generic(int dtype, const void* q, const void* k_pool, const void* v_pool, void* out,
                                  const StepBatch* sb, const int* tile_seq, const int* tile_q0, int n_tiles,
                                  const float* alibi_slopes, int heads, int kv_heads, int head_dim, float scale,
                                  int window, cudaStream_t stream) {
  if (n_tiles <= 0) return PTB_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || head_dim <= 0 || head_dim > MAX_D || heads > 65535)
    return PTB_ERR_SIZE;
  if (dtype == PTB_F32)
    return launch_attention<float>(q, k_pool, v_pool, out, *sb, tile_seq, tile_q0, n_tiles, alibi_slopes, heads,
                                   kv_heads, head_dim, scale, window, stream);
  if (dtype == PTB_BF16)
    return launch_attention<__nv_bfloat16>(q, k_pool, v_pool, out, *sb, tile_seq, tile_q0, n_tiles, alibi_slopes,
                                           heads, kv_heads, head_dim, scale, window, stream);
  return PTB_ERR_DTYPE;
}

// rows of a tile of the general kernel, for the host that builds the tile lists
PTB_API int ptb_attention_generic_tile_rows() { return BQ; }
