// Attention of a decode step in one kernel: for every sequence that brings a single token, take the
// token's row of the fused projection, rotate its queries and its key, put key and value into the
// paged cache, attend over the cache with all query heads of a K/V group in one tile, divide the key
// pages among blocks, and let the last block that finishes join the partial results.
//
// It does what split_rotate_store + attention_mma + attention_mma_reduce do for such steps, in one
// launch instead of three: the chain of small kernels between the two projections of a decode layer
// is what keeps a weight-bound step from the memory roofline.
//
//   grid = (sequences, K/V heads x head chunks, splits); block = 16 rows per warp, rows = heads.
//   Key pages are copied with cp.async into a three-stage ring of swizzled tiles.
//   The new token's key and value are written to the cache by one block per (sequence, K/V head)
//   and patched into the shared tile by every block that covers the token's page, so no block reads
//   a cache row that another block may still be writing.
//   Joining: the blocks that share a (sequence, head chunk) form one thread-block cluster
//   (cluster size = number of splits: 1, 2, 4 or 8). Each block leaves (max, sum, unnormalised
//   output) of its rows in its own shared memory; after a cluster barrier every block joins a
//   share of the rows, reading the other blocks' shared memory directly (distributed shared
//   memory), and writes them out. No workspace in global memory, no atomics, no second launch.
#include <cooperative_groups.h>

#include "mma_common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int STAGES = 3;

struct DecodeParams {
  int heads, kv_heads, hpk, n_splits, n_teams, rot_pairs, write_cache, window, interleaved;
  float scale;
  float* team_parts;   // [n_seqs][kv_heads * chunks][n_teams][hpk][D + 2] float32 when n_teams > 1
  int* tickets;        // [n_seqs][kv_heads * chunks][n_splits], zero before and after the launch
};

// KS: the 64 keys of a page are divided among KS groups of warps (KS = 1, 2 or 4). A group keeps its
// own running maximum, sum and output over its share of the keys of every page, like a block of a
// split set does over its pages, and the groups' results meet in the same join. A step of single
// tokens is a chain of dependent work per page and warp; with few query heads per K/V head (one
// warp of rows) this is what puts more warps on the chain's pages.
template <int D, int KS>
__global__ void __launch_bounds__(D == 64 ? 320 : 256)
attention_decode_kernel(const __nv_bfloat16* __restrict__ fused, __nv_bfloat16* __restrict__ k_pool,
                        __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out, StepBatch sb, const float* __restrict__ rope_cos, const float* __restrict__ rope_sin,
                        const float* __restrict__ alibi_slopes, DecodeParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int TILE_BYTES = KEYS * D * 2;
  const uint32_t smem_base = smem_u32(smem_raw);  // stage s: K at s * 2 * TILE_BYTES, V right after
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
  const int row_warps = (nthreads >> 5) / KS;
  const int rows_total = 16 * row_warps;
  const int rb = warp % row_warps;             // which 16 rows (query heads) this warp holds
  const int kp = warp / row_warps;             // which share of a page's keys it takes
  constexpr int PART = D + 2;                  // floats of a row in the teams' workspace: output, maximum, sum
  constexpr int NT = KEYS / 8 / KS;            // 8-key tiles of S per warp and page
  constexpr int KT = KEYS / 16 / KS;           // 16-key steps of P V per warp and page
  const int g4 = lane >> 2, t4 = lane & 3;

  const int seq = blockIdx.x;
  const int qpk = p.heads / p.kv_heads;
  const int chunks = (qpk + p.hpk - 1) / p.hpk;
  const int g = blockIdx.y / chunks;
  const int chunk = blockIdx.y % chunks;
  const int h0 = chunk * p.hpk;
  const int split = blockIdx.z % p.n_splits, team = blockIdx.z / p.n_splits;   // a cluster = consecutive z
  const int pos = sb.seq_past[seq];            // position of the new token
  const int tok = sb.seq_start[seq];           // its row in the step
  const int head_valid = min(p.hpk, qpk - h0);
  const int fused_width = p.kv_heads * (qpk + 2) * D;
  const __nv_bfloat16* frow = fused + size_t(tok) * fused_width + size_t(g) * (qpk + 2) * D;
  const float* rc = rope_cos ? rope_cos + size_t(tok) * p.rot_pairs : nullptr;
  const float* rs = rope_sin ? rope_sin + size_t(tok) * p.rot_pairs : nullptr;
  const int P = rc ? p.rot_pairs : 0;          // pairs (e, e + P), or (2 e, 2 e + 1), are rotated for e < P

  bool row_ok[2];
  int row_head[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    row_head[i] = rb * 16 + g4 + 8 * i;
    row_ok[i] = row_head[i] < head_valid;
  }
  float slope[2] = {0.f, 0.f};
  if (alibi_slopes) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (row_ok[i]) slope[i] = alibi_slopes[g * qpk + h0 + row_head[i]];
  }
  // pages of this block
  int kb_first = 0;
  if (p.window > 0) kb_first = max(0, pos - p.window + 1) / KEYS;
  const int kb_last = pos / KEYS;               // page that holds the new token
  const int n_pages = kb_last + 1 - kb_first;
  const int n_sharers = p.n_splits * p.n_teams;
  const int kb_begin = kb_first + int((long long)blockIdx.z * n_pages / n_sharers);
  const int kb_end = kb_first + int((long long)(blockIdx.z + 1) * n_pages / n_sharers);
  const int* pages = sb.pages + size_t(seq) * sb.pages_stride;
  const int n_mine = max(0, kb_end - kb_begin);

  auto issue = [&](int i) {  // copy page kb_begin + i into stage i % STAGES (or nothing), one group
    if (i < n_mine) {
      const int page = pages[kb_begin + i];
      const uint32_t dst = smem_base + (i % STAGES) * 2 * TILE_BYTES;
      load_page<D>(dst, k_pool + kv_offset(page, g, 0, p.kv_heads, D), tid, nthreads);
      load_page<D>(dst + TILE_BYTES, v_pool + kv_offset(page, g, 0, p.kv_heads, D), tid, nthreads);
    }
    cp_async_commit();
  };
  for (int i = 0; i < STAGES - 1; ++i) issue(i);   // the first pages travel while the token's row is prepared

  // The token's row of the fused projection, staged after the page ring: rows 0 .. hpk - 1 the query
  // heads of this chunk, row hpk its key, row hpk + 1 its value; 16-byte copies, then the rotation in
  // place (pairs (e, e + P)), rounded to bfloat16 as the stored queries of the three-kernel path are.
  __nv_bfloat16* rowbuf = reinterpret_cast<__nv_bfloat16*>(smem_raw + size_t(STAGES) * 2 * TILE_BYTES);
  float* cs = reinterpret_cast<float*>(rowbuf + size_t(p.hpk + 2) * D);   // cos[P], sin[P]
  {
    const uint4* src_q = reinterpret_cast<const uint4*>(frow + size_t(h0) * D);
    const uint4* src_kv = reinterpret_cast<const uint4*>(frow + size_t(qpk) * D);
    uint4* dst_q = reinterpret_cast<uint4*>(rowbuf);
    uint4* dst_kv = reinterpret_cast<uint4*>(rowbuf + size_t(p.hpk) * D);
    for (int i = tid; i < head_valid * (D / 8); i += nthreads) dst_q[i] = src_q[i];
    for (int i = tid; i < 2 * (D / 8); i += nthreads) dst_kv[i] = src_kv[i];
    for (int e = tid; e < P; e += nthreads) {
      cs[e] = rc[e];
      cs[P + e] = rs[e];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < (head_valid + 1) * P; idx += nthreads) {
    const int r = idx / P, e = idx % P;
    __nv_bfloat16* row = rowbuf + size_t(r < head_valid ? r : p.hpk) * D;
    float ra, rb;
    const int ia = p.interleaved ? 2 * e : e, ib = p.interleaved ? 2 * e + 1 : e + P;   // the pair's two dims
    rotate_pair(__bfloat162float(row[ia]), __bfloat162float(row[ib]), cs[e], cs[P + e], ra, rb);
    row[ia] = __float2bfloat16_rn(ra);
    row[ib] = __float2bfloat16_rn(rb);
  }
  __syncthreads();
  const __nv_bfloat16* krow = rowbuf + size_t(p.hpk) * D;   // rotated key, value
  const __nv_bfloat16* vrow = krow + D;
  // Q fragments
  uint32_t qa[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t lo = 0u, hi = 0u;
      if (row_ok[i]) {
        const __nv_bfloat16* qr = rowbuf + size_t(row_head[i]) * D + kk * 16 + t4 * 2;
        lo = *reinterpret_cast<const uint32_t*>(qr);
        hi = *reinterpret_cast<const uint32_t*>(qr + 8);
      }
      qa[kk][i] = lo;
      qa[kk][2 + i] = hi;
    }
  }

  // the new token's key and value go to the cache once per (sequence, K/V head)
  const bool covers_new = n_mine > 0 && kb_end == kb_last + 1;
  if (p.write_cache && chunk == 0 && covers_new) {
    const size_t off = kv_offset(pages[kb_last], g, pos % KEYS, p.kv_heads, D);
    for (int e = tid; e < D; e += nthreads) {
      k_pool[off + e] = krow[e];
      v_pool[off + e] = vrow[e];
    }
  }

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl2 = p.scale * 1.4426950408889634f;

  for (int i = 0; i < n_mine; ++i) {
    const int kb = kb_begin + i;
    issue(i + STAGES - 1);
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const uint32_t ks = smem_base + (i % STAGES) * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
    if (kb == kb_last && p.write_cache) {
      // the new token's row, from this block's staging rather than from the cache (another block
      // may still be writing it there). A layer that only reads another layer's cache finds the row
      // in the cache: the owner wrote it earlier in the step.
      unsigned char* kt = smem_raw + (i % STAGES) * 2 * TILE_BYTES;
      const int r = pos % KEYS;
      for (int e = tid; e < D; e += nthreads) {
        const uint32_t o2 = swz<D>(r, e >> 3) + (e & 7) * 2;
        *reinterpret_cast<__nv_bfloat16*>(kt + o2) = krow[e];
        *reinterpret_cast<__nv_bfloat16*>(kt + TILE_BYTES + o2) = vrow[e];
      }
      __syncthreads();
    }
    float s[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D / 16; kk += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, ks + swz<D>((kp * NT + j) * 8 + (lane & 7), 2 * kk + (lane >> 3)));
        mma_bf16(s[j], qa[kk], b0, b1);
        mma_bf16(s[j], qa[kk + 1], b2, b3);
      }
    }
    float m_blk[2] = {-INFINITY, -INFINITY};
    // a page that every row sees whole, without a bias: scale and maximum only (rows past the valid
    // heads have zero queries; their numbers are never written)
    const bool whole_page = kb < kb_last && !alibi_slopes && (p.window == 0 || kb * KEYS > pos - p.window);
    if (whole_page) {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[j][e] *= sl2;
          m_blk[e >> 1] = fmaxf(m_blk[e >> 1], s[j][e]);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i2 = e >> 1;
          const int key_pos = kb * KEYS + (kp * NT + j) * 8 + t4 * 2 + (e & 1);
          bool visible = row_ok[i2] && key_pos <= pos;
          if (p.window > 0) visible = visible && key_pos > pos - p.window;
          float v = s[j][e];
          if (alibi_slopes) v += alibi_bias(slope[i2], key_pos);
          v = visible ? v * sl2 : -INFINITY;
          s[j][e] = v;
          m_blk[i2] = fmaxf(m_blk[i2], v);
        }
      }
    }
    float corr[2];
#pragma unroll
    for (int i2 = 0; i2 < 2; ++i2) {
      m_blk[i2] = fmaxf(m_blk[i2], __shfl_xor_sync(0xffffffffu, m_blk[i2], 1));
      m_blk[i2] = fmaxf(m_blk[i2], __shfl_xor_sync(0xffffffffu, m_blk[i2], 2));
      const float m_new = fmaxf(m_run[i2], m_blk[i2]);
      corr[i2] = (m_run[i2] == -INFINITY) ? 0.f : fast_exp2(m_run[i2] - m_new);
      m_run[i2] = m_new;
    }
    uint32_t pa[KT][4];
    float l_blk[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i2 = e >> 1;
        pv[e] = (s[j][e] == -INFINITY) ? 0.f : fast_exp2(s[j][e] - m_run[i2]);
        l_blk[i2] += pv[e];
      }
      pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(pv[0], pv[1]);
      pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
    }
#pragma unroll
    for (int i2 = 0; i2 < 2; ++i2) l_run[i2] = l_run[i2] * corr[i2] + l_blk[i2];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0];
      o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < KT; ++kk) {
#pragma unroll
      for (int j = 0; j < D / 8; j += 2) {
        uint32_t b0, b1, b2, b3;
        const int m = lane >> 3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vs + swz<D>((kp * KT + kk) * 16 + (m & 1) * 8 + (lane & 7), j + (m >> 1)));
        mma_bf16(o[j], pa[kk], b0, b1);
        mma_bf16(o[j + 1], pa[kk], b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }

  __nv_bfloat16* out_tok = out + (size_t(tok) * p.heads + g * qpk + h0) * D;
  if (p.n_splits == 1 && KS == 1 && p.n_teams == 1) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (!row_ok[i]) continue;
      const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
      __nv_bfloat16* dst = out_tok + size_t(row_head[i]) * D + t4 * 2;
#pragma unroll
      for (int j = 0; j < D / 8; ++j)
        *reinterpret_cast<uint32_t*>(dst + j * 8) = pack_bf16(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
    }
    return;
  }
  // partial results of this block, in its own shared memory (the page ring is no longer needed):
  // po [KS][rows_total][D] float32, then pml [KS][rows_total][2]
  float* po = reinterpret_cast<float*>(smem_raw);
  float* pml = po + KS * rows_total * D;
  if (KS > 1) __syncthreads();   // every warp is past its last page: the ring may be overwritten
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = kp * rows_total + row_head[i];
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
      *reinterpret_cast<float2*>(po + size_t(r) * D + j * 8 + t4 * 2) = make_float2(o[j][2 * i], o[j][2 * i + 1]);
    if (t4 == 0) {
      pml[r * 2 + 0] = m_run[i];
      pml[r * 2 + 1] = l_run[i];
    }
  }
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();  // every block of the cluster has written its partial results
  const int n_splits = p.n_splits;
  // rows r with r % n_splits == split are joined by this block: thread -> (row, 4 dims)
  constexpr int VEC = 4;
  const int per_row = D / VEC;
  const int my_rows = (head_valid - split + n_splits - 1) / n_splits;  // rows split, split + n, ...
  for (int idx = tid; idx < my_rows * per_row; idx += nthreads) {
    const int r = split + (idx / per_row) * n_splits;
    const int d0 = (idx % per_row) * VEC;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) {
      const float* rml = cluster.map_shared_rank(pml, s);
#pragma unroll
      for (int k2 = 0; k2 < KS; ++k2) m = fmaxf(m, rml[(k2 * rows_total + r) * 2]);
    }
    float acc[VEC] = {0.f, 0.f, 0.f, 0.f};
    float l = 0.f;
    for (int s = 0; s < n_splits; ++s) {   // always in the same order: blocks of the split set, then key groups
      const float* rml = cluster.map_shared_rank(pml, s);
      const float* rpo = cluster.map_shared_rank(po, s);
#pragma unroll
      for (int k2 = 0; k2 < KS; ++k2) {
        const int rr = k2 * rows_total + r;
        const float ms = rml[rr * 2];
        const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
        l += rml[rr * 2 + 1] * w;
        const float4 v = *reinterpret_cast<const float4*>(rpo + size_t(rr) * D + d0);
        acc[0] += v.x * w; acc[1] += v.y * w; acc[2] += v.z * w; acc[3] += v.w * w;
      }
    }
    if (p.n_teams > 1) {
      // the cluster's rows as they are, for the join of the teams
      float* dst = p.team_parts + ((size_t(seq) * gridDim.y + blockIdx.y) * p.n_teams + team) * p.hpk * PART + size_t(r) * PART;
      *reinterpret_cast<float2*>(dst + d0) = make_float2(acc[0], acc[1]);
      *reinterpret_cast<float2*>(dst + d0 + 2) = make_float2(acc[2], acc[3]);
      if (d0 == 0) *reinterpret_cast<float2*>(dst + D) = make_float2(m, l);
      continue;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* dst = out_tok + size_t(r) * D + d0;
    *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc[0] * inv, acc[1] * inv), pack_bf16(acc[2] * inv, acc[3] * inv));
  }
  cluster.sync();  // no block leaves while another still reads its shared memory
  if (p.n_teams == 1) return;
  // The teams' join: every block takes a ticket for its share of the rows (r % n_splits == split); the one
  // that draws the last joins what the teams left, always in the order of the teams, and puts the
  // counter back to zero.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  int* ticket = p.tickets + (size_t(seq) * gridDim.y + blockIdx.y) * n_splits + split;
  if (tid == 0) s_last = (atomicAdd(ticket, 1) == p.n_teams - 1) ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* parts = p.team_parts + (size_t(seq) * gridDim.y + blockIdx.y) * p.n_teams * p.hpk * PART;
  for (int idx = tid; idx < my_rows * per_row; idx += nthreads) {
    const int r = split + (idx / per_row) * n_splits;
    const int d0 = (idx % per_row) * VEC;
    // eight teams' loads in flight at a time: this block alone reads what all teams left
    float m = -INFINITY;
    for (int t0 = 0; t0 < p.n_teams; t0 += 8) {
      float mt[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        mt[u] = (t0 + u < p.n_teams) ? __ldcg(parts + (size_t(t0 + u) * p.hpk + r) * PART + D) : -INFINITY;
#pragma unroll
      for (int u = 0; u < 8; ++u) m = fmaxf(m, mt[u]);
    }
    float acc[VEC] = {0.f, 0.f, 0.f, 0.f};
    float l = 0.f;
    for (int t0 = 0; t0 < p.n_teams; t0 += 8) {
      float2 ml[8], v0[8], v1[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float* pr = parts + (size_t(min(t0 + u, p.n_teams - 1)) * p.hpk + r) * PART;
        ml[u] = __ldcg(reinterpret_cast<const float2*>(pr + D));
        v0[u] = __ldcg(reinterpret_cast<const float2*>(pr + d0));
        v1[u] = __ldcg(reinterpret_cast<const float2*>(pr + d0 + 2));
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float w = (t0 + u >= p.n_teams || ml[u].x == -INFINITY) ? 0.f : exp2f(ml[u].x - m);
        l += ml[u].y * w;
        acc[0] += v0[u].x * w; acc[1] += v0[u].y * w; acc[2] += v1[u].x * w; acc[3] += v1[u].y * w;
      }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* dst = out_tok + size_t(r) * D + d0;
    *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc[0] * inv, acc[1] * inv), pack_bf16(acc[2] * inv, acc[3] * inv));
  }
  if (tid == 0) *ticket = 0;
}

template <int D, int KS>
int launch_decode(const void* fused, void* k_pool, void* v_pool, void* out, const StepBatch& sb,
                  const float* rope_cos, const float* rope_sin, const float* slopes, const DecodeParams& p,
                  int warps, cudaStream_t stream) {
  const int qpk = p.heads / p.kv_heads;
  const int chunks = (qpk + p.hpk - 1) / p.hpk;
  // page ring, then the token's row (query heads of the chunk, key, value) and its cos/sin
  const size_t ring = size_t(STAGES) * 2 * KEYS * D * 2;
  size_t smem = ring + size_t(p.hpk + 2) * D * 2 + size_t(D) * sizeof(float);
  const size_t join = size_t(KS) * warps * 16 * (D + 2) * sizeof(float);  // partial results reuse the ring
  if (join > smem) smem = join;
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(attention_decode_kernel<D, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) !=
        cudaSuccess)
      return PTB_ERR_LAUNCH;
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sb.n_seqs, p.kv_heads * chunks, p.n_splits * p.n_teams);
  cfg.blockDim = dim3(warps * KS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = p.n_splits;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, attention_decode_kernel<D, KS>, (const __nv_bfloat16*)fused, (__nv_bfloat16*)k_pool,
                         (__nv_bfloat16*)v_pool, (__nv_bfloat16*)out, sb, rope_cos, rope_sin, slopes,
                         p) != cudaSuccess) {
    (void)cudaGetLastError();
    return PTB_ERR_LAUNCH;
  }
  return launch_status();
}

}  // namespace

// Splits that a launch may use: the blocks of a split set form one cluster.
PTB_API int ptb_attention_decode_max_splits() { return 8; }

// Every sequence of the step brings exactly one token. fused [n_seqs, kv_heads * (q_per_kv + 2) *
// head_dim] bfloat16; out [n_seqs, heads * head_dim]. n_teams clusters of n_splits (1 to 8) blocks share a
// sequence's pages; more than one team needs `team_parts` (n_seqs * kv_heads * chunks * n_teams * hpk *
// (head_dim + 2) floats) and `tickets` (n_seqs * kv_heads * chunks * n_splits ints, zero before the launch
// and after it). key_split 1, 2 or 4 groups
// of `warps` warps each share the keys of every page (warps * key_split <= 10 for head size 64, 8 for 128). rope_cos/sin:
// [n_seqs, rot_pairs] float32 tables for the step's tokens, or null for no rotation; the rotated pairs are
// (e, e + rot_pairs), or with `interleaved` (2 e, 2 e + 1).
PTB_API int ptb_attention_decode(const void* fused, void* k_pool, void* v_pool, void* out, const StepBatch* sb,
                                 const float* rope_cos, const float* rope_sin, int rot_pairs, int interleaved,
                                 const float* alibi_slopes, int heads, int kv_heads, int head_dim, int hpk,
                                 int n_splits, int n_teams, int warps, int key_split, float scale, int window,
                                 int write_cache, float* team_parts, size_t team_floats, int* tickets, int n_tickets,
                                 cudaStream_t stream) {
  if (sb->n_seqs <= 0) return PTB_OK;
  if (sb->n_tokens != sb->n_seqs) return PTB_ERR_SIZE;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || warps < 1 || warps > 8 || hpk < 1 ||
      hpk > warps * 16 || rot_pairs < 0 || 2 * rot_pairs > head_dim)
    return PTB_ERR_SIZE;
  if (n_splits < 1 || n_splits > 8) return PTB_ERR_SIZE;   // a cluster holds at most 8 blocks
  if ((key_split != 1 && key_split != 2 && key_split != 4) || warps * key_split > (head_dim == 64 ? 10 : 8))
    return PTB_ERR_SIZE;
  if ((rope_cos == nullptr) != (rope_sin == nullptr)) return PTB_ERR_SIZE;
  const int qpk = heads / kv_heads;
  const int chunks = (qpk + hpk - 1) / hpk;
  if (kv_heads * chunks > 65535 || n_teams < 1 || n_splits * n_teams > 65535) return PTB_ERR_SIZE;
  if (n_teams > 1) {
    const size_t groups = size_t(sb->n_seqs) * kv_heads * chunks;
    if (team_parts == nullptr || tickets == nullptr || team_floats < groups * n_teams * hpk * (head_dim + 2) ||
        size_t(n_tickets) < groups * n_splits || (reinterpret_cast<uintptr_t>(team_parts) & 7))
      return PTB_ERR_SIZE;
  }
  DecodeParams p;
  p.heads = heads; p.kv_heads = kv_heads; p.hpk = hpk; p.n_splits = n_splits; p.n_teams = n_teams;
  p.rot_pairs = rot_pairs; p.write_cache = write_cache; p.window = window; p.scale = scale;
  p.interleaved = interleaved ? 1 : 0;
  p.team_parts = team_parts; p.tickets = tickets;
#define PTB_DECODE(DD, KK) \
  return launch_decode<DD, KK>(fused, k_pool, v_pool, out, *sb, rope_cos, rope_sin, alibi_slopes, p, warps, stream)
  if (head_dim == 64) {
    if (key_split == 1) PTB_DECODE(64, 1);
    if (key_split == 2) PTB_DECODE(64, 2);
    PTB_DECODE(64, 4);
  }
  if (head_dim == 128) {
    if (key_split == 1) PTB_DECODE(128, 1);
    if (key_split == 2) PTB_DECODE(128, 2);
    PTB_DECODE(128, 4);
  }
#undef PTB_DECODE
  return PTB_ERR_SIZE;
}
