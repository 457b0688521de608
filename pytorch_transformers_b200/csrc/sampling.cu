// Next-token selection on the device: one block per row of float32 logits.
//   processors, in the reference's order: repetition penalty, suppression of stop tokens (while a
//   minimum of new tokens is not reached), then for sampling: temperature, top-k, top-p, min-p;
//   selection: argmax (greedy) or a draw from softmax by inverse CDF with a counter-based uniform.
// `work` is scratch of the same shape as the logits; the logits themselves are left untouched.
//
// One block has to hide the latency of a whole row by itself (a pass over 65,024 floats takes it about
// 5 us), so the work is counted in passes over the row:
//   greedy: one pass. Sampling: one pass that scales the row into `work` and leaves each thread the
//   maximum of its own tokens. The top_k-th largest of these 1,024 maxima bounds the top_k-th largest
//   token from below, and closely, so one more pass gathers the few tokens above it into shared memory;
//   a sort by (value, token) there gives the exact top-k, the top-p cut, min-p and the draw. Top-p
//   without top-k looks among the 256 largest first and is done if the rest of the row weighs less than
//   1 - top_p. Rows with more candidates than the block has threads (flat distributions, a large top_k,
//   many equal values) take the exact ways: radix selection for top-k (12 + 12 + 8 bits), an interval of
//   keys narrowed by seven thresholds a pass for top-p, and a draw over the warps' ranges of the row.
//   Every sum runs in a fixed order, so a draw depends on (seed, stream, counter) and the row alone.
// Measured on B200 at 65,024 tokens a row, 8 to 64 rows, inside a CUDA graph: greedy 6 us, temperature
// 27 us, top_k = 50 with or without top_p 24 us, top_p on a peaked row 37 us, on a flat one 150 us.
#include "common.cuh"

namespace {

constexpr int ST = 1024;  // threads per row

// order-preserving map float -> uint32 (larger float <=> larger key); -inf is the smallest finite key
__device__ __forceinline__ uint32_t ordered_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// uniform in [0, 1) from (seed, stream, counter): the same three numbers give the same draw
// whatever else is in the batch
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t stream, uint64_t counter) {
  const uint64_t h = splitmix64(splitmix64(splitmix64(seed) ^ stream) ^ counter);
  return float(h >> 40) * (1.0f / 16777216.0f);
}

struct BlockScratch {
  float f[32];
  int i[32];
  unsigned int u[32];
};

// Scans over the ST threads of a block in thread order, always by the same tree: per warp by shuffles,
// then the 32 warp totals by the first warp. `buf` has 65 entries; the grand total is left in buf[64].
__device__ __forceinline__ float warp_inclusive_scan_f(float v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}
__device__ __forceinline__ unsigned int warp_inclusive_scan_u(unsigned int v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned int t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}
__device__ __forceinline__ float block_inclusive_scan_f(float v, float* buf) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_inclusive_scan_f(v, lane);
  __syncthreads();
  if (lane == 31) buf[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const float t = warp_inclusive_scan_f(buf[lane], lane);
    buf[32 + lane] = t;  // inclusive totals of the warps
    if (lane == 31) buf[64] = t;
  }
  __syncthreads();
  return v + (warp > 0 ? buf[32 + warp - 1] : 0.f);
}
__device__ __forceinline__ unsigned int block_exclusive_scan_u(unsigned int v, unsigned int* buf) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned int inc = warp_inclusive_scan_u(v, lane);
  __syncthreads();
  if (lane == 31) buf[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    const unsigned int t = warp_inclusive_scan_u(buf[lane], lane);
    buf[32 + lane] = t;
    if (lane == 31) buf[64] = t;
  }
  __syncthreads();
  return inc - v + (warp > 0 ? buf[32 + warp - 1] : 0u);
}

// A row is read in groups of four tokens (one 16-byte load where the row allows it), U groups of a thread
// in flight at a time: one block has to hide the latency of a whole row by itself.
struct RowView {
  int vocab;
  int groups;   // ceil(vocab / 4)
  bool vec;     // vocab % 4 == 0 and 16-byte aligned rows
};
__device__ __forceinline__ void load_group(const float* r, const RowView& rv, int j, float (&x)[4]) {
  if (rv.vec) {
    const float4 q = reinterpret_cast<const float4*>(r)[j];
    x[0] = q.x; x[1] = q.y; x[2] = q.z; x[3] = q.w;
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) x[c] = (4 * j + c < rv.vocab) ? r[4 * j + c] : -INFINITY;
  }
}
__device__ __forceinline__ void store_group(float* r, const RowView& rv, int j, const float (&x)[4]) {
  if (rv.vec) {
    reinterpret_cast<float4*>(r)[j] = make_float4(x[0], x[1], x[2], x[3]);
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c)
      if (4 * j + c < rv.vocab) r[4 * j + c] = x[c];
  }
}
// f(j, x, ok) for the groups first + id, first + id + step, ... below limit; every thread of the team
// (id = 0 .. step - 1) makes the same number of calls, with ok = false past the end, so f may vote.
template <int U, typename F>
__device__ __forceinline__ void sweep(const float* r, const RowView& rv, int first, int limit, int id, int step, F&& f) {
  for (int b = first; b < limit; b += step * U) {
    float x[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = b + u * step + id;
      if (j < limit) load_group(r, rv, j, x[u]);
      else x[u][0] = x[u][1] = x[u][2] = x[u][3] = -INFINITY;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = b + u * step + id;
      if (b + u * step < limit) f(j, x[u], j < limit);
    }
  }
}

struct SampleParams {
  int vocab;
  int do_sample;
  float temperature;
  int top_k;
  float top_p;
  float min_p;
  float repetition_penalty;
  int history_stride;    // row stride of `history`
  int n_suppress;        // stop tokens to suppress (0: none)
  unsigned long long seed;
};

// Ascending bitonic sort of the first n (a power of two) entries of `a` in shared memory by the whole block.
template <typename T>
__device__ __forceinline__ void block_sort_ascending(T* a, int n) {
  const int tid = threadIdx.x;
  for (int k2 = 2; k2 <= n; k2 <<= 1)
    for (int j = k2 >> 1; j > 0; j >>= 1) {
      const int other = tid ^ j;
      if (tid < n && other > tid) {
        const T x = a[tid], y = a[other];
        const bool up = (tid & k2) == 0;
        if (x != y && (x > y) == up) { a[tid] = y; a[other] = x; }
      }
      __syncthreads();
    }
}

__device__ __forceinline__ float key_value(uint32_t key) {  // the inverse of ordered_key
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// One pass of the radix selection: among the keys that agree with `prefix` on the bits above the digit,
// the digit (bits [shift, shift + bits)) of the want-th largest. Leaves the digit in *pick, the number of
// such keys with a larger digit in *above and the number with this digit in *same.
__device__ __forceinline__ void radix_pass(const float* w, const RowView& rv, uint32_t prefix, int shift, int bits,
                                           unsigned int want, unsigned int* hist, unsigned int* scan_buf,
                                           unsigned int* pick, unsigned int* above, unsigned int* same) {
  const int tid = threadIdx.x, lane = tid & 31;
  const int bins = 1 << bits;
  for (int i = tid; i < bins; i += ST) hist[i] = 0u;
  __syncthreads();
  const uint32_t high_mask = (shift + bits >= 32) ? 0u : (0xffffffffu << (shift + bits));
  const uint32_t digit_mask = uint32_t(bins - 1);
  sweep<4>(w, rv, 0, rv.groups, tid, ST, [&](int j, const float (&x)[4], bool ok) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t key = ordered_key(x[c]);
      const bool in = ok && 4 * j + c < rv.vocab && (key & high_mask) == prefix;
      if (__ballot_sync(0xffffffffu, in) == 0u) continue;
      // lanes of a warp with the same digit add once (whole numbers: the order of the additions is free)
      const uint32_t digit = in ? ((key >> shift) & digit_mask) : 0xffffffffu;
      const unsigned int peers = __match_any_sync(0xffffffffu, digit);
      if (in && lane == __ffs(peers) - 1) atomicAdd(&hist[digit], (unsigned int)__popc(peers));
    }
  });
  __syncthreads();
  // thread t looks after `per` digits, the largest digits first; the exclusive scan gives the keys above them
  const int per = bins >= ST ? bins / ST : 1;
  const int top = bins - 1 - tid * per;  // my largest digit
  unsigned int mine = 0u;
  if (top >= 0)
    for (int d = 0; d < per; ++d) mine += hist[top - d];
  unsigned int before = block_exclusive_scan_u(mine, scan_buf);
  if (top >= 0 && before < want && want <= before + mine) {
    for (int d = 0; d < per; ++d) {
      const unsigned int h = hist[top - d];
      if (want <= before + h) {
        *pick = (unsigned int)(top - d);
        *above = before;
        *same = h;
        break;
      }
      before += h;
    }
  }
  __syncthreads();
}

constexpr int HIST_BITS = 12;

__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, float* __restrict__ work, int* __restrict__ out,
              const int* __restrict__ history, const int* __restrict__ history_len,
              const int* __restrict__ suppress, const long long* __restrict__ streams,
              const long long* __restrict__ counters, SampleParams p) {
  __shared__ BlockScratch sc;
  __shared__ unsigned int s_hist[1 << HIST_BITS];
  __shared__ unsigned long long s_cand[ST];   // candidates: ordered key of the value above, token below
  __shared__ float s_scan_f[65];
  __shared__ unsigned int s_scan_u[65];
  __shared__ unsigned int s_pick, s_above, s_same, s_count;
  __shared__ float s_cut;
  const int row = blockIdx.x, tid = threadIdx.x, V = p.vocab;
  const int lane = tid & 31, warp = tid >> 5;
  if (tid == 0) { s_pick = 0u; s_above = 0u; s_same = 0u; s_count = 0u; s_cut = -INFINITY; }
  const float* lg = logits + size_t(row) * V;
  float* w = work + size_t(row) * V;   // scratch copy of the row that the processors may change
  RowView rv;
  rv.vocab = V;
  rv.groups = (V + 3) >> 2;
  rv.vec = (V & 3) == 0 && ((reinterpret_cast<uintptr_t>(lg) | reinterpret_cast<uintptr_t>(w)) & 15u) == 0;

  const bool touched = (p.repetition_penalty != 1.0f && history) || p.n_suppress > 0;
  const float* src = lg;  // where the row stands after the processors that run before the temperature
  if (touched) {
    sweep<4>(lg, rv, 0, rv.groups, tid, ST, [&](int j, const float (&x)[4], bool ok) {
      if (ok) store_group(w, rv, j, x);
    });
    __syncthreads();
    src = w;
  }
  if (p.repetition_penalty != 1.0f && history) {
    const int* hist = history + size_t(row) * p.history_stride;
    const int n = history_len[row];
    for (int i = tid; i < n; i += ST) {
      const int tok = hist[i];
      if (tok >= 0 && tok < V) {
        const float v = lg[tok];  // from the untouched logits: a token seen twice is penalised once
        w[tok] = v < 0.f ? v * p.repetition_penalty : v / p.repetition_penalty;
      }
    }
    __syncthreads();
  }
  if (p.n_suppress > 0) {
    for (int i = tid; i < p.n_suppress; i += ST) {
      const int tok = suppress[i];
      if (tok >= 0 && tok < V) w[tok] = -INFINITY;
    }
    __syncthreads();
  }

  if (!p.do_sample) {
    // argmax, the lowest index among equal maxima
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    sweep<4>(src, rv, 0, rv.groups, tid, ST, [&](int j, const float (&x)[4], bool ok) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = 4 * j + c;
        if (ok && i < V && (x[c] > best || (x[c] == best && i < best_i))) { best = x[c]; best_i = i; }
      }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { sc.f[warp] = best; sc.i[warp] = best_i; }
    __syncthreads();
    if (tid < 32) {
      best = sc.f[tid]; best_i = sc.i[tid];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
      }
      if (tid == 0) out[row] = (best_i == 0x7fffffff) ? 0 : best_i;
    }
    return;
  }

  // ---- sampling ----
  const float inv_t = 1.0f / p.temperature;
  float vmax = -INFINITY;   // of my own tokens first, then of the row
  sweep<4>(src, rv, 0, rv.groups, tid, ST, [&](int j, const float (&x)[4], bool ok) {
    if (!ok) return;
    float y[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      y[c] = x[c] * inv_t;
      vmax = fmaxf(vmax, y[c]);   // (what lies past the row's end was loaded as -inf)
    }
    store_group(w, rv, j, y);
  });
  const float my_max = vmax;
  vmax = block_max(vmax, sc.f);   // its barriers also make the scaled row visible to the whole block
  const float u01 = uniform01(p.seed, (uint64_t)streams[row], (uint64_t)counters[row]);

  // Candidates: the top_k largest values (ties with the last of them included). Without top-k, top-p looks
  // among the PROBE largest first: on a peaked distribution its cut lies there (`probe`), and if the rest
  // of the row weighs more than 1 - top_p the whole row is searched below instead.
  constexpr int PROBE = 256;
  int select = 0;
  bool probe = false;
  if (p.top_k > 0 && p.top_k < V) {
    select = p.top_k;
  } else if (p.top_p < 1.0f && V > ST) {
    select = PROBE;
    probe = true;
  }
  // Candidates are gathered in any order (a slot from a counter) and then sorted by (value, token), so what
  // follows does not depend on the order of arrival.
  uint32_t bound = 0u;  // keys >= bound are candidates
  auto gather = [&](uint32_t from, uint32_t upto) -> int {   // the tokens with from <= key <= upto
    __syncthreads();
    if (tid == 0) s_count = 0u;
    __syncthreads();
    sweep<4>(w, rv, 0, rv.groups, tid, ST, [&](int j, const float (&x)[4], bool ok) {
      const int valid = ok ? min(4, V - 4 * j) : 0;   // tokens of this group inside the row
      uint32_t key[4];
      unsigned int mine = 0u;                          // bit c: token c of my group is a candidate
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        key[c] = ordered_key(x[c]);
        if (c < valid && key[c] >= from && key[c] <= upto) mine |= 1u << c;
      }
      // candidates are rare: one vote per group of four tokens, and slots only where somebody has one
      const unsigned int votes = __ballot_sync(0xffffffffu, mine != 0u);
      if (votes == 0u) return;
      const unsigned int n_mine = __popc(mine);
      const unsigned int upto_me = warp_inclusive_scan_u(n_mine, lane);
      unsigned int base = 0u;
      if (lane == 31) base = atomicAdd(&s_count, upto_me);
      unsigned int slot = __shfl_sync(0xffffffffu, base, 31) + upto_me - n_mine;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (mine & (1u << c)) {
          if (slot < (unsigned int)ST) s_cand[slot] = ((unsigned long long)key[c] << 32) | (unsigned int)(4 * j + c);
          ++slot;
        }
    });
    __syncthreads();
    return (int)s_count;
  };
  int kept = V;
  if (select > 0 && select <= ST) {
    // The select-th largest of the threads' own maxima is a value that select tokens reach at least, so it
    // bounds the select-th largest of the row from below, and closely: few other tokens lie above it.
    float* tmax = reinterpret_cast<float*>(s_cand);
    tmax[tid] = my_max;
    __syncthreads();
    block_sort_ascending(tmax, ST);
    bound = ordered_key(tmax[ST - select]);
    kept = gather(bound, 0xffffffffu);
  } else if (select == 0 && V <= ST) {
    kept = gather(0u, 0xffffffffu);
  }
  if (select > 0 && kept > ST) {
    // too many (ties, or a top_k beyond the block): the exact key by radix selection, 12 + 12 + 8 bits
    radix_pass(w, rv, 0u, 32 - HIST_BITS, HIST_BITS, (unsigned int)select, s_hist, s_scan_u, &s_pick, &s_above, &s_same);
    uint32_t prefix = s_pick << (32 - HIST_BITS);
    unsigned int want = (unsigned int)select - s_above;
    __syncthreads();
    radix_pass(w, rv, prefix, 8, 32 - HIST_BITS - 8, want, s_hist, s_scan_u, &s_pick, &s_above, &s_same);
    prefix |= s_pick << 8;
    want -= s_above;
    __syncthreads();
    radix_pass(w, rv, prefix, 0, 8, want, s_hist, s_scan_u, &s_pick, &s_above, &s_same);
    bound = prefix | s_pick;
    kept = gather(bound, 0xffffffffu);
  }

  if (kept <= ST) {
    // ---- few candidates: sorted ascending by (value, token), the padding first; thread j holds entry j
    int n2 = 32;
    while (n2 < kept) n2 <<= 1;
    for (int i = kept + tid; i < n2; i += ST) s_cand[i] = 0ull;
    __syncthreads();
    block_sort_ascending(s_cand, n2);
    const bool have = tid < n2 && tid >= n2 - kept;
    const unsigned long long mine = tid < n2 ? s_cand[tid] : 0ull;
    const float v = have ? key_value((uint32_t)(mine >> 32)) : -INFINITY;
    const int token = (int)(uint32_t)mine;
    // below the select-th largest value a candidate is none after all
    const float floor_v = (select > 0 && !probe) ? key_value((uint32_t)(s_cand[n2 - select] >> 32)) : -INFINITY;
    float e = (have && v >= floor_v) ? expf(v - vmax) : 0.f;
    bool row_wide = false;
    if (p.top_p < 1.0f) {
      float outside = 0.f;  // the mass of the row below the candidates
      if (probe) {
        sweep<4>(w, rv, 0, rv.groups, tid, ST, [&](int j, const float (&x)[4], bool ok) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (ok && 4 * j + c < V && ordered_key(x[c]) < bound) outside += expf(x[c] - vmax);
        });
        outside = block_sum(outside, sc.f);
      }
      // the running sum of the masses in ascending order of the values: a value stays if the sum up to and
      // with the last entry equal to it exceeds (1 - top_p) of the total
      const float run = outside + block_inclusive_scan_f(e, s_scan_f);
      const float total = outside + s_scan_f[64];
      const float limit = (1.0f - p.top_p) * total;
      row_wide = probe && outside > limit;  // the cut may lie below the candidates
      const float next = tid + 1 < n2 ? key_value((uint32_t)(s_cand[tid + 1] >> 32)) : INFINITY;
      const unsigned int crosses = (e > 0.f && next != v && run > limit) ? 1u : 0u;
      const unsigned int crossed_before = block_exclusive_scan_u(crosses, s_scan_u);
      if (crosses && crossed_before == 0) s_cut = v;
      __syncthreads();
      if (v < s_cut) e = 0.f;
    }
    if (!row_wide) {
      if (p.min_p > 0.f && e < p.min_p && v != vmax) e = 0.f;
      // inverse CDF over the sorted candidates
      const float upto = block_inclusive_scan_f(e, s_scan_f);
      const float target = u01 * s_scan_f[64];
      const unsigned int hit = (e > 0.f && upto > target) ? 1u : 0u;
      const unsigned int hits_before = block_exclusive_scan_u(hit, s_scan_u);
      // rounding may leave the target at or past the total: then the last candidate, which is the largest
      if ((hit && hits_before == 0) || (tid == n2 - 1 && !(upto > target))) out[row] = token;
      return;
    }
    __syncthreads();
  }

  // warp w owns the groups [g_lo, g_hi): what runs in the order of the vocabulary goes warp by warp
  const int groups_per_warp = (rv.groups + 31) / 32;
  const int g_lo = min(rv.groups, warp * groups_per_warp), g_hi = min(rv.groups, g_lo + groups_per_warp);

  // ---- many candidates: the row stays as it is; `floor_key` says which of its tokens still have mass
  uint32_t floor_key = probe ? 0u : bound;  // (the probe's candidates were top-p's first look, not a top-k filter)
  if (p.top_p < 1.0f) {
    // The cut is the smallest key c whose lower tail (the mass of the keys <= c) exceeds 1 - top_p of the
    // total; keys below it go. It lies in (lo, hi], which each pass over the row narrows with seven
    // thresholds at once, until the tokens inside fit the block and their sorted list gives the cut.
    float tot = 0.f;
    unsigned int below = 0u;
    sweep<4>(w, rv, 0, rv.groups, tid, ST, [&](int j, const float (&x)[4], bool ok) {
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (ok && 4 * j + c < V) {
          if (ordered_key(x[c]) >= floor_key) tot += expf(x[c] - vmax);
          else ++below;
        }
    });
    tot = block_sum(tot, sc.f);
    below = block_exclusive_scan_u(below, s_scan_u);
    below = s_scan_u[64];
    const float limit = (1.0f - p.top_p) * tot;
    long long lo = (long long)floor_key - 1, hi = (long long)ordered_key(vmax);
    float m_lo = 0.f;                    // the mass of the keys <= lo
    unsigned int c_lo = below, c_hi = V; // the tokens with keys <= lo, <= hi
    // thresholds come from a sorted sample of the row while it has entries inside the interval
    uint32_t* samp = s_hist;
    __syncthreads();
    samp[tid] = ordered_key(w[(long long)tid * V / ST]);
    __syncthreads();
    block_sort_ascending(samp, ST);
    float* fbuf = reinterpret_cast<float*>(s_cand);
    unsigned int* ubuf = reinterpret_cast<unsigned int*>(s_cand) + 256;
    while (c_hi - c_lo > (unsigned int)ST && hi - lo > 1) {
      int a = 0, b = 0;  // sample entries <= lo, sample entries < hi
      for (int half = ST >> 1; half > 0; half >>= 1) {
        if ((long long)samp[a + half - 1] <= lo) a += half;
        if ((long long)samp[b + half - 1] < hi) b += half;
      }
      if (a < ST && (long long)samp[a] <= lo) ++a;
      if (b < ST && (long long)samp[b] < hi) ++b;
      const int inside = b - a;
      uint32_t t[7];
      float m[7];
      unsigned int n[7];
#pragma unroll
      for (int i = 0; i < 7; ++i) {
        const long long even = lo + ((i + 1) * (hi - lo)) / 8;  // without a sample: even steps through the keys
        t[i] = inside >= 7 ? samp[a + ((i + 1) * inside) / 8] : (uint32_t)(even > lo ? even : lo + 1);
        m[i] = 0.f;
        n[i] = 0u;
      }
      sweep<4>(w, rv, 0, rv.groups, tid, ST, [&](int j, const float (&x)[4], bool ok) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (!(ok && 4 * j + c < V)) continue;
          const uint32_t key = ordered_key(x[c]);
          const float e = key >= floor_key ? expf(x[c] - vmax) : 0.f;
#pragma unroll
          for (int i = 0; i < 7; ++i)
            if (key <= t[i]) { m[i] += e; ++n[i]; }
        }
      });
      // sums over the block in a fixed order: the lanes by a tree, the warps one after another
#pragma unroll
      for (int i = 0; i < 7; ++i) {
        m[i] = warp_sum(m[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) n[i] += __shfl_xor_sync(0xffffffffu, n[i], o);
      }
      __syncthreads();
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < 7; ++i) { fbuf[warp * 7 + i] = m[i]; ubuf[warp * 7 + i] = n[i]; }
      }
      __syncthreads();
      if (tid < 7) {
        float fm = 0.f;
        unsigned int un = 0u;
        for (int q = 0; q < 32; ++q) { fm += fbuf[q * 7 + tid]; un += ubuf[q * 7 + tid]; }
        fbuf[224 + tid] = fm;
        ubuf[224 + tid] = un;
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 7; ++i) {
        const float fm = fbuf[224 + i];
        const unsigned int un = ubuf[224 + i];
        if ((long long)t[i] <= lo || (long long)t[i] >= hi) continue;  // an earlier threshold moved the end
        if (fm <= limit) { lo = t[i]; m_lo = fm; c_lo = un; }
        else { hi = t[i]; c_hi = un; }
      }
      __syncthreads();
    }
    uint32_t cut = (uint32_t)hi;
    if (c_hi - c_lo <= (unsigned int)ST) {
      const int inside = gather((uint32_t)(lo + 1), (uint32_t)hi);
      int n2 = 32;
      while (n2 < inside) n2 <<= 1;
      for (int i = inside + tid; i < n2; i += ST) s_cand[i] = 0ull;
      if (tid == 0) s_pick = (uint32_t)hi;
      __syncthreads();
      block_sort_ascending(s_cand, n2);
      const bool have = tid < n2 && tid >= n2 - inside;
      const uint32_t key = have ? (uint32_t)(s_cand[tid] >> 32) : 0u;
      const float e = have ? expf(key_value(key) - vmax) : 0.f;
      const float run = m_lo + block_inclusive_scan_f(e, s_scan_f);
      const uint32_t next = tid + 1 < n2 ? (uint32_t)(s_cand[tid + 1] >> 32) : 0xffffffffu;
      const unsigned int crosses = (have && (next != key || tid + 1 == n2) && run > limit) ? 1u : 0u;
      const unsigned int crossed_before = block_exclusive_scan_u(crosses, s_scan_u);
      if (crosses && crossed_before == 0) s_pick = key;
      __syncthreads();
      cut = s_pick;
    }
    floor_key = max(floor_key, cut);
  }
  // probabilities below min_p times the largest one go: exp(v - vmax) < min_p
  const float min_p = p.min_p;
  const bool unfiltered = floor_key == 0u && !(min_p > 0.f);
  auto mass_of = [&](float x) {
    if (unfiltered) return expf(x - vmax);   // (the same for the whole block)
    if (ordered_key(x) < floor_key) return 0.f;
    const float e = expf(x - vmax);
    return (min_p > 0.f && e < min_p && x != vmax) ? 0.f : e;
  };
  // Inverse CDF. Each warp sums its range, 128 tokens at a time (four tokens in a lane, a scan tree over
  // the lanes, then the running sum); the running sums of the warps say whose range holds the target, and
  // that warp walks its range again with the same additions, so it finds the crossing its total promised.
  {
    float mine = 0.f;
    sweep<4>(w, rv, g_lo, g_hi, lane, 32, [&](int j, const float (&x)[4], bool ok) {
      float s4 = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) s4 += (ok && 4 * j + c < V) ? mass_of(x[c]) : 0.f;
      mine += __shfl_sync(0xffffffffu, warp_inclusive_scan_f(s4, lane), 31);
    });
    __syncthreads();
    if (lane == 0) sc.f[warp] = mine;
    __syncthreads();
    const float t = sc.f[lane];
    const float upto = warp_inclusive_scan_f(t, lane);            // lane l: ranges 0 .. l
    const float target = u01 * __shfl_sync(0xffffffffu, upto, 31);
    const float local = target - (upto - t);                       // lane l: the target inside range l
    const unsigned int hits = __ballot_sync(0xffffffffu, t > 0.f && t > local);
    const unsigned int massy = __ballot_sync(0xffffffffu, t > 0.f);
    // rounding may leave the target at or past the total: then the last range with mass, and its last token
    const int owner = hits ? __ffs(hits) - 1 : (massy ? 31 - __clz(massy) : 0);
    if (warp == owner) {
      const float goal = __shfl_sync(0xffffffffu, local, owner);
      float run = 0.f;
      int pick = -1, last = -1;
      sweep<4>(w, rv, g_lo, g_hi, lane, 32, [&](int j, const float (&x)[4], bool ok) {
        if (pick >= 0) return;  // the same for the whole warp
        float e[4], s4 = 0.f;
        int my_last = -1;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          e[c] = (ok && 4 * j + c < V) ? mass_of(x[c]) : 0.f;
          s4 += e[c];
          if (e[c] > 0.f) my_last = 4 * j + c;
        }
        const float inc = warp_inclusive_scan_f(s4, lane);
        const unsigned int live = __ballot_sync(0xffffffffu, s4 > 0.f);
        const unsigned int over = __ballot_sync(0xffffffffu, s4 > 0.f && run + inc > goal);
        if (over) {
          // inside the first lane whose running sum passes the goal: its tokens one by one
          const int l = __ffs(over) - 1;
          int mine_pick = my_last;
          float r = run + (inc - s4);
#pragma unroll
          for (int c = 3; c >= 0; --c) {
            // the first token with mass whose running sum passes the goal (found from the back)
            float upto_c = r;
#pragma unroll
            for (int d = 0; d <= c; ++d) upto_c += e[d];
            if (e[c] > 0.f && upto_c > goal) mine_pick = 4 * j + c;
          }
          pick = __shfl_sync(0xffffffffu, mine_pick, l);
        }
        if (live) last = __shfl_sync(0xffffffffu, my_last, 31 - __clz(live));
        run += __shfl_sync(0xffffffffu, inc, 31);
      });
      if (lane == 0) out[row] = pick >= 0 ? pick : (last >= 0 ? last : 0);
    }
  }
}

}  // namespace

PTB_API int ptb_sample(const float* logits, float* work, int* out, int rows, int vocab, int do_sample,
                       float temperature, int top_k, float top_p, float min_p, float repetition_penalty,
                       const int* history, const int* history_len, int history_stride, const int* suppress,
                       int n_suppress, unsigned long long seed, const long long* streams, const long long* counters,
                       cudaStream_t stream) {
  if (rows <= 0) return PTB_OK;
  if (vocab <= 0) return PTB_ERR_SIZE;
  if (do_sample && !(temperature > 0.f)) return PTB_ERR_SIZE;
  if (do_sample && (!(top_p > 0.f) || top_p > 1.f || min_p < 0.f || min_p > 1.f || top_k < 0)) return PTB_ERR_SIZE;
  if (!(repetition_penalty > 0.f)) return PTB_ERR_SIZE;
  SampleParams p;
  p.vocab = vocab;
  p.do_sample = do_sample;
  p.temperature = temperature;
  p.top_k = top_k;
  p.top_p = top_p;
  p.min_p = min_p;
  p.repetition_penalty = repetition_penalty;
  p.history_stride = history_stride;
  p.n_suppress = n_suppress;
  p.seed = seed;
  sample_kernel<<<rows, ST, 0, stream>>>(logits, work, out, history, history_len, suppress, streams, counters, p);
  return launch_status();
}
