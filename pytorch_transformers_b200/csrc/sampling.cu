// Next-token selection on the device: one block per row of float32 logits.
//   processors, in the reference's order: repetition penalty, suppression of stop tokens (while a
//   minimum of new tokens is not reached), then for sampling: temperature, top-k, top-p, min-p;
//   selection: argmax (greedy) or a draw from softmax by inverse CDF with a counter-based uniform.
// `work` is scratch of the same shape as the logits; the logits themselves are left untouched.
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

__device__ __forceinline__ unsigned int block_sum_u(unsigned int v, unsigned int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  unsigned int r = (lane < nwarp) ? scratch[lane] : 0u;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
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

__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, float* __restrict__ work, int* __restrict__ out,
              const int* __restrict__ history, const int* __restrict__ history_len,
              const int* __restrict__ suppress, const long long* __restrict__ streams,
              const long long* __restrict__ counters, SampleParams p) {
  __shared__ BlockScratch sc;
  __shared__ float s_thread_sum[ST];
  __shared__ int s_pick;
  const int row = blockIdx.x, tid = threadIdx.x, V = p.vocab;
  const float* lg = logits + size_t(row) * V;
  float* w = work + size_t(row) * V;   // scratch copy of the row that the processors may change

  const bool untouched = !p.do_sample && !(p.repetition_penalty != 1.0f && history) && p.n_suppress <= 0;
  if (untouched) {
    // plain greedy: nothing changes a logit, so the maximum is taken from the logits themselves
    w = const_cast<float*>(lg);
  } else {
    for (int i = tid; i < V; i += ST) w[i] = lg[i];
    __syncthreads();
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
    for (int i = tid; i < V; i += ST) {
      const float v = w[i];
      if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((tid & 31) == 0) { sc.f[tid >> 5] = best; sc.i[tid >> 5] = best_i; }
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
  for (int i = tid; i < V; i += ST) w[i] = w[i] * inv_t;
  __syncthreads();

  if (p.top_k > 0 && p.top_k < V) {
    // largest key c with count(key >= c) >= k: the k-th largest value; ties with it are kept
    uint32_t lo = 0u, hi = 0xffffffffu;
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1) + 1u;  // upper middle, lo < mid <= hi
      unsigned int cnt = 0;
      for (int i = tid; i < V; i += ST) cnt += (ordered_key(w[i]) >= mid) ? 1u : 0u;
      cnt = block_sum_u(cnt, sc.u);
      if (cnt >= (unsigned int)p.top_k) lo = mid; else hi = mid - 1u;
    }
    for (int i = tid; i < V; i += ST)
      if (ordered_key(w[i]) < lo) w[i] = -INFINITY;
    __syncthreads();
  }

  float vmax = -INFINITY;
  for (int i = tid; i < V; i += ST) vmax = fmaxf(vmax, w[i]);
  vmax = block_max(vmax, sc.f);

  if (p.top_p < 1.0f) {
    float tot = 0.f;
    for (int i = tid; i < V; i += ST) tot += expf(w[i] - vmax);
    tot = block_sum(tot, sc.f);
    // smallest key c whose lower tail mass (keys <= c) exceeds 1 - top_p: values below it go
    const float limit = (1.0f - p.top_p) * tot;
    uint32_t lo = 0u, hi = ordered_key(vmax);
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1);
      float mass = 0.f;
      for (int i = tid; i < V; i += ST)
        if (ordered_key(w[i]) <= mid) mass += expf(w[i] - vmax);
      mass = block_sum(mass, sc.f);
      if (mass > limit) hi = mid; else lo = mid + 1u;
    }
    for (int i = tid; i < V; i += ST)
      if (ordered_key(w[i]) < lo) w[i] = -INFINITY;
    __syncthreads();
  }

  if (p.min_p > 0.f) {
    // probabilities below min_p times the largest one go: exp(v - vmax) < min_p
    for (int i = tid; i < V; i += ST)
      if (expf(w[i] - vmax) < p.min_p && w[i] != vmax) w[i] = -INFINITY;
    __syncthreads();
  }

  // inverse CDF over contiguous chunks: thread t owns [t * chunk, (t + 1) * chunk)
  const int chunk = (V + ST - 1) / ST;
  const int lo_i = tid * chunk, hi_i = min(V, lo_i + chunk);
  float mine = 0.f;
  for (int i = lo_i; i < hi_i; ++i) mine += expf(w[i] - vmax);
  s_thread_sum[tid] = mine;
  if (tid == 0) s_pick = -1;
  __syncthreads();
  if (tid == 0) {
    float total = 0.f;
    for (int t = 0; t < ST; ++t) total += s_thread_sum[t];
    const float u = uniform01(p.seed, (uint64_t)streams[row], (uint64_t)counters[row]);
    const float target = u * total;
    float run = 0.f;
    int owner = ST - 1;
    for (int t = 0; t < ST; ++t) {
      if (run + s_thread_sum[t] > target) { owner = t; break; }
      run += s_thread_sum[t];
    }
    // walk the owner's chunk; fall back to the last token with non-zero mass
    int pick = -1;
    const int a = owner * chunk, b = min(V, a + chunk);
    for (int i = a; i < b; ++i) {
      const float e = expf(w[i] - vmax);
      if (e > 0.f) {
        pick = i;
        if (run + e > target) break;
        run += e;
      }
    }
    if (pick < 0) {
      for (int i = V - 1; i >= 0; --i)
        if (w[i] == vmax) { pick = i; break; }
    }
    s_pick = pick < 0 ? 0 : pick;
    out[row] = s_pick;
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
