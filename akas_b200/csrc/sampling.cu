// Sampling from float32 logits [M, V]: greedy, and temperature with optional top-k and top-p.
//
// argmax: ties go to the lowest index (kreasof-ai/akas, src/akas/ops/vocabulary/kernel.py:146-150).
//
// sample, per row with temperature T, top_k k, top_p p and a uniform u in [0, 1) from the caller:
//   T <= 0: the argmax. Else w_i = exp((x_i - max x) / T); the tokens are ranked by logit, larger first, equal
//   logits by id, lower first; token i is kept iff
//     its rank is below k (k <= 0 or k >= V: no limit; exactly k are kept, whatever is equal), and
//     the kept tokens ranked before it hold at most p of the kept mass (p >= 1: no limit);
//   the result is the first kept i, in index order, whose running kept mass exceeds u * (kept mass).
// The reference's only stochastic sampler (its audio model's `codebook_sample`,
// src/akas/ops/vocabulary/kernel.py:515-671) has the same stages: top-k, exp((v - peak) / T), a
// top-p cut on the mass before a token, inverse CDF with a supplied uniform, T <= 0 greedy. Here
// no sort is needed: both cuts are a threshold on the logit, found by bisection over the ordered
// bit patterns of float32 with one counting or summing pass over the row per step, and, for the tokens
// equal to the threshold, a largest id that is kept, found by a prefix count in index order.
// One block of 1024 threads per row. Softmax terms and sums are float32.
//
// adjust: the two stages that sampler applies before those, on the logits in place, per row:
//   softcap c > 0:  x = c * tanh(x / c)                                   (kernel.py:559)
//   penalty q != 1: a token found among the row's recent tokens (a window of the request's last generated
//                   tokens, -1 where there are fewer) becomes x / q if x > 0, else x * q, once however often it
//                   was generated                                          (kernel.py:560-575)
#include <math.h>

#include "common.cuh"

using namespace akas;

#define AKAS_SAMPLE_THREADS 1024

__device__ __forceinline__ uint32_t ordered_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}

__device__ __forceinline__ float key_value(uint32_t key) {  // the float whose ordered key this is
  return __uint_as_float(key ^ ((key >> 31) ? 0x80000000u : 0xffffffffu));
}

// (value, index) of the row maximum with the lowest index among equals; every thread gets it.
__device__ void block_argmax(const float* __restrict__ x, int V, float& best_out, int& idx_out) {
  __shared__ float vals[32];
  __shared__ int idxs[32];
  float best = -INFINITY;
  int idx = V;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = x[i];
    if (v > best || idx == V) { best = v; idx = i; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  if (lane == 0) { vals[warp] = best; idxs[warp] = idx; }
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  best = lane < warps ? vals[lane] : -INFINITY;
  idx = lane < warps ? idxs[lane] : V;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  best_out = best;
  idx_out = idx;
  __syncthreads();
}

// Greedy token in two launches, so that a handful of rows still keeps many SMs busy: the vocabulary is cut
// into `parts` slices, one block each; then one block per row picks the best of the slices' winners (the
// larger value, and among equals the lower index, so ties go to the lowest id as in one pass).
__global__ void __launch_bounds__(256)
argmax_parts_kernel(const float* __restrict__ logits, float* __restrict__ part_val, int* __restrict__ part_idx, int V,
                    int parts) {
  chain_release();
  chain_wait();
  const int row = blockIdx.x, part = blockIdx.y;
  const int per = (V + parts - 1) / parts;
  const int begin = min(V, part * per), count = min(V, begin + per) - begin;
  float best = -INFINITY;
  int idx = V;
  if (count > 0) {
    block_argmax(logits + (size_t)row * V + begin, count, best, idx);
    idx += begin;
  }
  if (threadIdx.x == 0) {
    part_val[row * parts + part] = count > 0 ? best : -INFINITY;
    part_idx[row * parts + part] = count > 0 ? idx : V;
  }
}

__global__ void argmax_pick_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                   int* __restrict__ out, int parts) {
  chain_release();
  chain_wait();
  const int row = blockIdx.x;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int p = threadIdx.x; p < parts; p += 32) {
    const float v = part_val[row * parts + p];
    const int i = part_idx[row * parts + p];
    if (v > best || (v == best && i < idx) || idx == 0x7fffffff) { best = v; idx = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  if (threadIdx.x == 0) out[row] = idx;
}

// Scratch: part_val float32 [M, parts], part_idx int32 [M, parts].
AKAS_API int akas_argmax(const float* logits, int* out, float* part_val, int* part_idx, int M, int V, int parts,
                         cudaStream_t stream) {
  if (M <= 0) return 0;
  if (parts < 1 || parts > 1024 || V <= 0) return (int)cudaErrorInvalidValue;
  int err = launch_chained(argmax_parts_kernel, dim3(M, parts), dim3(256), 0, stream, logits, part_val, part_idx, V, parts);
  if (err) return err;
  return launch_chained(argmax_pick_kernel, dim3(M), dim3(32), 0, stream, (const float*)part_val, (const int*)part_idx,
                        out, parts);
}

// The index of the `want`-th (1-based) position i, in index order, whose key equals `tie` and for which i <= limit;
// V - 1 if there are fewer (keep them all). Thread t owns the contiguous indices [t * chunk, (t + 1) * chunk).
// `counts` holds one int per warp; every thread gets the result.
__device__ int tie_cut(const float* __restrict__ x, int V, uint32_t tie, int limit, int want, int* counts, int* found) {
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int begin = min(V, (int)threadIdx.x * chunk), end = min(V, begin + chunk);
  int local = 0;
  for (int i = begin; i < end; ++i) local += (ordered_key(x[i]) == tie && i <= limit) ? 1 : 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  __syncthreads();  // counts and found may still be read from an earlier call
  if (threadIdx.x == 0) *found = V - 1;
  if (lane == 31) counts[warp] = incl;
  __syncthreads();
  int before = 0;
  for (int w = 0; w < warp; ++w) before += counts[w];
  int run = before + incl - local;
  if (run < want && run + local >= want) {  // the wanted one lies in this thread's chunk
    for (int i = begin; i < end; ++i)
      if (ordered_key(x[i]) == tie && i <= limit && ++run == want) { *found = i; break; }
  }
  __syncthreads();
  return *found;
}

// The order of the tokens is (logit descending, id ascending), the order in which the reference's rank loop takes
// them (src/akas/ops/vocabulary/kernel.py:586-622). top-k keeps the first k of that order exactly; top-p keeps a
// token while the kept mass before it, in that order, is at most p of the kept mass. Both cuts are a threshold on
// the logit plus, among the tokens equal to the threshold, an upper bound on the id.
__global__ void __launch_bounds__(AKAS_SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out, int V) {
  __shared__ float scratch[32];
  __shared__ float warp_tot[32];
  __shared__ int counts[32];
  __shared__ int found;
  __shared__ int pick, last_kept;
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * V;
  float top;
  int top_idx;
  block_argmax(x, V, top, top_idx);
  const float T = temperature[row];
  if (!(T > 0.f)) {
    if (threadIdx.x == 0) out[row] = top_idx;
    return;
  }
  const float inv_t = 1.f / T;
  uint32_t thr = 0u;  // keep tokens whose ordered key is > thr, and those == thr whose id is <= cut
  int cut = V - 1;

  const int k = top_k[row];
  if (k > 0 && k < V) {
    uint32_t lo = 0u, hi = 0xffffffffu;  // smallest t with count(key > t) < k: the key of the k-th largest logit
    while (lo < hi) {
      const uint32_t mid = lo + (hi - lo) / 2u;
      float c = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) c += ordered_key(x[i]) > mid ? 1.f : 0.f;
      c = block_sum(c, scratch);  // exact: counts stay far below 2^24
      if (c < (float)k) hi = mid; else lo = mid + 1u;
    }
    thr = lo;
    float above = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) above += ordered_key(x[i]) > thr ? 1.f : 0.f;
    above = block_sum(above, scratch);
    cut = tie_cut(x, V, thr, V - 1, k - (int)above, counts, &found);  // of the equals, the lowest ids fill up to k
  }

  const float p = top_p[row];
  if (p < 1.f) {
    float mass = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const uint32_t key = ordered_key(x[i]);
      if (key > thr || (key == thr && i <= cut)) mass += expf((x[i] - top) * inv_t);
    }
    mass = block_sum(mass, scratch);
    const float limit = p * mass;
    uint32_t lo = thr, hi = 0xffffffffu;  // smallest t >= thr with mass(key > t) <= limit
    while (lo < hi) {
      const uint32_t mid = lo + (hi - lo) / 2u;
      float g = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x)
        if (ordered_key(x[i]) > mid) g += expf((x[i] - top) * inv_t);
      g = block_sum(g, scratch);
      if (g <= limit) hi = mid; else lo = mid + 1u;
    }
    // Of the tokens equal to the new threshold, the j-th (from 0, by id) has above + j * w before it.
    float above = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (ordered_key(x[i]) > lo) above += expf((x[i] - top) * inv_t);
    above = block_sum(above, scratch);
    const float tie_w = expf((key_value(lo) - top) * inv_t);  // the weight of every token at the threshold
    int keep = 1;
    while (keep < V && tie_w > 0.f && above + (float)keep * tie_w <= limit) ++keep;  // few: equals of one value
    const int bound = lo == thr ? cut : V - 1;
    thr = lo;
    cut = tie_cut(x, V, thr, bound, keep, counts, &found);
  }

  // inverse CDF in index order: thread t owns the contiguous indices [t * chunk, (t + 1) * chunk)
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int begin = min(V, (int)threadIdx.x * chunk), end = min(V, begin + chunk);
  float local = 0.f;
  int my_last = -1;
  for (int i = begin; i < end; ++i) {
    const uint32_t key = ordered_key(x[i]);
    if (key > thr || (key == thr && i <= cut)) { local += expf((x[i] - top) * inv_t); my_last = i; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (threadIdx.x == 0) { pick = V; last_kept = -1; }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  float before = 0.f, total = 0.f;  // mass of the warps before mine, and of the whole row
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
    if (w < warp) before += warp_tot[w];
    total += warp_tot[w];
  }
  const float target = uniform[row] * total;
  float run = before + incl - local;
  for (int i = begin; i < end; ++i) {
    const uint32_t key = ordered_key(x[i]);
    if (key > thr || (key == thr && i <= cut)) {
      run += expf((x[i] - top) * inv_t);
      if (run > target) { atomicMin(&pick, i); break; }
    }
  }
  if (my_last >= 0) atomicMax(&last_kept, my_last);
  __syncthreads();
  if (threadIdx.x == 0) out[row] = pick < V ? pick : last_kept;
}

// One block per (slice of 4,096 logits, row): the softcap over the slice, then one thread per entry of the history
// whose token lies in the slice and did not occur earlier in the history applies the penalty.
__global__ void adjust_logits_kernel(float* __restrict__ logits, const float* __restrict__ softcap,
                                     const float* __restrict__ penalty, const int* __restrict__ history, int W, int V) {
  const int row = blockIdx.y, v0 = blockIdx.x * 4096, v1 = min(V, v0 + 4096);
  float* x = logits + (size_t)row * V;
  const float cap = softcap[row], q = penalty[row];
  if (cap > 0.f)
    for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) x[i] = cap * tanhf(x[i] / cap);
  if (q == 1.f) return;
  __syncthreads();
  const int* seen = history + (size_t)row * W;
  for (int w = threadIdx.x; w < W; w += blockDim.x) {
    const int token = seen[w];
    if (token < v0 || token >= v1) continue;
    bool first = true;
    for (int e = 0; e < w; ++e) first = first && seen[e] != token;
    if (first) x[token] = x[token] > 0.f ? x[token] / q : x[token] * q;
  }
}

// logits: float32 [M, V], changed in place; softcap, penalty: float32 [M]; history: int32 [M, W], -1 where empty.
AKAS_API int akas_adjust_logits(float* logits, const float* softcap, const float* penalty, const int* history, int W,
                                int M, int V, cudaStream_t stream) {
  if (M <= 0 || V <= 0) return 0;
  if (W < 0 || M > 65535) return (int)cudaErrorInvalidValue;
  adjust_logits_kernel<<<dim3((V + 4095) / 4096, M), 256, 0, stream>>>(logits, softcap, penalty, history, W, V);
  return launch_status();
}

AKAS_API int akas_sample(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                         const float* uniform, int* out, int M, int V, cudaStream_t stream) {
  if (M <= 0) return 0;
  sample_kernel<<<M, AKAS_SAMPLE_THREADS, 0, stream>>>(logits, temperature, top_k, top_p, uniform, out, V);
  return launch_status();
}
