// Rotary tables, and the fused per-head RMSNorm + rotation + write of keys and values into pages.
//
// Angles: theta = position * inv_freq[i] with inv_freq in float64 (made on the host), multiplied,
// reduced and evaluated in float64 and rounded to float32 last, so that long positions lose nothing.
// One table per step serves every layer that shares the encoding.
//
// qk_norm_rope_store works on the output of the stacked q/k/v product, [N, (heads + 2 kv_heads) * d]:
// one warp per (token, head). q heads: norm, rotate, write to q_out. k heads: norm, rotate, write
// back in place and into the key page of the token's (request, position). v heads: copy into the
// value page. Rotation pairs channel i with i + rotary/2; channels from `rotary` on pass through.
#include "common.cuh"
#include "qk_prep.cuh"

using namespace akas;

__global__ void rope_tables_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                   float* __restrict__ cos_out, float* __restrict__ sin_out, int N, int half) {
  chain_release();
  chain_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)N * half) return;
  const int n = (int)(i / half), f = (int)(i % half);
  // The angle is formed and reduced to [-pi, pi] in float64 (a product, a rounding and two fused multiply-adds with
  // 2 pi split in two), so that a position of a million still leaves it exact to 1e-10. The reduced angle goes to
  // float32 as a sum hi + lo; sine and cosine of hi are float32's own and lo enters by the first-order terms
  // sin(hi + lo) = sin hi + lo cos hi, cos(hi + lo) = cos hi - lo sin hi: accurate to an ulp of the table's type
  // at a fraction of the cost of a float64 sincos.
  const double angle = (double)positions[n] * inv_freq[f];
  const double turns = rint(angle * 0.15915494309189535);
  const double reduced = fma(-turns, 2.4492935982947064e-16, fma(-turns, 6.283185307179586, angle));
  const float hi = (float)reduced, lo = (float)(reduced - (double)hi);
  float s, c;
  sincosf(hi, &s, &c);
  cos_out[i] = fmaf(-lo, s, c);
  sin_out[i] = fmaf(lo, c, s);
}

AKAS_API int akas_rope_tables(const int* positions, const double* inv_freq, float* cos_out, float* sin_out, int N,
                              int half, cudaStream_t stream) {
  const size_t total = (size_t)N * half;
  if (total == 0) return 0;
  return launch_chained(rope_tables_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, positions,
                        inv_freq, cos_out, sin_out, N, half);
}

#define AKAS_ROPE_WARPS 4

template <typename T>
__global__ void qk_norm_rope_store_kernel(T* __restrict__ qkv, T* __restrict__ q_out,
                                          const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                          int zero_centered, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, int rotary, T* __restrict__ k_pool,
                                          T* __restrict__ v_pool, const int* __restrict__ block_table,
                                          int max_blocks, const int* __restrict__ seq_of_token,
                                          const int* __restrict__ positions, int page_size, int H, int KH, int D) {
  __shared__ float buf[AKAS_ROPE_WARPS][256];
  chain_release();
  chain_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head = blockIdx.y * AKAS_ROPE_WARPS + warp;
  if (head >= H + 2 * KH) return;
  const int width = (H + 2 * KH) * D;
  T* src = qkv + (size_t)t * width + (size_t)head * D;
  const int r = seq_of_token[t];
  const bool is_q = head < H, is_k = !is_q && head < H + KH;

  // where this token's key/value row lives, if it is to be stored
  T* page_row = nullptr;
  if (!is_q && k_pool != nullptr && r >= 0) {
    const int pos = positions[t];
    const int page = block_table[(size_t)r * max_blocks + pos / page_size];
    if (page >= 0) {
      const int kvh = is_k ? head - H : head - H - KH;
      T* pool = is_k ? k_pool : v_pool;
      page_row = pool + (((size_t)page * KH + kvh) * page_size + pos % page_size) * D;
    }
  }
  if (!is_q && !is_k) {  // value head: copy
    if (page_row)
      for (int e = lane; e < D; e += 32) page_row[e] = src[e];
    return;
  }

  float* x = buf[warp];
  const float* w = is_q ? q_w : k_w;
  float ss = 0.f;
  for (int e = lane; e < D; e += 32) {
    const float v = to_f32(src[e]);
    x[e] = v;
    ss = fmaf(v, v, ss);
  }
  if (w != nullptr) {
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)D + eps);
    for (int e = lane; e < D; e += 32) x[e] = x[e] * inv * (zero_centered ? 1.f + w[e] : w[e]);
  }
  __syncwarp();
  T* dst = is_q ? q_out + (size_t)t * H * D + (size_t)head * D : src;
  const int half = rotary / 2;
  for (int e = lane; e < D; e += 32) {
    float v = x[e];
    if (cos_t != nullptr && e < rotary) {
      const int f = e < half ? e : e - half;
      const float c = cos_t[(size_t)t * half + f], s = sin_t[(size_t)t * half + f];
      v = e < half ? x[e] * c - x[e + half] * s : x[e - half] * s + x[e] * c;
    }
    const T o = from_f32<T>(v);
    dst[e] = o;
    if (page_row) page_row[e] = o;
  }
}

// The same for head sizes 32, 64, 128 and 256 (and a rotary width that is a multiple of 16): a thread owns 8
// neighbouring channels, TPH = head_dim / 8 threads own a head, a warp 32 / TPH heads. Loads and stores are
// 16 bytes (32 for float32); the sum of squares and the rotation partner travel by shuffle.
template <typename T, int TPH>
__global__ void __launch_bounds__(128)
qk_norm_rope_store8_kernel(T* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ q_w,
                           const float* __restrict__ k_w, float eps, int zero_centered,
                           const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rotary,
                           T* __restrict__ k_pool, T* __restrict__ v_pool, const int* __restrict__ block_table,
                           int max_blocks, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                           int page_size, int H, int KH) {
  constexpr int D = TPH * 8, HEADS_PER_BLOCK = 128 / TPH;
  chain_release();
  chain_wait();
  const int t = blockIdx.x;
  const int head = blockIdx.y * HEADS_PER_BLOCK + threadIdx.x / TPH;
  const int j = threadIdx.x % TPH, e0 = j * 8;
  const int total = H + 2 * KH;
  const bool live = head < total;
  const int hd = live ? head : total - 1;  // threads past the last head shadow it (shuffles need every lane)
  const bool is_q = hd < H, is_k = !is_q && hd < H + KH;
  T* src = qkv + (size_t)t * total * D + (size_t)hd * D + e0;
  const int r = seq_of_token[t];

  T* page_row = nullptr;
  if (live && !is_q && k_pool != nullptr && r >= 0) {
    const int pos = positions[t];
    const int page = block_table[(size_t)r * max_blocks + pos / page_size];
    if (page >= 0) {
      const int kvh = is_k ? hd - H : hd - H - KH;
      page_row = (is_k ? k_pool : v_pool) + (((size_t)page * KH + kvh) * page_size + pos % page_size) * D + e0;
    }
  }
  float x[8];
  load8(src, x);
  if (!is_q && !is_k) {  // value head: copy into the page (every lane still takes part in the shuffles below)
    if (page_row) store8(page_row, x);
  }
  const int half = rotary / 2;
  head_norm_rotate8<TPH>(x, e0, is_q ? q_w : k_w, eps, zero_centered, cos_t ? cos_t + (size_t)t * half : nullptr,
                         cos_t ? sin_t + (size_t)t * half : nullptr, rotary);
  if (!live || (!is_q && !is_k)) return;
  if (is_q) {
    store8(q_out + (size_t)t * H * D + (size_t)hd * D + e0, x);
  } else {
    store8(src, x);
    if (page_row) store8(page_row, x);
  }
}

AKAS_API int akas_qk_norm_rope_store(void* qkv, void* q_out, const float* q_w, const float* k_w, float eps,
                                     int zero_centered, const float* cos_t, const float* sin_t, int rotary,
                                     void* k_pool, void* v_pool, const int* block_table, int max_blocks,
                                     const int* seq_of_token, const int* positions, int page_size, int N, int H,
                                     int KH, int D, int dtype, cudaStream_t stream) {
  if (D > 256 || D <= 0 || rotary > D || (rotary & 1)) return (int)cudaErrorInvalidValue;
  if (N <= 0) return 0;
  const bool wide = (D == 32 || D == 64 || D == 128 || D == 256) && rotary % 16 == 0 && (uintptr_t)qkv % 16 == 0 &&
                    (uintptr_t)q_out % 16 == 0 && (k_pool == nullptr || ((uintptr_t)k_pool % 16 == 0 && (uintptr_t)v_pool % 16 == 0)) &&
                    (cos_t == nullptr || ((uintptr_t)cos_t % 16 == 0 && (rotary / 2) % 8 == 0));
  if (wide) {
    const int tph = D / 8, per_block = 128 / tph;
    const dim3 grid8(N, (H + 2 * KH + per_block - 1) / per_block);
#define AKAS_QK8(T, TPH)                                                                                            \
  return launch_chained(qk_norm_rope_store8_kernel<T, TPH>, grid8, dim3(128), 0, stream, (T*)qkv, (T*)q_out, q_w, k_w, \
                        eps, zero_centered, cos_t, sin_t, rotary, (T*)k_pool, (T*)v_pool, block_table, max_blocks,      \
                        seq_of_token, positions, page_size, H, KH)
    if (dtype == AKAS_F32) {
      if (tph == 4) AKAS_QK8(float, 4);
      if (tph == 8) AKAS_QK8(float, 8);
      if (tph == 16) AKAS_QK8(float, 16);
      AKAS_QK8(float, 32);
    }
    if (tph == 4) AKAS_QK8(bf16, 4);
    if (tph == 8) AKAS_QK8(bf16, 8);
    if (tph == 16) AKAS_QK8(bf16, 16);
    AKAS_QK8(bf16, 32);
#undef AKAS_QK8
  }
  const dim3 grid(N, (H + 2 * KH + AKAS_ROPE_WARPS - 1) / AKAS_ROPE_WARPS);
  const int threads = 32 * AKAS_ROPE_WARPS;
  if (dtype == AKAS_F32)
    return launch_chained(qk_norm_rope_store_kernel<float>, grid, dim3(threads), 0, stream, (float*)qkv, (float*)q_out,
                          q_w, k_w, eps, zero_centered, cos_t, sin_t, rotary, (float*)k_pool, (float*)v_pool,
                          block_table, max_blocks, seq_of_token, positions, page_size, H, KH, D);
  return launch_chained(qk_norm_rope_store_kernel<bf16>, grid, dim3(threads), 0, stream, (bf16*)qkv, (bf16*)q_out, q_w,
                        k_w, eps, zero_centered, cos_t, sin_t, rotary, (bf16*)k_pool, (bf16*)v_pool, block_table,
                        max_blocks, seq_of_token, positions, page_size, H, KH, D);
}

// k, v: [N, KH * D] rows (row strides `stride` and `v_stride` elements) into the pages; for position encodings that
// rewrite k outside the fused kernel.
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ k, const T* __restrict__ v, size_t stride, size_t v_stride,
                                T* __restrict__ k_pool, T* __restrict__ v_pool, const int* __restrict__ block_table,
                                int max_blocks, const int* __restrict__ seq_of_token,
                                const int* __restrict__ positions, int page_size, int KH, int D) {
  const int t = blockIdx.x, kvh = blockIdx.y;
  const int r = seq_of_token[t];
  if (r < 0) return;
  const int pos = positions[t];
  const int page = block_table[(size_t)r * max_blocks + pos / page_size];
  if (page < 0) return;
  const size_t row = (((size_t)page * KH + kvh) * page_size + pos % page_size) * D;
  for (int e = threadIdx.x; e < D; e += blockDim.x) {
    k_pool[row + e] = k[(size_t)t * stride + kvh * D + e];
    v_pool[row + e] = v[(size_t)t * v_stride + kvh * D + e];
  }
}

AKAS_API int akas_kv_store(const void* k, const void* v, long long stride, long long v_stride, void* k_pool, void* v_pool,
                           const int* block_table, int max_blocks, const int* seq_of_token, const int* positions,
                           int page_size, int N, int KH, int D, int dtype, cudaStream_t stream) {
  if (N <= 0) return 0;
  const dim3 grid(N, KH);
  if (dtype == AKAS_F32)
    kv_store_kernel<float><<<grid, 64, 0, stream>>>((const float*)k, (const float*)v, (size_t)stride, (size_t)v_stride, (float*)k_pool,
                                                    (float*)v_pool, block_table, max_blocks, seq_of_token, positions,
                                                    page_size, KH, D);
  else
    kv_store_kernel<bf16><<<grid, 64, 0, stream>>>((const bf16*)k, (const bf16*)v, (size_t)stride, (size_t)v_stride, (bf16*)k_pool,
                                                   (bf16*)v_pool, block_table, max_blocks, seq_of_token, positions,
                                                   page_size, KH, D);
  return launch_status();
}
