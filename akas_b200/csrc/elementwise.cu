// Embedding gather, RMSNorm (optionally of gathered rows), SwiGLU and the reset of state rows.
//
// The residual stream is float32 in both precisions: the embedding writes float32, RMSNorm reads
// it and writes the compute dtype that the next matrix product takes. All sums are float32.
#include "common.cuh"

using namespace akas;

// out[n, :] = float(table[token[n], :])
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                 float* __restrict__ out, int C) {
  chain_release();
  chain_wait();
  const int n = blockIdx.x;
  const T* row = table + (size_t)tokens[n] * C;
  float* dst = out + (size_t)n * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) dst[c] = to_f32(row[c]);
}

AKAS_API int akas_embedding(const int* tokens, const void* table, float* out, int N, int C, int dtype,
                            cudaStream_t stream) {
  if (N <= 0) return 0;
  const int threads = C >= 1024 ? 256 : 128;
  if (dtype == AKAS_F32)
    return launch_chained(embedding_kernel<float>, dim3(N), dim3(threads), 0, stream, tokens, (const float*)table, out, C);
  return launch_chained(embedding_kernel<bf16>, dim3(N), dim3(threads), 0, stream, tokens, (const bf16*)table, out, C);
}

// y[i, :] = x[row(i), :] * rsqrt(mean(x^2) + eps) * (w or 1 + w); row(i) = rows[i] if rows else i.
// One block per row; the row is read twice (the second read hits L1/L2).
template <typename TI, typename TO>
__global__ void rmsnorm_kernel(const TI* __restrict__ x, const float* __restrict__ w, TO* __restrict__ y,
                               const int* __restrict__ rows, int C, float eps, int zero_centered) {
  chain_release();  // a kernel after this one that was launched as its programmatic dependent may set itself up meanwhile
  __shared__ float scratch[32];
  const int i = blockIdx.x;
  const TI* src = x + (size_t)(rows ? rows[i] : i) * C;
  float ss = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = to_f32(src[c]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)C + eps);
  TO* dst = y + (size_t)i * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float g = zero_centered ? 1.f + w[c] : w[c];
    dst[c] = from_f32<TO>(to_f32(src[c]) * inv * g);
  }
}

// The same for float32 rows whose width is a multiple of 8 and at most 8192: the row is read once, with
// 16-byte loads, and stays in registers between the sum of squares and the scaling.
template <typename TO, int PER_THREAD>  // PER_THREAD groups of 8 elements per thread, 256 threads
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ y,
                    const int* __restrict__ rows, int C, float eps, int zero_centered) {
  chain_release();  // a kernel after this one that was launched as its programmatic dependent may set itself up meanwhile
  __shared__ float scratch[32];
  const int i = blockIdx.x;
  // the weights and (what the host wrote for this step) the row's number do not wait for the kernel ahead
  const size_t row = rows ? rows[i] : i;
  float v[PER_THREAD][8], g[PER_THREAD][8];
#pragma unroll
  for (int p = 0; p < PER_THREAD; ++p) {
    const int c = (p * 256 + threadIdx.x) * 8;
    if (c < C) {
      const float4 wa = *reinterpret_cast<const float4*>(w + c);
      const float4 wb = *reinterpret_cast<const float4*>(w + c + 4);
      g[p][0] = wa.x; g[p][1] = wa.y; g[p][2] = wa.z; g[p][3] = wa.w;
      g[p][4] = wb.x; g[p][5] = wb.y; g[p][6] = wb.z; g[p][7] = wb.w;
    }
  }
  chain_wait();
  const float* src = x + row * C;
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < PER_THREAD; ++p) {
    const int c = (p * 256 + threadIdx.x) * 8;
    if (c < C) {
      const float4 a = *reinterpret_cast<const float4*>(src + c);
      const float4 b = *reinterpret_cast<const float4*>(src + c + 4);
      v[p][0] = a.x; v[p][1] = a.y; v[p][2] = a.z; v[p][3] = a.w;
      v[p][4] = b.x; v[p][5] = b.y; v[p][6] = b.z; v[p][7] = b.w;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(v[p][e], v[p][e], ss);
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)C + eps);
  TO* dst = y + (size_t)i * C;
#pragma unroll
  for (int p = 0; p < PER_THREAD; ++p) {
    const int c = (p * 256 + threadIdx.x) * 8;
    if (c < C) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v[p][e] * inv * (zero_centered ? 1.f + g[p][e] : g[p][e]);
      store8(dst + c, o);
    }
  }
}

AKAS_API int akas_rmsnorm(const void* x, const float* w, void* y, const int* rows, int M, int C, float eps,
                          int zero_centered, int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (in_dtype == AKAS_F32 && C % 8 == 0 && C >= 1024 && C <= 8192 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
#define AKAS_ROWS(TO, P) \
  return launch_chained(rmsnorm_rows_kernel<TO, P>, dim3(M), dim3(256), 0, stream, (const float*)x, w, (TO*)y, rows, C, eps, zero_centered)
    if (out_dtype == AKAS_F32) { if (C <= 2048) AKAS_ROWS(float, 1); else if (C <= 4096) AKAS_ROWS(float, 2); else AKAS_ROWS(float, 4); }
    else { if (C <= 2048) AKAS_ROWS(bf16, 1); else if (C <= 4096) AKAS_ROWS(bf16, 2); else AKAS_ROWS(bf16, 4); }
#undef AKAS_ROWS
  }
  const int threads = C >= 2048 ? 512 : C >= 512 ? 256 : 128;
#define AKAS_NORM(TI, TO) \
  rmsnorm_kernel<TI, TO><<<M, threads, 0, stream>>>((const TI*)x, w, (TO*)y, rows, C, eps, zero_centered)
  if (in_dtype == AKAS_F32 && out_dtype == AKAS_F32) AKAS_NORM(float, float);
  else if (in_dtype == AKAS_F32) AKAS_NORM(float, bf16);
  else if (out_dtype == AKAS_F32) AKAS_NORM(bf16, float);
  else AKAS_NORM(bf16, bf16);
#undef AKAS_NORM
  return launch_status();
}

// out[n, f] = silu(gu[n, f]) * gu[n, F + f], silu(g) = g / (1 + exp(-g)), in float32
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t n = i / F;
  const int f = (int)(i - n * F);
  const float g = to_f32(gu[n * 2 * F + f]);
  const float u = to_f32(gu[n * 2 * F + F + f]);
  out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
}

// Eight (bfloat16) or four (float32) neighbours per thread with 16-byte loads, for F a multiple of that.
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t groups) {
  constexpr int V = Vec<T>::N;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= groups) return;
  const int per_row = F / V;
  const size_t n = i / per_row;
  const int f = (int)(i - n * per_row) * V;
  float g[V], u[V], o[V];
  load_vec(gu + n * 2 * F + f, g);
  load_vec(gu + n * 2 * F + F + f, u);
#pragma unroll
  for (int e = 0; e < V; ++e) o[e] = g[e] / (1.f + expf(-g[e])) * u[e];
  store_vec(out + n * F + f, o);
}

AKAS_API int akas_swiglu(const void* gu, void* out, int N, int F, int dtype, cudaStream_t stream) {
  const size_t total = (size_t)N * F;
  if (total == 0) return 0;
  const int threads = 256;
  const int v = dtype == AKAS_F32 ? 4 : 8;
  if (F % v == 0 && (uintptr_t)gu % 16 == 0 && (uintptr_t)out % 16 == 0) {
    const size_t groups = total / v;
    const unsigned blocks = (unsigned)((groups + threads - 1) / threads);
    if (dtype == AKAS_F32)
      swiglu_vec_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, F, groups);
    else
      swiglu_vec_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, F, groups);
    return launch_status();
  }
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  if (dtype == AKAS_F32)
    swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, F, total);
  else
    swiglu_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, F, total);
  return launch_status();
}

// state[g, slot, :] = 0 for one slot of a [groups, slots, row] float32 tensor (groups: the layers whose states
// of one shape share an allocation)
__global__ void zero_row_kernel(float* __restrict__ state, size_t row, size_t group_stride, int slot) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < row) state[blockIdx.y * group_stride + (size_t)slot * row + i] = 0.f;
}

AKAS_API int akas_zero_row(float* state, long long row_elems, int slot, int groups, long long group_stride,
                           cudaStream_t stream) {
  if (row_elems <= 0 || groups <= 0) return 0;
  if (groups > 65535) return (int)cudaErrorInvalidValue;
  const int threads = 256;
  zero_row_kernel<<<dim3((unsigned)((row_elems + threads - 1) / threads), groups), threads, 0, stream>>>(
      state, (size_t)row_elems, (size_t)group_stride, slot);
  return launch_status();
}

// token_ids[i] = previous[source[i]] where source[i] >= 0: tokens that the step before sampled and that never
// went to the host.
__global__ void take_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ source,
                                   const int* __restrict__ previous, int previous_count, int N) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N) return;
  const int s = source[i];
  if (s >= 0 && s < previous_count) token_ids[i] = previous[s];
}

AKAS_API int akas_take_tokens(int* token_ids, const int* source, const int* previous, int previous_count, int N,
                              cudaStream_t stream) {
  if (N <= 0) return 0;
  take_tokens_kernel<<<(N + 255) / 256, 256, 0, stream>>>(token_ids, source, previous, previous_count, N);
  return launch_status();
}

// out[n, c] = x[n, c] + bias[c], x float32, out float32 or bfloat16 (out may be x): the bias of a product whose
// result was left in float32, added before the one rounding.
template <typename TO>
__global__ void add_bias_kernel(const float* __restrict__ x, const float* __restrict__ bias, TO* __restrict__ out, int C,
                                size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] = from_f32<TO>(x[i] + bias[i % C]);
}

AKAS_API int akas_add_bias(const float* x, const float* bias, void* out, int N, int C, int out_dtype, cudaStream_t stream) {
  const size_t total = (size_t)N * C;
  if (total == 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (out_dtype == AKAS_F32) add_bias_kernel<float><<<blocks, 256, 0, stream>>>(x, bias, (float*)out, C, total);
  else add_bias_kernel<bf16><<<blocks, 256, 0, stream>>>(x, bias, (bf16*)out, C, total);
  return launch_status();
}

// In place on float32: x = x * scale, then x = cap * tanh(x / cap) where cap > 0 (an embedding multiplier, a
// logit scale, a logit softcap).
__global__ void scale_cap_kernel(float* __restrict__ x, float scale, float cap, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = x[i] * scale;
  if (cap > 0.f) v = cap * tanhf(v / cap);
  x[i] = v;
}

AKAS_API int akas_scale_cap(float* x, float scale, float cap, long long total, cudaStream_t stream) {
  if (total <= 0) return 0;
  scale_cap_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(x, scale, cap, (size_t)total);
  return launch_status();
}
