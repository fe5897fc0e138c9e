// LFM2's gated causal depthwise short convolution over a flat batch, with per-request state.
//
// Per token t of request r (local index j = t - cu_seqlens[r]) and channel c:
//   u[t]   = B[t] * x[t]                      (bcx row = [B | C | x], three parts of width C)
//   s[t]   = sum_{i<L} u_i * taps[c, i]       u_i = u of local index j - (L-1-i), taken from this
//                                             step's rows when that index is >= 0, else from the
//                                             request's state (its last L-1 values of u, oldest first)
//   out[t] = C[t] * (s[t] + bias[c])
// and afterwards state[r] = the last L-1 values of u of (state ++ this step's u). Products, sums and
// the state are float32. Two launches: the forward reads the old state, the update then rewrites it;
// both are per-token/per-request parallel, so a prompt portion is not walked serially.
#include "common.cuh"

using namespace akas;

#define AKAS_CONV_MAX_TAPS 16

template <typename T>
__global__ void short_conv_forward_kernel(const T* __restrict__ bcx, const float* __restrict__ taps,
                                          const float* __restrict__ bias, const float* __restrict__ state,
                                          const int* __restrict__ cu_seqlens, const int* __restrict__ seq_of_token,
                                          const int* __restrict__ slots, T* __restrict__ out, int C, int L) {
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int r = seq_of_token[t];
  const int slot = r >= 0 ? slots[r] : -1;
  if (slot < 0) {
    out[(size_t)t * C + c] = from_f32<T>(0.f);
    return;
  }
  const int j = t - cu_seqlens[r];
  float acc = 0.f;
  for (int i = 0; i < L; ++i) {
    const int back = L - 1 - i;  // how many tokens before t
    float u;
    if (j - back >= 0) {
      const T* row = bcx + (size_t)(t - back) * 3 * C;
      u = to_f32(row[c]) * to_f32(row[2 * C + c]);
    } else {
      u = state[((size_t)slot * (L - 1) + (j + i)) * C + c];
    }
    acc = fmaf(u, taps[(size_t)c * L + i], acc);
  }
  if (bias) acc += bias[c];
  out[(size_t)t * C + c] = from_f32<T>(to_f32(bcx[(size_t)t * 3 * C + C + c]) * acc);
}

// The forward for widths that are a multiple of 8: a thread owns 8 neighbouring channels of one token.
template <typename T>
__global__ void short_conv_forward8_kernel(const T* __restrict__ bcx, const float* __restrict__ taps,
                                           const float* __restrict__ bias, const float* __restrict__ state,
                                           const int* __restrict__ cu_seqlens, const int* __restrict__ seq_of_token,
                                           const int* __restrict__ slots, T* __restrict__ out, int C, int L) {
  const int t = blockIdx.x;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int r = seq_of_token[t];
  const int slot = r >= 0 ? slots[r] : -1;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (slot >= 0) {
    const int j = t - cu_seqlens[r];
    for (int i = 0; i < L; ++i) {
      const int back = L - 1 - i;
      float u[8];
      if (j - back >= 0) {
        const T* row = bcx + (size_t)(t - back) * 3 * C;
        float b[8], x[8];
        load8(row + c, b);
        load8(row + 2 * C + c, x);
#pragma unroll
        for (int e = 0; e < 8; ++e) u[e] = b[e] * x[e];
      } else {
        load8(state + ((size_t)slot * (L - 1) + (j + i)) * C + c, u);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = fmaf(u[e], taps[(size_t)(c + e) * L + i], acc[e]);
    }
    float gate[8];
    load8(bcx + (size_t)t * 3 * C + C + c, gate);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = gate[e] * (bias ? acc[e] + bias[c + e] : acc[e]);
  }
  store8(out + (size_t)t * C + c, acc);
}

template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ bcx, float* __restrict__ state,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int C,
                                        int L) {
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int slot = slots[r];
  const int start = cu_seqlens[r];
  const int n = cu_seqlens[r + 1] - start;
  if (slot < 0 || n <= 0) return;
  float next[AKAS_CONV_MAX_TAPS - 1];
  float* rows = state + (size_t)slot * (L - 1) * C + c;
  for (int i = 0; i < L - 1; ++i) {
    const int j = n - (L - 1) + i;  // local index of the token whose u becomes state row i
    if (j >= 0) {
      const T* row = bcx + (size_t)(start + j) * 3 * C;
      next[i] = to_f32(row[c]) * to_f32(row[2 * C + c]);
    } else {
      next[i] = rows[(size_t)(n + i) * C];
    }
  }
  for (int i = 0; i < L - 1; ++i) rows[(size_t)i * C] = next[i];
}

// Steps that only decode: token t is the single token of request seq_of_token[t]. One thread per (token,
// channel) reads the state rows, forms the output and writes the shifted state: one launch instead of two.
template <typename T>
__global__ void short_conv_decode_kernel(const T* __restrict__ bcx, const float* __restrict__ taps,
                                         const float* __restrict__ bias, float* __restrict__ state,
                                         const int* __restrict__ seq_of_token, const int* __restrict__ slots,
                                         T* __restrict__ out, int C, int L) {
  chain_release();
  chain_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int r = seq_of_token[t];
  const int slot = r >= 0 ? slots[r] : -1;
  if (slot < 0) {
    out[(size_t)t * C + c] = from_f32<T>(0.f);
    return;
  }
  const T* row = bcx + (size_t)t * 3 * C;
  const float u = to_f32(row[c]) * to_f32(row[2 * C + c]);
  float* hist = state + (size_t)slot * (L - 1) * C + c;
  float acc = 0.f;
  for (int i = 0; i < L - 1; ++i) {
    const float h = hist[(size_t)i * C];
    acc = fmaf(h, taps[(size_t)c * L + i], acc);
    if (i > 0) hist[(size_t)(i - 1) * C] = h;
  }
  acc = fmaf(u, taps[(size_t)c * L + L - 1], acc);
  hist[(size_t)(L - 2) * C] = u;
  if (bias) acc += bias[c];
  out[(size_t)t * C + c] = from_f32<T>(to_f32(row[C + c]) * acc);
}

AKAS_API int akas_short_conv_decode(const void* bcx, const float* taps, const float* bias, float* state,
                                    const int* seq_of_token, const int* slots, void* out, int N, int C, int L,
                                    int dtype, cudaStream_t stream) {
  if (L < 2 || L > AKAS_CONV_MAX_TAPS) return (int)cudaErrorInvalidValue;
  if (N <= 0) return 0;
  const int threads = 128;
  const dim3 grid(N, (C + threads - 1) / threads);
  if (dtype == AKAS_F32)
    return launch_chained(short_conv_decode_kernel<float>, grid, dim3(threads), 0, stream, (const float*)bcx, taps, bias,
                          state, seq_of_token, slots, (float*)out, C, L);
  return launch_chained(short_conv_decode_kernel<bf16>, grid, dim3(threads), 0, stream, (const bf16*)bcx, taps, bias,
                        state, seq_of_token, slots, (bf16*)out, C, L);
}

AKAS_API int akas_short_conv(const void* bcx, const float* taps, const float* bias, float* state,
                             const int* cu_seqlens, const int* seq_of_token, const int* slots, void* out, int N,
                             int R, int C, int L, int dtype, cudaStream_t stream) {
  if (L < 2 || L > AKAS_CONV_MAX_TAPS) return (int)cudaErrorInvalidValue;
  if (N <= 0 || R <= 0) return 0;
  const int threads = 128;
  const dim3 fwd(N, (C + threads - 1) / threads), upd(R, (C + threads - 1) / threads);
  const bool wide = C % 8 == 0 && (uintptr_t)bcx % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)state % 16 == 0;
  const dim3 fwd8(N, (C / 8 + threads - 1) / threads);
  if (dtype == AKAS_F32) {
    if (wide)
      short_conv_forward8_kernel<float><<<fwd8, threads, 0, stream>>>((const float*)bcx, taps, bias, state, cu_seqlens,
                                                                      seq_of_token, slots, (float*)out, C, L);
    else
      short_conv_forward_kernel<float><<<fwd, threads, 0, stream>>>((const float*)bcx, taps, bias, state, cu_seqlens,
                                                                    seq_of_token, slots, (float*)out, C, L);
    short_conv_state_kernel<float><<<upd, threads, 0, stream>>>((const float*)bcx, state, cu_seqlens, slots, C, L);
  } else {
    if (wide)
      short_conv_forward8_kernel<bf16><<<fwd8, threads, 0, stream>>>((const bf16*)bcx, taps, bias, state, cu_seqlens,
                                                                     seq_of_token, slots, (bf16*)out, C, L);
    else
      short_conv_forward_kernel<bf16><<<fwd, threads, 0, stream>>>((const bf16*)bcx, taps, bias, state, cu_seqlens,
                                                                   seq_of_token, slots, (bf16*)out, C, L);
    short_conv_state_kernel<bf16><<<upd, threads, 0, stream>>>((const bf16*)bcx, state, cu_seqlens, slots, C, L);
  }
  return launch_status();
}
