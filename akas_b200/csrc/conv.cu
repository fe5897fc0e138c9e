// LFM2's gated causal depthwise short convolution over a flat batch, with per-request state.
//
// Per token t of request r (local index j = t - cu_seqlens[r]) and channel c:
//   u[t]   = B[t] * x[t]                      (bcx row = [B | C | x], three parts of width C)
//   s[t]   = sum_{i<L} u_i * taps[c, i]       u_i = u of local index j - (L-1-i), taken from this
//                                             step's rows when that index is >= 0, else from the
//                                             request's state (its last L-1 values of u, oldest first)
//   out[t] = C[t] * (s[t] + bias[c])
// and afterwards state[r] = the last L-1 values of u of (state ++ this step's u). Products, sums and
// the state are float32. With write == 0 the state is read and left as it is (a layer that reads another
// layer's state). Two launches: the forward reads the old state, the update then rewrites it;
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

// The forward for prompt portions, for the usual numbers of taps: a thread owns 8 neighbouring channels of TT
// consecutive tokens and slides the window along them, so that every u = B * x is formed once, and the taps and
// the bias are fetched once per thread. The sum runs in the same order as in the kernels above (tap 0 first), so
// the results are the same bits.
template <typename T, int L, int TT>
__global__ void __launch_bounds__(128)
short_conv_forward_run_kernel(const T* __restrict__ bcx, const float* __restrict__ taps, const float* __restrict__ bias,
                              const float* __restrict__ state, const int* __restrict__ cu_seqlens,
                              const int* __restrict__ seq_of_token, const int* __restrict__ slots, T* __restrict__ out,
                              int N, int C) {
  chain_release();  // a kernel after this one that was launched as its programmatic dependent may set itself up meanwhile
  chain_wait();
  const int t0 = blockIdx.x * TT;
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  float tap[8][L], bv[8], hist[L - 1][8];
  {
    float flat[8 * L];
#pragma unroll
    for (int i = 0; i < 8 * L; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(taps + (size_t)c * L + i);
      flat[i] = v.x; flat[i + 1] = v.y; flat[i + 2] = v.z; flat[i + 3] = v.w;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
      for (int i = 0; i < L; ++i) tap[e][i] = flat[e * L + i];
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) bv[e] = bias ? bias[c + e] : 0.f;
  bool have = false;  // hist holds the u of the L - 1 tokens before the current one
#pragma unroll
  for (int tt = 0; tt < TT; ++tt) {
    const int t = t0 + tt;
    if (t >= N) break;
    const int r = seq_of_token[t];
    const int slot = r >= 0 ? slots[r] : -1;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (slot < 0) {
      have = false;
      store8(out + (size_t)t * C + c, acc);
      continue;
    }
    const int j = t - cu_seqlens[r];
    if (!have || j == 0) {  // the first token of this thread's run or of a request: fetch the window
#pragma unroll
      for (int i = 0; i < L - 1; ++i) {
        const int back = L - 1 - i;
        if (j - back >= 0) {
          const T* row = bcx + (size_t)(t - back) * 3 * C;
          float b[8], x[8];
          load8(row + c, b);
          load8(row + 2 * C + c, x);
#pragma unroll
          for (int e = 0; e < 8; ++e) hist[i][e] = b[e] * x[e];
        } else {
          load8(state + ((size_t)slot * (L - 1) + (j + i)) * C + c, hist[i]);
        }
      }
    }
    const T* row = bcx + (size_t)t * 3 * C;
    float b[8], x[8], gate[8], u[8];
    load8(row + c, b);
    load8(row + 2 * C + c, x);
    load8(row + C + c, gate);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      u[e] = b[e] * x[e];
#pragma unroll
      for (int i = 0; i < L - 1; ++i) acc[e] = fmaf(hist[i][e], tap[e][i], acc[e]);
      acc[e] = fmaf(u[e], tap[e][L - 1], acc[e]);
      acc[e] = gate[e] * (bias ? acc[e] + bv[e] : acc[e]);
    }
    store8(out + (size_t)t * C + c, acc);
#pragma unroll
    for (int i = 0; i + 1 < L - 1; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) hist[i][e] = hist[i + 1][e];
#pragma unroll
    for (int e = 0; e < 8; ++e) hist[L - 2][e] = u[e];
    have = true;
  }
}

template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ bcx, float* __restrict__ state,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int C,
                                        int L) {
  chain_release();  // a kernel after this one that was launched as its programmatic dependent may set itself up meanwhile
  chain_wait();
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
                                         T* __restrict__ out, int C, int L, int write) {
  constexpr int FEW = 4;  // up to this many taps everything is fetched at once: one trip to memory, not one per tap
  chain_release();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  // What the host wrote for this step (which request, which state row) and the weights do not wait for the kernel ahead.
  const int r = seq_of_token[t];
  const int slot = r >= 0 ? slots[r] : -1;
  float tap[FEW] = {0.f, 0.f, 0.f, 0.f}, add = 0.f;
  if (c < C && L <= FEW) {
#pragma unroll
    for (int i = 0; i < FEW; ++i)
      if (i < L) tap[i] = taps[(size_t)c * L + i];
    if (bias) add = bias[c];
  }
  chain_wait();
  if (c >= C) return;
  if (slot < 0) {
    out[(size_t)t * C + c] = from_f32<T>(0.f);
    return;
  }
  const T* row = bcx + (size_t)t * 3 * C;
  float* hist = state + (size_t)slot * (L - 1) * C + c;
  if (L <= FEW) {
    float h[FEW - 1] = {0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < FEW - 1; ++i)
      if (i < L - 1) h[i] = hist[(size_t)i * C];
    const float b = to_f32(row[c]), gate = to_f32(row[C + c]), x = to_f32(row[2 * C + c]);
    const float u = b * x;
    float acc = 0.f, last = tap[0];
#pragma unroll
    for (int i = 0; i < FEW - 1; ++i) {
      if (i < L - 1) {
        acc = fmaf(h[i], tap[i], acc);
        if (i > 0 && write) hist[(size_t)(i - 1) * C] = h[i];
      }
      last = i + 1 == L - 1 ? tap[i + 1] : last;
    }
    acc = fmaf(u, last, acc);
    if (write) hist[(size_t)(L - 2) * C] = u;
    if (bias) acc += add;
    out[(size_t)t * C + c] = from_f32<T>(gate * acc);
    return;
  }
  const float u = to_f32(row[c]) * to_f32(row[2 * C + c]);
  float acc = 0.f;
  for (int i = 0; i < L - 1; ++i) {
    const float h = hist[(size_t)i * C];
    acc = fmaf(h, taps[(size_t)c * L + i], acc);
    if (i > 0 && write) hist[(size_t)(i - 1) * C] = h;
  }
  acc = fmaf(u, taps[(size_t)c * L + L - 1], acc);
  if (write) hist[(size_t)(L - 2) * C] = u;
  if (bias) acc += bias[c];
  out[(size_t)t * C + c] = from_f32<T>(to_f32(row[C + c]) * acc);
}

AKAS_API int akas_short_conv_decode(const void* bcx, const float* taps, const float* bias, float* state,
                                    const int* seq_of_token, const int* slots, void* out, int N, int C, int L,
                                    int dtype, int write, cudaStream_t stream) {
  if (L < 2 || L > AKAS_CONV_MAX_TAPS) return (int)cudaErrorInvalidValue;
  if (N <= 0) return 0;
  const int threads = 128;
  const dim3 grid(N, (C + threads - 1) / threads);
  if (dtype == AKAS_F32)
    return launch_chained(short_conv_decode_kernel<float>, grid, dim3(threads), 0, stream, (const float*)bcx, taps, bias,
                          state, seq_of_token, slots, (float*)out, C, L, write);
  return launch_chained(short_conv_decode_kernel<bf16>, grid, dim3(threads), 0, stream, (const bf16*)bcx, taps, bias,
                        state, seq_of_token, slots, (bf16*)out, C, L, write);
}

AKAS_API int akas_short_conv(const void* bcx, const float* taps, const float* bias, float* state,
                             const int* cu_seqlens, const int* seq_of_token, const int* slots, void* out, int N,
                             int R, int C, int L, int dtype, int write, cudaStream_t stream) {
  if (L < 2 || L > AKAS_CONV_MAX_TAPS) return (int)cudaErrorInvalidValue;
  if (N <= 0 || R <= 0) return 0;
  const int threads = 128;
  const dim3 fwd(N, (C + threads - 1) / threads), upd(R, (C + threads - 1) / threads);
  const bool wide = C % 8 == 0 && (uintptr_t)bcx % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)state % 16 == 0;
  const dim3 fwd8(N, (C / 8 + threads - 1) / threads);
  constexpr int TT = 4;
  const dim3 run((N + TT - 1) / TT, (C / 8 + threads - 1) / threads);
  const bool runs = wide && N >= 256 && L >= 2 && L <= 4 && (uintptr_t)taps % 16 == 0;
  // (both kernels as programmatic dependents; the state kernel writes what the run kernel ahead of it reads, after its wait)
#define AKAS_CONV_RUN(T, TAPS)                                                                                        \
  err = launch_chained(short_conv_forward_run_kernel<T, TAPS, TT>, run, dim3(threads), 0, stream, (const T*)bcx, taps, \
                       bias, (const float*)state, cu_seqlens, seq_of_token, slots, (T*)out, N, C)
  if (runs) {
    int err = 0;
    if (dtype == AKAS_F32) {
      if (L == 2) AKAS_CONV_RUN(float, 2); else if (L == 3) AKAS_CONV_RUN(float, 3); else AKAS_CONV_RUN(float, 4);
      if (!err && write) err = launch_chained(short_conv_state_kernel<float>, upd, dim3(threads), 0, stream, (const float*)bcx, state, cu_seqlens, slots, C, L);
    } else {
      if (L == 2) AKAS_CONV_RUN(bf16, 2); else if (L == 3) AKAS_CONV_RUN(bf16, 3); else AKAS_CONV_RUN(bf16, 4);
      if (!err && write) err = launch_chained(short_conv_state_kernel<bf16>, upd, dim3(threads), 0, stream, (const bf16*)bcx, state, cu_seqlens, slots, C, L);
    }
    return err;
  }
#undef AKAS_CONV_RUN
  if (dtype == AKAS_F32) {
    if (wide)
      short_conv_forward8_kernel<float><<<fwd8, threads, 0, stream>>>((const float*)bcx, taps, bias, state, cu_seqlens,
                                                                      seq_of_token, slots, (float*)out, C, L);
    else
      short_conv_forward_kernel<float><<<fwd, threads, 0, stream>>>((const float*)bcx, taps, bias, state, cu_seqlens,
                                                                    seq_of_token, slots, (float*)out, C, L);
    if (write) short_conv_state_kernel<float><<<upd, threads, 0, stream>>>((const float*)bcx, state, cu_seqlens, slots, C, L);
  } else {
    if (wide)
      short_conv_forward8_kernel<bf16><<<fwd8, threads, 0, stream>>>((const bf16*)bcx, taps, bias, state, cu_seqlens,
                                                                     seq_of_token, slots, (bf16*)out, C, L);
    else
      short_conv_forward_kernel<bf16><<<fwd, threads, 0, stream>>>((const bf16*)bcx, taps, bias, state, cu_seqlens,
                                                                   seq_of_token, slots, (bf16*)out, C, L);
    if (write) short_conv_state_kernel<bf16><<<upd, threads, 0, stream>>>((const bf16*)bcx, state, cu_seqlens, slots, C, L);
  }
  return launch_status();
}
