// What happens to a head of q or k between the qkv product and attention, for a thread that owns 8 neighbouring
// channels of the head (TPH = head_dim / 8 threads of one warp own a head): RMSNorm over the head's channels, then
// the rotation of its first `rotary` channels (channel e turns with channel e +- rotary / 2). The sum of squares and
// the rotation partner travel by shuffle, so every lane of the warp must call this together. All in float32.
#pragma once

#include "common.cuh"

namespace akas {

// x: the thread's channels e0..e0+7. w: the norm's weight over the head (nullptr: no norm). cos_row, sin_row: the
// token's rotary / 2 cosines and sines (nullptr: no rotation; rotary must be a multiple of 16).
template <int TPH>
__device__ __forceinline__ void head_norm_rotate8(float (&x)[8], int e0, const float* __restrict__ w, float eps,
                                                  int zero_centered, const float* __restrict__ cos_row,
                                                  const float* __restrict__ sin_row, int rotary) {
  constexpr int D = TPH * 8;
  if (w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(x[e], x[e], ss);
#pragma unroll
    for (int o = TPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.f / sqrtf(ss / (float)D + eps);
    float g[8];
    load8(w + e0, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = x[e] * inv * (zero_centered ? 1.f + g[e] : g[e]);
  }
  if (cos_row != nullptr) {
    const int half = rotary / 2, shift = half / 8;  // the partner of channel e is e +- half: `shift` threads away
    const bool low = e0 < half, rotated = e0 < rotary;
    const int lane = threadIdx.x & 31;
    const int partner = rotated ? (low ? lane + shift : lane - shift) : lane;
    float other[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) other[e] = __shfl_sync(0xffffffffu, x[e], partner);
    if (rotated) {
      float c[8], sn[8];
      const int f0 = low ? e0 : e0 - half;
      load8(cos_row + f0, c);
      load8(sin_row + f0, sn);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = low ? x[e] * c[e] - other[e] * sn[e] : other[e] * sn[e] + x[e] * c[e];
    }
  }
}

}  // namespace akas
