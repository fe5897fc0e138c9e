// Matrix products for a handful of tokens (decode steps): y[M, O] = f(x)[M, K] . W[O, K]^T with M <= 16,
// bfloat16 weights streamed once from HBM, float32 accumulation on the tensor cores.
//
// The weights are the A operand of mma.sync m16n8k16 (16 weight rows x 16 k), the tokens are the 8
// columns of B, so one block turns 16 rows of W into 16 output channels for all tokens. Its 8 warps
// split K in 32-wide chunks; in a chunk, thread (g, t) of a warp loads 16 contiguous bytes of W rows g
// and g + 8 and of the activations of token g at k = 32c + 8t. The 8 values feed two k-steps; the
// product does not care which physical k sits in which k-slot as long as A and B agree, which is
// what makes 16-byte loads possible. Partial sums of the 8 warps meet in shared memory.
//
// Input modes:   bf16   x is bfloat16 [M, K]
//                norm   x is the float32 residual stream (rows optionally gathered by index); the kernel
//                       forms bf16(x * norm_weight) for B, sums x^2 per token on the way and multiplies
//                       the result by rsqrt(mean(x^2) + eps): RMSNorm without a pass of its own.
// Output modes:  bf16 store | float32 store | float32 accumulate (y += ..., the residual stream) |
//                swiglu: the block's 16 rows are gate rows f0..f0+7 and up rows F+f0..F+f0+7 of the
//                stacked [2F, K] matrix, so silu(gate) * up is formed per thread and stored as bf16 [M, F].
// Needs K % 32 == 0. Results do not depend on what else runs; summation order is fixed.
#include <math.h>

#include "common.cuh"
#include "mma.cuh"

using namespace akas;

namespace {

constexpr int WARPS = 8;
enum { IN_BF16 = 0, IN_NORM = 1 };
enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_ACC = 2, OUT_SWIGLU = 3 };

template <int NT, int IN, int OUT>
__global__ void __launch_bounds__(WARPS * 32)
skinny_gemm_kernel(const void* __restrict__ x_, const int* __restrict__ rows, const float* __restrict__ norm_w,
                   float eps, int zero_centered, const bf16* __restrict__ W, void* __restrict__ y_, int M, int O,
                   int K) {
  __shared__ float red[WARPS][NT][16][8];
  __shared__ float ss_s[WARPS][NT * 8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  // weight rows of this block: output channels o0 .. o0+15, or 8 gate + 8 up rows
  const int F = O / 2;  // swiglu only: O is the stacked height 2F
  int row_a, row_b;
  bool ok_a, ok_b;
  if (OUT == OUT_SWIGLU) {
    const int f = blockIdx.x * 8 + g;
    ok_a = ok_b = f < F;
    row_a = ok_a ? f : 0;
    row_b = ok_a ? F + f : 0;
  } else {
    row_a = blockIdx.x * 16 + g;
    row_b = row_a + 8;
    ok_a = row_a < O;
    ok_b = row_b < O;
    if (!ok_a) row_a = 0;
    if (!ok_b) row_b = 0;
  }
  const bf16* wa = W + (size_t)row_a * K + 8 * t;
  const bf16* wb = W + (size_t)row_b * K + 8 * t;

  // the token this thread feeds into B, per n-block
  const bf16* xb[NT];
  const float* xf[NT];
  bool live[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int m = 8 * j + g;
    live[j] = m < M;
    const size_t src = live[j] ? (size_t)(rows ? rows[m] : m) : 0;
    xb[j] = (const bf16*)x_ + src * K + 8 * t;
    xf[j] = (const float*)x_ + src * K + 8 * t;
  }

  float acc[NT][4];
  float ss[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; ss[j] = 0.f; }

  const int chunks = K / 32;
#pragma unroll 4
  for (int c = warp; c < chunks; c += WARPS) {
    const int k = c * 32;
    const uint4 a_lo = *reinterpret_cast<const uint4*>(wa + k);
    const uint4 a_hi = *reinterpret_cast<const uint4*>(wb + k);
    const uint32_t a1[4] = {a_lo.x, a_hi.x, a_lo.y, a_hi.y};  // first k-step
    const uint32_t a2[4] = {a_lo.z, a_hi.z, a_lo.w, a_hi.w};  // second k-step
    float nw[8];
    if (IN == IN_NORM) {
      const float4 w0 = *reinterpret_cast<const float4*>(norm_w + k + 8 * t);
      const float4 w1 = *reinterpret_cast<const float4*>(norm_w + k + 8 * t + 4);
      nw[0] = w0.x; nw[1] = w0.y; nw[2] = w0.z; nw[3] = w0.w;
      nw[4] = w1.x; nw[5] = w1.y; nw[6] = w1.z; nw[7] = w1.w;
      if (zero_centered) {
#pragma unroll
        for (int i = 0; i < 8; ++i) nw[i] += 1.f;
      }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      uint32_t b[4] = {0u, 0u, 0u, 0u};
      if (live[j]) {
        if (IN == IN_BF16) {
          const uint4 v = *reinterpret_cast<const uint4*>(xb[j] + k);
          b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w;
        } else {
          const float4 v0 = *reinterpret_cast<const float4*>(xf[j] + k);
          const float4 v1 = *reinterpret_cast<const float4*>(xf[j] + k + 4);
          const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) ss[j] = fmaf(v[i], v[i], ss[j]);
#pragma unroll
          for (int i = 0; i < 4; ++i) b[i] = pack_bf16(v[2 * i] * nw[2 * i], v[2 * i + 1] * nw[2 * i + 1]);
        }
      }
      mma_bf16(acc[j], a1, b[0], b[1]);
      mma_bf16(acc[j], a2, b[2], b[3]);
    }
  }

  // partial sums of the 8 warps -> shared memory
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    red[warp][j][g][2 * t] = acc[j][0];
    red[warp][j][g][2 * t + 1] = acc[j][1];
    red[warp][j][g + 8][2 * t] = acc[j][2];
    red[warp][j][g + 8][2 * t + 1] = acc[j][3];
    if (IN == IN_NORM) {
      float s = ss[j];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      if (t == 0) ss_s[warp][j * 8 + g] = s;
    }
  }
  __syncthreads();

  const int per_tile = OUT == OUT_SWIGLU ? 64 : 128;  // (row, token) pairs per n-block handled in the epilogue
  for (int i = tid; i < NT * per_tile; i += WARPS * 32) {
    const int j = i / per_tile, row = (i % per_tile) / 8, tok = i % 8;
    const int m = 8 * j + tok;
    if (m >= M) continue;
    float v = 0.f, u = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      v += red[w][j][row][tok];
      if (OUT == OUT_SWIGLU) u += red[w][j][row + 8][tok];
    }
    if (IN == IN_NORM) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) s += ss_s[w][j * 8 + tok];
      const float inv = 1.f / sqrtf(s / (float)K + eps);
      v *= inv;
      u *= inv;
    }
    if (OUT == OUT_SWIGLU) {
      const int f = blockIdx.x * 8 + row;
      if (f < F) ((bf16*)y_)[(size_t)m * F + f] = __float2bfloat16_rn(v / (1.f + expf(-v)) * u);
    } else {
      const int o = blockIdx.x * 16 + row;
      if (o >= O) continue;
      const size_t at = (size_t)m * O + o;
      if (OUT == OUT_BF16) ((bf16*)y_)[at] = __float2bfloat16_rn(v);
      else if (OUT == OUT_F32) ((float*)y_)[at] = v;
      else ((float*)y_)[at] += v;
    }
  }
}

template <int NT, int IN>
int launch_out(int out_mode, const void* x, const int* rows, const float* norm_w, float eps, int zero_centered,
               const void* W, void* y, int M, int O, int K, cudaStream_t stream) {
  const int threads = WARPS * 32;
#define AKAS_SKINNY(OUTM, GRID)                                                                                   \
  skinny_gemm_kernel<NT, IN, OUTM><<<GRID, threads, 0, stream>>>(x, rows, norm_w, eps, zero_centered,             \
                                                                 (const bf16*)W, y, M, O, K)
  switch (out_mode) {
    case OUT_BF16: AKAS_SKINNY(OUT_BF16, (O + 15) / 16); break;
    case OUT_F32: AKAS_SKINNY(OUT_F32, (O + 15) / 16); break;
    case OUT_ACC: AKAS_SKINNY(OUT_ACC, (O + 15) / 16); break;
    case OUT_SWIGLU: AKAS_SKINNY(OUT_SWIGLU, (O / 2 + 7) / 8); break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef AKAS_SKINNY
  return launch_status();
}

}  // namespace

// x: bfloat16 [M, K] (in_mode 0) or float32 [*, K] rows gathered by `rows` (or 0..M-1) with RMSNorm fused (in_mode 1).
// W: bfloat16 [O, K]. y: [M, O] in the output mode's type, or bfloat16 [M, O / 2] for swiglu (out_mode 3).
AKAS_API int akas_skinny_gemm(const void* x, const int* rows, const float* norm_w, float eps, int zero_centered,
                              const void* W, void* y, int M, int O, int K, int in_mode, int out_mode,
                              cudaStream_t stream) {
  if (M <= 0 || O <= 0) return 0;
  if (M > 16 || K <= 0 || K % 32 || (out_mode == OUT_SWIGLU && O % 2)) return (int)cudaErrorInvalidValue;
  if (in_mode == IN_NORM && norm_w == nullptr) return (int)cudaErrorInvalidValue;
  if (M <= 8) {
    if (in_mode == IN_BF16) return launch_out<1, IN_BF16>(out_mode, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, stream);
    return launch_out<1, IN_NORM>(out_mode, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, stream);
  }
  if (in_mode == IN_BF16) return launch_out<2, IN_BF16>(out_mode, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, stream);
  return launch_out<2, IN_NORM>(out_mode, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, stream);
}
