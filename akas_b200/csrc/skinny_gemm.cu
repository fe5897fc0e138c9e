// Matrix products for a handful of tokens (decode steps): y[M, O] = f(x)[M, K] . W[O, K]^T with M <= 16,
// bfloat16 weights streamed once from HBM, float32 accumulation on the tensor cores.
//
// The weights are the A operand of mma.sync m16n8k16 (16 weight rows x 16 k), the tokens are the 8
// columns of B, so one block turns 16 rows of W into 16 output channels for all tokens. Its 8 warps
// split K in 32-wide chunks; in a chunk, thread (g, t) of a warp loads 16 contiguous bytes of W rows g
// and g + 8 and of the activations of token g at k = 32c + 8t. The 8 values feed two k-steps; the
// product does not care which physical k sits in which k-slot as long as A and B agree, which is
// what makes 16-byte loads possible. The weight rows arrive through a six-stage ring of 256-wide
// chunks in shared memory filled by cp.async (40 KB of loads in flight per block, several blocks per
// SM), the activations come from L1/L2 one chunk ahead. Partial sums of the 8 warps meet in shared memory.
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

constexpr int WARPS = 8, KC = 256, STAGES = 6, AS = KC + 32;  // AS: row stride of a stage, 16 words off a multiple of 32 banks
enum { IN_BF16 = 0, IN_NORM = 1 };
enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_ACC = 2, OUT_SWIGLU = 3 };

template <int NT, int IN>
struct BFrag {
  uint4 raw[NT];        // IN_BF16: 8 bfloat16 of the token's activations
  float4 lo[NT], hi[NT];  // IN_NORM: 8 float32 of the residual stream
  float4 w_lo, w_hi;    // IN_NORM: 8 norm weights
};

template <int NT, int IN, int OUT>
__global__ void __launch_bounds__(WARPS * 32)
skinny_gemm_kernel(const void* __restrict__ x_, const int* __restrict__ rows, const float* __restrict__ norm_w,
                   float eps, int zero_centered, const bf16* __restrict__ W, void* __restrict__ y_, int M, int O,
                   int K) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* ring = reinterpret_cast<bf16*>(smem_raw);  // [STAGES][16][AS]
  __shared__ float ss_s[WARPS][NT * 8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int F = O / 2;  // swiglu only: O is the stacked height 2F

  // weight row that stage row i of this block holds, or -1
  auto weight_row = [&](int i) -> int {
    if (OUT == OUT_SWIGLU) {
      const int f = blockIdx.x * 8 + (i & 7);
      return f < F ? (i < 8 ? f : F + f) : -1;
    }
    const int o = blockIdx.x * 16 + i;
    return o < O ? o : -1;
  };
  const int chunks = (K + KC - 1) / KC;
  auto load_stage = [&](int c) {
    const int k0 = c * KC, len = min(KC, K - k0), per_row = len / 8;
    bf16* dst = ring + (size_t)(c % STAGES) * 16 * AS;
    for (int i = tid; i < 16 * per_row; i += WARPS * 32) {
      const int row = i / per_row, col = (i % per_row) * 8;
      const int wr = weight_row(row);
      cp_async16(dst + row * AS + col, W + (size_t)max(wr, 0) * K + k0 + col, wr >= 0 ? 16 : 0);
    }
  };
#pragma unroll
  for (int c = 0; c < STAGES - 1; ++c) {
    if (c < chunks) load_stage(c);
    cp_async_commit();
  }

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
  auto load_b = [&](BFrag<NT, IN>& f, int k) {  // k: first of this thread's 8 consecutive k
    if (k >= K) return;
    if (IN == IN_NORM) {
      f.w_lo = *reinterpret_cast<const float4*>(norm_w + k + 8 * t);
      f.w_hi = *reinterpret_cast<const float4*>(norm_w + k + 8 * t + 4);
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      if (!live[j]) continue;
      if (IN == IN_BF16) {
        f.raw[j] = *reinterpret_cast<const uint4*>(xb[j] + k);
      } else {
        f.lo[j] = *reinterpret_cast<const float4*>(xf[j] + k);
        f.hi[j] = *reinterpret_cast<const float4*>(xf[j] + k + 4);
      }
    }
  };

  float acc[NT][4];
  float ss[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; ss[j] = 0.f; }

  BFrag<NT, IN> cur, next;
  load_b(cur, warp * 32);
  for (int c = 0; c < chunks; ++c) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();  // chunk c has landed for everyone, and everyone is done with chunk c - 1
    if (c + STAGES - 1 < chunks) load_stage(c + STAGES - 1);
    cp_async_commit();
    const int k = c * KC + warp * 32;  // this warp's 32 k of the chunk
    load_b(next, k + KC);
    if (k < K) {
      const bf16* st = ring + (size_t)(c % STAGES) * 16 * AS + warp * 32 + 8 * t;
      const uint4 a_lo = *reinterpret_cast<const uint4*>(st + g * AS);
      const uint4 a_hi = *reinterpret_cast<const uint4*>(st + (g + 8) * AS);
      const uint32_t a1[4] = {a_lo.x, a_hi.x, a_lo.y, a_hi.y};  // first k-step: this thread's k 0..3
      const uint32_t a2[4] = {a_lo.z, a_hi.z, a_lo.w, a_hi.w};  // second k-step: its k 4..7
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        uint32_t b[4] = {0u, 0u, 0u, 0u};
        if (live[j]) {
          if (IN == IN_BF16) {
            b[0] = cur.raw[j].x; b[1] = cur.raw[j].y; b[2] = cur.raw[j].z; b[3] = cur.raw[j].w;
          } else {
            const float v[8] = {cur.lo[j].x, cur.lo[j].y, cur.lo[j].z, cur.lo[j].w,
                                cur.hi[j].x, cur.hi[j].y, cur.hi[j].z, cur.hi[j].w};
            float nw[8] = {cur.w_lo.x, cur.w_lo.y, cur.w_lo.z, cur.w_lo.w, cur.w_hi.x, cur.w_hi.y, cur.w_hi.z, cur.w_hi.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              ss[j] = fmaf(v[i], v[i], ss[j]);
              if (zero_centered) nw[i] += 1.f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) b[i] = pack_bf16(v[2 * i] * nw[2 * i], v[2 * i + 1] * nw[2 * i + 1]);
          }
        }
        mma_bf16(acc[j], a1, b[0], b[1]);
        mma_bf16(acc[j], a2, b[2], b[3]);
      }
    }
    cur = next;
  }
  cp_async_wait<0>();
  __syncthreads();  // the ring is free: it becomes the buffer where the 8 warps' partial sums meet

  float* red = reinterpret_cast<float*>(smem_raw);  // [WARPS][NT][16][8]
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    float* r0 = red + (((size_t)warp * NT + j) * 16 + g) * 8 + 2 * t;
    r0[0] = acc[j][0];
    r0[1] = acc[j][1];
    r0[64] = acc[j][2];  // row g + 8
    r0[65] = acc[j][3];
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
      const float* r0 = red + (((size_t)w * NT + j) * 16 + row) * 8 + tok;
      v += r0[0];
      if (OUT == OUT_SWIGLU) u += r0[64];
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

constexpr int kSmemBytes = STAGES * 16 * AS * (int)sizeof(bf16);

template <int NT, int IN>
int launch_out(int out_mode, const void* x, const int* rows, const float* norm_w, float eps, int zero_centered,
               const void* W, void* y, int M, int O, int K, cudaStream_t stream) {
  const int threads = WARPS * 32;
#define AKAS_SKINNY(OUTM, GRID)                                                                                   \
  {                                                                                                               \
    static bool configured = false;                                                                               \
    if (!configured) {                                                                                            \
      const cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<NT, IN, OUTM>,                                \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);        \
      if (e != cudaSuccess) return (int)e;                                                                        \
      configured = true;                                                                                          \
    }                                                                                                             \
    skinny_gemm_kernel<NT, IN, OUTM><<<GRID, threads, kSmemBytes, stream>>>(x, rows, norm_w, eps, zero_centered,  \
                                                                            (const bf16*)W, y, M, O, K);          \
  }
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
