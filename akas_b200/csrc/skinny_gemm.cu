// Matrix products for a handful of tokens (decode steps): y[M, O] = f(x)[M, K] . W[O, K]^T with M <= 16,
// bfloat16 weights streamed once from HBM, float32 accumulation on the tensor cores.
//
// The weights are the A operand of mma.sync m16n8k16 (16 weight rows x 16 k), the tokens are the 8
// columns of B, so one block turns 16 rows of W into 16 output channels for all tokens. Its 8 warps
// split K in 32-wide chunks; in a chunk, thread (g, t) of a warp loads 16 contiguous bytes of W rows g
// and g + 8 and of the activations of token g at k = 32c + 8t. The 8 values feed two k-steps; the
// product does not care which physical k sits in which k-slot as long as A and B agree, which is
// what makes 16-byte loads possible. Blocks are persistent: one or two per SM, each taking row tiles
// blockIdx.x, blockIdx.x + gridDim.x, ... The weight rows arrive through an eight-stage ring of
// 256-wide chunks in shared memory filled by cp.async (56 KB of loads in flight per block) that runs
// on across row tiles; the tokens' activations are put into shared memory once per block (converted
// and weighted by the norm there, if the norm rides along), so the inner loop reads shared memory
// only. At the end of a row tile the 8 warps' partial sums meet in shared memory.
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

constexpr int WARPS = 8, KC = 256, STAGES = 8, AS = KC + 32;  // AS: row stride of a stage, 16 words off a multiple of 32 banks
enum { IN_BF16 = 0, IN_NORM = 1 };
enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_ACC = 2, OUT_SWIGLU = 3 };

template <int NT, int IN, int OUT>
__global__ void __launch_bounds__(WARPS * 32)
skinny_gemm_kernel(const void* __restrict__ x_, const int* __restrict__ rows, const float* __restrict__ norm_w,
                   float eps, int zero_centered, const bf16* __restrict__ W, void* __restrict__ y_, int M, int O,
                   int K, int num_tiles) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* ring = reinterpret_cast<bf16*>(smem_raw);               // [STAGES][16][AS]: weight rows, chunk by chunk
  float* red = reinterpret_cast<float*>(ring + STAGES * 16 * AS);  // [WARPS][NT][16][8]: the warps' partial sums
  bf16* xs = reinterpret_cast<bf16*>(red + WARPS * NT * 128);    // [NT * 8][XS]: the tokens' activations, whole K
  const int XS = K + 32;
  __shared__ float ss_s[NT * 8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int F = O / 2;  // swiglu only: O is the stacked height 2F

  // weight row that stage row i of row tile `tile` holds, or -1
  auto weight_row = [&](int tile, int i) -> int {
    if (OUT == OUT_SWIGLU) {
      const int f = tile * 8 + (i & 7);
      return f < F ? (i < 8 ? f : F + f) : -1;
    }
    const int o = tile * 16 + i;
    return o < O ? o : -1;
  };
  const int chunks = (K + KC - 1) / KC;
  // this block's row tiles: blockIdx.x, blockIdx.x + gridDim.x, ...; its work is the sequence of their chunks
  const int my_tiles = (num_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int items = my_tiles * chunks;
  int load_tile = blockIdx.x, load_chunk = 0, loaded = 0;  // the next item whose copies are to be issued
  auto issue_next = [&]() {
    if (loaded < items) {
      const int k0 = load_chunk * KC, len = min(KC, K - k0);
      bf16* dst = ring + (size_t)(loaded % STAGES) * 16 * AS;
      if (len == KC) {  // the common case: two 16-byte copies per thread, no division
#pragma unroll
        for (int i = tid; i < 16 * (KC / 8); i += WARPS * 32) {
          const int row = i / (KC / 8), col = (i % (KC / 8)) * 8;
          const int wr = weight_row(load_tile, row);
          cp_async16(dst + row * AS + col, W + (size_t)max(wr, 0) * K + k0 + col, wr >= 0 ? 16 : 0);
        }
      } else {
        const int per_row = len / 8;
        for (int i = tid; i < 16 * per_row; i += WARPS * 32) {
          const int row = i / per_row, col = (i % per_row) * 8;
          const int wr = weight_row(load_tile, row);
          cp_async16(dst + row * AS + col, W + (size_t)max(wr, 0) * K + k0 + col, wr >= 0 ? 16 : 0);
        }
      }
      ++loaded;
      if (++load_chunk == chunks) { load_chunk = 0; load_tile += gridDim.x; }
    }
    cp_async_commit();
  };

  // The weights do not depend on anything an earlier kernel wrote: their first chunks are requested before
  // this kernel waits for its predecessor, whose tail they overlap.
  chain_release();
#pragma unroll
  for (int c = 0; c < STAGES - 2; ++c) issue_next();
  chain_wait();

  // Activations into shared memory, once per block. bfloat16 input is a cp.async group of its own (empty
  // when the norm rides along), then the last chunk of the prologue follows.
  if (IN == IN_BF16) {
    const int per_row = K / 8;
    for (int i = tid; i < NT * 8 * per_row; i += WARPS * 32) {
      const int m = i / per_row, col = (i % per_row) * 8;
      const size_t src = m < M ? (size_t)(rows ? rows[m] : m) : 0;
      cp_async16(xs + (size_t)m * XS + col, (const bf16*)x_ + src * K + col, m < M ? 16 : 0);
    }
  }
  cp_async_commit();
  issue_next();
  if (IN == IN_NORM) {
    // float32 residual rows -> bf16(x * norm weight); each warp owns tokens warp, warp + 8 and sums x^2
    for (int m = warp; m < NT * 8; m += WARPS) {
      float ss = 0.f;
      bf16* dst = xs + (size_t)m * XS;
      if (m < M) {
        const float* src = (const float*)x_ + (size_t)(rows ? rows[m] : m) * K;
#pragma unroll 8
        for (int k = lane * 4; k < K; k += 128) {
          const float4 v = *reinterpret_cast<const float4*>(src + k);
          float4 w = *reinterpret_cast<const float4*>(norm_w + k);
          if (zero_centered) { w.x += 1.f; w.y += 1.f; w.z += 1.f; w.w += 1.f; }
          ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
          uint2 packed;
          packed.x = pack_bf16(v.x * w.x, v.y * w.y);
          packed.y = pack_bf16(v.z * w.z, v.w * w.w);
          *reinterpret_cast<uint2*>(dst + k) = packed;
        }
        ss = warp_sum(ss);
      } else {
        for (int k = lane * 4; k < K; k += 128) *reinterpret_cast<uint2*>(dst + k) = make_uint2(0u, 0u);
      }
      if (lane == 0) ss_s[m] = ss;
    }
  }

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }

  int tile = blockIdx.x, c = 0;
  for (int n = 0; n < items; ++n) {
    // Groups in flight, oldest first: chunks 0 .. STAGES-3, the activations, chunk STAGES-2, ... The first
    // item waits until only the newest is pending (so the activations are in); later ones keep STAGES-2 going.
    if (n == 0) cp_async_wait<1>(); else cp_async_wait<STAGES - 2>();
    __syncthreads();  // item n (and the activations) are there for everyone; everyone is done with item n - 1
    issue_next();
    const int k = c * KC + warp * 32 + 8 * t;  // this thread's 8 consecutive k of the chunk
    if (k < K) {
      const bf16* st = ring + (size_t)(n % STAGES) * 16 * AS + warp * 32 + 8 * t;
      const uint4 a_lo = *reinterpret_cast<const uint4*>(st + g * AS);
      const uint4 a_hi = *reinterpret_cast<const uint4*>(st + (g + 8) * AS);
      const uint32_t a1[4] = {a_lo.x, a_hi.x, a_lo.y, a_hi.y};  // first k-step: this thread's k 0..3
      const uint32_t a2[4] = {a_lo.z, a_hi.z, a_lo.w, a_hi.w};  // second k-step: its k 4..7
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint4 b = *reinterpret_cast<const uint4*>(xs + (size_t)(8 * j + g) * XS + k);
        mma_bf16(acc[j], a1, b.x, b.y);
        mma_bf16(acc[j], a2, b.z, b.w);
      }
    }
    if (++c < chunks) continue;

    // the row tile is complete: the 8 warps' partial sums meet in shared memory, then the epilogue
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      float* r0 = red + (((size_t)warp * NT + j) * 16 + g) * 8 + 2 * t;
      r0[0] = acc[j][0];
      r0[1] = acc[j][1];
      r0[64] = acc[j][2];  // row g + 8
      r0[65] = acc[j][3];
      acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    }
    __syncthreads();  // (the next write to `red` is a whole item, and so a barrier, away)
    constexpr int per_tile = OUT == OUT_SWIGLU ? 64 : 128;  // (row, token) pairs per n-block
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
        const float inv = 1.f / sqrtf(ss_s[m] / (float)K + eps);
        v *= inv;
        u *= inv;
      }
      if (OUT == OUT_SWIGLU) {
        const int f = tile * 8 + row;
        if (f < F) ((bf16*)y_)[(size_t)m * F + f] = __float2bfloat16_rn(v / (1.f + expf(-v)) * u);
      } else {
        const int o = tile * 16 + row;
        if (o >= O) continue;
        const size_t at = (size_t)m * O + o;
        if (OUT == OUT_BF16) ((bf16*)y_)[at] = __float2bfloat16_rn(v);
        else if (OUT == OUT_F32) ((float*)y_)[at] = v;
        else ((float*)y_)[at] += v;
      }
    }
    c = 0;
    tile += gridDim.x;
  }
  cp_async_wait<0>();
}

constexpr int kMaxSmemBytes = 226 * 1024;  // the block also has a few bytes of static shared memory

template <int NT>
constexpr int fixed_smem() { return STAGES * 16 * AS * (int)sizeof(bf16) + WARPS * NT * 128 * (int)sizeof(float); }

template <int NT, int IN, int OUTM>
int launch_one(int num_tiles, const void* x, const int* rows, const float* norm_w, float eps, int zero_centered,
               const void* W, void* y, int M, int O, int K, cudaStream_t stream) {
  const int smem = fixed_smem<NT>() + NT * 8 * (K + 32) * (int)sizeof(bf16);
  if (smem > kMaxSmemBytes) return (int)cudaErrorInvalidValue;
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<NT, IN, OUTM>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemBytes);
    if (e != cudaSuccess) { sms = 0; return (int)e; }
  }
  const int per_sm = max(1, min(3, kMaxSmemBytes / (smem + 1024)));  // resident blocks per SM by shared memory
  // every block gets the same number of row tiles (to within one): blocks advance at the same rate, so a
  // grid that leaves some blocks with one tile more than others would idle the rest of the GPU meanwhile
  const int rounds = (num_tiles + sms * per_sm - 1) / (sms * per_sm);
  const int grid = (num_tiles + rounds - 1) / rounds;
  return launch_chained(skinny_gemm_kernel<NT, IN, OUTM>, dim3(grid), dim3(WARPS * 32), (size_t)smem, stream, x, rows,
                        norm_w, eps, zero_centered, (const bf16*)W, y, M, O, K, num_tiles);
}

template <int NT, int IN>
int launch_out(int out_mode, const void* x, const int* rows, const float* norm_w, float eps, int zero_centered,
               const void* W, void* y, int M, int O, int K, cudaStream_t stream) {
  const int tiles = (O + 15) / 16;
  switch (out_mode) {
    case OUT_BF16: return launch_one<NT, IN, OUT_BF16>(tiles, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, stream);
    case OUT_F32: return launch_one<NT, IN, OUT_F32>(tiles, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, stream);
    case OUT_ACC: return launch_one<NT, IN, OUT_ACC>(tiles, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, stream);
    case OUT_SWIGLU:
      return launch_one<NT, IN, OUT_SWIGLU>((O / 2 + 7) / 8, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, stream);
    default: return (int)cudaErrorInvalidValue;
  }
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
