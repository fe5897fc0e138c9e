// float32 matrix product on the CUDA cores: y[N, O] = x[N, K] . w[O, K]^T (+ residual, in place).
//
// This is the 32-bit path's product: plain FFMA, no tensor cores, no reduced-precision mode. Each
// output element is one chain of fused multiply-adds over k = 0 .. K-1 in ascending order, whatever
// the tile shape and however many rows the launch has, so a row's result does not depend on what
// else is in the batch (bitwise). Both operands are contiguous along K.
//
// Tiles BM x BN x 16 through shared memory (stored k-major so the inner loop reads vectors), each
// thread a TM x TN micro-tile. Three shapes: 128x128 (8x8) for prompts, 32x64 (2x4) and 16x64 (1x4)
// for few rows; and a kernel of its own for up to 16 rows against a wide w, which streams w once. kreasof-ai/akas's plain float32 `linear` is a per-row tree reduction
// (src/akas/ops/linear/kernel.py:403-447).
#include "common.cuh"

using namespace akas;

#define AKAS_BK 16

template <int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
sgemm_tn_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                const float* __restrict__ residual, int N, int O, int K, int vec_ok) {
  constexpr int NT = (BM / TM) * (BN / TN);
  __shared__ float As[AKAS_BK][BM + 4];
  __shared__ float Bs[AKAS_BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += AKAS_BK) {
    // each tile row has AKAS_BK / 4 = 4 groups of four consecutive k
    for (int i = tid; i < BM * (AKAS_BK / 4); i += NT) {
      const int r = i / (AKAS_BK / 4), kq = (i % (AKAS_BK / 4)) * 4;
      const int gr = row0 + r, gk = k0 + kq;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (gr < N) {
        const float* p = x + (size_t)gr * K + gk;
        if (vec_ok && gk + 3 < K) {
          const float4 f = *reinterpret_cast<const float4*>(p);
          v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (gk + j < K) v[j] = p[j];
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) As[kq + j][r] = v[j];
    }
    for (int i = tid; i < BN * (AKAS_BK / 4); i += NT) {
      const int r = i / (AKAS_BK / 4), kq = (i % (AKAS_BK / 4)) * 4;
      const int gr = col0 + r, gk = k0 + kq;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (gr < O) {
        const float* p = w + (size_t)gr * K + gk;
        if (vec_ok && gk + 3 < K) {
          const float4 f = *reinterpret_cast<const float4*>(p);
          v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (gk + j < K) v[j] = p[j];
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) Bs[kq + j][r] = v[j];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < AKAS_BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gr = row0 + ty * TM + i;
    if (gr >= N) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gc = col0 + tx * TN + j;
      if (gc >= O) continue;
      const size_t at = (size_t)gr * O + gc;
      y[at] = residual ? residual[at] + acc[i][j] : acc[i][j];
    }
  }
}

// A handful of rows (decode steps): the time goes to reading w once. A block owns 32 rows of w (32 output
// channels): its 128 threads fetch them 64 k at a time with coalesced 16-byte loads into a double-buffered
// shared-memory tile (the next tile is on its way while the current one is multiplied); then lane l of every warp
// reads row l of the tile, and the block's four warps split the tokens. x is staged in shared memory 256 k at a
// time and read from there by broadcast. Each output is the same ascending chain of fused multiply-adds as in the
// tiled kernel above, so the two give the same bits.
template <int TOK>  // tokens per thread; the block's 4 warps cover 4 * TOK tokens
__global__ void __launch_bounds__(128)
sgemm_few_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                 const float* __restrict__ residual, int N, int O, int K) {
  constexpr int KC = 256, KS = 64, PITCH = KS + 4;  // rows of the tile 16-byte aligned and conflict-free to read
  __shared__ __align__(16) float xs[4 * TOK][KC];
  __shared__ __align__(16) float tile[2][32][PITCH];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = blockIdx.x * 32;
  const int load_row = tid >> 4, load_k = (tid & 15) * 4;  // this thread's 16 bytes of rows load_row + 8 j
  float acc[TOK];
#pragma unroll
  for (int i = 0; i < TOK; ++i) acc[i] = 0.f;

  float4 next[4];
  auto fetch = [&](int k) {  // the tile that starts at column k of w (a multiple of 64)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = row0 + load_row + 8 * j;
      next[j] = (r < O && k + load_k < K) ? *reinterpret_cast<const float4*>(w + (size_t)r * K + k + load_k)
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  auto put = [&](int buffer) {
#pragma unroll
    for (int j = 0; j < 4; ++j) *reinterpret_cast<float4*>(&tile[buffer][load_row + 8 * j][load_k]) = next[j];
  };

  fetch(0);
  int buffer = 0;
  for (int k0 = 0; k0 < K; k0 += KC) {
    __syncthreads();  // the last chunk's x has been read
    for (int i = tid; i < 4 * TOK * (KC / 4); i += 128) {
      const int t = i / (KC / 4), q = (i % (KC / 4)) * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t < N && k0 + q < K) v = *reinterpret_cast<const float4*>(x + (size_t)t * K + k0 + q);
      *reinterpret_cast<float4*>(&xs[t][q]) = v;
    }
    for (int q0 = 0; q0 < KC && k0 + q0 < K; q0 += KS) {
      put(buffer);
      __syncthreads();  // the tile (and, the first time, x) is in shared memory
      if (k0 + q0 + KS < K) fetch(k0 + q0 + KS);
#pragma unroll 4
      for (int kk = 0; kk < KS; kk += 4) {
        const float4 wv = *reinterpret_cast<const float4*>(&tile[buffer][lane][kk]);
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
          const float4 xv = *reinterpret_cast<const float4*>(&xs[warp * TOK + i][q0 + kk]);
          acc[i] = fmaf(xv.x, wv.x, acc[i]);
          acc[i] = fmaf(xv.y, wv.y, acc[i]);
          acc[i] = fmaf(xv.z, wv.z, acc[i]);
          acc[i] = fmaf(xv.w, wv.w, acc[i]);
        }
      }
      buffer ^= 1;
    }
  }
  const int row = row0 + lane;
  if (row >= O) return;
#pragma unroll
  for (int i = 0; i < TOK; ++i) {
    const int t = warp * TOK + i;
    if (t >= N) continue;
    const size_t at = (size_t)t * O + row;
    y[at] = residual ? residual[at] + acc[i] : acc[i];
  }
}

// residual may alias y (in-place accumulation into the residual stream) or be null.
AKAS_API int akas_sgemm(const float* x, const float* w, float* y, const float* residual, int N, int O, int K,
                        cudaStream_t stream) {
  if (N <= 0 || O <= 0) return 0;
  if (K <= 0) return (int)cudaErrorInvalidValue;
  const int vec_ok = (K % 4 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0);
  if (N <= 16 && vec_ok && O >= 256) {
    const dim3 grid((O + 31) / 32);
    if (N <= 4) sgemm_few_kernel<1><<<grid, 128, 0, stream>>>(x, w, y, residual, N, O, K);
    else if (N <= 8) sgemm_few_kernel<2><<<grid, 128, 0, stream>>>(x, w, y, residual, N, O, K);
    else sgemm_few_kernel<4><<<grid, 128, 0, stream>>>(x, w, y, residual, N, O, K);
  } else if (N > 64) {
    const dim3 grid((O + 127) / 128, (N + 127) / 128);
    sgemm_tn_kernel<128, 128, 8, 8><<<grid, 256, 0, stream>>>(x, w, y, residual, N, O, K, vec_ok);
  } else if (N > 16) {
    const dim3 grid((O + 63) / 64, (N + 31) / 32);
    sgemm_tn_kernel<32, 64, 2, 4><<<grid, 256, 0, stream>>>(x, w, y, residual, N, O, K, vec_ok);
  } else {
    const dim3 grid((O + 63) / 64, 1);
    sgemm_tn_kernel<16, 64, 1, 4><<<grid, 256, 0, stream>>>(x, w, y, residual, N, O, K, vec_ok);
  }
  return launch_status();
}
