// Grouped-query attention over the paged cache, float32 softmax and accumulation.
//
// Pages: [num_pages, kv_heads, page_size, head_dim]; key j of request r lives in page
// block_table[r, j / page_size] at row j % page_size. A query at absolute position p sees keys
// first..p of its own request, first = max(0, p - window + 1) with a window, else 0. The step has
// already written this step's keys, so a prompt portion attends to earlier pages and to itself.
//
// Two kernels:
//  * paged_attention_kernel: one block per (token, query head); works for any mix of portions and
//    decoded tokens. Its warps walk 32-key tiles aligned to absolute position 0, so the sequence
//    of operations for a query does not depend on how the tokens were cut into steps or batched.
//  * decode_splitk_kernel + decode_merge_kernel: for steps that only decode. One block per
//    (token, tile of query heads that share a kv head, split of the keys); the key rows of a kv head
//    are read once for the whole tile of query heads. Partial (acc, max, sum) per split go to scratch
//    and are merged by log-sum-exp.
//
// In both, a lane owns one key of the tile for q.k (the row is read with 16-byte loads, q comes
// from shared memory), and owns head_dim/32 output channels for p.v (p is broadcast by shuffle).
#include <math.h>

#include "common.cuh"

using namespace akas;

#define AKAS_ATT_WARPS 4

struct KeyRange {
  int first_key, first_tile, last_tile;
};

__device__ __forceinline__ KeyRange key_range(int pos, int window) {
  KeyRange k;
  k.first_key = window > 0 ? max(0, pos - window + 1) : 0;
  k.first_tile = k.first_key >> 5;
  k.last_tile = pos >> 5;
  return k;
}

// Row index (in units of head_dim elements) of `key` of request r for kv head kvh, or -1.
__device__ __forceinline__ int key_row(const int* __restrict__ block_table, int max_blocks, int r, int key,
                                       int page_size, int KH, int kvh) {
  const int page = block_table[(size_t)r * max_blocks + key / page_size];
  return page < 0 ? -1 : (page * KH + kvh) * page_size + key % page_size;
}

template <typename T, int NE>
__global__ void __launch_bounds__(AKAS_ATT_WARPS * 32)
paged_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                       const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_of_token,
                       const int* __restrict__ positions, T* __restrict__ out, float scale, int window,
                       int page_size, int H, int KH, int D) {
  __shared__ float q_s[NE * 32];
  __shared__ float acc_s[AKAS_ATT_WARPS][NE * 32];
  __shared__ float m_s[AKAS_ATT_WARPS], l_s[AKAS_ATT_WARPS];
  const int t = blockIdx.x, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = seq_of_token[t];
  T* dst = out + ((size_t)t * H + head) * D;
  if (r < 0) {
    for (int e = threadIdx.x; e < D; e += blockDim.x) dst[e] = from_f32<T>(0.f);
    return;
  }
  const int pos = positions[t];
  const int kvh = head / (H / KH);
  const T* qp = q + ((size_t)t * H + head) * D;
  for (int e = threadIdx.x; e < D; e += blockDim.x) q_s[e] = to_f32(qp[e]);
  __syncthreads();

  const KeyRange range = key_range(pos, window);
  float m = -INFINITY, l = 0.f, acc[NE];
#pragma unroll
  for (int i = 0; i < NE; ++i) acc[i] = 0.f;

  for (int tile = range.first_tile + warp; tile <= range.last_tile; tile += AKAS_ATT_WARPS) {
    const int key = tile * 32 + lane;
    int row = -1;
    float s = -INFINITY;
    if (key >= range.first_key && key <= pos) row = key_row(block_table, max_blocks, r, key, page_size, KH, kvh);
    if (row >= 0) {
      const T* kp = k_pool + (size_t)row * D;
      float dot = 0.f;
      for (int c = 0; c < D; c += Vec<T>::N) {
        float kv[Vec<T>::N];
        load_vec(kp + c, kv);
#pragma unroll
        for (int i = 0; i < Vec<T>::N; ++i) dot = fmaf(q_s[c + i], kv[i], dot);
      }
      s = dot * scale;
    }
    const float tile_max = warp_max(s);
    if (tile_max == -INFINITY) continue;
    const float m_new = fmaxf(m, tile_max);
    const float p = row >= 0 ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < NE; ++i) acc[i] *= corr;
    const int keys = min(32, pos - tile * 32 + 1);
    for (int j = 0; j < keys; ++j) {
      const int rj = __shfl_sync(0xffffffffu, row, j);
      const float pj = __shfl_sync(0xffffffffu, p, j);
      if (rj < 0) continue;
      const T* vp = v_pool + (size_t)rj * D;
#pragma unroll
      for (int i = 0; i < NE; ++i) {
        const int e = lane + 32 * i;
        if (e < D) acc[i] = fmaf(pj, to_f32(vp[e]), acc[i]);
      }
    }
    m = m_new;
  }

  if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
  for (int i = 0; i < NE; ++i) acc_s[warp][lane + 32 * i] = acc[i];
  __syncthreads();
  float top = m_s[0];
#pragma unroll
  for (int w = 1; w < AKAS_ATT_WARPS; ++w) top = fmaxf(top, m_s[w]);
  for (int e = threadIdx.x; e < D; e += blockDim.x) {
    float sum = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < AKAS_ATT_WARPS; ++w) {
      const float f = m_s[w] == -INFINITY ? 0.f : expf(m_s[w] - top);
      sum = fmaf(l_s[w], f, sum);
      o = fmaf(acc_s[w][e], f, o);
    }
    dst[e] = from_f32<T>(o / sum);
  }
}

// Decode: grid (token, kv_head * head_tiles, split). GT query heads of one kv head per block.
template <typename T, int NE, int GT>
__global__ void __launch_bounds__(AKAS_ATT_WARPS * 32)
decode_splitk_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                     const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_of_token,
                     const int* __restrict__ positions, float* __restrict__ part_o, float* __restrict__ part_ml,
                     float scale, int window, int page_size, int H, int KH, int D, int head_tiles, int splits) {
  __shared__ float q_s[GT][NE * 32];
  __shared__ float acc_s[AKAS_ATT_WARPS][GT][NE * 32];
  __shared__ float m_s[AKAS_ATT_WARPS][GT], l_s[AKAS_ATT_WARPS][GT];
  const int t = blockIdx.x, split = blockIdx.z;
  const int kvh = blockIdx.y / head_tiles, head_tile = blockIdx.y % head_tiles;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = seq_of_token[t];
  if (r < 0) return;
  const int G = H / KH;
  const int g0 = head_tile * GT;            // first query head of this tile inside the group
  const int gn = min(GT, G - g0);           // live heads in the tile
  const int pos = positions[t];
  for (int i = threadIdx.x; i < GT * D; i += blockDim.x) {
    const int g = i / D, e = i % D;
    q_s[g][e] = g < gn ? to_f32(q[((size_t)t * H + kvh * G + g0 + g) * D + e]) : 0.f;
  }
  __syncthreads();

  const KeyRange range = key_range(pos, window);
  const int tiles = range.last_tile - range.first_tile + 1;
  const int per_split = (tiles + splits - 1) / splits;
  const int tile_lo = range.first_tile + split * per_split;
  const int tile_hi = min(tile_lo + per_split, range.last_tile + 1);

  float m[GT], l[GT], acc[GT][NE];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < NE; ++i) acc[g][i] = 0.f;
  }

  for (int tile = tile_lo + warp; tile < tile_hi; tile += AKAS_ATT_WARPS) {
    const int key = tile * 32 + lane;
    int row = -1;
    if (key >= range.first_key && key <= pos) row = key_row(block_table, max_blocks, r, key, page_size, KH, kvh);
    float s[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) s[g] = 0.f;
    if (row >= 0) {
      const T* kp = k_pool + (size_t)row * D;
      for (int c = 0; c < D; c += Vec<T>::N) {
        float kv[Vec<T>::N];
        load_vec(kp + c, kv);
#pragma unroll
        for (int g = 0; g < GT; ++g)
#pragma unroll
          for (int i = 0; i < Vec<T>::N; ++i) s[g] = fmaf(q_s[g][c + i], kv[i], s[g]);
      }
    }
    if (__ballot_sync(0xffffffffu, row >= 0) == 0u) continue;
    float p[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      const float sg = row >= 0 ? s[g] * scale : -INFINITY;
      const float m_new = fmaxf(m[g], warp_max(sg));
      p[g] = row >= 0 ? expf(sg - m_new) : 0.f;
      const float corr = expf(m[g] - m_new);
      l[g] = l[g] * corr + warp_sum(p[g]);
#pragma unroll
      for (int i = 0; i < NE; ++i) acc[g][i] *= corr;
      m[g] = m_new;
    }
    const int keys = min(32, pos - tile * 32 + 1);
    for (int j = 0; j < keys; ++j) {
      const int rj = __shfl_sync(0xffffffffu, row, j);
      if (rj < 0) continue;
      const T* vp = v_pool + (size_t)rj * D;
      float v[NE];
#pragma unroll
      for (int i = 0; i < NE; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < D ? to_f32(vp[e]) : 0.f;
      }
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        const float pj = __shfl_sync(0xffffffffu, p[g], j);
#pragma unroll
        for (int i = 0; i < NE; ++i) acc[g][i] = fmaf(pj, v[i], acc[g][i]);
      }
    }
  }

#pragma unroll
  for (int g = 0; g < GT; ++g) {
    if (lane == 0) { m_s[warp][g] = m[g]; l_s[warp][g] = l[g]; }
#pragma unroll
    for (int i = 0; i < NE; ++i) acc_s[warp][g][lane + 32 * i] = acc[g][i];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < gn * D; i += blockDim.x) {
    const int g = i / D, e = i % D;
    float top = m_s[0][g];
#pragma unroll
    for (int w = 1; w < AKAS_ATT_WARPS; ++w) top = fmaxf(top, m_s[w][g]);
    float sum = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < AKAS_ATT_WARPS; ++w) {
      const float f = m_s[w][g] == -INFINITY ? 0.f : expf(m_s[w][g] - top);
      sum = fmaf(l_s[w][g], f, sum);
      o = fmaf(acc_s[w][g][e], f, o);
    }
    const size_t slot = ((size_t)t * H + kvh * G + g0 + g) * splits + split;
    part_o[slot * D + e] = o;
    if (e == 0) { part_ml[slot * 2] = top; part_ml[slot * 2 + 1] = sum; }
  }
}

template <typename T>
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ seq_of_token, T* __restrict__ out, int H, int D,
                                    int splits) {
  const int t = blockIdx.x, head = blockIdx.y;
  T* dst = out + ((size_t)t * H + head) * D;
  if (seq_of_token[t] < 0) {
    for (int e = threadIdx.x; e < D; e += blockDim.x) dst[e] = from_f32<T>(0.f);
    return;
  }
  const size_t base = ((size_t)t * H + head) * splits;
  float top = -INFINITY;
  for (int s = 0; s < splits; ++s) top = fmaxf(top, part_ml[(base + s) * 2]);
  for (int e = threadIdx.x; e < D; e += blockDim.x) {
    float sum = 0.f, o = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = part_ml[(base + s) * 2];
      const float f = ms == -INFINITY ? 0.f : expf(ms - top);
      sum = fmaf(part_ml[(base + s) * 2 + 1], f, sum);
      o = fmaf(part_o[(base + s) * D + e], f, o);
    }
    dst[e] = from_f32<T>(o / sum);
  }
}

template <typename T>
static int launch_generic(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                          int max_blocks, const int* seq_of_token, const int* positions, void* out, float scale,
                          int window, int page_size, int N, int H, int KH, int D, cudaStream_t stream) {
  const dim3 grid(N, H);
  const int threads = AKAS_ATT_WARPS * 32;
#define AKAS_GEN(NE)                                                                                              \
  paged_attention_kernel<T, NE><<<grid, threads, 0, stream>>>((const T*)q, (const T*)k_pool, (const T*)v_pool,    \
                                                              block_table, max_blocks, seq_of_token, positions,   \
                                                              (T*)out, scale, window, page_size, H, KH, D)
  if (D <= 32) AKAS_GEN(1);
  else if (D <= 64) AKAS_GEN(2);
  else if (D <= 128) AKAS_GEN(4);
  else AKAS_GEN(8);
#undef AKAS_GEN
  return launch_status();
}

AKAS_API int akas_paged_attention(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                  int max_blocks, const int* seq_of_token, const int* positions, void* out,
                                  float scale, int window, int page_size, int N, int H, int KH, int D, int dtype,
                                  cudaStream_t stream) {
  if (D <= 0 || D > 256 || D % 16 || H % KH || H > 65535) return (int)cudaErrorInvalidValue;
  if (N <= 0) return 0;
  if (dtype == AKAS_F32)
    return launch_generic<float>(q, k_pool, v_pool, block_table, max_blocks, seq_of_token, positions, out, scale,
                                 window, page_size, N, H, KH, D, stream);
  return launch_generic<bf16>(q, k_pool, v_pool, block_table, max_blocks, seq_of_token, positions, out, scale,
                              window, page_size, N, H, KH, D, stream);
}

template <typename T, int NE>
static int launch_decode(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                         int max_blocks, const int* seq_of_token, const int* positions, void* out, float* part_o,
                         float* part_ml, float scale, int window, int page_size, int N, int H, int KH, int D,
                         int splits, cudaStream_t stream) {
  const int G = H / KH;
  const int gt = G >= 8 ? 8 : G > 2 ? 4 : G;  // 1, 2, 4 or 8 query heads per block
  const int head_tiles = (G + gt - 1) / gt;
  const dim3 grid(N, KH * head_tiles, splits);
  const int threads = AKAS_ATT_WARPS * 32;
#define AKAS_DEC(GT)                                                                                               \
  decode_splitk_kernel<T, NE, GT><<<grid, threads, 0, stream>>>(                                                   \
      (const T*)q, (const T*)k_pool, (const T*)v_pool, block_table, max_blocks, seq_of_token, positions, part_o,   \
      part_ml, scale, window, page_size, H, KH, D, head_tiles, splits)
  if (gt == 1) AKAS_DEC(1);
  else if (gt == 2) AKAS_DEC(2);
  else if (gt == 4) AKAS_DEC(4);
  else AKAS_DEC(8);
#undef AKAS_DEC
  int err = launch_status();
  if (err) return err;
  decode_merge_kernel<T><<<dim3(N, H), 64, 0, stream>>>(part_o, part_ml, seq_of_token, (T*)out, H, D, splits);
  return launch_status();
}

// Scratch: part_o float32 [N, H, splits, D], part_ml float32 [N, H, splits, 2].
AKAS_API int akas_paged_attention_decode(const void* q, const void* k_pool, const void* v_pool,
                                         const int* block_table, int max_blocks, const int* seq_of_token,
                                         const int* positions, void* out, float* part_o, float* part_ml,
                                         float scale, int window, int page_size, int N, int H, int KH, int D,
                                         int splits, int dtype, cudaStream_t stream) {
  if (D <= 0 || D > 256 || D % 16 || H % KH || splits < 1 || splits > 65535 || H > 65535)
    return (int)cudaErrorInvalidValue;
  if (N <= 0) return 0;
#define AKAS_DECODE(T, NE)                                                                                       \
  return launch_decode<T, NE>(q, k_pool, v_pool, block_table, max_blocks, seq_of_token, positions, out, part_o,  \
                              part_ml, scale, window, page_size, N, H, KH, D, splits, stream)
  if (dtype == AKAS_F32) {
    if (D <= 32) AKAS_DECODE(float, 1);
    if (D <= 64) AKAS_DECODE(float, 2);
    if (D <= 128) AKAS_DECODE(float, 4);
    AKAS_DECODE(float, 8);
  }
  if (D <= 32) AKAS_DECODE(bf16, 1);
  if (D <= 64) AKAS_DECODE(bf16, 2);
  if (D <= 128) AKAS_DECODE(bf16, 4);
  AKAS_DECODE(bf16, 8);
#undef AKAS_DECODE
}
