// Paged GQA attention for prompt portions in bfloat16 on the tensor cores (flash-attention style).
//
// One block per (tile of 64 consecutive query tokens of one request, query head); 4 warps, each
// owning 16 query rows. The block walks 64-key tiles aligned to absolute position 0, from the first
// key any of its queries may see to its last query's own position; K and V rows are fetched from the
// pages with 16-byte cp.async copies (row by row through the block table, so any page size works;
// rows beyond the visible range are zero-filled), two tiles in flight. S = Q.K^T and O += P.V run as
// mma.sync m16n8k16 (bf16 in, float32 accumulate) with fragments read by ldmatrix from padded shared
// memory; scale, causal/window mask, running max and sum are float32 in registers; P is rounded to
// bfloat16 for the second product, as the values it multiplies are.
//
// Tiles are found on the device: a block scans cu_seqlens for the request whose tiles contain its tile number.
// Head sizes 16, 32, 64 and 128; others use the general kernel in attention.cu.
#include <math.h>

#include "common.cuh"
#include "mma.cuh"

using namespace akas;

namespace {

constexpr int BQ = 64, BK = 64, WARPS = 4;

template <int D>
__global__ void __launch_bounds__(WARPS * 32)
prefill_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_seqlens,
                         const int* __restrict__ positions, bf16* __restrict__ out, float scale, int window,
                         int page_size, int H, int KH, int R) {
  constexpr int STRIDE = D + 8;         // elements per shared row: 16 bytes of padding keep ldmatrix conflict-free
  constexpr int CHUNKS = D / 8;         // 16-byte chunks per row
  constexpr int KS = D / 16;            // k-steps of Q.K^T
  constexpr int NB = D / 8;             // 8-wide output blocks of P.V
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* k_s = reinterpret_cast<bf16*>(smem_raw);          // [2][BK][STRIDE]; stage 0 first holds Q
  bf16* v_s = k_s + 2 * BK * STRIDE;                      // [2][BK][STRIDE]

  // Which tile of which request is this block? Blocks are handed out with x fastest, so heads are x and tiles y,
  // last tile first: the tiles with the most keys to walk (the ends of long portions) start first and the short
  // ones fill the tail.
  int tile = (int)gridDim.y - 1 - (int)blockIdx.y, r = 0, n = 0;
  for (; r < R; ++r) {
    n = cu_seqlens[r + 1] - cu_seqlens[r];
    const int tiles = (n + BQ - 1) / BQ;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (r >= R) return;
  const int head = blockIdx.x, kvh = head / (H / KH);
  const int q0 = cu_seqlens[r] + tile * BQ;
  const int rows = min(BQ, n - tile * BQ);
  const int pos0 = positions[q0];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;

  // Q tile -> shared (rows beyond the tile are zero) -> A fragments in registers
  for (int c = tid; c < BQ * CHUNKS; c += WARPS * 32) {
    const int row = c / CHUNKS, col = (c % CHUNKS) * 8;
    const bf16* src = q + ((size_t)(q0 + min(row, rows - 1)) * H + head) * D + col;
    cp_async16(k_s + row * STRIDE + col, src, row < rows ? 16 : 0);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
    ldmatrix_x4(qf[ks], k_s + (warp * 16 + (lane & 15)) * STRIDE + ks * 16 + (lane >> 4) * 8);
  __syncthreads();

  const int last_key = pos0 + rows - 1;
  const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int kt0 = first_key / BK, kt1 = last_key / BK;

  auto load_tile = [&](int kt, int stage) {
    bf16* ks_ = k_s + stage * BK * STRIDE;
    bf16* vs_ = v_s + stage * BK * STRIDE;
    for (int c = tid; c < BK * CHUNKS; c += WARPS * 32) {
      const int row = c / CHUNKS, col = (c % CHUNKS) * 8;
      const int key = kt * BK + row;
      size_t at = 0;
      int bytes = 0;
      if (key >= first_key && key <= last_key) {
        const int page = block_table[(size_t)r * max_blocks + key / page_size];
        if (page >= 0) {
          at = (((size_t)page * KH + kvh) * page_size + key % page_size) * D + col;
          bytes = 16;
        }
      }
      cp_async16(ks_ + row * STRIDE + col, k_pool + at, bytes);
      cp_async16(vs_ + row * STRIDE + col, v_pool + at, bytes);
    }
    cp_async_commit();
  };

  float o[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) { o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl2 = scale * 1.4426950408889634f;  // scores are kept in units of log2(e) so that exp is exp2
  const int qpos[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};

  load_tile(kt0, 0);
  for (int kt = kt0; kt <= kt1; ++kt) {
    const int stage = (kt - kt0) & 1;
    if (kt < kt1) {
      load_tile(kt + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* ks_ = k_s + stage * BK * STRIDE;
    const bf16* vs_ = v_s + stage * BK * STRIDE;

    // S = Q.K^T for this warp's 16 rows and the tile's 64 keys
    float s[BK / 8][4];
#pragma unroll
    for (int nb = 0; nb < BK / 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int np = 0; np < BK / 16; ++np) {  // two 8-key blocks per ldmatrix
        uint32_t b[4];
        ldmatrix_x4(b, ks_ + (np * 16 + (lane & 7) + (lane >> 4) * 8) * STRIDE + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
        mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
      }
    }

    // scale, mask by absolute position, running softmax (rows g and g + 8 of the warp's 16). Most tiles lie
    // wholly before every query of the warp (and inside every window): those need no mask.
    float m_new[2] = {m_run[0], m_run[1]};
    const int warp_first = pos0 + warp * 16, warp_last = warp_first + 15;
    const bool whole = kt * BK + BK - 1 <= warp_first && (window <= 0 || kt * BK > warp_last - window);
    if (whole) {
#pragma unroll
      for (int nb = 0; nb < BK / 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[nb][e] *= sl2;
          m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nb][e]);
        }
      }
    } else {
#pragma unroll
      for (int nb = 0; nb < BK / 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = kt * BK + nb * 8 + 2 * t + (e & 1);
          const int qp = qpos[e >> 1];
          const bool seen = key <= qp && (window <= 0 || key > qp - window);
          s[nb][e] = seen ? s[nb][e] * sl2 : -INFINITY;
          m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nb][e]);
        }
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      m_new[h2] = fmaxf(m_new[h2], __shfl_xor_sync(0xffffffffu, m_new[h2], 1));
      m_new[h2] = fmaxf(m_new[h2], __shfl_xor_sync(0xffffffffu, m_new[h2], 2));
      m_use[h2] = m_new[h2] == -INFINITY ? 0.f : m_new[h2];  // a row that sees nothing yet
      corr[h2] = fast_exp2(m_run[h2] - m_use[h2]);
      m_run[h2] = m_new[h2];
    }
    float l_add[2] = {0.f, 0.f};
    uint32_t pf[BK / 16][4];
#pragma unroll
    for (int nb = 0; nb < BK / 8; ++nb) {
      const float p0 = fast_exp2(s[nb][0] - m_use[0]), p1 = fast_exp2(s[nb][1] - m_use[0]);
      const float p2 = fast_exp2(s[nb][2] - m_use[1]), p3 = fast_exp2(s[nb][3] - m_use[1]);
      l_add[0] += p0 + p1;
      l_add[1] += p2 + p3;
      pf[nb >> 1][(nb & 1) * 2] = pack_bf16(p0, p1);
      pf[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) l_run[h2] = l_run[h2] * corr[h2] + l_add[h2];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      o[nb][0] *= corr[0]; o[nb][1] *= corr[0];
      o[nb][2] *= corr[1]; o[nb][3] *= corr[1];
    }

    // O += P.V
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < NB / 2; ++np) {  // two 8-wide output blocks per ldmatrix
        uint32_t b[4];
        ldmatrix_x4_trans(b, vs_ + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + np * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * np], pf[kk], b[0], b[1]);
        mma_bf16(o[2 * np + 1], pf[kk], b[2], b[3]);
      }
    }
    __syncthreads();  // everyone is done with this stage before the next load overwrites it
  }

  // the row sums were accumulated per thread: add the four threads of a row, then normalise and store
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
    l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
  }
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    const int row = warp * 16 + g + h2 * 8;
    if (row >= rows) continue;
    const float inv = 1.f / l_run[h2];
    bf16* dst = out + ((size_t)(q0 + row) * H + head) * D;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
      *reinterpret_cast<uint32_t*>(dst + nb * 8 + 2 * t) = pack_bf16(o[nb][h2 * 2] * inv, o[nb][h2 * 2 + 1] * inv);
  }
}

template <int D>
int launch(const void* q, const void* k_pool, const void* v_pool, const int* block_table, int max_blocks,
           const int* cu_seqlens, const int* positions, void* out, float scale, int window, int page_size, int tiles,
           int H, int KH, int R, cudaStream_t stream) {
  constexpr int smem = 4 * BK * (D + 8) * (int)sizeof(bf16);
  static bool configured[64] = {};  // by device ordinal: the attribute belongs to a device's copy of the kernel
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  if (!configured[device]) {
    const cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured[device] = true;
  }
  prefill_attention_kernel<D><<<dim3(H, tiles), WARPS * 32, smem, stream>>>(
      (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table, max_blocks, cu_seqlens, positions,
      (bf16*)out, scale, window, page_size, H, KH, R);
  return launch_status();
}

}  // namespace

// tiles: sum over requests of ceil(tokens / 64). Returns cudaErrorInvalidValue for a head size it does not take.
AKAS_API int akas_prefill_attention_bf16(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                         int max_blocks, const int* cu_seqlens, const int* positions, void* out,
                                         float scale, int window, int page_size, int tiles, int H, int KH, int D, int R,
                                         cudaStream_t stream) {
  if (H % KH || tiles > 65535 || R <= 0) return (int)cudaErrorInvalidValue;
  if (tiles <= 0) return 0;
#define AKAS_PREFILL(DD)                                                                                          \
  case DD:                                                                                                        \
    return launch<DD>(q, k_pool, v_pool, block_table, max_blocks, cu_seqlens, positions, out, scale, window,      \
                      page_size, tiles, H, KH, R, stream)
  switch (D) {
    AKAS_PREFILL(16);
    AKAS_PREFILL(32);
    AKAS_PREFILL(64);
    AKAS_PREFILL(128);
    default:
      return (int)cudaErrorInvalidValue;
  }
#undef AKAS_PREFILL
}
