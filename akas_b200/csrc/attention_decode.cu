// Paged GQA attention for steps that only decode, bfloat16, keys split across blocks (flash-decoding).
//
// One block per (token, kv head x tile of up to 16 query heads of its group, split of the keys). The
// query heads that share a kv head are the rows of one mma tile (rows beyond the group are zero), so
// the K and V rows of a kv head are read once for the whole group. The block's share of the 64-key
// tiles is streamed through a three-stage cp.async pipeline (48 KB of loads in flight per block at
// head size 64); in every tile each of the 4 warps takes 16 of the 64 keys: S = Q.K^T (mma.sync
// m16n8k16), mask by absolute position, running max/sum in float32, O += P.V. At the end the four
// warps' (max, sum, O) are merged through shared memory. With one split the block writes the output;
// otherwise it writes float32 partials [token, head, split] (+ max and sum), which
// decode_merge_bf16_kernel combines by log-sum-exp.
//
// Launch shapes depend only on (tokens, heads, splits); lengths are read on the device, so the
// kernel can sit in a captured graph. Tokens of request -1 (padding) write zeros and touch no page.
#include <math.h>

#include "common.cuh"
#include "qk_prep.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"

using namespace akas;

namespace {

constexpr int BK = 64, WARPS = 4, STAGES = 3, ROWS = 16;

template <int D>
__global__ void __launch_bounds__(WARPS * 32)
decode_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_of_token,
                        const int* __restrict__ positions, bf16* __restrict__ out, float* __restrict__ part_o,
                        float* __restrict__ part_ml, float scale, int window, int page_size, int H, int KH,
                        int row_tiles, int splits) {
  constexpr int STRIDE = D + 8, CHUNKS = D / 8, KS = D / 16, NB = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);        // [ROWS][STRIDE]
  bf16* k_s = q_s + ROWS * STRIDE;                      // [STAGES][BK][STRIDE]
  bf16* v_s = k_s + STAGES * BK * STRIDE;               // [STAGES][BK][STRIDE]

  chain_release();
  chain_wait();
  const int tok = blockIdx.x, split = blockIdx.z;
  const int kvh = blockIdx.y / row_tiles, row_tile = blockIdx.y % row_tiles;
  const int G = H / KH;
  const int g0 = row_tile * ROWS, gn = min(ROWS, G - g0);
  const int head0 = kvh * G + g0;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int r = seq_of_token[tok];
  if (r < 0) {
    if (split == 0)
      for (int i = tid; i < gn * D; i += WARPS * 32) out[((size_t)tok * H + head0) * D + i] = __float2bfloat16_rn(0.f);
    return;
  }
  const int pos = positions[tok];
  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  const int kt_first = first_key / BK, kt_last = pos / BK;
  const int tiles = kt_last - kt_first + 1;
  const int per_split = (tiles + splits - 1) / splits;
  const int lo = kt_first + split * per_split, hi = min(lo + per_split, kt_last + 1);

  // A thread copies the same 16-byte column of rows tid / CHUNKS, + 128 / CHUNKS, ... of every tile. When pages hold
  // whole tiles (page size a multiple of 64) a tile needs one look-up in the block table; else one per row.
  constexpr int ROWS_PER_PASS = WARPS * 32 / CHUNKS;
  const int my_row = tid / CHUNKS, my_col = (tid % CHUNKS) * 8;
  const bool whole_pages = page_size % BK == 0;
  auto load_tile = [&](int kt, int stage) {
    bf16* ks_ = k_s + stage * BK * STRIDE + my_col;
    bf16* vs_ = v_s + stage * BK * STRIDE + my_col;
    const int key0 = kt * BK;
    long long tile_row = -1;  // first pool row of the tile (in rows of D elements), if one page holds it
    if (whole_pages) {
      const int page = block_table[(size_t)r * max_blocks + key0 / page_size];
      if (page >= 0) tile_row = ((long long)page * KH + kvh) * page_size + key0 % page_size;
    }
#pragma unroll
    for (int row = my_row; row < BK; row += ROWS_PER_PASS) {
      const int key = key0 + row;
      size_t at = 0;
      int bytes = 0;
      if (key >= first_key && key <= pos) {
        if (whole_pages) {
          if (tile_row >= 0) { at = (size_t)(tile_row + row) * D + my_col; bytes = 16; }
        } else {
          const int page = block_table[(size_t)r * max_blocks + key / page_size];
          if (page >= 0) { at = (((size_t)page * KH + kvh) * page_size + key % page_size) * D + my_col; bytes = 16; }
        }
      }
      cp_async16(ks_ + row * STRIDE, k_pool + at, bytes);
      cp_async16(vs_ + row * STRIDE, v_pool + at, bytes);
    }
  };

  // Q rows (one per query head of the group) and the first tiles, all in flight together
  for (int c = tid; c < ROWS * CHUNKS; c += WARPS * 32) {
    const int row = c / CHUNKS, col = (c % CHUNKS) * 8;
    const bf16* src = q + ((size_t)tok * H + head0 + min(row, gn - 1)) * D + col;
    cp_async16(q_s + row * STRIDE + col, src, row < gn ? 16 : 0);
  }
  cp_async_commit();
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (lo + s < hi) load_tile(lo + s, s);
    cp_async_commit();
  }

  float o[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) { o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl2 = scale * 1.4426950408889634f;
  uint32_t qf[KS][4];

  for (int kt = lo; kt < hi; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (kt == lo) {
#pragma unroll
      for (int ks = 0; ks < KS; ++ks)
        ldmatrix_x4(qf[ks], q_s + (lane & 15) * STRIDE + ks * 16 + (lane >> 4) * 8);
    }
    const int next = kt + STAGES - 1;
    if (next < hi) load_tile(next, (next - lo) % STAGES);
    cp_async_commit();
    const int stage = (kt - lo) % STAGES;
    const bf16* ks_ = k_s + stage * BK * STRIDE + warp * 16 * STRIDE;  // this warp's 16 keys of the tile
    const bf16* vs_ = v_s + stage * BK * STRIDE + warp * 16 * STRIDE;

    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t b[4];
      ldmatrix_x4(b, ks_ + ((lane & 7) + (lane >> 4) * 8) * STRIDE + ks * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(s[0], qf[ks], b[0], b[1]);
      mma_bf16(s[1], qf[ks], b[2], b[3]);
    }
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kt * BK + warp * 16 + nb * 8 + 2 * t + (e & 1);
        const bool seen = key <= pos && key >= first_key;
        s[nb][e] = seen ? s[nb][e] * sl2 : -INFINITY;
        m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nb][e]);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      m_new[h2] = fmaxf(m_new[h2], __shfl_xor_sync(0xffffffffu, m_new[h2], 1));
      m_new[h2] = fmaxf(m_new[h2], __shfl_xor_sync(0xffffffffu, m_new[h2], 2));
      m_use[h2] = m_new[h2] == -INFINITY ? 0.f : m_new[h2];
      corr[h2] = exp2f(m_run[h2] - m_use[h2]);
      m_run[h2] = m_new[h2];
    }
    uint32_t pf[4];
    float l_add[2] = {0.f, 0.f};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      const float p0 = exp2f(s[nb][0] - m_use[0]), p1 = exp2f(s[nb][1] - m_use[0]);
      const float p2 = exp2f(s[nb][2] - m_use[1]), p3 = exp2f(s[nb][3] - m_use[1]);
      l_add[0] += p0 + p1;
      l_add[1] += p2 + p3;
      pf[nb * 2] = pack_bf16(p0, p1);
      pf[nb * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) l_run[h2] = l_run[h2] * corr[h2] + l_add[h2];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      o[nb][0] *= corr[0]; o[nb][1] *= corr[0];
      o[nb][2] *= corr[1]; o[nb][3] *= corr[1];
    }
#pragma unroll
    for (int np = 0; np < NB / 2; ++np) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, vs_ + ((lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + np * 16 + (lane >> 4) * 8);
      mma_bf16(o[2 * np], pf, b[0], b[1]);
      mma_bf16(o[2 * np + 1], pf, b[2], b[3]);
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // all warps are done with the tiles: the stages become the merge buffers

  // merge the four warps: (m, l) per row and O[16][D] per warp, in float32 through shared memory
  float* o_s = reinterpret_cast<float*>(k_s);            // [WARPS][ROWS][D]
  float* ml_s = o_s + WARPS * ROWS * D;                  // [WARPS][ROWS][2]
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
    l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
    const int row = g + h2 * 8;
    if (t == 0) {
      ml_s[(warp * ROWS + row) * 2] = m_run[h2];
      ml_s[(warp * ROWS + row) * 2 + 1] = l_run[h2];
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float* dst = o_s + ((size_t)warp * ROWS + row) * D + nb * 8 + 2 * t;
      dst[0] = o[nb][h2 * 2];
      dst[1] = o[nb][h2 * 2 + 1];
    }
  }
  __syncthreads();
  for (int i = tid; i < gn * D; i += WARPS * 32) {
    const int row = i / D, e = i % D;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) top = fmaxf(top, ml_s[(w * ROWS + row) * 2]);
    float sum = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float mw = ml_s[(w * ROWS + row) * 2];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - top);
      sum = fmaf(ml_s[(w * ROWS + row) * 2 + 1], f, sum);
      acc = fmaf(o_s[((size_t)w * ROWS + row) * D + e], f, acc);
    }
    const size_t head = (size_t)tok * H + head0 + row;
    if (splits == 1) {
      out[head * D + e] = __float2bfloat16_rn(acc / sum);
    } else {
      part_o[(head * splits + split) * D + e] = acc;
      if (e == 0) {
        part_ml[(head * splits + split) * 2] = top;  // in units of log2(e)
        part_ml[(head * splits + split) * 2 + 1] = sum;
      }
    }
  }
}

__global__ void decode_merge_bf16_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         const int* __restrict__ seq_of_token, bf16* __restrict__ out, int H, int D,
                                         int splits) {
  chain_release();
  chain_wait();
  const int tok = blockIdx.x, head = blockIdx.y;
  if (seq_of_token[tok] < 0) return;  // the split kernel wrote the zeros
  const size_t base = ((size_t)tok * H + head) * splits;
  float top = -INFINITY;
  for (int s = 0; s < splits; ++s) top = fmaxf(top, part_ml[(base + s) * 2]);
  for (int e = threadIdx.x; e < D; e += blockDim.x) {
    float sum = 0.f, acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = part_ml[(base + s) * 2];
      const float f = ms == -INFINITY ? 0.f : exp2f(ms - top);
      sum = fmaf(part_ml[(base + s) * 2 + 1], f, sum);
      acc = fmaf(part_o[(base + s) * D + e], f, acc);
    }
    out[((size_t)tok * H + head) * D + e] = __float2bfloat16_rn(acc / sum);
  }
}

// The same for head size 64 and pages that hold whole 64-key tiles, with the K and V tiles fetched by TMA: a fifth
// warp's one thread issues two tensor loads per tile (128-byte swizzle) into a four-stage ring guarded by "full" and
// "empty" mbarriers, instead of every thread computing addresses and issuing eight 16-byte copies per tile; the four
// consumer warps read their fragments from the swizzled tiles. Rows of V past the request's position are zeroed in
// shared memory (a page may hold anything there, and nothing may meet a zero probability as NaN). Waits are bounded
// (akas_decode_attention_status).
constexpr int TMA_STAGES = 4, TMA_TILE = BK * 128;  // a tile: 64 rows of 64 bfloat16

__device__ int g_decode_status = 0;

// The address of a shared-memory location of block `rank` of this cluster, and a store there.
__device__ __forceinline__ unsigned peer_address(const void* local, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(akas::tc::smem_u32(local)), "r"(rank));
  return r;
}
__device__ __forceinline__ void peer_store(unsigned address, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(address), "f"(v) : "memory");
}

// One 64-key tile (128-byte rows in the swizzle that TMA wrote) against a warp's query fragments, head size 64: the
// warp takes 16 of the tile's keys (scores, the running maximum and sum in units of log2(e), probabilities times V).
// UPPER: rows 8..15 of the query tile are alive (more than 8 query heads per KV head); without it their softmax is
// left out. edge: the tile may hold keys that the token does not see (past its position, before its window); other
// tiles skip the comparisons. The accumulators are rescaled only when some row's maximum moved (the factor is
// exactly 1 otherwise), which after the first tiles is rare.
template <bool UPPER>
__device__ __forceinline__ void attend_tile64(const unsigned char* kt_, const unsigned char* vt_, const uint32_t (&qf)[4][4],
                                              float (&o)[8][4], float (&m_run)[2], float (&l_run)[2], int kt, int pos,
                                              int first_key, float sl2, bool edge, int warp, int lane) {
  constexpr int KS = 4, NB = 8, HALVES = UPPER ? 2 : 1, LIVE = UPPER ? 4 : 2;
  const int t = lane & 3;
  // this lane's rows inside the warp's 16 keys of a tile, and the 16-byte units it reads there
  const int k_row = warp * 16 + (lane & 7) + (lane >> 4) * 8, k_unit = (lane >> 3) & 1;
  const int v_row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, v_unit = lane >> 4;
  float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    uint32_t b[4];
    ldmatrix_x4(b, kt_ + k_row * 128 + (((ks * 2 + k_unit) ^ (k_row & 7)) << 4));
    mma_bf16(sc[0], qf[ks], b[0], b[1]);
    mma_bf16(sc[1], qf[ks], b[2], b[3]);
  }
  float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
  for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
    for (int e = 0; e < LIVE; ++e) {
      bool seen = true;
      if (edge) {
        const int key = kt * BK + warp * 16 + nb * 8 + 2 * t + (e & 1);
        seen = key <= pos && key >= first_key;
      }
      sc[nb][e] = seen ? sc[nb][e] * sl2 : -INFINITY;
      m_new[e >> 1] = fmaxf(m_new[e >> 1], sc[nb][e]);
    }
  }
  float m_use[2] = {0.f, 0.f};
  bool moved = false;
#pragma unroll
  for (int h2 = 0; h2 < HALVES; ++h2) {
    m_new[h2] = fmaxf(m_new[h2], __shfl_xor_sync(0xffffffffu, m_new[h2], 1));
    m_new[h2] = fmaxf(m_new[h2], __shfl_xor_sync(0xffffffffu, m_new[h2], 2));
    m_use[h2] = m_new[h2] == -INFINITY ? 0.f : m_new[h2];
    moved = moved || m_new[h2] != m_run[h2];
  }
  if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
    for (int h2 = 0; h2 < HALVES; ++h2) {
      const float corr = exp2f(m_run[h2] - m_use[h2]);
      m_run[h2] = m_new[h2];
      l_run[h2] *= corr;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) { o[nb][h2 * 2] *= corr; o[nb][h2 * 2 + 1] *= corr; }
    }
  }
  uint32_t pf[4] = {0u, 0u, 0u, 0u};
#pragma unroll
  for (int nb = 0; nb < 2; ++nb) {
    const float p0 = exp2f(sc[nb][0] - m_use[0]), p1 = exp2f(sc[nb][1] - m_use[0]);
    l_run[0] += p0 + p1;
    pf[nb * 2] = pack_bf16(p0, p1);
    if (UPPER) {
      const float p2 = exp2f(sc[nb][2] - m_use[1]), p3 = exp2f(sc[nb][3] - m_use[1]);
      l_run[1] += p2 + p3;
      pf[nb * 2 + 1] = pack_bf16(p2, p3);
    }
  }
#pragma unroll
  for (int np = 0; np < NB / 2; ++np) {
    uint32_t b[4];
    ldmatrix_x4_trans(b, vt_ + v_row * 128 + (((np * 2 + v_unit) ^ (v_row & 7)) << 4));
    mma_bf16(o[2 * np], pf, b[0], b[1]);
    mma_bf16(o[2 * np + 1], pf, b[2], b[3]);
  }
}

// The token's own q, k and v as the qkv product left them, [N, (H + 2 KH) * 64], for a kernel that does what lies
// between that product and attention itself: the per-head RMSNorm and rotation of q (every block, for its own rows,
// on the way into shared memory) and of k, and the write of k and v into the pages. The block that holds the last key
// tile does the latter and puts the two rows into its tile in shared memory as well, since its TMA load may have read
// the page before the write landed. With qkv == nullptr, q is ready and the pages hold the token already.
struct Fresh {
  const bf16* qkv;
  const float* q_w;    // the norms' weights over a head (nullptr: no norm)
  const float* k_w;
  float eps;
  int zero_centered;
  const float* cos_t;  // [N, rotary / 2] each (nullptr: no rotation)
  const float* sin_t;
  int rotary;
  bf16* k_pool;        // nullptr: a layer that only reads the pages; they are attended as they are
  bf16* v_pool;
};

__global__ void __launch_bounds__((WARPS + 1) * 32)
decode_attention_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const bf16* __restrict__ q, const int* __restrict__ block_table, int max_blocks,
                            const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                            bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, float scale,
                            int window, int page_size, int H, int KH, int row_tiles, int splits, int in_cluster,
                            const Fresh fresh) {
  // in_cluster: the blocks of a (token, KV head)'s key parts form a thread-block cluster; their partial results meet in
  // the first block's shared memory and that block writes the output, instead of a second kernel over global scratch.
  using namespace akas::tc;
  constexpr int D = 64, STRIDE = D + 8, CHUNKS = D / 8, KS = D / 16, NB = D / 8;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* k_t = tiles;                              // [TMA_STAGES][64 keys][128 bytes], swizzled
  unsigned char* v_t = k_t + TMA_STAGES * TMA_TILE;        // [TMA_STAGES][64 keys][128 bytes], swizzled
  bf16* q_s = reinterpret_cast<bf16*>(v_t + TMA_STAGES * TMA_TILE);  // [ROWS][STRIDE]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(q_s + ROWS * STRIDE);
  uint64_t* empty_bar = full_bar + TMA_STAGES;
  uint64_t* gathered = empty_bar + TMA_STAGES;  // first block of a cluster: the other parts have arrived
  int* abort_s = reinterpret_cast<int*>(gathered + 1);
  float* gather = reinterpret_cast<float*>(abort_s + 2);  // [splits - 1][rows of this tile][D + 2], in_cluster only

  chain_release();
  chain_wait();
  const int tok = blockIdx.x, split = blockIdx.z;
  const int kvh = blockIdx.y / row_tiles, row_tile = blockIdx.y % row_tiles;
  const int G = H / KH;
  const int g0 = row_tile * ROWS, gn = min(ROWS, G - g0);
  const int head0 = kvh * G + g0;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int r = seq_of_token[tok];
  if (r < 0) {
    if (split == 0)
      for (int i = tid; i < gn * D; i += (WARPS + 1) * 32) out[((size_t)tok * H + head0) * D + i] = __float2bfloat16_rn(0.f);
    return;
  }
  const int pos = positions[tok];
  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  const int kt_first = first_key / BK, kt_last = pos / BK;
  const int per_split = (kt_last - kt_first + 1 + splits - 1) / splits;
  const int lo = kt_first + split * per_split, hi = min(lo + per_split, kt_last + 1);

  if (tid == 0) {
    *abort_s = 0;
    for (int s = 0; s < TMA_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], WARPS); }
    mbar_init(gathered, in_cluster ? (unsigned)(splits - 1) : 1u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // Every block of the cluster says that its barriers exist; whoever writes into a peer waits for that first (at the
  // end, when it has long happened). A padding token's blocks have all left above, before any of this.
  if (in_cluster) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  auto wait_for = [&](uint64_t* bar, unsigned parity, int code) {
    if (*(volatile int*)abort_s) return;
    if (!mbar_wait(bar, parity)) {
      *(volatile int*)abort_s = 1;
      atomicExch(&g_decode_status, code);
    }
  };

  if (warp == WARPS) {
    // ------------------------------------------------------------------ producer (a whole warp: the page numbers of up
    // to 32 tiles are fetched at once, one by each lane, instead of one trip to memory before every tile's copies)
    for (int base = lo; base < hi; base += 32) {
      int page = 0;
      if (base + lane < hi) page = block_table[(size_t)r * max_blocks + (base + lane) * BK / page_size];
      if (page < 0) page = 0;  // cannot happen for keys up to the request's position
      const int n = min(32, hi - base);
      for (int j = 0; j < n; ++j) {
        const int kt = base + j, i = kt - lo, s = i % TMA_STAGES;
        const int row = (__shfl_sync(0xffffffffu, page, j) * KH + kvh) * page_size + (kt * BK) % page_size;
        if (lane == 0) {
          if (i >= TMA_STAGES) wait_for(&empty_bar[s], ((i / TMA_STAGES) & 1) ^ 1, 2);
          if (!*(volatile int*)abort_s) {
            mbar_expect_tx(&full_bar[s], 2 * TMA_TILE);
            tma_load_2d(k_t + s * TMA_TILE, &map_k, 0, row, &full_bar[s]);
            tma_load_2d(v_t + s * TMA_TILE, &map_v, 0, row, &full_bar[s]);
          }
        }
      }
    }
    return;  // the consumers wait for every load before the block ends
  }

  // -------------------------------------------------------------------- consumers: warps 0..3
  auto consumers_meet = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory"); };
  uint4 new_row = make_uint4(0u, 0u, 0u, 0u);  // first warp, lanes 0..7: the token's k row; lanes 8..15: its v row
  const bool holds_last = lo <= kt_last && kt_last < hi;
  const bool patches = fresh.qkv != nullptr && fresh.k_pool != nullptr && holds_last;
  if (fresh.qkv == nullptr) {
    for (int c = tid; c < ROWS * CHUNKS; c += WARPS * 32) {
      const int row = c / CHUNKS, col = (c % CHUNKS) * 8;
      const bf16* src = q + ((size_t)tok * H + head0 + min(row, gn - 1)) * D + col;
      cp_async16(q_s + row * STRIDE + col, src, row < gn ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
  } else {
    static_assert(ROWS * CHUNKS == WARPS * 32, "one thread per 8 channels of the query tile");
    const int total = H + 2 * KH, half = fresh.rotary / 2;
    const float* cos_row = fresh.cos_t ? fresh.cos_t + (size_t)tok * half : nullptr;
    const float* sin_row = fresh.cos_t ? fresh.sin_t + (size_t)tok * half : nullptr;
    const bf16* token = fresh.qkv + (size_t)tok * total * D;
    const int row = tid / CHUNKS, e0 = (tid % CHUNKS) * 8;
    float x[8];
    load8(token + (size_t)(head0 + min(row, gn - 1)) * D + e0, x);
    head_norm_rotate8<CHUNKS>(x, e0, fresh.q_w, fresh.eps, fresh.zero_centered, cos_row, sin_row, fresh.rotary);
    if (row >= gn) {
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = 0.f;
    }
    store8(q_s + row * STRIDE + e0, x);
    if (patches && warp == 0) {  // (a whole warp: the norm and the rotation shuffle)
      const int which = lane / CHUNKS;  // 0: k; 1: v; the others shadow k
      load8(token + (size_t)(which == 1 ? H + KH + kvh : H + kvh) * D + e0, x);
      float turned[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) turned[e] = x[e];
      head_norm_rotate8<CHUNKS>(turned, e0, fresh.k_w, fresh.eps, fresh.zero_centered, cos_row, sin_row, fresh.rotary);
      if (which != 1) {  // v goes as it is (its lanes took part in the shuffles above all the same)
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = turned[e];
      }
      new_row = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
      if (row_tile == 0 && which < 2) {  // one block per (token, KV head) writes the pages
        const int page = block_table[(size_t)r * max_blocks + pos / page_size];
        if (page >= 0) {
          bf16* pool = which == 0 ? fresh.k_pool : fresh.v_pool;
          *reinterpret_cast<uint4*>(pool + (((size_t)page * KH + kvh) * page_size + pos % page_size) * D + e0) = new_row;
        }
      }
    }
  }
  consumers_meet();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) ldmatrix_x4(qf[ks], q_s + (lane & 15) * STRIDE + ks * 16 + (lane >> 4) * 8);

  float o[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) { o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl2 = scale * 1.4426950408889634f;

  for (int kt = lo; kt < hi; ++kt) {
    const int i = kt - lo, s = i % TMA_STAGES;
    wait_for(&full_bar[s], (i / TMA_STAGES) & 1, 1);
    unsigned char* kt_ = k_t + s * TMA_TILE;
    unsigned char* vt_ = v_t + s * TMA_TILE;
    if (kt == kt_last && (patches || pos % BK != BK - 1)) {
      if (patches && warp == 0 && lane < 2 * CHUNKS) {  // the token's own k and v rows, whatever the load found there
        const int p = pos % BK;
        *reinterpret_cast<uint4*>((lane < CHUNKS ? kt_ : vt_) + p * 128 + (((lane % CHUNKS) ^ (p & 7)) << 4)) = new_row;
      }
      // rows of V past the position: zero
      for (int c = tid + (pos % BK + 1) * 8; c < BK * 8; c += WARPS * 32)
        *reinterpret_cast<uint4*>(vt_ + c * 16) = make_uint4(0u, 0u, 0u, 0u);
      consumers_meet();
    }
    {
        const bool edge = kt == kt_last || kt * BK < first_key;  // keys past the position, or before the window
        if (gn > 8) attend_tile64<true>(kt_, vt_, qf, o, m_run, l_run, kt, pos, first_key, sl2, edge, warp, lane);
        else attend_tile64<false>(kt_, vt_, qf, o, m_run, l_run, kt, pos, first_key, sl2, edge, warp, lane);
      }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);  // this warp has read the stage
  }
  consumers_meet();  // every warp is done with the tiles: their memory becomes the merge buffers

  float* o_s = reinterpret_cast<float*>(k_t);            // [WARPS][ROWS][D]
  float* ml_s = o_s + WARPS * ROWS * D;                  // [WARPS][ROWS][2]
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
    l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
    const int row = g + h2 * 8;
    if (t == 0) {
      ml_s[(warp * ROWS + row) * 2] = m_run[h2];
      ml_s[(warp * ROWS + row) * 2 + 1] = l_run[h2];
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float* dst = o_s + ((size_t)warp * ROWS + row) * D + nb * 8 + 2 * t;
      dst[0] = o[nb][h2 * 2];
      dst[1] = o[nb][h2 * 2 + 1];
    }
  }
  consumers_meet();
  for (int i = tid; i < gn * D; i += WARPS * 32) {
    const int row = i / D, e = i % D;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) top = fmaxf(top, ml_s[(w * ROWS + row) * 2]);
    float sum = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float mw = ml_s[(w * ROWS + row) * 2];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - top);
      sum = fmaf(ml_s[(w * ROWS + row) * 2 + 1], f, sum);
      acc = fmaf(o_s[((size_t)w * ROWS + row) * D + e], f, acc);
    }
    const size_t head = (size_t)tok * H + head0 + row;
    if (splits == 1) {
      out[head * D + e] = __float2bfloat16_rn(acc / sum);
    } else if (!in_cluster) {
      part_o[(head * splits + split) * D + e] = acc;
      if (e == 0) {
        part_ml[(head * splits + split) * 2] = top;  // in units of log2(e)
        part_ml[(head * splits + split) * 2 + 1] = sum;
      }
    } else if (split == 0) {  // the first block keeps its own part where the merge below finds it: the tiles are done with
      o_s[(size_t)WARPS * ROWS * (D + 2) + row * (D + 2) + e] = acc;
      if (e == 0) {
        o_s[(size_t)WARPS * ROWS * (D + 2) + row * (D + 2) + D] = top;
        o_s[(size_t)WARPS * ROWS * (D + 2) + row * (D + 2) + D + 1] = sum;
      }
    } else {  // into the first block's shared memory
      const unsigned to = peer_address(gather, 0) + (unsigned)((((split - 1) * gn + row) * (D + 2) + e) * 4);
      peer_store(to, acc);
      if (e == 0) {
        peer_store(to + (unsigned)(D * 4), top);
        peer_store(to + (unsigned)((D + 1) * 4), sum);
      }
    }
  }
  if (!in_cluster) return;
  __syncwarp();
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // (arrived long ago) the first block's barrier exists
  consumers_meet();  // all of this block's part is written or on its way
  if (split > 0) {
    if (tid == 0) {
      asm volatile("fence.acq_rel.cluster;" ::: "memory");
      asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(peer_address(gathered, 0)) : "memory");
    }
    return;
  }
  // the first block: the parts in the order of their numbers, as the merge kernel adds them
  bool ok = !*(volatile int*)abort_s;
  if (ok) {
    const unsigned addr = smem_u32(gathered);
    ok = false;
    for (unsigned spin = 0; spin < kSpinLimit && !ok; ++spin) {
      unsigned done;
      asm volatile(
          "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
          : "=r"(done) : "r"(addr), "r"(0u) : "memory");
      ok = done != 0;
    }
    if (!ok) atomicExch(&g_decode_status, 3);
  }
  if (!ok) return;
  const float* own = o_s + (size_t)WARPS * ROWS * (D + 2);
  for (int i = tid; i < gn * D; i += WARPS * 32) {
    const int row = i / D, e = i % D;
    float top = own[row * (D + 2) + D];
    for (int p = 1; p < splits; ++p) top = fmaxf(top, gather[((p - 1) * gn + row) * (D + 2) + D]);
    float sum = 0.f, acc = 0.f;
    for (int p = 0; p < splits; ++p) {
      const float* part = p == 0 ? own + row * (D + 2) : gather + ((p - 1) * gn + row) * (D + 2);
      const float f = part[D] == -INFINITY ? 0.f : exp2f(part[D] - top);
      sum = fmaf(part[D + 1], f, sum);
      acc = fmaf(part[e], f, acc);
    }
    out[((size_t)tok * H + head0 + row) * D + e] = __float2bfloat16_rn(acc / sum);
  }
}

constexpr int kMaxDevices = 64;  // device ordinals that per-device set-up is remembered for

// The same work handed out differently, for steps with more (token, KV head, key part) items than blocks that fit the
// GPU at once: as many blocks as fit, each walking the items blockIdx.x, blockIdx.x + gridDim.x, ... with one ring of
// tiles that runs on across items. The producer warp fetches the next item's tiles while the consumers finish this one
// (its query load, the meeting of the four warps' partial results, the store), so an item's fixed cost hides behind the
// stream, and parts can be small enough (a few tiles) that the last round of items leaves little of the GPU idle. With
// one block per item, 64 requests of 8 KV heads in 2 parts are 1,024 blocks for 444 places: the third round runs a
// third full. The producer warp reads an item's page numbers 32 at a time. Partial results always go to the scratch
// (a merge kernel follows) unless splits == 1.
constexpr int RING = 3;  // stages here: the four warps' partial results need memory of their own beside the ring

__global__ void __launch_bounds__((WARPS + 1) * 32, 4)
decode_attention_items_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                              const bf16* __restrict__ q, const int* __restrict__ block_table, int max_blocks,
                              const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                              bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                              float scale, int window, int page_size, int H, int KH, int row_tiles, int splits,
                              int items, const Fresh fresh) {
  using namespace akas::tc;
  constexpr int D = 64, STRIDE = D + 8, CHUNKS = D / 8, KS = D / 16, NB = D / 8;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* k_t = tiles;                        // [RING][64 keys][128 bytes], swizzled
  unsigned char* v_t = k_t + RING * TMA_TILE;        // [RING][64 keys][128 bytes], swizzled
  bf16* q_s = reinterpret_cast<bf16*>(v_t + RING * TMA_TILE);  // [ROWS][STRIDE]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(q_s + ROWS * STRIDE);
  uint64_t* empty_bar = full_bar + RING;
  int* abort_s = reinterpret_cast<int*>(empty_bar + RING);
  float* o_s = reinterpret_cast<float*>(abort_s + 4);  // [WARPS][rows of a tile][D], then [WARPS][rows of a tile][2]

  chain_release();
  chain_wait();
  const int G = H / KH, rows_most = min(ROWS, G);
  float* ml_s = o_s + WARPS * rows_most * D;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  if (tid == 0) {
    *abort_s = 0;
    for (int s = 0; s < RING; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  auto wait_for = [&](uint64_t* bar, unsigned parity, int code) {
    if (*(volatile int*)abort_s) return;
    if (!mbar_wait(bar, parity)) {
      *(volatile int*)abort_s = 1;
      atomicExch(&g_decode_status, code);
    }
  };
  const int per_token = KH * row_tiles * splits;
  unsigned filled = 0;  // tiles that have gone through the ring so far: the same count in the producer and the consumers

  if (warp == WARPS) {
    // ------------------------------------------------------------------ producer (a whole warp: page numbers by lane)
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int tok = item / per_token, rest = item % per_token;
      const int kvh = rest / splits / row_tiles, split = rest % splits;
      const int r = seq_of_token[tok];
      if (r < 0) continue;
      const int pos = positions[tok];
      const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
      const int kt_first = first_key / BK, kt_last = pos / BK;
      const int per_split = (kt_last - kt_first + 1 + splits - 1) / splits;
      const int lo = kt_first + split * per_split, hi = min(lo + per_split, kt_last + 1);
      for (int base = lo; base < hi; base += 32) {
        int page = 0;
        if (base + lane < hi) page = block_table[(size_t)r * max_blocks + (base + lane) * BK / page_size];
        if (page < 0) page = 0;  // cannot happen for keys up to the request's position
        const int n = min(32, hi - base);
        for (int j = 0; j < n; ++j) {
          const int kt = base + j;
          const int row = (__shfl_sync(0xffffffffu, page, j) * KH + kvh) * page_size + (kt * BK) % page_size;
          if (lane == 0) {
            const unsigned s = filled % RING;
            if (filled >= RING) wait_for(&empty_bar[s], ((filled / RING) & 1) ^ 1, 2);
            if (!*(volatile int*)abort_s) {
              mbar_expect_tx(&full_bar[s], 2 * TMA_TILE);
              tma_load_2d(k_t + s * TMA_TILE, &map_k, 0, row, &full_bar[s]);
              tma_load_2d(v_t + s * TMA_TILE, &map_v, 0, row, &full_bar[s]);
            }
          }
          ++filled;
        }
      }
    }
    return;  // the consumers wait for every load before the block ends
  }

  // -------------------------------------------------------------------- consumers: warps 0..3
  auto consumers_meet = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory"); };
  const float sl2 = scale * 1.4426950408889634f;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int tok = item / per_token, rest = item % per_token;
    const int y = rest / splits, split = rest % splits;
    const int kvh = y / row_tiles, row_tile = y % row_tiles;
    const int g0 = row_tile * ROWS, gn = min(ROWS, G - g0);
    const int head0 = kvh * G + g0;
    const int r = seq_of_token[tok];
    if (r < 0) {
      if (split == 0)
        for (int i = tid; i < gn * D; i += WARPS * 32) out[((size_t)tok * H + head0) * D + i] = __float2bfloat16_rn(0.f);
      continue;
    }
    const int pos = positions[tok];
    const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
    const int kt_first = first_key / BK, kt_last = pos / BK;
    const int per_split = (kt_last - kt_first + 1 + splits - 1) / splits;
    const int lo = kt_first + split * per_split, hi = min(lo + per_split, kt_last + 1);

    uint4 new_row = make_uint4(0u, 0u, 0u, 0u);  // first warp, lanes 0..7: the token's k row; lanes 8..15: its v row
    const bool holds_last = lo <= kt_last && kt_last < hi;
    const bool patches = fresh.qkv != nullptr && fresh.k_pool != nullptr && holds_last;
    if (fresh.qkv == nullptr) {
      for (int c = tid; c < ROWS * CHUNKS; c += WARPS * 32) {
        const int row = c / CHUNKS, col = (c % CHUNKS) * 8;
        const bf16* src = q + ((size_t)tok * H + head0 + min(row, gn - 1)) * D + col;
        cp_async16(q_s + row * STRIDE + col, src, row < gn ? 16 : 0);
      }
      cp_async_commit();
      cp_async_wait<0>();
    } else {
      static_assert(ROWS * CHUNKS == WARPS * 32, "one thread per 8 channels of the query tile");
      const int total = H + 2 * KH, half = fresh.rotary / 2;
      const float* cos_row = fresh.cos_t ? fresh.cos_t + (size_t)tok * half : nullptr;
      const float* sin_row = fresh.cos_t ? fresh.sin_t + (size_t)tok * half : nullptr;
      const bf16* token = fresh.qkv + (size_t)tok * total * D;
      const int row = tid / CHUNKS, e0 = (tid % CHUNKS) * 8;
      float x[8];
      load8(token + (size_t)(head0 + min(row, gn - 1)) * D + e0, x);
      head_norm_rotate8<CHUNKS>(x, e0, fresh.q_w, fresh.eps, fresh.zero_centered, cos_row, sin_row, fresh.rotary);
      if (row >= gn) {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = 0.f;
      }
      store8(q_s + row * STRIDE + e0, x);
      if (patches && warp == 0) {  // (a whole warp: the norm and the rotation shuffle)
        const int which = lane / CHUNKS;  // 0: k; 1: v; the others shadow k
        load8(token + (size_t)(which == 1 ? H + KH + kvh : H + kvh) * D + e0, x);
        float turned[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) turned[e] = x[e];
        head_norm_rotate8<CHUNKS>(turned, e0, fresh.k_w, fresh.eps, fresh.zero_centered, cos_row, sin_row, fresh.rotary);
        if (which != 1) {  // v goes as it is (its lanes took part in the shuffles above all the same)
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] = turned[e];
        }
        new_row = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
        if (row_tile == 0 && which < 2) {  // one item per (token, KV head) writes the pages
          const int page = block_table[(size_t)r * max_blocks + pos / page_size];
          if (page >= 0) {
            bf16* pool = which == 0 ? fresh.k_pool : fresh.v_pool;
            *reinterpret_cast<uint4*>(pool + (((size_t)page * KH + kvh) * page_size + pos % page_size) * D + e0) = new_row;
          }
        }
      }
    }
    consumers_meet();
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) ldmatrix_x4(qf[ks], q_s + (lane & 15) * STRIDE + ks * 16 + (lane >> 4) * 8);

    float o[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) { o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    for (int kt = lo; kt < hi; ++kt) {
      const unsigned s = filled % RING;
      wait_for(&full_bar[s], (filled / RING) & 1, 1);
      ++filled;
      unsigned char* kt_ = k_t + s * TMA_TILE;
      unsigned char* vt_ = v_t + s * TMA_TILE;
      if (kt == kt_last && (patches || pos % BK != BK - 1)) {
        if (patches && warp == 0 && lane < 2 * CHUNKS) {  // the token's own k and v rows, whatever the load found there
          const int p = pos % BK;
          *reinterpret_cast<uint4*>((lane < CHUNKS ? kt_ : vt_) + p * 128 + (((lane % CHUNKS) ^ (p & 7)) << 4)) = new_row;
        }
        // rows of V past the position: zero
        for (int c = tid + (pos % BK + 1) * 8; c < BK * 8; c += WARPS * 32)
          *reinterpret_cast<uint4*>(vt_ + c * 16) = make_uint4(0u, 0u, 0u, 0u);
        consumers_meet();
      }
      {
        const bool edge = kt == kt_last || kt * BK < first_key;  // keys past the position, or before the window
        if (gn > 8) attend_tile64<true>(kt_, vt_, qf, o, m_run, l_run, kt, pos, first_key, sl2, edge, warp, lane);
        else attend_tile64<false>(kt_, vt_, qf, o, m_run, l_run, kt, pos, first_key, sl2, edge, warp, lane);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);  // this warp has read the stage
    }

    // the four warps' partial results meet in memory of their own (the ring is already filling for the next item)
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
      l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
      const int row = g + h2 * 8;
      if (row < rows_most) {
        if (t == 0) {
          ml_s[(warp * rows_most + row) * 2] = m_run[h2];
          ml_s[(warp * rows_most + row) * 2 + 1] = l_run[h2];
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          float* dst = o_s + ((size_t)warp * rows_most + row) * D + nb * 8 + 2 * t;
          dst[0] = o[nb][h2 * 2];
          dst[1] = o[nb][h2 * 2 + 1];
        }
      }
    }
    consumers_meet();
    for (int i = tid; i < gn * D; i += WARPS * 32) {
      const int row = i / D, e = i % D;
      float top = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) top = fmaxf(top, ml_s[(w * rows_most + row) * 2]);
      float sum = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float mw = ml_s[(w * rows_most + row) * 2];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - top);
        sum = fmaf(ml_s[(w * rows_most + row) * 2 + 1], f, sum);
        acc = fmaf(o_s[((size_t)w * rows_most + row) * D + e], f, acc);
      }
      const size_t head = (size_t)tok * H + head0 + row;
      if (splits == 1) {
        out[head * D + e] = __float2bfloat16_rn(acc / sum);
      } else {
        part_o[(head * splits + split) * D + e] = acc;
        if (e == 0) {
          part_ml[(head * splits + split) * 2] = top;  // in units of log2(e)
          part_ml[(head * splits + split) * 2 + 1] = sum;
        }
      }
    }
    consumers_meet();  // q_s and the partial results are free for the next item
  }
}

template <int D>
int launch(const void* q, const void* k_pool, const void* v_pool, const int* block_table, int max_blocks,
           const int* seq_of_token, const int* positions, void* out, float* part_o, float* part_ml, float scale,
           int window, int page_size, int N, int H, int KH, int splits, cudaStream_t stream) {
  constexpr int STRIDE = D + 8;
  constexpr int tiles_bytes = (ROWS + 2 * STAGES * BK) * STRIDE * (int)sizeof(bf16);
  constexpr int merge_bytes = ROWS * STRIDE * (int)sizeof(bf16) + WARPS * ROWS * (D + 2) * (int)sizeof(float);
  constexpr int smem = tiles_bytes > merge_bytes ? tiles_bytes : merge_bytes;
  // The attribute belongs to a device, like the scratch address of the entry point that allocates nothing.
  static bool configured[kMaxDevices] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  if (!configured[device]) {
    const cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured[device] = true;
  }
  const int G = H / KH, row_tiles = (G + ROWS - 1) / ROWS;
  int err = launch_chained(decode_attention_kernel<D>, dim3(N, KH * row_tiles, splits), dim3(WARPS * 32), smem, stream,
                           (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table, max_blocks,
                           seq_of_token, positions, (bf16*)out, part_o, part_ml, scale, window, page_size, H, KH,
                           row_tiles, splits);
  if (err || splits == 1) return err;
  return launch_chained(decode_merge_bf16_kernel, dim3(N, H), dim3(D >= 64 ? 64 : 32), 0, stream,
                        (const float*)part_o, (const float*)part_ml, seq_of_token, (bf16*)out, H, D, splits);
}

// Head size 64, pages of whole tiles: the TMA-fed kernel. pool_rows: pages x kv heads x page size.
int launch_tma(const void* q, const void* k_pool, const void* v_pool, long long pool_rows, const int* block_table,
               int max_blocks, const int* seq_of_token, const int* positions, void* out, float* part_o, float* part_ml,
               float scale, int window, int page_size, int N, int H, int KH, int splits, cudaStream_t stream,
               const Fresh& fresh = Fresh{}) {
  constexpr int D = 64, MAX_CLUSTER = 8;
  constexpr int smem = 1024 + 2 * TMA_STAGES * TMA_TILE + ROWS * (D + 8) * (int)sizeof(bf16) + (2 * TMA_STAGES + 1) * 8 + 16;
  constexpr int gather_most = (MAX_CLUSTER - 1) * ROWS * (D + 2) * (int)sizeof(float);  // the other parts, in the first block
  static_assert(2 * TMA_STAGES * TMA_TILE >= (WARPS + 1) * ROWS * (D + 2) * (int)sizeof(float), "the merge buffers fit the tiles");
  static bool configured[kMaxDevices] = {};
  static int cluster_ok[kMaxDevices][MAX_CLUSTER + 1] = {};  // 0 unknown, 1 a cluster of that many blocks can run, -1 it cannot
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  if (!configured[device]) {
    const cudaError_t e = cudaFuncSetAttribute(decode_attention_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               smem + gather_most);
    if (e != cudaSuccess) return (int)e;
    configured[device] = true;
  }
  CUtensorMap map_k, map_v;
  int err = akas::tc::cached_map(&map_k, k_pool, (int)pool_rows, D, BK, true);
  if (!err) err = akas::tc::cached_map(&map_v, v_pool, (int)pool_rows, D, BK, true);
  if (err) return err;
  const int G = H / KH, row_tiles = (G + ROWS - 1) / ROWS;
  // The parts of a (token, KV head) as a thread-block cluster whose first block merges them, where a cluster can be
  // that large; else every part writes to the scratch and a second kernel merges.
  static const bool clusters_wanted = [] { const char* v = getenv("AKAS_B200_DECODE_CLUSTER_MERGE"); return !(v && v[0] == '0'); }();
  // Only while the blocks are few (up to four per SM): with more, a cluster's blocks wait for one another to be placed
  // and the second kernel costs less than that (64 requests: 43.1k tokens/s merged in clusters, 44.3k with the kernel).
  static int sms[kMaxDevices] = {};
  if (sms[device] == 0) cudaDeviceGetAttribute(&sms[device], cudaDevAttrMultiProcessorCount, device);
  int in_cluster = clusters_wanted && splits >= 2 && splits <= MAX_CLUSTER &&
                   (long long)N * KH * row_tiles * splits <= 4ll * sms[device] ? 1 : 0;
  const int gather_bytes = in_cluster ? (splits - 1) * (G < ROWS ? G : ROWS) * (D + 2) * (int)sizeof(float) : 0;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(N, KH * row_tiles, splits);
  config.blockDim = dim3((WARPS + 1) * 32);
  config.dynamicSmemBytes = smem + gather_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  int n = 0;
  if (chained_launches_enabled()) {
    attribute[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (in_cluster) {
    attribute[n].id = cudaLaunchAttributeClusterDimension;
    attribute[n].val.clusterDim.x = 1;
    attribute[n].val.clusterDim.y = 1;
    attribute[n].val.clusterDim.z = splits;
    config.attrs = attribute;
    config.numAttrs = n + 1;
    if (cluster_ok[device][splits] == 0) {
      int room = 0;
      if (cudaOccupancyMaxActiveClusters(&room, decode_attention_tma_kernel, &config) != cudaSuccess) { cudaGetLastError(); room = 0; }
      cluster_ok[device][splits] = room > 0 ? 1 : -1;
    }
    if (cluster_ok[device][splits] < 0) {
      in_cluster = 0;
      config.dynamicSmemBytes = smem;
    } else {
      ++n;
    }
  }
  config.attrs = attribute;
  config.numAttrs = n;
  if (!in_cluster && splits > 1 && (part_o == nullptr || part_ml == nullptr)) return (int)cudaErrorInvalidValue;
  err = (int)cudaLaunchKernelEx(&config, decode_attention_tma_kernel, map_k, map_v, (const bf16*)q, block_table, max_blocks,
                                seq_of_token, positions, (bf16*)out, part_o, part_ml, scale, window, page_size, H, KH,
                                row_tiles, splits, in_cluster, fresh);
  if (err || splits == 1 || in_cluster) return err;
  return launch_chained(decode_merge_bf16_kernel, dim3(N, H), dim3(64), 0, stream, (const float*)part_o,
                        (const float*)part_ml, seq_of_token, (bf16*)out, H, D, splits);
}

// The items kernel: as many blocks as the device holds at once (or as there are items).
constexpr int items_smem(int rows_most) {
  return 1024 + 2 * RING * TMA_TILE + ROWS * (64 + 8) * (int)sizeof(bf16) + 2 * RING * 8 + 16 +
         WARPS * rows_most * (64 + 2) * (int)sizeof(float);
}

// Blocks of the items kernel that are resident at once on the current device for H / KH query heads per KV head
// (0: the kernel cannot run here).
int items_places(int G) {
  static int places[kMaxDevices][ROWS + 1] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return 0;
  const int rows_most = G < ROWS ? G : ROWS;
  if (places[device][rows_most] == 0) {
    static bool configured[kMaxDevices] = {};
    if (!configured[device]) {
      if (cudaFuncSetAttribute(decode_attention_items_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, items_smem(ROWS)) != cudaSuccess) {
        cudaGetLastError();
        return 0;
      }
      configured[device] = true;
    }
    int per_sm = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_attention_items_kernel, (WARPS + 1) * 32,
                                                      items_smem(rows_most)) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    places[device][rows_most] = per_sm * sms > 0 ? per_sm * sms : -1;
  }
  return places[device][rows_most] > 0 ? places[device][rows_most] : 0;
}

int launch_items(const void* q, const void* k_pool, const void* v_pool, long long pool_rows, const int* block_table,
                 int max_blocks, const int* seq_of_token, const int* positions, void* out, float* part_o, float* part_ml,
                 float scale, int window, int page_size, int N, int H, int KH, int splits, cudaStream_t stream,
                 const Fresh& fresh) {
  constexpr int D = 64;
  const int G = H / KH, row_tiles = (G + ROWS - 1) / ROWS;
  const int places = items_places(G);
  if (places <= 0) return (int)cudaErrorInvalidConfiguration;
  if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) return (int)cudaErrorInvalidValue;
  const long long items = (long long)N * KH * row_tiles * splits;
  if (items >= (1ll << 31)) return (int)cudaErrorInvalidValue;
  CUtensorMap map_k, map_v;
  int err = akas::tc::cached_map(&map_k, k_pool, (int)pool_rows, D, BK, true);
  if (!err) err = akas::tc::cached_map(&map_v, v_pool, (int)pool_rows, D, BK, true);
  if (err) return err;
  err = launch_chained(decode_attention_items_kernel, dim3((unsigned)(items < places ? items : places)), dim3((WARPS + 1) * 32),
                       items_smem(G < ROWS ? G : ROWS), stream, map_k, map_v, (const bf16*)q, block_table, max_blocks,
                       seq_of_token, positions, (bf16*)out, part_o, part_ml, scale, window, page_size, H, KH, row_tiles,
                       splits, (int)items, fresh);
  if (err || splits == 1) return err;
  return launch_chained(decode_merge_bf16_kernel, dim3(N, H), dim3(64), 0, stream, (const float*)part_o,
                        (const float*)part_ml, seq_of_token, (bf16*)out, H, D, splits);
}


}  // namespace

// The same as akas_decode_attention_bf16 below for callers that know the size of the pools (pool_pages pages): with
// head size 64 and a page size that is a multiple of 64 the K and V tiles are fetched by TMA.
AKAS_API int akas_decode_attention_bf16_paged(const void* q, const void* k_pool, const void* v_pool, int pool_pages,
                                              const int* block_table, int max_blocks, const int* seq_of_token,
                                              const int* positions, void* out, float* part_o, float* part_ml, float scale,
                                              int window, int page_size, int N, int H, int KH, int D, int splits,
                                              cudaStream_t stream);

// 0 if no bounded wait of the TMA-fed kernel has ever run out on the current device (1: consumers, 2: producer).
AKAS_API int akas_decode_attention_status() {
  int status = -1;
  const cudaError_t e = cudaMemcpyFromSymbol(&status, g_decode_status, sizeof(int));
  return e == cudaSuccess ? status : -(int)e;
}

// Scratch (untouched when splits == 1): part_o float32 [N, H, splits, D], part_ml float32 [N, H, splits, 2].
AKAS_API int akas_decode_attention_bf16(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                        int max_blocks, const int* seq_of_token, const int* positions, void* out,
                                        float* part_o, float* part_ml, float scale, int window, int page_size, int N,
                                        int H, int KH, int D, int splits, cudaStream_t stream) {
  if (H % KH || splits < 1 || splits > 65535 || (long long)KH * ((H / KH + ROWS - 1) / ROWS) > 65535)
    return (int)cudaErrorInvalidValue;
  if (N <= 0) return 0;
#define AKAS_DECODE(DD)                                                                                             \
  case DD:                                                                                                          \
    return launch<DD>(q, k_pool, v_pool, block_table, max_blocks, seq_of_token, positions, out, part_o, part_ml,    \
                      scale, window, page_size, N, H, KH, splits, stream)
  switch (D) {
    AKAS_DECODE(16);
    AKAS_DECODE(32);
    AKAS_DECODE(64);
    AKAS_DECODE(128);
    default:
      return (int)cudaErrorInvalidValue;
  }
#undef AKAS_DECODE
}

AKAS_API int akas_decode_attention_bf16_paged(const void* q, const void* k_pool, const void* v_pool, int pool_pages,
                                              const int* block_table, int max_blocks, const int* seq_of_token,
                                              const int* positions, void* out, float* part_o, float* part_ml, float scale,
                                              int window, int page_size, int N, int H, int KH, int D, int splits,
                                              cudaStream_t stream) {
  const long long pool_rows = (long long)pool_pages * KH * page_size;
  if (D == 64 && page_size % BK == 0 && H % KH == 0 && splits >= 1 && splits <= 65535 && pool_rows > 0 &&
      pool_rows < (1ll << 31) && (long long)KH * ((H / KH + ROWS - 1) / ROWS) <= 65535 && (uintptr_t)k_pool % 16 == 0 &&
      (uintptr_t)v_pool % 16 == 0) {
    if (N <= 0) return 0;
    return launch_tma(q, k_pool, v_pool, pool_rows, block_table, max_blocks, seq_of_token, positions, out, part_o, part_ml,
                      scale, window, page_size, N, H, KH, splits, stream);
  }
  return akas_decode_attention_bf16(q, k_pool, v_pool, block_table, max_blocks, seq_of_token, positions, out, part_o,
                                    part_ml, scale, window, page_size, N, H, KH, D, splits, stream);
}

// How many blocks of the kernel below the current device holds at once (0: it cannot run here): a step with more
// (token, KV head, 16 query heads, key part) items than that is better off there than with a block per item.
AKAS_API int akas_decode_attention_items_places(int H, int KH) { return KH > 0 && H % KH == 0 ? items_places(H / KH) : 0; }

// Decode attention by a fixed number of blocks that walk the (token, KV head, 16 query heads, key part) items, from q
// [N, H * 64] (qkv null) or straight from the qkv product (q null; the arguments of akas_decode_attention_from_qkv).
// Head size 64 and a page size that is a multiple of 64 only: 3999 otherwise.
AKAS_API int akas_decode_attention_items(const void* q, const void* qkv, const float* q_w, const float* k_w, float eps,
                                         int zero_centered, const float* cos_t, const float* sin_t, int rotary, int write,
                                         void* k_pool, void* v_pool, int pool_pages, const int* block_table, int max_blocks,
                                         const int* seq_of_token, const int* positions, void* out, float* part_o,
                                         float* part_ml, float scale, int window, int page_size, int N, int H, int KH,
                                         int D, int splits, cudaStream_t stream) {
  const long long pool_rows = (long long)pool_pages * KH * page_size;
  if (D != 64 || page_size % BK || KH <= 0 || H % KH || splits < 1 || splits > 65535 || pool_rows <= 0 || pool_rows >= (1ll << 31) ||
      (q == nullptr) == (qkv == nullptr) || rotary < 0 || rotary > D || rotary % 16 ||
      (cos_t != nullptr && (rotary == 0 || sin_t == nullptr)) || (uintptr_t)q % 16 ||
      (uintptr_t)qkv % 16 || (uintptr_t)k_pool % 16 || (uintptr_t)v_pool % 16 || (uintptr_t)out % 16 ||
      (uintptr_t)q_w % 16 || (uintptr_t)k_w % 16 || (uintptr_t)cos_t % 16 || (uintptr_t)sin_t % 16)
    return 3999;
  if (N <= 0) return 0;
  Fresh fresh = {};
  if (qkv != nullptr) {
    fresh.qkv = (const bf16*)qkv;
    fresh.q_w = q_w;
    fresh.k_w = k_w;
    fresh.eps = eps;
    fresh.zero_centered = zero_centered;
    fresh.cos_t = cos_t;
    fresh.sin_t = sin_t;
    fresh.rotary = cos_t ? rotary : 0;
    fresh.k_pool = write ? (bf16*)k_pool : nullptr;
    fresh.v_pool = write ? (bf16*)v_pool : nullptr;
  }
  return launch_items(q, k_pool, v_pool, pool_rows, block_table, max_blocks, seq_of_token, positions, out, part_o, part_ml,
                      scale, window, page_size, N, H, KH, splits, stream, fresh);
}

// Decode attention straight from the qkv product, [N, (H + 2 KH) * D] bfloat16: the per-head RMSNorm (q_w, k_w:
// float32 [D], or null) and rotation (cos_t, sin_t: float32 [N, rotary / 2], or null) of q and k, the write of the
// token's k and v rows into the pages (write == 0: a layer that only reads them) and attention, as one kernel.
// Returns 3999 where that kernel does not take the sizes (head size 64, page size a multiple of 64, a rotary width
// that is a multiple of 16, 16-byte aligned pointers): the caller then runs the steps as separate kernels.
AKAS_API int akas_decode_attention_from_qkv(const void* qkv, const float* q_w, const float* k_w, float eps, int zero_centered,
                                            const float* cos_t, const float* sin_t, int rotary, int write, void* k_pool,
                                            void* v_pool, int pool_pages, const int* block_table, int max_blocks,
                                            const int* seq_of_token, const int* positions, void* out, float* part_o,
                                            float* part_ml, float scale, int window, int page_size, int N, int H, int KH,
                                            int D, int splits, cudaStream_t stream) {
  const long long pool_rows = (long long)pool_pages * KH * page_size;
  if (D != 64 || page_size % BK || KH <= 0 || H % KH || splits < 1 || splits > 65535 || pool_rows <= 0 || pool_rows >= (1ll << 31) ||
      (long long)KH * ((H / KH + ROWS - 1) / ROWS) > 65535 || rotary < 0 || rotary > D || rotary % 16 ||
      (cos_t != nullptr && (rotary == 0 || sin_t == nullptr)) ||
      (uintptr_t)qkv % 16 || (uintptr_t)k_pool % 16 || (uintptr_t)v_pool % 16 || (uintptr_t)out % 16 ||
      (uintptr_t)q_w % 16 || (uintptr_t)k_w % 16 || (uintptr_t)cos_t % 16 || (uintptr_t)sin_t % 16)
    return 3999;
  if (N <= 0) return 0;
  Fresh fresh;
  fresh.qkv = (const bf16*)qkv;
  fresh.q_w = q_w;
  fresh.k_w = k_w;
  fresh.eps = eps;
  fresh.zero_centered = zero_centered;
  fresh.cos_t = cos_t;
  fresh.sin_t = sin_t;
  fresh.rotary = cos_t ? rotary : 0;
  fresh.k_pool = write ? (bf16*)k_pool : nullptr;
  fresh.v_pool = write ? (bf16*)v_pool : nullptr;
  return launch_tma(nullptr, k_pool, v_pool, pool_rows, block_table, max_blocks, seq_of_token, positions, out, part_o,
                    part_ml, scale, window, page_size, N, H, KH, splits, stream, fresh);
}

// ---------------------------------------------------------------------------------------------------------
// The same kernels for callers that cannot allocate: scratch inside the library. See noalloc.h.
#include <mutex>

#include "noalloc.h"

namespace {

// Partials of the key splits: [tokens, heads, splits, head_dim] sums, then [tokens, heads, splits, 2] (max, sum).
// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer a kernel may be given.
static __device__ __align__(256) float g_decode_scratch[AKAS_DECODE_NOALLOC_FLOATS];

float* g_decode_scratch_address[kMaxDevices] = {};  // device address of the array, per device ordinal
std::mutex g_decode_scratch_mutex;

// The device address of g_decode_scratch on the current device; looked up once per device.
int decode_scratch(float** address) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= kMaxDevices) return AKAS_NOALLOC_NO_SYMBOL;
  std::lock_guard<std::mutex> lock(g_decode_scratch_mutex);
  if (g_decode_scratch_address[device] == nullptr) {
    float* found = nullptr;
    e = cudaGetSymbolAddress((void**)&found, g_decode_scratch);
    if (e != cudaSuccess || found == nullptr) return e != cudaSuccess ? (int)e : AKAS_NOALLOC_NO_SYMBOL;
    g_decode_scratch_address[device] = found;
  }
  *address = g_decode_scratch_address[device];
  return 0;
}

}  // namespace

long long akas_decode_attention_bf16_noalloc_needs(int tokens, int heads, int splits, int head_dim) {
  if (tokens <= 0 || heads <= 0 || splits <= 1 || head_dim <= 0) return 0;  // a single split writes the output directly
  // Four ints can overflow 64 bits: once a partial product is past the array, the answer is "too many" whatever follows.
  const long long limit = (long long)AKAS_DECODE_NOALLOC_FLOATS + 1;
  long long need = (long long)tokens * heads;          // < 2^62
  if (need >= limit) return limit;
  need *= splits;                                       // < 2^20 * 2^31
  if (need >= limit) return limit;
  need *= (long long)head_dim + 2;                      // < 2^20 * 2^32
  return need >= limit ? limit : need;
}

const char* akas_noalloc_error_string(int code) {
  switch (code) {
    case 0: return "no error";
    case AKAS_NOALLOC_TOO_LARGE:
      return "the call needs more than AKAS_DECODE_NOALLOC_FLOATS float32 of scratch (tokens * heads * splits * "
             "(head_dim + 2)); use fewer splits or tokens, or akas_decode_attention_bf16 with scratch of your own";
    case AKAS_NOALLOC_NO_SYMBOL: return "the device address of the library's scratch array could not be found";
    case AKAS_NOALLOC_BAD_ARGUMENT: return "a size is out of range or a pointer is null";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
  }
}

int akas_decode_attention_bf16_noalloc(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                       int max_blocks, const int* seq_of_token, const int* positions, void* out,
                                       float scale, int window, int page_size, int tokens, int heads, int kv_heads,
                                       int head_dim, int splits, cudaStream_t stream) {
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || splits < 1 || page_size <= 0 || max_blocks <= 0 ||
      !q || !k_pool || !v_pool || !block_table || !seq_of_token || !positions || !out)
    return AKAS_NOALLOC_BAD_ARGUMENT;
  const long long need = akas_decode_attention_bf16_noalloc_needs(tokens, heads, splits, head_dim);
  if (need > (long long)AKAS_DECODE_NOALLOC_FLOATS) return AKAS_NOALLOC_TOO_LARGE;
  float* scratch = nullptr;
  const int err = decode_scratch(&scratch);
  if (err) return err;
  float* part_o = scratch;
  float* part_ml = scratch + (size_t)tokens * heads * splits * head_dim;
  return akas_decode_attention_bf16(q, k_pool, v_pool, block_table, max_blocks, seq_of_token, positions, out, part_o,
                                    part_ml, scale, window, page_size, tokens, heads, kv_heads, head_dim, splits,
                                    stream);
}
