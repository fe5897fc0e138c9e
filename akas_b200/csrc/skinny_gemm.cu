// Matrix products for a handful of tokens (decode steps): y[M, O] = f(x)[M, K] . W[O, K]^T with M <= 16,
// bfloat16 weights streamed once from HBM by TMA, float32 accumulation on the tensor cores.
//
// The weights are the A operand of mma.sync m16n8k16 (16 weight rows x 16 k), the tokens are the 8
// columns of B, so 16 rows of W become 16 output channels for all tokens. Blocks are persistent: one or
// two per SM, each taking row tiles blockIdx.x, blockIdx.x + gridDim.x, ...
//
// A block has one producer warp and 8 consumer warps. The producer streams the block's weight rows, in
// 512-wide chunks, into a four-stage ring in shared memory: one TMA tensor load per stage (a box of 64 k x 16
// rows x 8 groups of k from a three-dimensional view [K/64][O][64] of the matrix, 128-byte swizzle; for SwiGLU
// two boxes of 8 rows), completion counted in bytes on the stage's "full" mbarrier. An instruction that starts a
// TMA copy costs the issuing thread some 300 cycles whatever the copy holds, so a box is as large as it can be:
// with 4 KB boxes one thread could not feed an SM's share of the memory bandwidth.
// It runs ahead across row tiles, held back only by the stages' "empty" mbarriers, on which the consumer
// warps arrive when they have read a stage. So up to 64 KB of loads are in flight per block with one thread
// issuing them, and the consumers' loop is: wait for the stage, 16-byte reads from shared memory, four
// products, arrive. The 8 consumer warps split a chunk 64 k each; in each 32 k of it, thread (g, t) reads 16
// contiguous bytes of W rows g and g + 8 and of token g at k = 8t. These 8 values feed two k-steps: the
// product does not care which physical k sits in which k-slot as long as A and B agree, which is what makes
// 16-byte reads possible. The tokens' activations are put into shared memory once per block (converted and
// weighted by the norm there, if the norm rides along). At the end of a row tile the consumers' partial sums
// meet in shared memory (a barrier of the consumer warps only).
//
// The producer starts before the kernel waits for its predecessor (weights depend on nothing).
// Every wait on an mbarrier is bounded: a wait that runs out sets a status flag that the host can read
// (akas_skinny_gemm_status), everyone stops waiting and the block runs to its end; results of such a launch
// are not valid.
//
// Input modes:   bf16   x is bfloat16 [M, K]
//                norm   x is the float32 residual stream (rows optionally gathered by index); the kernel
//                       forms bf16(x * norm_weight), sums x^2 per token on the way and multiplies the
//                       result by rsqrt(mean(x^2) + eps): RMSNorm without a pass of its own.
// Output modes:  bf16 store | float32 store | float32 accumulate (y += ..., the residual stream) |
//                swiglu: the block's 16 rows are gate rows f0..f0+7 and up rows F+f0..F+f0+7 of the
//                stacked [2F, K] matrix, so silu(gate) * up is formed per thread and stored as bf16 [M, F].
//                conv: W is the in projection [3C, K] of a gated short convolution and every token is the single
//                token of its request (a decode step). A tile is 8 channels: 8 rows each of the projection's B, C
//                and x parts (three boxes a stage, three stages), a second product per k-step for the x rows; the
//                read-out rounds the three values to bfloat16 as the product by itself would, then does what the
//                convolution's decode kernel does (u = B x; the taps over the request's state rows and u; the
//                state shifted; bias; times C) and stores bf16 [M, C]: one launch and no [M, 3C] round trip.
// Parts of K. A block must hold its tokens' activations for all the k it multiplies, and fetching them costs the
// SM as much as fetching weights does; with a long K and few rows (the down projection of a feed-forward) they
// are a third of what a block fetches, and they leave room for one block per SM only. Such a product is cut
// along K as well: the `ksplit` blocks of a thread-block cluster take one part of K each for the same row
// tiles, keep their sums in shared memory, and at the end send them to the cluster's first block
// (st.shared::cluster, one arrival per block on its mbarrier), which adds the parts in rank order and writes
// the result. Not for the SwiGLU read-out.
// Needs K % 64 == 0. Results do not depend on what else runs; summation order is fixed.
#include <cuda.h>
#include <math.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "mma.cuh"

using namespace akas;

namespace {

constexpr int CONSUMERS = 8, KC = 512, STAGES = 4;
constexpr int MAX_KSPLIT = 8, SPLIT_TILES = 4;  // parts of K; row tiles a cluster may take when K is cut
constexpr int STAGE_BYTES = 16 * KC * 2;  // one box of [8 groups of k][16 rows][128 bytes], or (SwiGLU) two of 8 rows
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr unsigned kSpinLimit = 1u << 22;  // try_wait calls before a wait gives up (each may block for a while)
enum { IN_BF16 = 0, IN_NORM = 1 };
enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_ACC = 2, OUT_SWIGLU = 3, OUT_CONV = 4 };
// Bytes of a stage, stages of the ring and weight rows of a tile, by read-out: the convolution's three boxes of 8 rows
// make a stage of 24 KB, and three of them leave room for two blocks on an SM.
template <int OUT> struct Ring {
  static constexpr int BYTES = OUT == OUT_CONV ? 24 * KC * 2 : STAGE_BYTES;
  static constexpr int DEPTH = OUT == OUT_CONV ? 3 : STAGES;
  static constexpr int ROWS = OUT == OUT_CONV ? 24 : 16;
};
// What the convolution's read-out needs beside the product's operands (all null or zero for the other read-outs).
struct ConvTail {
  const float* taps;        // [C, L]
  const float* bias;        // [C] or null
  float* state;             // [slots, L - 1, C]
  const int* seq_of_token;  // [M]: the request of a token, or -1 for padding
  const int* slots;         // [requests]: the state row of a request
  int L, write;
};

__device__ int g_skinny_status = 0;  // 0, or the code of a wait that ran out (1: a full stage, 2: an empty stage)

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Waits for the phase of the given parity to complete; false if the bounded wait ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
  const unsigned addr = smem_u32(bar);
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity), "r"(200u) : "memory");
    if (done) return true;
  }
  return false;
}
// One box of the weights: 64 k x 8 rows x 4 groups of k, starting at row `row` and k-group `group`.
__device__ __forceinline__ void tma_load_box(void* smem_dst, const CUtensorMap* map, int row, int group, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(smem_u32(smem_dst)), "l"(map), "r"(0), "r"(row), "r"(group), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory"); }

__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned peer_address(const void* local, unsigned rank) {  // the same location in block `rank`
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
  return r;
}
__device__ __forceinline__ void peer_store(unsigned address, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(address), "f"(v) : "memory");
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, unsigned parity) {
  const unsigned addr = smem_u32(bar);
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void cluster_meet() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int NT, int IN, int OUT, bool GROUPED>
__global__ void __launch_bounds__(THREADS, 2)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const void* __restrict__ x_, const int* __restrict__ rows,
                   const float* __restrict__ norm_w, float eps, int zero_centered, void* __restrict__ y_, int M, int O,
                   int K, int num_tiles, int ksplit, int groups, const ConvTail tail) {
  constexpr int STAGES = Ring<OUT>::DEPTH, STAGE_BYTES = Ring<OUT>::BYTES, RT = Ring<OUT>::ROWS;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);  // [STAGES][STAGE_BYTES]
  float* red = reinterpret_cast<float*>(ring + STAGES * STAGE_BYTES);   // [CONSUMERS][NT][RT][8]: partial sums
  // ksplit > 1: this block's sums of its row tiles, then (first block only) the other blocks' sums and sums of x^2
  float* part = red + CONSUMERS * NT * RT * 8;                           // [SPLIT_TILES][NT * 128]
  float* peer = part + (ksplit > 1 ? SPLIT_TILES * NT * 128 : 0);        // [ksplit - 1][SPLIT_TILES][NT * 128]
  float* peer_ss = peer + (ksplit > 1 ? (ksplit - 1) * SPLIT_TILES * NT * 128 : 0);  // [ksplit - 1][NT * 8]
  bf16* xs = reinterpret_cast<bf16*>(peer_ss + (ksplit > 1 ? (ksplit - 1) * NT * 8 : 0));  // [NT * 8][XS]: activations
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], gathered;
  __shared__ float ss_s[CONSUMERS][NT * 8];  // sums of x^2 per token, one part per consumer warp (added in warp order)
  __shared__ int slot_s[NT * 8];  // convolution read-out: the state row of each token's request, or -1
  __shared__ int abort_s;  // set by the first wait that runs out; from then on nobody waits on an mbarrier
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int F = O / 2;  // swiglu only: O is the stacked height 2F
  const int all_chunks = (K + KC - 1) / KC;
  // this block's part of K: chunks [chunk0, chunk0 + chunks) of all_chunks, k from k0 on
  const int rank = ksplit > 1 ? (int)cluster_rank() : 0;
  const int chunk0 = all_chunks * rank / ksplit, chunks = all_chunks * (rank + 1) / ksplit - chunk0;
  const int k0 = chunk0 * KC, k_len = min(K, (chunk0 + chunks) * KC) - k0;
  const int XS = ((all_chunks + ksplit - 1) / ksplit) * KC + 32;
  // Token groups (9 to 16 tokens on the kernel for 8): every row tile is the work of `groups` blocks (clusters), one per
  // group of NT * 8 tokens, that run side by side and read the same weights, the second one mostly from the L2. A
  // block's group is fixed (the host makes the number of clusters a multiple of `groups`); from here on it sees only
  // its own tokens.
  // (GROUPED is a template argument so that the kernel for a single group keeps its registers: with the group's offsets
  // computed in every instance the staging of the normed rows spilled)
  const int item0 = (int)blockIdx.x / ksplit, item_step = (int)gridDim.x / ksplit;  // of this block's cluster
  const int first_tile = GROUPED ? item0 / groups : item0, tile_step = GROUPED ? item_step / groups : item_step;
  const int* token_request = tail.seq_of_token;
  if (GROUPED) {
    const int m0 = (item0 % groups) * NT * 8;
    if (rows) rows += m0;
    else x_ = IN == IN_NORM ? (const void*)((const float*)x_ + (size_t)m0 * K) : (const void*)((const bf16*)x_ + (size_t)m0 * K);
    const size_t width = OUT == OUT_SWIGLU ? O / 2 : OUT == OUT_CONV ? O / 3 : O;
    y_ = OUT == OUT_F32 || OUT == OUT_ACC ? (void*)((float*)y_ + m0 * width) : (void*)((bf16*)y_ + m0 * width);
    if (OUT == OUT_CONV) token_request += m0;
    M = max(0, min(M - m0, NT * 8));
  }
  const int my_tiles = first_tile < num_tiles ? (num_tiles - first_tile + tile_step - 1) / tile_step : 0;
  const int items = my_tiles * chunks;  // this block's work: the chunks of its row tiles, in order

  if (tid == 0) {
    abort_s = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], CONSUMERS);
    }
    mbar_init(&gathered, ksplit > 1 ? (unsigned)(ksplit - 1) : 1u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (ksplit > 1) cluster_meet();  // the first block's barrier exists before a peer arrives on it
  chain_release();
  // A bounded wait. When one runs out the launch is lost (the status flag says so), but every thread keeps
  // following the same path through the barriers, so the block still ends.
  auto wait_for = [&](uint64_t* bar, unsigned parity, int code) {
    if (*(volatile int*)&abort_s) return;
    if (!mbar_wait(bar, parity)) {
      *(volatile int*)&abort_s = 1;
      if (lane == 0) atomicExch(&g_skinny_status, code);
    }
  };

  if (warp == CONSUMERS) {
    // ---------------------------------------------------------------- producer: one thread, one box per stage (SwiGLU: two)
    if (lane == 0) {
      int tile = first_tile, chunk = 0;
      for (int n = 0; n < items; ++n) {
        const int s = n % STAGES;
        if (n >= STAGES) wait_for(&empty_bar[s], ((n / STAGES) & 1) ^ 1, 2);
        if (*(volatile int*)&abort_s) break;  // no more copies
        // rows 0-7 and 8-15 of the tile: 16 consecutive weight rows, or 8 gate rows and the 8 up rows under them
        const int row_lo = OUT == OUT_SWIGLU ? tile * 8 : tile * 16;
        const int row_hi = OUT == OUT_SWIGLU ? F + tile * 8 : tile * 16 + 8;
        unsigned char* dst = ring + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);  // rows or k past the matrix arrive as zeros and count too
        // An instruction that starts a TMA copy costs the issuing thread some 300 cycles whatever the copy holds, so
        // the boxes are as large as they can be: 16 rows x 512 k (16 KB), or two of 8 rows for SwiGLU's two halves.
        // (SwiGLU as a run of stages over 16 gate rows and then one over 16 up rows, one box a stage, measured
        // slower here: 0.926 against 0.898 ms a decode step of the 1.2B shape.)
        if (OUT == OUT_CONV) {  // 8 rows each of the projection's B, C and x parts, C = O / 3 rows apart
          for (int h = 0; h < 3; ++h)
            tma_load_box(dst + h * (STAGE_BYTES / 3), &map_w, h * (O / 3) + tile * 8, (chunk0 + chunk) * (KC / 64), &full_bar[s]);
        } else if (OUT == OUT_SWIGLU) {
          tma_load_box(dst, &map_w, row_lo, (chunk0 + chunk) * (KC / 64), &full_bar[s]);
          tma_load_box(dst + STAGE_BYTES / 2, &map_w, row_hi, (chunk0 + chunk) * (KC / 64), &full_bar[s]);
        } else {
          tma_load_box(dst, &map_w, row_lo, (chunk0 + chunk) * (KC / 64), &full_bar[s]);
        }
        if (++chunk == chunks) { chunk = 0; tile += tile_step; }
      }
    }
    // Copies may still be in flight: the block must not exit before they have landed. The consumers wait for
    // every stage they read; the producer stays until they are through (the block-wide barrier below).
  } else {
    // ---------------------------------------------------------------- consumers
    const int g = lane >> 2, t = lane & 3;
    if (OUT == OUT_CONV && tid < NT * 8) {
      // which request a token belongs to and where its state lies is what the host wrote for this step: looked up while
      // the kernel ahead is still at work, not once per tile in the read-out (two loads, one after the other)
      const int r = tid < M ? token_request[tid] : -1;
      slot_s[tid] = r >= 0 ? tail.slots[r] : -1;
    }
    if (IN == IN_BF16) {
      chain_wait();  // from here on the kernel reads what its predecessor wrote
#pragma unroll
      for (int m = 0; m < NT * 8; ++m) {  // all copies in flight together
        const size_t src = m < M ? (size_t)(rows ? rows[m] : m) : 0;
        for (int col = tid * 8; col < k_len; col += CONSUMERS * 32 * 8)
          cp_async16(xs + (size_t)m * XS + col, (const bf16*)x_ + src * K + k0 + col, m < M ? 16 : 0);
      }
      cp_async_commit();
      cp_async_wait<0>();
    } else {
      // float32 residual rows -> bf16(x * norm weight), with the sum of x^2 on the way. A warp takes 128-float blocks
      // of k (blocks warp, warp + 8, ...) for every token, two blocks a pass: the pass's 16 loads per lane (8 tokens x
      // 2 blocks) are all in flight at once, so a pass costs one trip to the L2, and the first pass's norm weights
      // are fetched before the kernel waits for its predecessor (they depend on nothing).
      constexpr int PER = 2;
      const int kblocks = (k_len + 127) / 128;
      float4 wv[PER];
#pragma unroll
      for (int p = 0; p < PER; ++p) {
        const int k = (warp + CONSUMERS * p) * 128 + lane * 4;
        wv[p] = k < k_len ? *reinterpret_cast<const float4*>(norm_w + k0 + k) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      chain_wait();  // from here on the kernel reads what its predecessor wrote
#pragma unroll 1
      for (int half = 0; half < NT; ++half) {  // 8 tokens at a time
        float ss[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) ss[i] = 0.f;
        for (int b0 = warp; b0 < kblocks; b0 += CONSUMERS * PER) {
          if (b0 != warp || half > 0) {
#pragma unroll
            for (int p = 0; p < PER; ++p) {
              const int k = (b0 + CONSUMERS * p) * 128 + lane * 4;
              wv[p] = k < k_len ? *reinterpret_cast<const float4*>(norm_w + k0 + k) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
          float4 v[PER][8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int m = half * 8 + i;
            const float* src = (const float*)x_ + (size_t)(m < M ? (rows ? rows[m] : m) : 0) * K + k0;
#pragma unroll
            for (int p = 0; p < PER; ++p) {
              const int k = (b0 + CONSUMERS * p) * 128 + lane * 4;
              v[p][i] = m < M && k < k_len ? *reinterpret_cast<const float4*>(src + k) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
#pragma unroll
          for (int p = 0; p < PER; ++p) {
            const int k = (b0 + CONSUMERS * p) * 128 + lane * 4;
            float4 w = wv[p];
            if (zero_centered) { w.x += 1.f; w.y += 1.f; w.z += 1.f; w.w += 1.f; }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 a = v[p][i];
              ss[i] = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, ss[i]))));
              uint2 packed;
              packed.x = pack_bf16(a.x * w.x, a.y * w.y);
              packed.y = pack_bf16(a.z * w.z, a.w * w.w);
              if (k < k_len) *reinterpret_cast<uint2*>(xs + (size_t)(half * 8 + i) * XS + k) = packed;
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float total = warp_sum(ss[i]);
          if (lane == 0) ss_s[warp][half * 8 + i] = total;
        }
      }
    }
    consumer_barrier();  // the activations are in shared memory for every consumer warp
    auto sum_sq = [&](int m) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < CONSUMERS; ++w) total += ss_s[w][m];
      return total;
    };

    // Where this thread's 16 bytes of weight rows g and g + 8 lie inside a stage: group of 64 k, row, and the 16-byte
    // unit (slice & 1) * 4 + t XOR g of the 128-byte swizzle. One box holds 16 rows to a group of k, SwiGLU's two boxes
    // 8 rows each. A warp multiplies 64 of a chunk's 512 k: slices 2 * warp and 2 * warp + 1 of 32 k.
    constexpr bool BOXES8 = OUT == OUT_SWIGLU || OUT == OUT_CONV;  // boxes of 8 rows: a group of 64 k is 1 KB
    constexpr int kg_stride = BOXES8 ? 1024 : 2048;
    constexpr int hi_off = OUT == OUT_CONV ? STAGE_BYTES / 3 : OUT == OUT_SWIGLU ? STAGE_BYTES / 2 : 1024;
    float acc[NT][4], acc_x[OUT == OUT_CONV ? NT : 1][4];  // acc_x: the convolution's x rows (rows g; rows g + 8 unused)
#pragma unroll
    for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
#pragma unroll
    for (int j = 0; j < (OUT == OUT_CONV ? NT : 1); ++j) { acc_x[j][0] = acc_x[j][1] = acc_x[j][2] = acc_x[j][3] = 0.f; }
    int tile = first_tile, c = 0, tiles_done = 0;
    for (int n = 0; n < items; ++n) {
      const int s = n % STAGES;
      wait_for(&full_bar[s], (n / STAGES) & 1, 1);
#pragma unroll
      for (int i2 = 0; i2 < 2; ++i2) {
        const int k = c * KC + warp * 64 + i2 * 32 + 8 * t;  // this thread's 8 consecutive k, counted from k0
        if (k < k_len) {
          const unsigned char* st = ring + (size_t)s * STAGE_BYTES + warp * kg_stride + g * 128 + (((i2 * 4 + t) ^ g) << 4);
          const uint4 a_lo = *reinterpret_cast<const uint4*>(st);
          const uint4 a_hi = *reinterpret_cast<const uint4*>(st + hi_off);
          const uint32_t a1[4] = {a_lo.x, a_hi.x, a_lo.y, a_hi.y};  // first k-step: this thread's k 0..3
          const uint32_t a2[4] = {a_lo.z, a_hi.z, a_lo.w, a_hi.w};  // second k-step: its k 4..7
          uint4 a_x = make_uint4(0u, 0u, 0u, 0u);
          if (OUT == OUT_CONV) a_x = *reinterpret_cast<const uint4*>(st + 2 * hi_off);
          const uint32_t x1[4] = {a_x.x, 0u, a_x.y, 0u}, x2[4] = {a_x.z, 0u, a_x.w, 0u};
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            const uint4 b = *reinterpret_cast<const uint4*>(xs + (size_t)(8 * j + g) * XS + k);
            mma_bf16(acc[j], a1, b.x, b.y);
            mma_bf16(acc[j], a2, b.z, b.w);
            if (OUT == OUT_CONV) {
              mma_bf16(acc_x[j], x1, b.x, b.y);
              mma_bf16(acc_x[j], x2, b.z, b.w);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);  // this warp has read the stage
      if (++c < chunks) continue;

      // the row tile is complete: the consumer warps' partial sums meet in shared memory, then the epilogue
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        float* r0 = red + (((size_t)warp * NT + j) * RT + g) * 8 + 2 * t;
        r0[0] = acc[j][0];
        r0[1] = acc[j][1];
        r0[64] = acc[j][2];  // row g + 8
        r0[65] = acc[j][3];
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        if (OUT == OUT_CONV) {
          r0[128] = acc_x[j][0];  // row g + 16: the x part
          r0[129] = acc_x[j][1];
          acc_x[j][0] = acc_x[j][1] = acc_x[j][2] = acc_x[j][3] = 0.f;
        }
      }
      constexpr int per_tile = BOXES8 ? 64 : 128;  // (row, token) pairs per n-block
      static_assert(2 * 128 <= CONSUMERS * 32, "a thread reads out at most one (row, token) pair of a tile");
      float before = 0.f;  // the residual stream's value, on its way while the sums meet
      if (OUT == OUT_ACC && ksplit == 1 && tid < NT * per_tile) {
        const int m = 8 * (tid / per_tile) + tid % 8, o = tile * 16 + (tid % per_tile) / 8;
        if (m < M && o < O) before = ((const float*)y_)[(size_t)m * O + o];
      }
      // The convolution's taps, bias and state rows of this thread's (channel, token), likewise (up to 4 taps; longer
      // ones are read where they are used).
      constexpr int TAPS = 4;
      float taps_r[TAPS] = {0.f, 0.f, 0.f, 0.f}, hist_r[TAPS - 1] = {0.f, 0.f, 0.f}, bias_r = 0.f;
      if (OUT == OUT_CONV && tail.L <= TAPS && tid < NT * per_tile) {
        const int m = 8 * (tid / per_tile) + tid % 8, C = O / 3, c = tile * 8 + (tid % per_tile) / 8;
        const int slot = m < M ? slot_s[m] : -1;
        if (slot >= 0 && c < C) {
          const float* hist = tail.state + (size_t)slot * (tail.L - 1) * C + c;
#pragma unroll
          for (int l = 0; l < TAPS; ++l) {
            if (l < tail.L) taps_r[l] = tail.taps[(size_t)c * tail.L + l];
            if (l < tail.L - 1) hist_r[l] = hist[(size_t)l * C];
          }
          if (tail.bias) bias_r = tail.bias[c];
        }
      }
      consumer_barrier();
      for (int i = tid; i < NT * per_tile; i += CONSUMERS * 32) {
        const int j = i / per_tile, row = (i % per_tile) / 8, tok = i % 8;
        const int m = 8 * j + tok;
        if (m >= M) continue;
        float v = 0.f, u = 0.f, xv = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) {
          const float* r0 = red + (((size_t)w * NT + j) * RT + row) * 8 + tok;
          v += r0[0];
          if (BOXES8) u += r0[64];
          if (OUT == OUT_CONV) xv += r0[128];
        }
        if (ksplit > 1) {  // a part of K: kept until the parts meet
          part[tiles_done * NT * 128 + i] = v;
          continue;
        }
        if (IN == IN_NORM) {
          const float inv = 1.f / sqrtf(sum_sq(m) / (float)K + eps);
          v *= inv;
          u *= inv;
          xv *= inv;
        }
        if (OUT == OUT_CONV) {
          // v, u, xv: the B, C and x parts of channel c for token m, rounded as the projection's own read-out would
          const int C = O / 3, c = tile * 8 + row, L = tail.L;
          if (c >= C) continue;
          const int slot = slot_s[m];
          bf16* out = (bf16*)y_ + (size_t)m * C + c;
          if (slot < 0) {
            *out = __float2bfloat16_rn(0.f);
            continue;
          }
          const float bq = to_f32(__float2bfloat16_rn(v)), cq = to_f32(__float2bfloat16_rn(u)), xq = to_f32(__float2bfloat16_rn(xv));
          const float uu = bq * xq;
          float* hist = tail.state + (size_t)slot * (L - 1) * C + c;
          float sum = 0.f;
          if (L <= TAPS) {  // (everything is in registers already)
#pragma unroll
            for (int l = 0; l < TAPS - 1; ++l) {
              if (l < L - 1) {
                sum = fmaf(hist_r[l], taps_r[l], sum);
                if (l > 0 && tail.write) hist[(size_t)(l - 1) * C] = hist_r[l];
              }
            }
            float last = taps_r[0];
#pragma unroll
            for (int l = 1; l < TAPS; ++l) last = l == L - 1 ? taps_r[l] : last;
            sum = fmaf(uu, last, sum);
            if (tail.write) hist[(size_t)(L - 2) * C] = uu;
            if (tail.bias) sum += bias_r;
          } else {
            for (int l = 0; l < L - 1; ++l) {
              const float h = hist[(size_t)l * C];
              sum = fmaf(h, tail.taps[(size_t)c * L + l], sum);
              if (l > 0 && tail.write) hist[(size_t)(l - 1) * C] = h;
            }
            sum = fmaf(uu, tail.taps[(size_t)c * L + L - 1], sum);
            if (tail.write) hist[(size_t)(L - 2) * C] = uu;
            if (tail.bias) sum += tail.bias[c];
          }
          *out = __float2bfloat16_rn(cq * sum);
        } else if (OUT == OUT_SWIGLU) {
          const int f = tile * 8 + row;
          if (f < F) ((bf16*)y_)[(size_t)m * F + f] = __float2bfloat16_rn(v / (1.f + expf(-v)) * u);
        } else {
          const int o = tile * 16 + row;
          if (o >= O) continue;
          const size_t at = (size_t)m * O + o;
          if (OUT == OUT_BF16) ((bf16*)y_)[at] = __float2bfloat16_rn(v);
          else if (OUT == OUT_F32) ((float*)y_)[at] = v;
          else ((float*)y_)[at] = before + v;
        }
      }
      consumer_barrier();  // `red` is free again before the next tile's sums are written
      c = 0;
      tile += tile_step;
      ++tiles_done;
    }

    if (ksplit > 1 && !BOXES8) {
      // ---------------------------------------------------------------- the parts of K meet in the first block
      const int count = my_tiles * NT * 128;
      if (rank > 0) {
        const unsigned to = peer_address(peer, 0) + (unsigned)((rank - 1) * SPLIT_TILES * NT * 128 * 4);
        for (int i = tid; i < count; i += CONSUMERS * 32) peer_store(to + (unsigned)i * 4u, part[i]);
        if (IN == IN_NORM && tid < NT * 8) peer_store(peer_address(peer_ss, 0) + (unsigned)(((rank - 1) * NT * 8 + tid) * 4), sum_sq(tid));
        consumer_barrier();  // all of this block's sums are on their way; one thread tells the first block
        if (tid == 0) {
          asm volatile("fence.acq_rel.cluster;" ::: "memory");
          asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(peer_address(&gathered, 0)) : "memory");
        }
      } else {
        constexpr int MOST = (SPLIT_TILES * NT * 128 + CONSUMERS * 32 - 1) / (CONSUMERS * 32);  // pairs a thread writes
        float before[MOST];  // the residual stream's values, fetched while the other parts are on their way
#pragma unroll
        for (int n = 0; n < MOST; ++n) {
          before[n] = 0.f;
          const int i = tid + n * CONSUMERS * 32;
          if (OUT == OUT_ACC && i < count) {
            const int tl = i / (NT * 128), e = i % (NT * 128);
            const int m = 8 * (e / 128) + e % 8, o = (first_tile + tl * tile_step) * 16 + (e % 128) / 8;
            if (m < M && o < O) before[n] = ((const float*)y_)[(size_t)m * O + o];
          }
        }
        if (!*(volatile int*)&abort_s && !mbar_wait_cluster(&gathered, 0)) {
          *(volatile int*)&abort_s = 1;
          if (lane == 0) atomicExch(&g_skinny_status, 3);
        }
        if (!*(volatile int*)&abort_s) {
#pragma unroll
          for (int n = 0; n < MOST; ++n) {
            const int i = tid + n * CONSUMERS * 32;
            if (i >= count) continue;
            const int tl = i / (NT * 128), e = i % (NT * 128);
            const int j = e / 128, row = (e % 128) / 8, tok = e % 8;
            const int m = 8 * j + tok, o = (first_tile + tl * tile_step) * 16 + row;
            if (m >= M || o >= O) continue;
            float v = part[i], ss = IN == IN_NORM ? sum_sq(m) : 0.f;
            for (int r = 0; r < ksplit - 1; ++r) {  // in rank order
              v += peer[(r * SPLIT_TILES + tl) * NT * 128 + e];
              if (IN == IN_NORM) ss += peer_ss[r * NT * 8 + m];
            }
            if (IN == IN_NORM) v *= 1.f / sqrtf(ss / (float)K + eps);
            const size_t at = (size_t)m * O + o;
            if (OUT == OUT_BF16) ((bf16*)y_)[at] = __float2bfloat16_rn(v);
            else if (OUT == OUT_F32) ((float*)y_)[at] = v;
            else ((float*)y_)[at] = before[n] + v;
          }
        }
      }
    }
  }
  if (*(volatile int*)&abort_s) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // a lost launch: give copies still in flight time to land
  }
  __syncthreads();  // nobody leaves while a copy into this block's shared memory may be in flight
  if (ksplit > 1) cluster_meet();  // nor while a peer may still write its sums there
}

// ------------------------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (EncodeTiled)p;
  }();
  return fn;
}

std::mutex g_map_mutex;
std::map<std::tuple<const void*, int, int, int>, CUtensorMap> g_maps;  // one map per weight matrix and box height

// The matrix [O, K] seen as [K / 64][O][64]: boxes of 64 k x 16 (SwiGLU: 8) rows x 8 groups of k, 128-byte swizzle, zeros outside.
int weight_map(CUtensorMap* out, const void* w, int O, int K, int box_rows) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const auto key = std::make_tuple(w, O, K, box_rows);
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    EncodeTiled fn = encode_tiled();
    if (!fn) return 3001;
    const cuuint64_t dims[3] = {64, (cuuint64_t)O, (cuuint64_t)(K / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
    const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, KC / 64};
    const cuuint32_t elem[3] = {1, 1, 1};
    CUtensorMap map;
    const CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(w), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 3000 + (int)r;
    it = g_maps.emplace(key, map).first;
  }
  *out = it->second;
  return 0;
}

constexpr int kMaxSmemBytes = 226 * 1024;  // the block also has a few hundred bytes of static shared memory

// Shared memory of a block with `ksplit` parts of K: alignment slack, the ring, the consumers' partial sums, the
// parts' meeting place, and the activations of this block's part of K.
template <int NT, int OUTM>
int block_smem(int K, int ksplit) {
  const int chunks = (K + KC - 1) / KC, part_k = (chunks + ksplit - 1) / ksplit * KC;
  int bytes = 1024 + Ring<OUTM>::DEPTH * Ring<OUTM>::BYTES + CONSUMERS * NT * Ring<OUTM>::ROWS * 8 * (int)sizeof(float) +
              NT * 8 * (part_k + 32) * (int)sizeof(bf16);
  if (ksplit > 1) bytes += (ksplit * SPLIT_TILES * NT * 128 + (ksplit - 1) * NT * 8) * (int)sizeof(float);
  return bytes;
}

struct SplitPlan {
  int ksplit, grid, smem;
};

template <int NT, int IN, int OUTM>
int launch_one(int num_tiles, const void* x, const int* rows, const float* norm_w, float eps, int zero_centered,
               const void* W, void* y, int M, int O, int K, const ConvTail& tail, int groups, cudaStream_t stream) {
  auto kernel = groups > 1 ? skinny_gemm_kernel<NT, IN, OUTM, true> : skinny_gemm_kernel<NT, IN, OUTM, false>;
  constexpr bool UNCUT = OUTM == OUT_SWIGLU || OUTM == OUT_CONV;  // read-outs that need a tile's whole K in one block
  if (block_smem<NT, OUTM>(K, 1) > kMaxSmemBytes && (UNCUT || block_smem<NT, OUTM>(K, MAX_KSPLIT) > kMaxSmemBytes))
    return (int)cudaErrorInvalidValue;
  static int sms_of[64] = {};  // by device ordinal, like the plans below: a launch attribute belongs to a device
  static std::mutex mutex;
  static std::map<std::tuple<int, int, int, int>, SplitPlan> plans;  // (device, tiles, token groups, K) -> how the product is cut
  static std::map<std::tuple<int, int, int>, int> cluster_room;  // (device, ksplit, smem) -> clusters resident at once
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  SplitPlan plan;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (sms_of[device] == 0) {
      cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<NT, IN, OUTM, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemBytes);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(skinny_gemm_kernel<NT, IN, OUTM, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemBytes);
      if (e != cudaSuccess) return (int)e;
      cudaDeviceGetAttribute(&sms_of[device], cudaDevAttrMultiProcessorCount, device);
    }
    const int sms = sms_of[device];
    const auto key = std::make_tuple(device, num_tiles, groups, K);
    auto found = plans.find(key);
    if (found == plans.end()) {
      // What the busiest SM must fetch, in bytes, if the product is cut into `ksplit` parts of K: its blocks' weights
      // and activations. A cut costs an exchange at the end that grows with the number of parts, counted as the
      // bytes the SM could have fetched meanwhile (30 KB a part; AKAS_B200_SKINNY_PART_COST sets another figure); an
      // SM with a single block streams about 30 % slower than one with two. On the 1.2B shape this cuts only the down
      // projection (4 parts) and leaves the out and qkv projections whole. Measured, a decode step of 8 requests:
      // 0.811 ms at 6 KB a part, 0.757 at 12 KB (out projection in 2 parts, qkv in 4), 0.740 at 30 KB, 0.742 at 60 KB
      // (nothing cut).
      const int chunks = (K + KC - 1) / KC;
      long long best = -1;
      plan = SplitPlan{1, 0, 0};
      for (int ksplit = 1; ksplit <= MAX_KSPLIT; ksplit *= 2) {
        if (ksplit > 1 && (UNCUT || ksplit > chunks)) break;
        const int smem = block_smem<NT, OUTM>(K, ksplit);
        if (smem > kMaxSmemBytes) continue;
        static const int per_sm_cap = [] { const char* v = getenv("AKAS_B200_SKINNY_PER_SM"); return v ? atoi(v) : 3; }();
        const int per_sm = max(1, min(per_sm_cap, kMaxSmemBytes / (smem + 1024)));
        int clusters = sms * per_sm / ksplit;
        if (ksplit > 1) {
          const auto room_key = std::make_tuple(device, ksplit, smem);
          if (!cluster_room.count(room_key)) {
            cudaLaunchConfig_t config = {};
            config.gridDim = dim3(ksplit * 64);
            config.blockDim = dim3(THREADS);
            config.dynamicSmemBytes = smem;
            cudaLaunchAttribute attribute[1];
            attribute[0].id = cudaLaunchAttributeClusterDimension;
            attribute[0].val.clusterDim.x = ksplit;
            attribute[0].val.clusterDim.y = 1;
            attribute[0].val.clusterDim.z = 1;
            config.attrs = attribute;
            config.numAttrs = 1;
            int room = 0;
            if (cudaOccupancyMaxActiveClusters(&room, kernel, &config) != cudaSuccess) { cudaGetLastError(); room = 0; }
            cluster_room[room_key] = room;
          }
          clusters = min(clusters, cluster_room[room_key]);
          if (clusters < 1) continue;
        }
        // every row tile is the work of `groups` clusters (one per group of tokens) that run side by side: the
        // clusters come in sets of that many, and every set gets the same number of row tiles (to within one)
        int sets = min(max(1, clusters / groups), num_tiles);
        const int rounds = (num_tiles + sets - 1) / sets;
        if (ksplit > 1 && rounds > SPLIT_TILES) continue;
        sets = (num_tiles + rounds - 1) / rounds;
        clusters = sets * groups;
        const int blocks = clusters * ksplit, on_busiest_sm = (blocks + sms - 1) / sms;
        const long long part_k = (long long)(chunks + ksplit - 1) / ksplit * KC;
        long long fetched = on_busiest_sm * (rounds * 16 * part_k * 2 + NT * 8 * part_k * 2);
        if (on_busiest_sm == 1) fetched += fetched * 3 / 10;  // one ring per SM keeps too few bytes in flight
        static const int part_cost = [] { const char* v = getenv("AKAS_B200_SKINNY_PART_COST"); return v ? atoi(v) : 30000; }();
        if (ksplit > 1) fetched += (long long)part_cost * ksplit;
        if (best < 0 || fetched < best) {
          best = fetched;
          plan = SplitPlan{ksplit, blocks, smem};
        }
      }
      if (best < 0) return (int)cudaErrorInvalidValue;
      plans[key] = plan;
    } else {
      plan = found->second;
    }
  }
  CUtensorMap map;
  const int err = weight_map(&map, W, O, K, UNCUT ? 8 : 16);
  if (err) return err;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(plan.grid);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = plan.smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  int n = 0;
  if (chained_launches_enabled()) {
    attribute[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (plan.ksplit > 1) {
    attribute[n].id = cudaLaunchAttributeClusterDimension;
    attribute[n].val.clusterDim.x = plan.ksplit;
    attribute[n].val.clusterDim.y = 1;
    attribute[n].val.clusterDim.z = 1;
    ++n;
  }
  config.attrs = attribute;
  config.numAttrs = n;
  return (int)cudaLaunchKernelEx(&config, kernel, map, x, rows, norm_w, eps, zero_centered, y, M, O, K, num_tiles, plan.ksplit, groups, tail);
}

template <int NT, int IN>
int launch_out(int out_mode, const void* x, const int* rows, const float* norm_w, float eps, int zero_centered,
               const void* W, void* y, int M, int O, int K, const ConvTail& tail, int groups, cudaStream_t stream) {
  const int tiles = (O + 15) / 16;
  switch (out_mode) {
    case OUT_BF16: return launch_one<NT, IN, OUT_BF16>(tiles, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, tail, groups, stream);
    case OUT_F32: return launch_one<NT, IN, OUT_F32>(tiles, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, tail, groups, stream);
    case OUT_ACC: return launch_one<NT, IN, OUT_ACC>(tiles, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, tail, groups, stream);
    case OUT_SWIGLU:
      return launch_one<NT, IN, OUT_SWIGLU>((O / 2 + 7) / 8, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, tail, groups, stream);
    case OUT_CONV:
      return launch_one<NT, IN, OUT_CONV>((O / 3 + 7) / 8, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, tail, groups, stream);
    default: return (int)cudaErrorInvalidValue;
  }
}

}  // namespace

// x: bfloat16 [M, K] (in_mode 0) or float32 [*, K] rows gathered by `rows` (or 0..M-1) with RMSNorm fused (in_mode 1).
// W: bfloat16 [O, K]. y: [M, O] in the output mode's type, or bfloat16 [M, O / 2] for swiglu (out_mode 3).
// Returns 0, a CUDA error code, or 3000 + a driver error from building the weights' tensor map.
static int skinny_dispatch(const void* x, const int* rows, const float* norm_w, float eps, int zero_centered, const void* W,
                           void* y, int M, int O, int K, int in_mode, int out_mode, const ConvTail& tail, cudaStream_t stream) {
  if (M <= 0 || O <= 0) return 0;
  if (M > 16 || K <= 0 || K % 64 || (out_mode == OUT_SWIGLU && O % 2) || (out_mode == OUT_CONV && O % 3)) return (int)cudaErrorInvalidValue;
  if (in_mode == IN_NORM && norm_w == nullptr) return (int)cudaErrorInvalidValue;
  if ((uintptr_t)W % 16 || (uintptr_t)x % 16) return (int)cudaErrorInvalidValue;  // TMA and 16-byte loads
  // 9 to 16 tokens: as two groups of 8 on the kernel for 8, whose blocks then come in pairs that read the same weights
  // (the second mostly from the L2), rather than on the kernel for 16, whose activations leave room for one block per
  // SM only (AKAS_B200_SKINNY_GROUPS=0: that kernel).
  static const bool in_groups = [] { const char* v = getenv("AKAS_B200_SKINNY_GROUPS"); return !(v && v[0] == '0'); }();
  if (M <= 8 || in_groups) {
    const int groups = M <= 8 ? 1 : 2;
    if (in_mode == IN_BF16) return launch_out<1, IN_BF16>(out_mode, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, tail, groups, stream);
    return launch_out<1, IN_NORM>(out_mode, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, tail, groups, stream);
  }
  if (in_mode == IN_BF16) return launch_out<2, IN_BF16>(out_mode, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, tail, 1, stream);
  return launch_out<2, IN_NORM>(out_mode, x, rows, norm_w, eps, zero_centered, W, y, M, O, K, tail, 1, stream);
}

AKAS_API int akas_skinny_gemm(const void* x, const int* rows, const float* norm_w, float eps, int zero_centered,
                              const void* W, void* y, int M, int O, int K, int in_mode, int out_mode,
                              cudaStream_t stream) {
  if (out_mode < OUT_BF16 || out_mode > OUT_SWIGLU) return (int)cudaErrorInvalidValue;
  return skinny_dispatch(x, rows, norm_w, eps, zero_centered, W, y, M, O, K, in_mode, out_mode, ConvTail{}, stream);
}

// The in projection of a gated short convolution and the convolution itself, for a decode step: W bfloat16 [3C, K]
// (the B, C and x parts), x as for akas_skinny_gemm, every token the single token of request seq_of_token[t] (or -1:
// padding, its output is zero) whose state row is slots[request]; taps float32 [C, L], bias float32 [C] or null,
// state float32 [slots, L - 1, C] (read, and shifted by the token unless write is 0); y bfloat16 [M, C].
AKAS_API int akas_skinny_gemm_conv(const void* x, const int* rows, const float* norm_w, float eps, int zero_centered,
                                   const void* W, void* y, int M, int C, int K, int in_mode, const float* taps,
                                   const float* bias, float* state, const int* seq_of_token, const int* slots, int L,
                                   int write, cudaStream_t stream) {
  if (L < 2 || L > 16 || C <= 0 || taps == nullptr || state == nullptr || seq_of_token == nullptr || slots == nullptr)
    return (int)cudaErrorInvalidValue;
  const ConvTail tail{taps, bias, state, seq_of_token, slots, L, write};
  return skinny_dispatch(x, rows, norm_w, eps, zero_centered, W, y, M, 3 * C, K, in_mode, OUT_CONV, tail, stream);
}

// 0 if no bounded wait of the kernel has ever run out on the current device, else the code of the last one
// (1: consumers waited for a stage that never filled, 2: the producer waited for a stage that never emptied).
// Synchronises with the device.
AKAS_API int akas_skinny_gemm_status() {
  int status = -1;
  const cudaError_t e = cudaMemcpyFromSymbol(&status, g_skinny_status, sizeof(int));
  return e == cudaSuccess ? status : -(int)e;
}
