// A decode step's chain of small operations as ONE persistent launch: a program of matrix products for a
// handful of tokens (with RMSNorm, SwiGLU and the residual add fused as in skinny_gemm.cu), short-convolution
// steps and the embedding look-up, run by one block per SM with a grid-wide barrier between operations.
//
// Why. A decode step of a 16-layer model is about a hundred launches of a few microseconds each. Every launch
// pays for its ramp and its tail: the weight stream starts from an empty pipe and the last blocks finish alone,
// so that products of 8 to 70 MB reach a third to a half of the memory bandwidth. Here the weight stream never
// stops: in every block one producer thread walks the WHOLE program and keeps a ring of weight chunks full by
// TMA, whatever the other warps are doing, so that while they meet at the barrier between two operations and
// fetch the next operation's activations, the next operation's weights are already on their way.
//
// A block has one producer warp, 8 consumer warps and one writer warp.
//   producer   for every product of the program, in order: for every row tile of this block, for every 512-wide
//              chunk of K, ONE TMA box load of 16 rows x 512 k (16 KB) into the next stage of the ring, bytes
//              counted on the stage's "full" mbarrier; held back only by the stage's "empty" mbarrier. (An
//              instruction that starts a TMA copy costs the issuing thread some 300 cycles whatever the copy
//              holds: with 4 KB boxes one thread could not feed an SM's share of the memory bandwidth.)
//   consumers  per operation: fetch the activations into shared memory (bfloat16 rows as they are; float32 rows
//              of the residual stream weighted by the norm's weights, with the sum of squares on the way), then
//              two warps share a stage, half of its k each: 16-byte reads of the weight rows, mma.sync m16n8k16
//              with the weights as A and the tokens as B (8 tokens per n-block). At the end of a row tile the
//              warps put their sums into one of two buffers in shared memory and go on with the next tile.
//   writer     adds the warps' sums of a finished tile (always in the same order) and writes bf16 / f32 / y += /
//              silu(gate) * up, while the consumers multiply the next tile: stores to global memory never hold
//              them up. At the end of an operation it goes to the grid's meeting straight from its last store.
// Row tiles. A tile is 16 consecutive rows of W. For SwiGLU a tile is 16 channels: a run of stages over the 16 gate
// rows, then a run over the 16 up rows under them of the stacked [2F, K] matrix; the writer keeps the gate sums in
// registers until the up sums arrive. Block b takes tiles b, b + grid, ...
// Inner sizes beyond 4,096 (a down projection) do not fit the activations' room in shared memory: such a product
// (residual add only) is cut along K into parts of at most 4,096; block b takes part b % parts of tiles b / parts,
// b / parts + grid / parts, ..., so it needs one part of the activations only, and the parts of a tile are added to
// the residual stream in the order of their numbers (the writer of part p waits for a per-tile counter to reach p),
// so that the sum does not depend on timing.
// Other operations are run by the consumer warps alone, spread over the blocks: the short convolution of decode
// steps (a block owns channels, so it may read and rewrite their state), the embedding look-up.
//
// The grid barrier is one word in global memory that every block's writer adds to and then polls (block 0 adds what
// makes the top bit flip when all have arrived: no reset is needed, whatever the word held). The kernel is launched
// cooperatively, so all blocks are resident. Every wait (mbarriers, the grid barrier, the tile counters) is bounded;
// a wait that runs out sets a status word (akas_chain_status), everyone stops waiting, and the launch runs to its
// end with results that are not valid. Results do not depend on what else runs: summation order is fixed.
#include <cuda.h>
#include <math.h>

#include "mma.cuh"
#include "tcgen05.cuh"

using namespace akas;
using akas::tc::mbar_arrive;
using akas::tc::mbar_expect_tx;
using akas::tc::mbar_init;
using akas::tc::mbar_wait;
using akas::tc::smem_u32;

namespace {

constexpr int CONSUMERS = 8, KC = 512;                  // consumer warps; k per chunk
constexpr int XK = 4096;                                // the most k of activations that shared memory holds
constexpr int STAGE_BYTES = 16 * KC * 2;                // 16 weight rows x KC: [8 groups of 64 k][16 rows][128 bytes]
constexpr int WPS = 2;                                  // consumer warps that share a stage, half of its k each
constexpr int PAIRS = CONSUMERS / WPS;                  // stages that are multiplied at the same time
constexpr int THREADS = (CONSUMERS + 2) * 32;           // consumer warps, the producer warp, the writer warp
constexpr int BAR_FULL = 2, BAR_FREE = 4, BAR_OP = 6, BAR_PRE = 7;  // named barriers (1: the consumers; FULL, FREE: two each)
constexpr int WORKERS = (CONSUMERS + 1) * 32;           // the threads that meet at an operation's end: consumers and writer
constexpr int NW_MAX = 2048;                            // norm weights of the next operation kept in shared memory (NT = 1)
constexpr int XSTRIDE = XK + 32;                        // elements per activation row in shared memory
constexpr int MAX_OPS = 24;
constexpr int MAX_SPLIT_TILES = 8192;                   // tile counters of a product that is cut along K
constexpr unsigned kBarrierSpins = 1u << 24;
enum { OP_GEMM = 0, OP_CONV = 1, OP_EMBED = 2 };
enum { IN_BF16 = 0, IN_NORM = 1 };
enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_ACC = 2, OUT_SWIGLU = 3 };

struct alignas(64) ChainOp {
  CUtensorMap map;       // product: the weights as [K / 64][O][64]
  const void* x;         // product: activations; conv: bcx; embed: token ids
  const void* aux0;      // product: rows (int32) or null; conv: taps; embed: table
  const void* aux1;      // product: norm weights; conv: bias or null
  const void* aux2;      // conv: seq_of_token
  const void* aux3;      // conv: slots
  void* y;               // output
  void* y2;              // conv: state
  int kind, in_mode, out_mode;
  int M, O, K;           // product sizes; conv: tokens, channels, taps; embed: tokens, columns, -
  int tiles;             // product: row tiles (SwiGLU: tiles of 16 channels)
  int flag;              // product: zero_centered; conv: write; embed: dtype of the table
  float eps;
  int parts;             // product: parts of K (1 unless K > XK)
  int part_chunks;       // product: chunks of K in a part
  int pad;
};

struct Program {
  ChainOp ops[MAX_OPS];
  int count;
  unsigned* barrier;     // the grid's meeting word
  int* counters;         // [MAX_SPLIT_TILES] zero between operations
};

__device__ int g_chain_status = 0;  // 0, or the code of a wait that ran out (1 full stage, 2 empty stage, 3 grid barrier, 4 tile counter)

// This block's share of a product: tiles first, first + step, ... (count of them), chunks [chunk0, chunk0 + chunks)
// of K, and `runs` runs of stages per tile (2 for SwiGLU: the gate rows, then the up rows).
struct Share {
  int first, step, count, chunk0, chunks, runs, part;
  __device__ Share(const ChainOp& op, int b, int G) {
    const int total = (op.K + KC - 1) / KC;
    runs = op.out_mode == OUT_SWIGLU ? 2 : 1;
    if (op.parts > 1) {
      step = G / op.parts;
      part = b % op.parts;
      first = b / op.parts;
      chunk0 = part * op.part_chunks;
      chunks = min(op.part_chunks, total - chunk0);
      count = first < step && first < op.tiles && chunks > 0 ? (op.tiles - first + step - 1) / step : 0;
    } else {
      step = G;
      part = 0;
      first = b;
      chunk0 = 0;
      chunks = total;
      count = first < op.tiles ? (op.tiles - first + step - 1) / step : 0;
    }
  }
  // the first weight row of run `run` of tile `tile`
  __device__ int row(const ChainOp& op, int tile, int run) const { return (run ? op.O / 2 : 0) + tile * 16; }
};

__device__ __forceinline__ void tma_load_box(void* smem_dst, const CUtensorMap* map, int row, int group, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(smem_u32(smem_dst)), "l"(map), "r"(0), "r"(row), "r"(group), "r"(smem_u32(bar)) : "memory");
}
// What another block wrote earlier in this launch is read from the L2, never from this SM's L1.
__device__ __forceinline__ float ldcg_bf16(const bf16* p) {
  return to_f32(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(p))));
}
__device__ __forceinline__ unsigned load_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory"); }
__device__ __forceinline__ void named_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
// Arrives without waiting and without a fence: a fence would wait for every earlier store of the thread, stores to
// global memory included, and under a busy memory system those take microseconds to be acknowledged. The writer warp
// has only read the buffer it hands back (its global stores are fenced once, at the operation's end); the consumers
// fence by themselves before they arrive (they have no global stores in flight).
__device__ __forceinline__ void named_arrive(int id, int count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// The same once `value` has been computed: the arrival's count is made to depend on it, so the instruction cannot issue
// while a load that feeds the value is still in flight. For a thread that hands back a buffer it has only read.
__device__ __forceinline__ void named_arrive_after(int id, int count, float value) {
  unsigned zero;
  asm volatile("and.b32 %0, %1, 0;" : "=r"(zero) : "r"(__float_as_uint(value)));
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count + (int)zero) : "memory");
}

template <int NT, int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
decode_chain_kernel(const __grid_constant__ Program prog) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  float* red = reinterpret_cast<float*>(ring + STAGES * STAGE_BYTES);  // [2][CONSUMERS][NT][16][8] partial sums
  bf16* xs = reinterpret_cast<bf16*>(red + 2 * CONSUMERS * NT * 128);  // [NT * 8][XSTRIDE] activations
  float* nw_s = reinterpret_cast<float*>(xs + NT * 8 * XSTRIDE);       // [NW_MAX] norm weights fetched ahead (NT = 1 only)
  constexpr bool kNormAhead = NT == 1;
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES];
  __shared__ float ss_s[NT * 8];
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = (int)gridDim.x, b = (int)blockIdx.x;

  if (tid == 0) {
    abort_s = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], WPS);  // the consumer warps that multiply the stage
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  auto wait_for = [&](uint64_t* bar, unsigned parity, int code) {
    if (*(volatile int*)&abort_s) return;
    if (!mbar_wait(bar, parity)) {
      *(volatile int*)&abort_s = 1;
      if (lane == 0) atomicExch(&g_chain_status, code);
    }
  };

  if (warp == CONSUMERS) {
    // ---------------------------------------------------------------- producer: one thread, the whole program
    if (lane == 0) {
      unsigned n = 0;
      for (int i = 0; i < prog.count; ++i) {
        const ChainOp& op = prog.ops[i];
        if (op.kind != OP_GEMM) continue;
        const Share sh(op, b, G);
        for (int t = 0; t < sh.count; ++t) {
          for (int run = 0; run < sh.runs; ++run) {
            const int row = sh.row(op, sh.first + t * sh.step, run);
            for (int c = 0; c < sh.chunks; ++c, ++n) {
              const unsigned s = n % STAGES;
              if (n >= (unsigned)STAGES) wait_for(&empty_bar[s], ((n / STAGES) & 1) ^ 1, 2);
              if (*(volatile int*)&abort_s) break;
              mbar_expect_tx(&full_bar[s], STAGE_BYTES);  // rows or k past the matrix arrive as zeros and count too
              tma_load_box(ring + (size_t)s * STAGE_BYTES, &op.map, row, (sh.chunk0 + c) * (KC / 64), &full_bar[s]);
            }
            if (*(volatile int*)&abort_s) break;
          }
          if (*(volatile int*)&abort_s) break;
        }
        if (*(volatile int*)&abort_s) break;
      }
    }
  } else if (warp < CONSUMERS) {
    // ---------------------------------------------------------------- consumers
    const int g = lane >> 2, t = lane & 3;
    unsigned n = 0, deposits = 0;
    chain_wait();  // what came before this launch on the stream is complete
    for (int i = 0; i < prog.count; ++i) {
      const ChainOp& op = prog.ops[i];
      if (op.kind == OP_GEMM) {
        const int M = op.M, K = op.K;
        const Share sh(op, b, G);
        const int k0 = sh.chunk0 * KC, k_len = min(K, (sh.chunk0 + sh.chunks) * KC) - k0;  // this block's k
        const int* rows = (const int*)op.aux0;
        if (sh.count > 0) {
          if (op.in_mode == IN_BF16) {
            const int per_row = k_len / 8;
            for (int e = tid; e < NT * 8 * per_row; e += CONSUMERS * 32) {  // all copies in flight together
              const int m = e / per_row, col = (e % per_row) * 8;
              const size_t src = m < M ? (size_t)(rows ? rows[m] : m) : 0;
              cp_async16(xs + (size_t)m * XSTRIDE + col, (const bf16*)op.x + src * K + k0 + col, m < M ? 16 : 0);
            }
            cp_async_commit();
            cp_async_wait<0>();
          } else {
            // float32 residual rows -> bf16(x * norm weight); each warp owns tokens warp, warp + 8 and sums x^2
            const bool ahead = kNormAhead && i > 0 && K <= NW_MAX;  // fetched into shared memory before the barrier
            const float* norm_w = ahead ? nw_s : (const float*)op.aux1;
            if (ahead) {
              cp_async_wait<0>();
              consumer_barrier();
            }
            for (int m = warp; m < NT * 8; m += CONSUMERS) {
              float ss = 0.f;
              bf16* dst = xs + (size_t)m * XSTRIDE;
              if (m < M) {
                const float* src = (const float*)op.x + (size_t)(rows ? rows[m] : m) * K;
                // Sixteen 16-byte loads of the row and sixteen of the weights are asked for before any is used: under a
                // busy memory system a round trip takes microseconds, and this staging sits between two operations.
                for (int kb = lane * 4; kb < K; kb += 128 * 16) {
                  float4 v[16], w[16];
#pragma unroll
                  for (int u = 0; u < 16; ++u) {
                    const int k = kb + u * 128;
                    v[u] = k < K ? __ldcg(reinterpret_cast<const float4*>(src + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
                  }
#pragma unroll
                  for (int u = 0; u < 16; ++u) {
                    const int k = kb + u * 128;
                    w[u] = k < K ? *reinterpret_cast<const float4*>(norm_w + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                  }
#pragma unroll
                  for (int u = 0; u < 16; ++u) {
                    const int k = kb + u * 128;
                    if (k >= K) break;
                    if (op.flag) { w[u].x += 1.f; w[u].y += 1.f; w[u].z += 1.f; w[u].w += 1.f; }
                    ss = fmaf(v[u].x, v[u].x, fmaf(v[u].y, v[u].y, fmaf(v[u].z, v[u].z, fmaf(v[u].w, v[u].w, ss))));
                    uint2 packed;
                    packed.x = pack_bf16(v[u].x * w[u].x, v[u].y * w[u].y);
                    packed.y = pack_bf16(v[u].z * w[u].z, v[u].w * w[u].w);
                    *reinterpret_cast<uint2*>(dst + k) = packed;
                  }
                }
                ss = warp_sum(ss);
              } else {
                for (int k = lane * 4; k < K; k += 128) *reinterpret_cast<uint2*>(dst + k) = make_uint2(0u, 0u);
              }
              if (lane == 0) ss_s[m] = ss;
            }
          }
          consumer_barrier();
        }
        // Two warps share a stage (half of its k each): warps 2p and 2p + 1 multiply chunks p, p + 4, ... of every run of
        // stages, with two sets of sums so that consecutive products do not wait for each other.
        float acc[2][NT][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int j = 0; j < NT; ++j) { acc[h][j][0] = acc[h][j][1] = acc[h][j][2] = acc[h][j][3] = 0.f; }
        // Chunk number `at` of the whole program goes to pair at % PAIRS and lies in stage at % STAGES; STAGES is a
        // multiple of PAIRS, so a stage is always the same pair's and the pair sees every filling of it in turn. (A
        // pair that skipped stages could ask for a stage's second filling before the first had landed, and the
        // barrier would answer that the phase of that parity was complete: the one before the first.)
        static_assert(STAGES % PAIRS == 0, "a stage of the ring belongs to one pair of warps");
        const int pair = warp / WPS, half = warp % WPS;
        for (int run = 0; run < sh.count * sh.runs; ++run, n += sh.chunks) {
          for (int c = (pair + PAIRS - (int)(n % PAIRS)) % PAIRS; c < sh.chunks; c += PAIRS) {
            const unsigned at = n + (unsigned)c, s = at % STAGES;
            wait_for(&full_bar[s], (at / STAGES) & 1, 1);
            // a stage: [group of 64 k][row][128 bytes]; row g's 16-byte unit u lies at unit u XOR g (the 128-byte swizzle)
            const unsigned char* st = ring + (size_t)s * STAGE_BYTES + g * 128;
            const bf16* xrow = xs + (size_t)g * XSTRIDE + c * KC + 8 * t;
            constexpr int SLICES = KC / 32 / WPS;  // 32 k at a time: 16 bytes of rows g and g + 8, two products
#pragma unroll
            for (int i8 = 0; i8 < SLICES; ++i8) {
              const int sl = half * SLICES + i8;
              if (c * KC + sl * 32 < k_len) {
                const int a_off = (sl >> 1) * 2048 + ((((sl & 1) * 4 + t) ^ g) << 4);
                const uint4 a_lo = *reinterpret_cast<const uint4*>(st + a_off);
                const uint4 a_hi = *reinterpret_cast<const uint4*>(st + 1024 + a_off);  // row g + 8
                const uint32_t a1[4] = {a_lo.x, a_hi.x, a_lo.y, a_hi.y};  // first k-step: this thread's k 0..3
                const uint32_t a2[4] = {a_lo.z, a_hi.z, a_lo.w, a_hi.w};  // second k-step: its k 4..7
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                  const uint4 bv = *reinterpret_cast<const uint4*>(xrow + (size_t)8 * j * XSTRIDE + sl * 32);
                  mma_bf16(acc[0][j], a1, bv.x, bv.y);
                  mma_bf16(acc[1][j], a2, bv.z, bv.w);
                }
              }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
          }
          // The run is complete: the warps' sums go to one of two buffers in shared memory, from where the writer
          // warp reads them out while these warps go on with the next run. The buffer was last used two runs ago.
          const int buf = (int)(deposits & 1);
          if (deposits >= 2) named_sync(BAR_FREE + buf, WORKERS);
          float* mine = red + (size_t)buf * CONSUMERS * NT * 128;
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            float* r0 = mine + (((size_t)warp * NT + j) * 16 + g) * 8 + 2 * t;
            r0[0] = acc[0][j][0] + acc[1][j][0];
            r0[1] = acc[0][j][1] + acc[1][j][1];
            r0[64] = acc[0][j][2] + acc[1][j][2];
            r0[65] = acc[0][j][3] + acc[1][j][3];
#pragma unroll
            for (int h = 0; h < 2; ++h) acc[h][j][0] = acc[h][j][1] = acc[h][j][2] = acc[h][j][3] = 0.f;
          }
          __threadfence_block();  // the sums are in shared memory for the writer
          named_arrive(BAR_FULL + buf, WORKERS);
          ++deposits;
        }
      } else if (op.kind == OP_CONV) {
        // The short convolution of a decode step (conv.cu's short_conv_decode_kernel): token t is the single token of
        // request seq_of_token[t]. A thread owns a (token, channel); blocks take channels b, b + G, ... in groups of 32.
        const int N = op.M, C = op.O, L = op.K;
        const bf16* bcx = (const bf16*)op.x;
        const float* taps = (const float*)op.aux0;
        const float* bias = (const float*)op.aux1;
        const int* seq_of_token = (const int*)op.aux2;
        const int* slots = (const int*)op.aux3;
        float* state = (float*)op.y2;
        bf16* out = (bf16*)op.y;
        const int groups = (C + 31) / 32;
        for (int item = b * (CONSUMERS * 32) + tid; item < groups * 32 * N; item += G * CONSUMERS * 32) {
          const int c = (item / (32 * N)) * 32 + (item & 31), tk = (item / 32) % N;
          if (c >= C) continue;
          const int r = seq_of_token[tk];
          const int slot = r >= 0 ? slots[r] : -1;
          if (slot < 0) {
            out[(size_t)tk * C + c] = __float2bfloat16_rn(0.f);
            continue;
          }
          const bf16* row = bcx + (size_t)tk * 3 * C;
          const float bb = ldcg_bf16(row + c), gg = ldcg_bf16(row + C + c), xx = ldcg_bf16(row + 2 * C + c);
          const float uu = bb * xx;
          float* hist = state + (size_t)slot * (L - 1) * C + c;
          float acc1 = 0.f;
          for (int l = 0; l < L - 1; ++l) {
            const float h = __ldcg(hist + (size_t)l * C);
            acc1 = fmaf(h, taps[(size_t)c * L + l], acc1);
            if (l > 0 && op.flag) hist[(size_t)(l - 1) * C] = h;
          }
          acc1 = fmaf(uu, taps[(size_t)c * L + L - 1], acc1);
          if (op.flag) hist[(size_t)(L - 2) * C] = uu;
          if (bias) acc1 += bias[c];
          out[(size_t)tk * C + c] = __float2bfloat16_rn(gg * acc1);
        }
      } else if (op.kind == OP_EMBED) {
        // h[t, :] = table[token[t], :] as float32; blocks take (token, 256-column piece) pairs in turn
        const int N = op.M, C = op.O;
        const int* ids = (const int*)op.x;
        float* h = (float*)op.y;
        const int pieces = (C + 255) / 256;
        for (int item = b; item < N * pieces; item += G) {
          const int tk = item / pieces, c = (item % pieces) * 256 + tid;
          if (c >= C) continue;
          const size_t src = (size_t)ids[tk] * C + c;
          h[(size_t)tk * C + c] = op.flag == AKAS_BF16 ? to_f32(((const bf16*)op.aux0)[src]) : ((const float*)op.aux0)[src];
        }
      }
      // ---------------------------------------------------------------- the grid meets before the next operation
      // The writer warp does the meeting (see there). What these warps wrote to global memory themselves (a convolution,
      // an embedding) they hand over at BAR_PRE; of a product they wrote nothing. While the grid meets they fetch
      // what the next operation needs and no other block makes: its norm weights.
      if (i + 1 < prog.count) {
        if (op.kind != OP_GEMM) named_sync(BAR_PRE, WORKERS);
        const ChainOp& next = prog.ops[i + 1];
        if (kNormAhead && next.kind == OP_GEMM && next.in_mode == IN_NORM && next.K <= NW_MAX && b < next.tiles) {
          for (int k = tid * 4; k < next.K; k += CONSUMERS * 32 * 4)
            cp_async16(nw_s + k, (const float*)next.aux1 + k, 16);
          cp_async_commit();
        }
        named_sync(BAR_OP, WORKERS);
      }
    }
  } else {
    // ---------------------------------------------------------------- the writer warp: read-outs of the products
    chain_wait();
    unsigned deposits = 0;
    for (int i = 0; i < prog.count; ++i) {
      const ChainOp& op = prog.ops[i];
      if (op.kind == OP_GEMM) {
        const int M = op.M, O = op.O, K = op.K, F = O / 2;
        const bool swiglu = op.out_mode == OUT_SWIGLU;
        const Share sh(op, b, G);
        for (int ti = 0; ti < sh.count; ++ti) {
          const int tile = sh.first + ti * sh.step;
          float v[NT * 4], u[NT * 4];  // this lane's (row, token) pairs: pair e = lane + 32 * q of NT * 128
          for (int run = 0; run < sh.runs; ++run, ++deposits) {
            const int buf = (int)(deposits & 1);
            named_sync(BAR_FULL + buf, WORKERS);  // the consumers' sums of this run are in the buffer
            const float* sums = red + (size_t)buf * CONSUMERS * NT * 128;
            float all = 0.f;
#pragma unroll
            for (int q = 0; q < NT * 4; ++q) {
              const int e = lane + 32 * q, j = e >> 7, row = (e & 127) >> 3, tok = e & 7;
              float sum = 0.f;
#pragma unroll
              for (int w = 0; w < CONSUMERS; ++w)  // always in this order: results do not depend on timing
                sum += sums[(((size_t)w * NT + j) * 16 + row) * 8 + tok];
              if (run == 0) v[q] = sum; else u[q] = sum;
              all += sum;
            }
            // The buffer may take the sums of the run after next - once every load from it has come back: an arrival
            // that went out while loads were in flight let the consumers overwrite what was still being read.
            named_arrive_after(BAR_FREE + buf, WORKERS, all);
          }
          // A product that is cut along K: the parts of a tile are added in the order of their numbers.
          int* counter = op.parts > 1 ? prog.counters + tile : nullptr;
          if (op.parts > 1 && sh.part > 0 && !*(volatile int*)&abort_s) {
            unsigned spins = 0;
            while (load_acquire((const unsigned*)counter) != (unsigned)sh.part) {
              if (++spins > kBarrierSpins) {
                *(volatile int*)&abort_s = 1;
                atomicExch(&g_chain_status, 4);
                break;
              }
            }
          }
#pragma unroll
          for (int q = 0; q < NT * 4; ++q) {
            const int e = lane + 32 * q, j = e >> 7, row = (e & 127) >> 3, tok = e & 7;
            const int m = 8 * j + tok, o = tile * 16 + row;
            if (m >= M) continue;
            float a = v[q], c = swiglu ? u[q] : 0.f;
            if (op.in_mode == IN_NORM) {
              const float inv = 1.f / sqrtf(ss_s[m] / (float)K + op.eps);
              a *= inv;
              c *= inv;
            }
            if (swiglu) {
              if (o < F) ((bf16*)op.y)[(size_t)m * F + o] = __float2bfloat16_rn(a / (1.f + expf(-a)) * c);
            } else if (o < O) {
              const size_t at = (size_t)m * O + o;
              if (op.out_mode == OUT_BF16) ((bf16*)op.y)[at] = __float2bfloat16_rn(a);
              else if (op.out_mode == OUT_F32) ((float*)op.y)[at] = a;
              else atomicAdd((float*)op.y + at, a);  // no value comes back: the L2 adds; who adds when is fixed, so is the sum
            }
          }
          if (op.parts > 1) {
            __syncwarp();
            if (lane == 0) {
              __threadfence();  // this part's additions come before the next part's
              *(volatile int*)counter = sh.part + 1 < op.parts ? sh.part + 1 : 0;  // the last part leaves the counter at zero
            }
          }
        }
      }
      // ---------------------------------------------------------------- the grid meets before the next operation
      // This warp has stored the block's results of a product (the consumers store nothing then), so it goes to the
      // meeting straight from its last store; after other operations the consumers hand over first.
      if (i + 1 < prog.count) {
        if (op.kind != OP_GEMM) named_sync(BAR_PRE, WORKERS);
        __syncwarp();
        if (lane == 0 && !*(volatile int*)&abort_s) {
          __threadfence();  // the block's stores are visible to every SM before its arrival is
          const unsigned add = b == 0 ? 0x80000000u - (unsigned)(G - 1) : 1u;
          const unsigned old = atomicAdd(prog.barrier, add);
          unsigned spins = 0;
          while (((old ^ load_acquire(prog.barrier)) & 0x80000000u) == 0) {
            if (++spins > kBarrierSpins) {
              *(volatile int*)&abort_s = 1;
              atomicExch(&g_chain_status, 3);
              break;
            }
          }
        }
        named_sync(BAR_OP, WORKERS);  // lets the consumers go on: what the other blocks stored is visible
      }
    }
  }
  chain_release();
  if (*(volatile int*)&abort_s) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // a lost launch: give copies still in flight time to land
  }
  __syncthreads();  // nobody leaves while a copy into this block's shared memory may be in flight
}

// ------------------------------------------------------------------------------------------------ host side

std::mutex g_mutex;
Program g_program;            // the program under construction (one builder per process: the engine runs on one thread)
int g_tokens = 0;             // the most tokens of any product so far
unsigned* g_scratch[64] = {}; // per device: the barrier word, then the tile counters (given by the caller, zeroed once)

// The matrix [O, K] seen as [K / 64][O][64]: boxes of 64 k x 16 rows x 8 groups of k, 128-byte swizzle, zeros outside.
std::map<std::tuple<const void*, int, int>, CUtensorMap> g_maps;

int weight_map(CUtensorMap* out, const void* w, int O, int K) {
  const auto key = std::make_tuple(w, O, K);
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    akas::tc::EncodeTiled fn = akas::tc::encode_tiled();
    if (!fn) return 3001;
    const cuuint64_t dims[3] = {64, (cuuint64_t)O, (cuuint64_t)(K / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
    const cuuint32_t box[3] = {64, 16, KC / 64};
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

template <int NT, int STAGES>
constexpr int smem_bytes() {
  return 1024 + STAGES * STAGE_BYTES + 2 * CONSUMERS * NT * 128 * (int)sizeof(float) + NT * 8 * XSTRIDE * (int)sizeof(bf16) +
         (NT == 1 ? NW_MAX * (int)sizeof(float) : 0);
}
constexpr int STAGES_1 = 8, STAGES_2 = 4;  // multiples of the number of warp pairs
static_assert(smem_bytes<1, STAGES_1>() <= 226 * 1024 && smem_bytes<2, STAGES_2>() <= 226 * 1024, "the block fits an SM");

template <int NT, int STAGES>
int launch(cudaStream_t stream) {
  auto kernel = decode_chain_kernel<NT, STAGES>;
  constexpr int smem = smem_bytes<NT, STAGES>();
  static int sms[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  if (sms[device] == 0) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    int count = 0;
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, smem);
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) return (int)cudaErrorInvalidConfiguration;
    sms[device] = count;
  }
  if (g_scratch[device] == nullptr) return (int)cudaErrorInvalidValue;
  g_program.barrier = g_scratch[device];
  g_program.counters = (int*)(g_scratch[device] + 16);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(sms[device]);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeCooperative;
  attribute[0].val.cooperative = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&config, kernel, g_program);
}

}  // namespace

// How many 32-bit words of device memory the chain needs on a device: the grid's meeting word and the tile counters.
AKAS_API int akas_chain_scratch_words() { return 16 + MAX_SPLIT_TILES; }

// Gives the chain its scratch on the current device: akas_chain_scratch_words() words of device memory that the caller
// has zeroed and keeps alive (the library allocates nothing). The kernel leaves every word as it found it.
AKAS_API int akas_chain_set_scratch(void* words) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mutex);
  g_scratch[device] = (unsigned*)words;
  return 0;
}

// Starts a new program. Operations are added with the functions below and run, in order, by akas_chain_run.
AKAS_API int akas_chain_begin() {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_program.count = 0;
  g_tokens = 0;
  return 0;
}

// How many operations the program holds.
AKAS_API int akas_chain_count() { return g_program.count; }

// Whether a product of these sizes can join a chain (1) or not (0): at most 16 tokens, K a multiple of 64; beyond
// K = 4,096 only a residual add of bfloat16 activations (it is cut along K); the fused norm weights its rows in one pass.
AKAS_API int akas_chain_takes(int M, int O, int K, int in_mode, int out_mode) {
  if (M <= 0 || M > 16 || O <= 0 || K <= 0 || K % 64) return 0;
  if (K > XK && (in_mode != IN_BF16 || out_mode != OUT_ACC || (O + 15) / 16 > MAX_SPLIT_TILES)) return 0;
  if (in_mode == IN_NORM && K % 4) return 0;
  if (out_mode == OUT_SWIGLU && O % 2) return 0;
  return 1;
}

// y = f(x) . W^T as in akas_skinny_gemm (same modes). Returns 0, 1 if the program is full (run it and begin
// another), or an error code.
AKAS_API int akas_chain_gemm(const void* x, const int* rows, const float* norm_w, float eps, int zero_centered,
                             const void* W, void* y, int M, int O, int K, int in_mode, int out_mode) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!akas_chain_takes(M, O, K, in_mode, out_mode)) return (int)cudaErrorInvalidValue;
  if ((uintptr_t)W % 16 || (uintptr_t)x % 16 || (in_mode == IN_NORM && norm_w == nullptr)) return (int)cudaErrorInvalidValue;
  if (g_program.count >= MAX_OPS) return 1;
  ChainOp& op = g_program.ops[g_program.count];
  op = ChainOp{};
  const int err = weight_map(&op.map, W, O, K);
  if (err) return err;
  op.kind = OP_GEMM;
  op.x = x; op.aux0 = rows; op.aux1 = norm_w; op.y = y;
  op.in_mode = in_mode; op.out_mode = out_mode;
  op.M = M; op.O = O; op.K = K;
  op.tiles = out_mode == OUT_SWIGLU ? (O / 2 + 15) / 16 : (O + 15) / 16;
  op.flag = zero_centered; op.eps = eps;
  const int chunks = (K + KC - 1) / KC;
  op.parts = K > XK ? (K + XK - 1) / XK : 1;
  op.part_chunks = (chunks + op.parts - 1) / op.parts;
  if ((op.parts - 1) * op.part_chunks >= chunks) return (int)cudaErrorInvalidValue;  // every part must have chunks of its own
  ++g_program.count;
  if (M > g_tokens) g_tokens = M;
  return 0;
}

// The short convolution of a decode step on bfloat16 activations (akas_short_conv_decode's arguments).
AKAS_API int akas_chain_conv(const void* bcx, const float* taps, const float* bias, float* state, const int* seq_of_token,
                             const int* slots, void* out, int N, int C, int L, int write) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (N <= 0 || C <= 0 || L < 2 || L > 16) return (int)cudaErrorInvalidValue;
  if (g_program.count >= MAX_OPS) return 1;
  ChainOp& op = g_program.ops[g_program.count];
  op = ChainOp{};
  op.kind = OP_CONV;
  op.x = bcx; op.aux0 = taps; op.aux1 = bias; op.aux2 = seq_of_token; op.aux3 = slots; op.y = out; op.y2 = state;
  op.M = N; op.O = C; op.K = L; op.flag = write;
  ++g_program.count;
  return 0;
}

// h[t, :] = table[token[t], :] as float32.
AKAS_API int akas_chain_embed(const int* token_ids, const void* table, float* h, int N, int C, int dtype) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (N <= 0 || C <= 0) return (int)cudaErrorInvalidValue;
  if (g_program.count >= MAX_OPS) return 1;
  ChainOp& op = g_program.ops[g_program.count];
  op = ChainOp{};
  op.kind = OP_EMBED;
  op.x = token_ids; op.aux0 = table; op.y = h;
  op.M = N; op.O = C; op.flag = dtype;
  ++g_program.count;
  return 0;
}

// Runs the program on the stream (one launch) and leaves it empty.
AKAS_API int akas_chain_run(cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_program.count == 0) return 0;
  const int err = g_tokens > 8 ? launch<2, STAGES_2>(stream) : launch<1, STAGES_1>(stream);
  g_program.count = 0;
  g_tokens = 0;
  return err;
}

// 0 if no bounded wait of the kernel has ever run out on the current device, else the code of the last one
// (1: a stage that never filled, 2: a stage that never emptied, 3: the grid barrier, 4: a tile counter). Synchronises
// with the device.
AKAS_API int akas_chain_status() {
  int status = -1;
  const cudaError_t e = cudaMemcpyFromSymbol(&status, g_chain_status, sizeof(int));
  return e == cudaSuccess ? status : -(int)e;
}
