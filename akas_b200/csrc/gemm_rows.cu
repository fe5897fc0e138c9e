// bfloat16 matrix products for 17 to 128 tokens (a decode step of many requests, a short prompt portion):
// y[M, O] = x[M, K] . W[O, K]^T with tcgen05.mma, float32 accumulation in tensor memory, epilogues fused into the
// read-out and written by TMA. The time of such a product is the time to read W once, so the kernel is a stream
// of weights through as many SMs as there are, one block per SM (a long K is cut over a cluster, see "Parts of K").
//
// The token rows are the 128 lanes of the accumulator (rows past M are never read), the channels its columns. The
// output is cut into tiles of TILE_N channels, TILE_N the multiple of 16 that gives every SM one tile (or two, three
// ... for a wide matrix: 48 channels for 6,144, 16 for 2,048, 224 for a vocabulary of 65,536 on 148 SMs); a block
// walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... and, where it has more than one, with two sets of accumulators,
// so that a tile is read out while the next is summed.
//   warp 0   producer: TMA loads into a ring of stages. A stage holds `G` 64-wide steps of K: the RT token rows of x
//            (RT = M rounded up to 16) and the tile's TILE_N rows of W (SwiGLU: TILE_N gate rows and the TILE_N up rows
//            under them in the stacked [2F, K] matrix), each with ONE copy of a box of a view [K / 64][rows][64] (SwiGLU:
//            [K / 64][2][F][64]) of the matrix (starting a copy costs the issuing thread some hundreds of cycles
//            whatever it moves; K that is no multiple of 64 takes a copy per step). The weights of the first stages
//            are asked for before the kernel waits for its predecessor on the stream (programmatic dependent launch):
//            no kernel writes them.
//   warps 1-4 tensor cores: one thread of each of up to four warps issues the products of every fourth (third, second)
//            stage: per step of K four tcgen05.mma (M 128, N TILE_N, or 2 TILE_N for SwiGLU, whose gate and up rows lie
//            behind one another in a stage; K 16), then a commit to the stage's "empty" barrier. Issuing a product costs
//            its thread some 55 cycles however small the product is, which for these thin tiles is more than the tensor
//            cores need for it: several issuing threads, each with an accumulator of its own, keep them busy. Each of
//            them waits for every stage in order, also for those it leaves to the others (see there). The
//            operand of the token rows is read as 128 rows although only RT were loaded: the rest is whatever lies
//            behind in shared memory, and lands in accumulator lanes that nobody reads.
//   warps 5-8 read-out: each warp owns the 32 accumulator lanes (token rows) of its sub-partition; those whose rows lie
//            inside M read 16 columns of every issuing warp's accumulator with tcgen05.ld, add them in the warps'
//            order, write them into a staging tile in shared memory in the swizzle
//            TMA expects, and one lane hands the tile (32 rows x 16 channels) to TMA, which writes whole rows and clips
//            at the matrix's edges:
//              BF16    y bfloat16 [M, O]          a TMA store
//              ACC     y float32 [M, O] +=        a TMA reduce-add: the residual stream is added to in the L2; every
//                                                 element is added to once, so the sum does not depend on timing
//              F32     y float32 [M, O]           a TMA store
//              SWIGLU  y bfloat16 [M, F]          silu(gate) * up, a TMA store
// Parts of K. Every block reads all token rows of x for the k it multiplies, from the L2 at the 64 bytes a cycle an SM
// takes in; where K is long and the tile narrow (the down projection of a feed-forward: 1 MB of x beside 256 KB of
// weights at 64 tokens) that is what the block waits for. Such a product (residual read-out only) is cut along K into
// 2 or 4 parts with tiles that many times as wide: the blocks of a thread-block cluster take one part each for the same
// tile, the others put their sums into their own shared memory (the ring is free by then) and send them to the first
// block's with ONE bulk copy each (cp.async.bulk shared::cta -> shared::cluster, its bytes counted on the first block's
// mbarrier; stores from registers into a peer's shared memory, 16 bytes a thread and rows 256 bytes apart, took 10 us
// for 48 KB), and the first block adds the parts in the order of their numbers and hands the tile to TMA. One tile per
// block then (the meeting place is used once). The cluster's barrier is passed twice: once so that the first block's
// mbarrier exists before a peer's copy counts on it, once so that a peer's shared memory lives until its copy has
// been received.
// Every wait on an mbarrier is bounded (akas_gemm_rows_status): one that runs out sets a status word, every role
// falls through, tensor memory is freed and the block returns; that launch's results are not valid. The cluster's
// barrier has no bounded form; every thread arrives at it without condition, or after a bounded wait of its own.
#include <math.h>

#include "tcgen05.cuh"

using namespace akas;
using namespace akas::tc;

namespace {

constexpr int ISSUERS = 4, THREADS = 32 * (1 + ISSUERS + 4), MAX_STAGES = 16, MAX_TOKENS = 128;
constexpr int STAGING = 2048;  // bytes of one staging tile: 32 rows x 64 bytes (float32) or x 32 bytes (bfloat16)
constexpr int SMEM_LIMIT = 227 * 1024;
enum { EPI_BF16 = 0, EPI_ACC = 1, EPI_SWIGLU = 2, EPI_F32 = 3 };

__device__ int g_rows_status = 0;  // 0, or which bounded wait ran out last (1 producer, 2 tensor cores, 3 read-out, 4 the parts of K)

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int row, int group, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(smem_u32(smem_dst)), "l"(map), "r"(0), "r"(row), "r"(group), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, int row, int group, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
               ::"r"(smem_u32(smem_dst)), "l"(map), "r"(0), "r"(row), "r"(0), "r"(group), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_add_2d(const CUtensorMap* map, const void* smem_src, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 16 consecutive float32 columns of this thread's accumulator lane, asked for but not waited for.
__device__ __forceinline__ void tmem_ask16(unsigned taddr, unsigned (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
// Waits for the loads asked for. The registers pass through the statement, so that no use of them moves above it.
__device__ __forceinline__ void tmem_wait(unsigned (&a)[16], unsigned (&b)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]), "+r"(a[8]),
                 "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15]), "+r"(b[0]), "+r"(b[1]),
                 "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]), "+r"(b[8]), "+r"(b[9]), "+r"(b[10]),
                 "+r"(b[11]), "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15])
               :: "memory");
}
// The sum over the issuing warps' accumulators (in the warps' order) of 16 columns, two accumulators per wait.
__device__ __forceinline__ void tmem_sum16(unsigned taddr, int warps, int pitch, float (&v)[16]) {
#pragma unroll
  for (int w0 = 0; w0 < ISSUERS; w0 += 2) {
    if (w0 >= warps) break;
    unsigned r[2][16];
    tmem_ask16(taddr + w0 * pitch, r[0]);
    if (w0 + 1 < warps) {
      tmem_ask16(taddr + (w0 + 1) * pitch, r[1]);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) r[1][i] = 0u;
    }
    tmem_wait(r[0], r[1]);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = w0 == 0 ? __uint_as_float(r[0][i]) : v[i] + __uint_as_float(r[0][i]);
    if (w0 + 1 < warps) {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] += __uint_as_float(r[1][i]);
    }
  }
}

__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address of a shared-memory location of block `rank` of this cluster, and a 16-byte store there.
__device__ __forceinline__ unsigned peer_address(const void* local, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
  return r;
}
__device__ __forceinline__ void peer_store4(unsigned address, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(address), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

struct Shape {
  int M, O, K, F;     // F: output channels of SwiGLU (O = 2F), else unused
  int RT;             // token rows a stage holds (M rounded up to 16)
  int tile_n;         // output channels of a tile = N of a product
  int G;              // 64-wide steps of K in a stage
  int stages;
  int wide;           // 1: one copy per operand and stage (K % 64 == 0), 0: a copy per step of K
  int tmem_cols;
  int issuers;        // warps that issue products, each with accumulators of its own
  int buffers;        // sets of accumulators: 2 where a block walks several tiles, else 1
  unsigned suspend_ns;  // how long a waiting thread may sleep before it looks at its barrier again
  int parts;          // blocks of a cluster that share a tile, one part of K each (1: no cluster)
  int part_blocks;    // 64-wide steps of K in a part (a multiple of G)
};

template <int EPI>
__global__ void __launch_bounds__(THREADS, 2)  // registers for two blocks to an SM, should their shared memory allow it
gemm_rows_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_y, const Shape sh) {
  constexpr bool SWIGLU = EPI == EPI_SWIGLU;
  constexpr int HALVES = SWIGLU ? 2 : 1;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2], gathered;
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int M = sh.M, K = sh.K, RT = sh.RT, TN = sh.tile_n, G = sh.G, stages = sh.stages;
  const int out_cols = SWIGLU ? sh.F : sh.O;
  const int tiles = (out_cols + TN - 1) / TN;
  // this block's part of K: 64-wide steps [kb0, kb0 + k_blocks); its place among the blocks that walk the tiles
  const int P = sh.parts, rank = P > 1 ? (int)cluster_rank() : 0;
  const int kb0 = rank * sh.part_blocks;
  const int k_blocks = P > 1 ? min(sh.part_blocks, (K + BK - 1) / BK - kb0) : (K + BK - 1) / BK;
  const int bid = (int)blockIdx.x / P, nb = (int)gridDim.x / P;
  const int steps = (k_blocks + G - 1) / G;  // stages' worth of K in a tile
  const int x_bytes = G * RT * 128, w_bytes = G * HALVES * TN * 128;  // of a stage; W as [G][gate rows, up rows][64]
  const int stage_bytes = x_bytes + w_bytes;
  unsigned char* staging = smem + (size_t)stages * stage_bytes;  // [4 warps][2][STAGING], behind the ring
  float* gather = reinterpret_cast<float*>(staging + 8 * STAGING);  // first block of a cluster: [P - 1][RT][TN + 4] sums of the other parts
  const int acc_cols = HALVES * TN, W = sh.issuers < steps ? sh.issuers : steps;  // warps that issue at all

  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_y) : "memory");
  }
  if (warp == 1 + ISSUERS) {  // a lane per barrier
    if (lane < stages) { mbar_init(&full_bar[lane], 1); mbar_init(&empty_bar[lane], 1); }
    if (lane >= 16 && lane < 18) { mbar_init(&acc_full[lane - 16], (unsigned)W); mbar_init(&acc_empty[lane - 16], 4); }
    if (lane == 18) abort_s = 0;
    if (lane == 19) {  // the bytes of the other parts' copies are counted here (first block of a cluster)
      mbar_init(&gathered, 1);
      if (P > 1 && rank == 0) mbar_expect_tx(&gathered, (unsigned)((P - 1) * RT * (TN + 4) * 4));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(sh.tmem_cols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_base_s;
  // Every block of a cluster says that its barriers exist; who writes into the first block waits for that, at the end.
  if (P > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  // Every thread of a cluster's block passes here once, when its own work is done: the first meeting is over by then;
  // it arrives at the second, and in a block that sent its sums away it stays until the first block has them.
  auto cluster_leave = [&]() {
    if (P > 1) {
      asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
      asm volatile("barrier.cluster.arrive.release;" ::: "memory");
      if (rank > 0) asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    }
  };
  chain_release();

  // A bounded wait that also ends when another role has given up; nothing but the poll itself on the fast path.
  auto wait_for = [&](uint64_t* bar, unsigned parity, int code) -> bool {
    const unsigned addr = smem_u32(bar);
    for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
      unsigned done;
      asm volatile(
          "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
          : "=r"(done) : "r"(addr), "r"(parity), "r"(sh.suspend_ns) : "memory");
      if (done) return true;
      if (*(volatile int*)&abort_s) return false;
    }
    *(volatile int*)&abort_s = 1;
    atomicExch(&g_rows_status, code);
    return false;
  };

  // Loads of this block in all, and how many of them fill the ring for the first time.
  const int my_tiles = bid < tiles ? (tiles - bid + nb - 1) / nb : 0;
  const int total = my_tiles * steps, head = total < stages ? total : stages;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      // Where the next load goes: tile, step of K within it, stage of the ring; counted up, never divided.
      struct Cursor { int tile, st, s; unsigned char* dst; };
      auto advance = [&](Cursor& c) {
        if (++c.st == steps) { c.st = 0; c.tile += nb; }
        c.dst += stage_bytes;
        if (++c.s == stages) { c.s = 0; c.dst = smem; }
      };
      auto load_w = [&](const Cursor& c) {
        unsigned char* dst = c.dst + x_bytes;
        const int kb = kb0 + c.st * G, row = c.tile * TN;
        mbar_expect_tx(&full_bar[c.s], stage_bytes);
        if (sh.wide) {
          if (SWIGLU) tma_load_4d(dst, &map_w, row, kb, &full_bar[c.s]); else tma_load_3d(dst, &map_w, row, kb, &full_bar[c.s]);
        } else {
          for (int g = 0; g < G; ++g)
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
              tma_load_2d(dst + (g * HALVES + h) * TN * 128, &map_w, (kb + g) * BK, row + h * sh.F, &full_bar[c.s]);
        }
      };
      auto load_x = [&](const Cursor& c) {
        const int kb = kb0 + c.st * G;
        if (sh.wide) {
          tma_load_3d(c.dst, &map_x, 0, kb, &full_bar[c.s]);
        } else {
          for (int g = 0; g < G; ++g) tma_load_2d(c.dst + g * RT * 128, &map_x, (kb + g) * BK, 0, &full_bar[c.s]);
        }
      };
      // The ring's first filling: the weights from here, at once (no kernel writes them); the token rows from a thread
      // of the read-out warps, which has nothing else to do yet, as soon as the predecessor on the stream is done.
      Cursor c = {bid, 0, 0, smem};
      for (int i = 0; i < head; ++i, advance(c)) load_w(c);
      chain_wait();
      unsigned parity = 0;  // of the "empty" barriers in this round of the ring
      for (int i = head; i < total; ++i, advance(c)) {
        if (!wait_for(&empty_bar[c.s], parity, 1)) break;
        load_w(c);
        load_x(c);
        if (c.s == stages - 1) parity ^= 1;
      }
    }
    cluster_leave();
  } else if (warp <= ISSUERS) {
    // ------------------------------------------------------------------ tensor cores: warps 1..W, stage i to warp 1 + i % W
    const int me = warp - 1;
    if (lane == 0 && me < W) {
      // instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, N = the tile's stacked rows, M = 128
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(acc_cols >> 3) << 17) | ((unsigned)(128 >> 4) << 24);
      // Shared-memory descriptors differ in their address field only (16-byte units, all of the block's shared memory
      // fits the field), so the descriptor of a tile further on is a sum.
      const uint64_t ring_desc = smem_desc(smem);
      const unsigned stage_units = (unsigned)stage_bytes >> 4, x_units = (unsigned)x_bytes >> 4;
      const unsigned a_step = (unsigned)RT * 8, b_step = (unsigned)acc_cols * 8;  // one 64-wide step of K further, in 16-byte units
      int s = 0, turn = 0;  // the stage of the ring, and whose turn it is
      unsigned parity = 0, t = 0;
      uint64_t stage_desc = ring_desc;
      bool lost = false;
      for (int tile = bid; tile < tiles && !lost; tile += nb, ++t) {
        const unsigned acc = t % (unsigned)sh.buffers;
        if (!wait_for(&acc_empty[acc], ((t / (unsigned)sh.buffers) & 1) ^ 1, 2)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned d = tmem_base + (acc * W + me) * acc_cols;
        int left = k_blocks;  // steps of K of this tile still to add
        unsigned on = 0;      // 0 for this warp's first product of the tile, which overwrites its accumulator
        for (int st = 0; st < steps; ++st) {
          const int gs = left < G ? left : G;  // a stage's steps past the end of K hold zeros: nothing to add
          left -= gs;
          // Every issuing warp sees every stage fill, in order, also those it leaves to the others: a warp that looked at
          // a slot of the ring only every few fillings could ask its barrier for a phase whose parity reads "complete"
          // before the slot has been filled at all (the phase before the first has that parity). In order, and with the
          // producer held back by this warp's own uncommitted stage, it can never fall two fillings of a slot behind.
          if (!wait_for(&full_bar[s], parity, 2)) { lost = true; break; }
          if (turn == me) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint64_t a_desc = stage_desc, b_desc = stage_desc + x_units;
            for (int g = 0; g < gs; ++g) {
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k)  // 32 bytes further along the swizzled row per product
                umma(d, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, k ? 1u : on);
              on = 1u;
              a_desc += a_step;
              b_desc += b_step;
            }
            umma_commit(&empty_bar[s]);
          }
          if (++turn == W) turn = 0;
          stage_desc += stage_units;
          if (++s == stages) { s = 0; parity ^= 1; stage_desc = ring_desc; }
        }
        if (lost) break;
        umma_commit(&acc_full[acc]);  // this warp's share of the tile is summed (every issuing warp has a stage in every tile)
      }
    }
    cluster_leave();
  } else {
    // ------------------------------------------------------------------ read-out: the last four warps
    const int sub = warp & 3;  // the tensor-memory sub-partition (32 lanes) this warp may read
    unsigned char* stage_of_warp = staging + (size_t)sub * 2 * STAGING;
    const int row0 = sub * 32;  // this warp's 32 token rows; lane l holds row0 + l
    unsigned t = 0, stores = 0;
    bool left = false;  // whether this thread has passed the cluster's second meeting (every thread must, once)
    chain_wait();  // the residual stream that ACC adds to is an earlier kernel's, and so are the token rows
    if (warp == THREADS / 32 - 1 && lane == 0) {  // the token rows of the ring's first filling
      for (int i = 0; i < head; ++i) {
        const int kb = kb0 + (i % steps) * G;
        unsigned char* dst = smem + (size_t)i * stage_bytes;
        if (sh.wide) {
          tma_load_3d(dst, &map_x, 0, kb, &full_bar[i]);
        } else {
          for (int g = 0; g < G; ++g) tma_load_2d(dst + g * RT * 128, &map_x, (kb + g) * BK, 0, &full_bar[i]);
        }
      }
    }
    for (int tile = bid; tile < tiles; tile += nb, ++t) {
      const unsigned acc = t % (unsigned)sh.buffers;
      const int n0 = tile * TN;
      int ok = 1;
      if (lane == 0) ok = wait_for(&acc_full[acc], (t / (unsigned)sh.buffers) & 1, 3) ? 1 : 0;  // one lane polls
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const unsigned taddr = tmem_base + acc * W * acc_cols + ((unsigned)row0 << 16);
      if (EPI == EPI_ACC && P > 1 && rank > 0) {
        // A part of K that is not the first: this block's sums go into its own shared memory, [token row][TN + 4]
        // float32 (the ring is free: every stage has been multiplied), and from there to the first block with one copy.
        float* mine = reinterpret_cast<float*>(smem);
        const int pitch = TN + 4;  // 16 bytes of padding a row: a warp's 16-byte stores and loads meet no bank twice
        if (row0 < M) {  // the whole warp reads tensor memory (the loads are warp-wide); rows past RT are not kept
#pragma unroll 1
          for (int c = 0; c < TN; c += 16) {
            float v[16];
            tmem_sum16(taddr + c, W, acc_cols, v);
            if (row0 + lane < RT) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                *reinterpret_cast<float4*>(mine + (size_t)(row0 + lane) * pitch + c + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        fence_async_smem();
        asm volatile("bar.sync 2, 128;" ::: "memory");  // the four read-out warps: the block's sums are in place
        if (warp == 1 + ISSUERS && lane == 0) {
          asm volatile("barrier.cluster.wait.acquire;" ::: "memory");  // (arrived at the start) the first block's barrier exists
          const unsigned bytes = (unsigned)(RT * pitch * 4);
          asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(peer_address(gather, 0) + (unsigned)(rank - 1) * bytes), "r"(smem_u32(mine)), "r"(bytes),
                         "r"(peer_address(&gathered, 0)) : "memory");
          asm volatile("barrier.cluster.arrive.release;" ::: "memory");
          asm volatile("barrier.cluster.wait.acquire;" ::: "memory");  // the first block has the sums: this block may go
        } else {
          cluster_leave();
        }
        left = true;
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        continue;
      }
      if (EPI == EPI_ACC && P > 1) {  // the first part: the others' sums have arrived in this block's shared memory
        int here = 1;
        if (lane == 0) {
          here = 0;
          const unsigned addr = smem_u32(&gathered);
          for (unsigned spin = 0; spin < kSpinLimit && !here; ++spin) {
            unsigned done;
            asm volatile(
                "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                : "=r"(done) : "r"(addr), "r"(0u) : "memory");
            here = done != 0;
            if (!here && *(volatile int*)&abort_s) break;
          }
          if (!here) { *(volatile int*)&abort_s = 1; atomicExch(&g_rows_status, 4); }
        }
        const int got = __shfl_sync(0xffffffffu, here, 0);
        cluster_leave();  // (the peers may go: their sums are here, or are given up)
        left = true;
        if (!got) break;
      }
      if (row0 < M) {
#pragma unroll 1
        for (int c = 0; c < TN; c += 16, ++stores) {
          if (n0 + c >= out_cols) break;
          unsigned char* buf = stage_of_warp + (stores & 1) * STAGING;
          if (lane == 0) bulk_wait_read<1>();  // the store before last has read this tile
          __syncwarp();
          float v[16];
          tmem_sum16(taddr + c, W, acc_cols, v);
          if (EPI == EPI_ACC && P > 1 && row0 + lane < RT) {  // the parts in the order of their numbers
            for (int r = 0; r < P - 1; ++r) {
              const float4* part = reinterpret_cast<const float4*>(gather + ((size_t)r * RT + row0 + lane) * (TN + 4) + c);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float4 q = part[j];
                v[4 * j] += q.x; v[4 * j + 1] += q.y; v[4 * j + 2] += q.z; v[4 * j + 3] += q.w;
              }
            }
          }
          if (EPI == EPI_ACC || EPI == EPI_F32) {
            // row `lane` of 64 bytes, its 16-byte units XORed with bits 7-8 of the address (the 64-byte swizzle)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<float4*>(buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
                  make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
            if (SWIGLU) {
              float u[16];
              tmem_sum16(taddr + TN + c, W, acc_cols, u);
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = __fdividef(v[i], 1.f + __expf(-v[i])) * u[i];  // the fast division: IEEE division cost more than the tile's loads
            }
            // row `lane` of 32 bytes, its two 16-byte units XORed with bit 7 of the address (the 32-byte swizzle)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              uint4 o;
              o.x = pack2(v[8 * j], v[8 * j + 1]); o.y = pack2(v[8 * j + 2], v[8 * j + 3]);
              o.z = pack2(v[8 * j + 4], v[8 * j + 5]); o.w = pack2(v[8 * j + 6], v[8 * j + 7]);
              *reinterpret_cast<uint4*>(buf + lane * 32 + ((j ^ ((lane >> 2) & 1)) << 4)) = o;
            }
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (EPI == EPI_ACC) tma_add_2d(&map_y, buf, n0 + c, row0); else tma_store_2d(&map_y, buf, n0 + c, row0);
            bulk_commit();
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
    if (lane == 0) bulk_wait_all();  // what this warp handed to TMA has been written before the block may leave
    __syncwarp();
    if (!left) cluster_leave();  // (a wait gave up before the parts met)
  }

  // wind down: everyone meets, then the allocating warp frees tensor memory
  if (*(volatile int*)&abort_s) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // a lost launch: let copies and products in flight finish
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(sh.tmem_cols));
  }
}

// ------------------------------------------------------------------------------------------------ host side

// A tensor map of a row-major matrix [rows, cols] of 2- or 4-byte elements for the read-out's staging tiles: boxes of
// 32 rows x 16 columns (64 or 32 bytes), in the swizzle of that width.
int make_out_map(CUtensorMap* map, void* base, int rows, int cols, int elem_bytes) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return 3001;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * elem_bytes};
  const cuuint32_t box[2] = {16, 32};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims,
                        strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        elem_bytes == 4 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 3000 + (int)r;
}

// A tensor map of a row-major bfloat16 matrix [rows, K], K a multiple of 64, seen as [K / 64][rows][64]: boxes of
// 64 k x box_rows x `groups` groups of k, 128-byte swizzle, zeros outside.
int make_wide_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows, int groups) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return 3001;
  const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(K / 64)};
  const cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)groups};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 3000 + (int)r;
}

// The stacked [2F, K] gate and up matrices, K a multiple of 64, seen as [K / 64][2][F][64]: boxes of 64 k x box_rows gate
// rows and the box_rows up rows under them x `groups` groups of k.
int make_stacked_map(CUtensorMap* map, const void* base, int F, int K, int box_rows, int groups) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return 3001;
  const cuuint64_t dims[4] = {64, (cuuint64_t)F, 2, (cuuint64_t)(K / 64)};
  const cuuint64_t strides[3] = {(cuuint64_t)K * 2, (cuuint64_t)F * K * 2, 128};
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 2, (cuuint32_t)groups};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 3000 + (int)r;
}

std::mutex g_rows_mutex;
std::map<std::tuple<const void*, int, int, int, int>, CUtensorMap> g_rows_maps;  // weights keep their maps

int weight_map(CUtensorMap* out, const void* base, int rows, int K, int box_rows, int groups, bool wide, bool stacked) {
  if (!wide) return cached_map(out, base, rows, K, box_rows, true);
  std::lock_guard<std::mutex> lock(g_rows_mutex);
  const auto key = std::make_tuple(base, stacked ? -rows : rows, K, box_rows, groups);
  auto it = g_rows_maps.find(key);
  if (it == g_rows_maps.end()) {
    CUtensorMap map;
    const int err = stacked ? make_stacked_map(&map, base, rows / 2, K, box_rows, groups) : make_wide_map(&map, base, rows, K, box_rows, groups);
    if (err) return err;
    it = g_rows_maps.emplace(key, map).first;
  }
  *out = it->second;
  return 0;
}

int env_int(const char* name, int fallback) {
  const char* v = getenv(name);
  return v && v[0] ? atoi(v) : fallback;
}

// How a product is cut: the tile width that gives every SM the same number of tiles, the steps of K per stage and the
// depth of the ring that fit the shared memory. Returns false if the kernel does not take these sizes.
bool plan(Shape* sh, int M, int O, int K, int epilogue, int sms, int budget, int parts = 0) {
  const bool swiglu = epilogue == EPI_SWIGLU;
  const int out_cols = swiglu ? O / 2 : O, halves = swiglu ? 2 : 1;
  const int widest = 256 / halves;  // two accumulators of halves * tile_n columns in 512 columns of tensor memory
  sh->M = M; sh->O = O; sh->K = K; sh->F = O / 2;
  sh->RT = (M + 15) / 16 * 16;
  const int rounds = (out_cols + widest * sms - 1) / (widest * sms);  // tiles a block walks
  int tile_n = ((out_cols + rounds * sms - 1) / (rounds * sms) + 15) / 16 * 16;
  if (tile_n > widest) tile_n = widest;
  const int all_blocks = (K + BK - 1) / BK;
  // Parts of K (the residual read-out, K a multiple of 64, one tile per block): tiles `parts` times as wide, so that a
  // block reads a part of x only. Taken where x is most of what a block reads: from K = 4,096 on, the cut that leaves
  // a block the fewest bytes of 1, 2 and 4 (AKAS_B200_ROWS_PARTS forces one).
  if (parts == 0) {
    parts = 1;
    const int forced = env_int("AKAS_B200_ROWS_PARTS", 0);
    if (epilogue == EPI_ACC && K % 64 == 0 && rounds == 1 && (forced > 1 || (forced == 0 && K >= 4096))) {
      long long best = (long long)(sh->RT + tile_n) * K;
      for (int p = 2; p <= 4; p *= 2) {
        if (forced > 1 && p != forced) continue;
        const int wide_n = ((out_cols * p + sms - 1) / sms + 15) / 16 * 16;
        if (wide_n > widest || ((out_cols + wide_n - 1) / wide_n) * p > sms || all_blocks < 4 * p) continue;
        const long long bytes = (long long)(sh->RT + wide_n) * K / p;
        if (forced > 1 || bytes * 4 <= best * 3) { best = bytes; parts = p; }
      }
    }
  }
  if (parts > 1) tile_n = ((out_cols * parts + sms - 1) / sms + 15) / 16 * 16;
  sh->tile_n = tile_n;
  sh->wide = K % 64 == 0 ? 1 : 0;
  sh->parts = parts;
  const int gather_bytes = parts > 1 ? (parts - 1) * sh->RT * (tile_n + 4) * (int)sizeof(float) : 0;
  budget -= gather_bytes;
  int k_blocks = all_blocks;  // of a part
  const int step_bytes = (sh->RT + halves * tile_n) * 128;
  // All of an SM's shared memory by default. AKAS_B200_ROWS_SMEM_KB gives a block less (and at most half of tensor
  // memory), so that a block of the next kernel on the stream can set itself up and fetch its first weights beside a
  // block of this one that is still summing or reading out: measured on a B200 at 64 tokens that loses more (thinner
  // rings, two blocks sharing an SM's 64 bytes a cycle from the L2) than the overlap wins, 1.72 ms a step against 1.40.
  const int share = env_int("AKAS_B200_ROWS_SMEM_KB", 227) * 1024;
  int g = 1, stages = 0, tmem_cap = 256;
  for (int attempt = 0; attempt < 2; ++attempt) {
    const int have = attempt == 0 && share < budget ? share : budget;
    tmem_cap = have < budget ? 256 : 512;
    const int room = have - 8 * STAGING - 1024;  // staging tiles (the products' reads past RT rows end inside them), alignment
    // Stages of up to 48 KB: fewer copies to start and fewer barriers to pass, yet three or more stages in flight.
    g = env_int("AKAS_B200_ROWS_STEPS", 0);
    if (g <= 0) {
      g = 1;
      while (g < 4 && 2 * g * step_bytes <= 48 * 1024 && 2 * g <= k_blocks) g *= 2;
    }
    if (g > k_blocks) g = k_blocks;
    stages = room / (g * step_bytes);
    while (stages < 3 && g > 1) { g /= 2; stages = room / (g * step_bytes); }
    if (stages >= 3 || have == budget) break;
  }
  if (stages < 2) return false;
  const int cap = env_int("AKAS_B200_ROWS_STAGES", MAX_STAGES);
  if (stages > cap) stages = cap;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  sh->G = g;
  sh->part_blocks = all_blocks;
  if (parts > 1) {  // a part: a whole number of stages, and the last part is not empty
    sh->part_blocks = ((all_blocks + parts - 1) / parts + g - 1) / g * g;
    if ((parts - 1) * sh->part_blocks >= all_blocks) return false;
    k_blocks = sh->part_blocks;
  }
  const int tiles = (out_cols + tile_n - 1) / tile_n;
  sh->buffers = tiles > sms ? 2 : 1;
  // As many issuing warps as tensor memory has accumulators for, at most one per stage of a tile or of the ring.
  const int steps = (k_blocks + g - 1) / g;
  int issuers = env_int("AKAS_B200_ROWS_ISSUERS", ISSUERS);
  if (issuers > ISSUERS) issuers = ISSUERS;
  if (issuers > steps) issuers = steps;
  if (issuers > stages) issuers = stages;
  while (issuers > 1 && sh->buffers * issuers * halves * tile_n > tmem_cap) --issuers;
  if (issuers < 1) issuers = 1;
  sh->stages = stages;
  sh->issuers = issuers;
  sh->suspend_ns = (unsigned)env_int("AKAS_B200_ROWS_SUSPEND_NS", 200);
  sh->tmem_cols = 32;
  while (sh->tmem_cols < sh->buffers * issuers * halves * tile_n) sh->tmem_cols *= 2;
  return sh->tmem_cols <= 512;
}

// The launch of a product that is not cut along K (also where a cut was planned and the device cannot place its clusters).
template <int EPI, typename Kernel>
int launch_uncut(Kernel kernel, const void* x, const void* w, const CUtensorMap& map_y, const Shape& sh, int M, int O,
                 int K, int sms, cudaStream_t stream) {
  constexpr bool SWIGLU = EPI == EPI_SWIGLU;
  const int out_cols = SWIGLU ? O / 2 : O, halves = SWIGLU ? 2 : 1;
  CUtensorMap map_x, map_w;
  int err = sh.wide ? make_wide_map(&map_x, x, M, K, sh.RT, sh.G) : make_map(&map_x, x, M, K, sh.RT);
  if (!err) err = weight_map(&map_w, w, O, K, sh.tile_n, sh.G, sh.wide, SWIGLU);
  if (err) return err;
  const int tiles = (out_cols + sh.tile_n - 1) / sh.tile_n, per = (tiles + sms - 1) / sms;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((tiles + per - 1) / per);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = sh.stages * sh.G * (sh.RT + halves * sh.tile_n) * 128 + 8 * STAGING + 1024;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = chained_launches_enabled() ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&config, kernel, map_x, map_w, map_y, sh);
  return e != cudaSuccess ? (int)e : launch_status();
}

template <int EPI>
int launch(const void* x, const void* w, void* y, int M, int O, int K, bool dry, cudaStream_t stream) {
  auto kernel = gemm_rows_kernel<EPI>;
  static int budget[64] = {}, sms[64] = {};
  static std::mutex mutex;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (budget[device] == 0) {
      cudaFuncAttributes attributes;
      cudaError_t e = cudaFuncGetAttributes(&attributes, kernel);
      if (e != cudaSuccess) return (int)e;
      const int room = SMEM_LIMIT - (int)attributes.sharedSizeBytes;
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, room);
      if (e != cudaSuccess) return (int)e;
      cudaDeviceGetAttribute(&sms[device], cudaDevAttrMultiProcessorCount, device);
      budget[device] = room;
    }
  }
  Shape sh;
  if (!plan(&sh, M, O, K, EPI, sms[device], budget[device])) {
    // (a cut along K that does not fit after all: the product uncut)
    if (!plan(&sh, M, O, K, EPI, sms[device], budget[device], 1)) return 3999;
  }
  if (dry) return 0;
  constexpr bool SWIGLU = EPI == EPI_SWIGLU;
  const int out_cols = SWIGLU ? O / 2 : O;
  CUtensorMap map_x, map_w, map_y;
  int err = sh.wide ? make_wide_map(&map_x, x, M, K, sh.RT, sh.G) : make_map(&map_x, x, M, K, sh.RT);
  if (err) return err;
  err = weight_map(&map_w, w, O, K, sh.tile_n, sh.G, sh.wide, SWIGLU);
  if (err) return err;
  err = make_out_map(&map_y, y, M, out_cols, EPI == EPI_ACC || EPI == EPI_F32 ? 4 : 2);
  if (err) return err;
  const int tiles = (out_cols + sh.tile_n - 1) / sh.tile_n;
  const int per = (tiles + sms[device] - 1) / sms[device];  // tiles per block, and as few blocks as do it in that many rounds
  const int halves = SWIGLU ? 2 : 1;
  auto smem_of = [&](const Shape& s) {
    return s.stages * s.G * (s.RT + halves * s.tile_n) * 128 + 8 * STAGING + 1024 +
           (s.parts > 1 ? (s.parts - 1) * s.RT * (s.tile_n + 4) * (int)sizeof(float) : 0);
  };
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(sh.parts > 1 ? tiles * sh.parts : (tiles + per - 1) / per);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem_of(sh);
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  int n = 0;
  if (chained_launches_enabled()) {
    attribute[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (sh.parts > 1) {  // the parts of a tile: a thread-block cluster, if the device can place one
    attribute[n].id = cudaLaunchAttributeClusterDimension;
    attribute[n].val.clusterDim.x = sh.parts;
    attribute[n].val.clusterDim.y = 1;
    attribute[n].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = n + 1;
    static std::map<std::tuple<int, int, int>, int> room;  // (device, parts, shared memory) -> clusters resident at once
    int clusters = 0;
    {
      std::lock_guard<std::mutex> lock(mutex);
      const auto key = std::make_tuple(device, sh.parts, (int)config.dynamicSmemBytes);
      if (!room.count(key)) {
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) { cudaGetLastError(); clusters = 0; }
        room[key] = clusters;
      }
      clusters = room[key];
    }
    if (clusters * sh.parts < (int)config.gridDim.x) {  // all of a launch's clusters are resident at once, or the product goes uncut
      if (!plan(&sh, M, O, K, EPI, sms[device], budget[device], 1)) return 3999;
      return launch_uncut<EPI>(kernel, x, w, map_y, sh, M, O, K, sms[device], stream);
    }
    ++n;
  }
  config.attrs = attribute;
  config.numAttrs = n;
  const cudaError_t e = cudaLaunchKernelEx(&config, kernel, map_x, map_w, map_y, sh);
  return e != cudaSuccess ? (int)e : launch_status();
}

int dispatch(const void* x, const void* w, void* y, int M, int O, int K, int epilogue, bool dry, cudaStream_t stream) {
  if (M <= 0 || O <= 0) return 0;
  if (M > MAX_TOKENS || K <= 0 || K % 8) return 3999;
  if (epilogue == EPI_SWIGLU && (O % 2 || (O / 2) % 8)) return 3999;
  if (epilogue == EPI_BF16 && O % 8) return 3999;
  if ((epilogue == EPI_ACC || epilogue == EPI_F32) && O % 4) return 3999;
  if (!dry && ((uintptr_t)x % 16 || (uintptr_t)w % 16 || (uintptr_t)y % 16)) return (int)cudaErrorInvalidValue;
  switch (epilogue) {
    case EPI_BF16: return launch<EPI_BF16>(x, w, y, M, O, K, dry, stream);
    case EPI_ACC: return launch<EPI_ACC>(x, w, y, M, O, K, dry, stream);
    case EPI_SWIGLU: return launch<EPI_SWIGLU>(x, w, y, M, O, K, dry, stream);
    case EPI_F32: return launch<EPI_F32>(x, w, y, M, O, K, dry, stream);
    default: return (int)cudaErrorInvalidValue;
  }
}

}  // namespace

// x: bfloat16 [M, K], M <= 128; w: bfloat16 [O, K]; epilogue 0: y bfloat16 [M, O]; 1: y float32 [M, O] +=; 3: y float32
// [M, O]; 2 (SwiGLU, w the stacked [2F, K] gate and up matrices, O = 2F): y bfloat16 [M, F]. Returns 0, a CUDA error
// code, 3000 + a driver error from building a tensor map, or 3999 if the kernel does not take these sizes (nothing was
// launched): K and the row pitch of y must be multiples of 16 bytes' worth of elements (K % 8, O % 8 for bfloat16 y,
// O % 4 for float32 y, F % 8), since TMA moves every operand.
AKAS_API int akas_gemm_rows(const void* x, const void* w, void* y, int M, int O, int K, int epilogue, cudaStream_t stream) {
  return dispatch(x, w, y, M, O, K, epilogue, false, stream);
}

// 1 if akas_gemm_rows takes these sizes on the current device, else 0. Launches nothing.
AKAS_API int akas_gemm_rows_takes(int M, int O, int K, int epilogue) {
  return dispatch(nullptr, nullptr, nullptr, M, O, K, epilogue, true, 0) == 0 ? 1 : 0;
}

// 0 if no bounded wait of the kernel has ever run out on the current device (1: producer, 2: tensor cores,
// 3: read-out). Synchronises with the device.
AKAS_API int akas_gemm_rows_status() {
  int status = -1;
  const cudaError_t e = cudaMemcpyFromSymbol(&status, g_rows_status, sizeof(int));
  return e == cudaSuccess ? status : -(int)e;
}
