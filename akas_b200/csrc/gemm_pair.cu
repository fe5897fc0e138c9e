// bfloat16 matrix product for prompt portions on pairs of SMs: y[M, N] = x[M, K] . W[N, K]^T with
// tcgen05.mma.cta_group::2, float32 accumulation in the tensor memory of both SMs, epilogues fused into the read-out
// and written by TMA.
//
// A thread-block cluster of two blocks (two SMs) walks output tiles of 256 tokens x BN channels (BN 256, 192, 128 or
// 64: the width that finishes first by a count of rounds over the pairs and of what a stage costs, see launch_width). Each block stages its own 128 token rows of x and HALF of
// the tile's channels of W, 32 KB a step of K at BN = 256 instead of the 48 KB a lone block needs for a 128 x 256
// tile: a product of the pair reads the channels from both blocks' shared memory. That halves what a block writes
// into and reads out of its shared memory per multiply-add, which is what bounds a one-block kernel (its TMA writes
// and operand reads ask for 192 bytes a cycle of a shared memory that gives 128).
//   The kernel is launched as a programmatic dependent of the kernel before it on the stream: it sets itself up and
//   asks for its first weights while that kernel drains, and waits for it before it touches the token rows.
//   warp 0   producer, in both blocks: TMA loads of the block's slice of x and of W into a ring of stages of two
//            64-wide steps of K each: ONE copy per operand and stage (a box of two groups of 64 k from a view
//            [K / 64][rows][64] of the matrix; starting a copy costs the issuing thread some 300 cycles whatever it
//            moves, and with a copy per step the producer fell behind the tensor cores; K that is no multiple of 64
//            takes a copy per step). Every load of either block counts its bytes on the LEADER's "full" barrier of
//            the stage (the block of cluster rank 0), on which the leader has announced the bytes of both.
//   warp 1   tensor cores: both blocks allocate tensor memory together (two accumulators of BN columns); one thread
//            of the leader issues, per stage, eight tcgen05.mma.cta_group::2 (M 256, N BN, K 16) and commits them to
//            the stage's "empty" barrier of BOTH blocks (multicast commit: a commit to both blocks costs the issuing
//            thread about as much as four products, hence two steps of K per stage); after a tile's last stage it
//            commits to both blocks' "accumulator full" barrier.
//   warps 2-5 read-out, in both blocks: each warp owns the 32 accumulator lanes (token rows) of its sub-partition
//            of its own block's tensor memory. A lane holds a token row, so storing from registers would touch 32
//            rows per instruction; instead the warp reads 32 columns with tcgen05.ld, writes them into a staging
//            tile in shared memory in the swizzle that TMA expects (no bank conflicts), and one lane hands the tile
//            (32 rows x 128 or 64 bytes) to TMA, which writes whole rows and clips at the matrix's edges:
//              BF16    y bfloat16 [M, N]          a TMA store of 32 x 64 channels
//              ACC     y float32 [M, N] +=        a TMA reduce-add of 32 x 32 channels: the residual stream is added
//                                                 to in the L2, no SM reads it
//              F32     y float32 [M, N]           a TMA store of 32 x 32 channels
//              SWIGLU  y bfloat16 [M, F]          silu(gate) * up of 32 channels, a TMA store of 32 x 32
//            Two staging tiles per warp: the next is filled while TMA reads the last. The warp then arrives on the
//            leader's "accumulator empty" barrier (the peer through the cluster's shared memory window).
// For SWIGLU the leader stages the tile's BN/2 gate rows and the peer the BN/2 up rows under them of the stacked
// [2F, K] matrix, so columns 0..BN/2-1 of an accumulator are gate and the rest up, in both blocks.
// No load is multicast. Every wait on an mbarrier is bounded (akas_gemm_pair_status); the cluster meets before any
// block leaves, so that no block writes into or reads from a peer that is gone.
#include <math.h>

#include "tcgen05.cuh"

using namespace akas;
using namespace akas::tc;

namespace {

constexpr int BM = 128;    // token rows a block stages; a pair's tile has 256
constexpr int STEPS = 2;    // 64-wide steps of K in a stage
constexpr int THREADS = 192;
constexpr int STAGING = 4096;  // bytes of one staging tile: 32 rows x 128 bytes
enum { EPI_BF16 = 0, EPI_ACC = 1, EPI_SWIGLU = 2, EPI_F32 = 3 };

template <int BN> struct Shape {
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, HALF_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGE_BYTES = STEPS * HALF_BYTES;  // x of both steps of K, then W of both steps
  static constexpr int STAGES = BN >= 192 ? 3 : 4;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 8 * STAGING + 1024;
  static constexpr int TMEM_COLS = BN > 128 ? 512 : 2 * BN;  // two accumulators of BN columns, a power of two
};

__device__ int g_pair_status = 0;  // 0, or which bounded wait ran out last (1 producer, 2 tensor cores, 3 read-out)

__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared memory window, of a location of block `rank`.
__device__ __forceinline__ unsigned peer_address(const void* local, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_at(unsigned cluster_address) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}
__device__ __forceinline__ void cluster_meet() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A tile load into this block's shared memory whose bytes are counted on a barrier given by its address in the
// cluster's window (the leader's). Not a multicast: one destination.
__device__ __forceinline__ void tma_load_2d_for(void* smem_dst, const CUtensorMap* map, int c0, int c1, unsigned bar_address) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(bar_address) : "memory");
}
// The same with a box of a three-dimensional view [K / 64][rows][64] of the matrix: rows x 64 k x `STEPS` groups of k
// in ONE copy (an instruction that starts a TMA copy costs the issuing thread some 300 cycles whatever it moves; with
// a copy per step of K the producer could not keep up with the tensor cores).
__device__ __forceinline__ void tma_load_3d_for(void* smem_dst, const CUtensorMap* map, int row, int group, unsigned bar_address) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(0), "r"(row), "r"(group), "r"(bar_address) : "memory");
}
__device__ __forceinline__ void umma_pair(unsigned tmem_d, uint64_t a_desc, uint64_t b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once the products issued so far have run, on the barrier at this offset in both blocks of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
}
// 32 consecutive float32 columns of this thread's accumulator lane.
__device__ __forceinline__ void tmem_load32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      "tcgen05.wait::ld.sync.aligned;\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// A staging tile in shared memory to the matrix behind `map`, at column c0, row c1; rows and columns past the
// matrix's edges are not written.
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

template <int BN, int EPI, bool WIDE>
__global__ void __launch_bounds__(THREADS)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_y, int M, int N, int K, int F) {
  // N: channels of the product (for SWIGLU the stacked height 2F); a tile covers BN of them (SWIGLU: BN/2 gate
  // rows f0.. and BN/2 up rows F + f0..).
  using S = Shape<BN>;
  constexpr int STAGES = S::STAGES, A_BYTES = S::A_BYTES, STAGE_BYTES = S::STAGE_BYTES;
  constexpr int TILE_N = EPI == EPI_SWIGLU ? BN / 2 : BN;  // output columns a tile yields
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* staging = smem + STAGES * STAGE_BYTES;  // [4 warps][2][STAGING], 1,024-byte aligned
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const unsigned rank = cluster_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int out_cols = EPI == EPI_SWIGLU ? F : N;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (out_cols + TILE_N - 1) / TILE_N;
  const int tiles = tiles_m * tiles_n, k_blocks = (K + BK - 1) / BK;

  if (tid == 0) {
    abort_s = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }  // four warps of each block
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory of both SMs: two accumulators of BN float32 columns, 128 lanes in each block
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(S::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_meet();  // the peer's barriers exist and its tensor memory is allocated before anything arrives there
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_base_s;
  chain_release();  // (programmatic dependent launch) the next kernel on the stream may set itself up beside this one

  auto wait_for = [&](uint64_t* bar, unsigned parity, int code) {
    if (*(volatile int*)&abort_s) return;
    if (!mbar_wait(bar, parity)) {
      *(volatile int*)&abort_s = 1;
      atomicExch(&g_pair_status, code);
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both blocks)
    if (lane == 0) {
      // The ring's first filling asks for the weights at once (no kernel writes them) and for the token rows only when
      // the kernel before this one on the stream is done; from then on a stage's two copies go out together.
      const int per_tile = (k_blocks + STEPS - 1) / STEPS;  // stages of a tile
      const int my_tiles = pair < tiles ? (tiles - pair + pairs - 1) / pairs : 0;
      const int total = my_tiles * per_tile, head = total < STAGES ? total : STAGES;
      auto load = [&](int i, bool weights, bool rows) {
        const int tile = pair + (i / per_tile) * pairs, kb = (i % per_tile) * STEPS, s = i % STAGES;
        const int m0 = (tile / tiles_n) * 2 * BM + (int)rank * BM, n0 = (tile % tiles_n) * TILE_N;
        // this block's half of the tile's channels: rows of W
        const int w_row = EPI == EPI_SWIGLU ? (rank == 0 ? n0 : F + n0) : n0 + (int)rank * (BN / 2);
        unsigned char* a = smem + (size_t)s * STAGE_BYTES;
        const unsigned leader_full = peer_address(&full_bar[s], 0);
        if (weights && rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);  // the bytes of both blocks
        if (WIDE) {  // K is a multiple of 64: both steps of K in one copy per operand (groups past K: zeros)
          if (rows) tma_load_3d_for(a, &map_x, m0, kb, leader_full);
          if (weights) tma_load_3d_for(a + STEPS * A_BYTES, &map_w, w_row, kb, leader_full);
        } else {
#pragma unroll
          for (int h = 0; h < STEPS; ++h) {  // a step past the end of K is filled with zeros
            if (rows) tma_load_2d_for(a + h * A_BYTES, &map_x, (kb + h) * BK, m0, leader_full);
            if (weights) tma_load_2d_for(a + STEPS * A_BYTES + h * S::B_BYTES, &map_w, (kb + h) * BK, w_row, leader_full);
          }
        }
      };
      for (int i = 0; i < head; ++i) load(i, true, false);
      chain_wait();
      for (int i = 0; i < head; ++i) load(i, false, true);
      for (int i = head; i < total; ++i) {
        wait_for(&empty_bar[i % STAGES], ((i / STAGES) & 1) ^ 1, 1);
        if (*(volatile int*)&abort_s) break;
        load(i, true, true);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tensor cores (the leader issues for the pair)
    if (lane == 0 && rank == 0) {
      // instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, N = BN, M = 256 over the pair
      constexpr unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(2 * BM >> 4) << 24);
      unsigned it = 0, t = 0;
      for (int tile = pair; tile < tiles; tile += pairs, ++t) {
        const unsigned acc = t & 1;
        wait_for(&acc_empty[acc], ((t >> 1) & 1) ^ 1, 2);  // both blocks' read-outs have drained this accumulator
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; kb += STEPS, ++it) {
          const int s = it % STAGES;
          wait_for(&full_bar[s], (it / STAGES) & 1, 2);
          if (*(volatile int*)&abort_s) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned char* a = smem + (size_t)s * STAGE_BYTES;
#pragma unroll
          for (int h = 0; h < STEPS; ++h) {
            if (kb + h >= k_blocks) break;  // zeros: nothing to add
            const uint64_t a_desc = smem_desc(a + h * A_BYTES), b_desc = smem_desc(a + STEPS * A_BYTES + h * S::B_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)  // 32 bytes further along the swizzled row per step
              umma_pair(d, a_desc + (uint64_t)(k * UMMA_K * 2 >> 4), b_desc + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
                        (kb | h | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[s]);  // the stage is free in both blocks once these products have read it
        }
        if (*(volatile int*)&abort_s) break;
        umma_commit_pair(&acc_full[acc]);  // the tile's sums are complete, in both blocks
      }
    }
  } else {
    // ------------------------------------------------------------------ read-out: warps 2..5 (both blocks)
    const int sub = warp & 3;  // the tensor-memory sub-partition (32 lanes) this warp may read
    unsigned char* stage_of_warp = staging + (size_t)sub * 2 * STAGING;
    unsigned t = 0, stores = 0;
    chain_wait();  // what the read-out adds to is an earlier kernel's
    for (int tile = pair; tile < tiles; tile += pairs, ++t) {
      const unsigned acc = t & 1;
      const int m0 = (tile / tiles_n) * 2 * BM + (int)rank * BM, n0 = (tile % tiles_n) * TILE_N;
      wait_for(&acc_full[acc], (t >> 1) & 1, 3);
      if (*(volatile int*)&abort_s) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row0 = m0 + sub * 32;  // this warp's 32 token rows; lane l holds row0 + l
      const unsigned taddr = tmem_base + acc * BN + ((unsigned)(sub * 32) << 16);
      constexpr int COLS = EPI == EPI_BF16 ? 64 : 32;  // output columns per staging tile
#pragma unroll 1
      for (int c = 0; c < TILE_N; c += COLS, ++stores) {
        if (n0 + c >= out_cols || row0 >= M) break;  // nothing of this warp's rows or of these columns is inside
        unsigned char* buf = stage_of_warp + (stores & 1) * STAGING;
        if (lane == 0) bulk_wait_read<1>();  // the store before last has read this tile
        __syncwarp();
        if (EPI == EPI_ACC || EPI == EPI_F32) {
          float v[32];
          tmem_load32(taddr + c, v);
          // row `lane` of 128 bytes, its 16-byte units XORed with the row's number within eight (the 128-byte swizzle)
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (EPI == EPI_ACC) tma_add_2d(&map_y, buf, n0 + c, row0); else tma_store_2d(&map_y, buf, n0 + c, row0);
            bulk_commit();
          }
        } else if (EPI == EPI_BF16) {
          float v[32], u[32];
          tmem_load32(taddr + c, v);
          tmem_load32(taddr + c + 32, u);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o, p;
            o.x = pack2(v[8 * j], v[8 * j + 1]); o.y = pack2(v[8 * j + 2], v[8 * j + 3]);
            o.z = pack2(v[8 * j + 4], v[8 * j + 5]); o.w = pack2(v[8 * j + 6], v[8 * j + 7]);
            p.x = pack2(u[8 * j], u[8 * j + 1]); p.y = pack2(u[8 * j + 2], u[8 * j + 3]);
            p.z = pack2(u[8 * j + 4], u[8 * j + 5]); p.w = pack2(u[8 * j + 6], u[8 * j + 7]);
            *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
            *reinterpret_cast<uint4*>(buf + lane * 128 + (((j + 4) ^ (lane & 7)) << 4)) = p;
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) { tma_store_2d(&map_y, buf, n0 + c, row0); bulk_commit(); }
        } else {
          float v[32], u[32];
          tmem_load32(taddr + c, v);
          tmem_load32(taddr + BN / 2 + c, u);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __fdividef(v[i], 1.f + __expf(-v[i])) * u[i];  // the fast division: IEEE division cost more than the tile's loads
          // row `lane` of 64 bytes, its 16-byte units XORed with bits 7-8 of the address (the 64-byte swizzle)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack2(v[8 * j], v[8 * j + 1]); o.y = pack2(v[8 * j + 2], v[8 * j + 3]);
            o.z = pack2(v[8 * j + 4], v[8 * j + 5]); o.w = pack2(v[8 * j + 6], v[8 * j + 7]);
            *reinterpret_cast<uint4*>(buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) = o;
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) { tma_store_2d(&map_y, buf, n0 + c, row0); bulk_commit(); }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {  // the leader's tensor-core thread waits for all eight warps
        if (rank == 0) mbar_arrive(&acc_empty[acc]);
        else mbar_arrive_at(peer_address(&acc_empty[acc], 0));
      }
    }
    if (lane == 0) bulk_wait_all();  // what this warp handed to TMA has been written before the block may leave
    __syncwarp();
  }

  // wind down: everyone meets, the pair meets, then the allocating warps free tensor memory
  if (*(volatile int*)&abort_s) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // a lost launch: let copies and products in flight finish
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_meet();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(S::TMEM_COLS));
  }
}

// ------------------------------------------------------------------------------------------------ host side

// A tensor map of a row-major matrix [rows, cols] of 2- or 4-byte elements for the read-out's staging tiles:
// boxes of 32 rows x box_cols (128 or 64 bytes), in the swizzle of that width.
int make_out_map(CUtensorMap* map, void* base, int rows, int cols, int elem_bytes, int box_cols) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return 3001;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, 32};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims,
                        strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        box_cols * elem_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 3000 + (int)r;
}

// A tensor map of a row-major bfloat16 matrix [rows, K], K a multiple of 64, seen as [K / 64][rows][64]: boxes of 64 k x
// box_rows x `STEPS` groups of k, 128-byte swizzle, zeros outside.
int make_wide_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return 3001;
  const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(K / 64)};
  const cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, STEPS};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 3000 + (int)r;
}

std::mutex g_wide_mutex;
std::map<std::tuple<const void*, int, int, int>, CUtensorMap> g_wide_maps;  // weights keep their maps

int cached_wide_map(CUtensorMap* out, const void* base, int rows, int K, int box_rows, bool cache) {
  if (!cache) return make_wide_map(out, base, rows, K, box_rows);
  std::lock_guard<std::mutex> lock(g_wide_mutex);
  const auto key = std::make_tuple(base, rows, K, box_rows);
  auto it = g_wide_maps.find(key);
  if (it == g_wide_maps.end()) {
    CUtensorMap map;
    const int err = make_wide_map(&map, base, rows, K, box_rows);
    if (err) return err;
    it = g_wide_maps.emplace(key, map).first;
  }
  *out = it->second;
  return 0;
}

template <int BN, int EPI, bool WIDE>
int launch(const void* x, const void* w, void* y, int M, int N, int K, cudaStream_t stream) {
  constexpr int smem = Shape<BN>::SMEM;
  static int pairs_room[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  if (pairs_room[device] == 0) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<BN, EPI, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(sms & ~1);
    probe.blockDim = dim3(THREADS);
    probe.dynamicSmemBytes = smem;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 2;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    probe.attrs = attribute;
    probe.numAttrs = 1;
    int room = 0;
    e = cudaOccupancyMaxActiveClusters(&room, gemm_pair_kernel<BN, EPI, WIDE>, &probe);
    if (e != cudaSuccess) return (int)e;
    if (room < 1) return (int)cudaErrorInvalidConfiguration;
    pairs_room[device] = room < sms / 2 ? room : sms / 2;
  }
  const int F = N / 2;
  const int out_cols = EPI == EPI_SWIGLU ? F : N, tile_n = EPI == EPI_SWIGLU ? BN / 2 : BN;
  CUtensorMap map_x, map_w, map_y;
  int err = WIDE ? cached_wide_map(&map_x, x, M, K, BM, false) : cached_map(&map_x, x, M, K, BM, false);
  if (err) return err;
  err = WIDE ? cached_wide_map(&map_w, w, N, K, BN / 2, true) : cached_map(&map_w, w, N, K, BN / 2, true);
  if (err) return err;
  err = EPI == EPI_ACC || EPI == EPI_F32 ? make_out_map(&map_y, y, M, out_cols, 4, 32)
                                         : make_out_map(&map_y, y, M, out_cols, 2, EPI == EPI_BF16 ? 64 : 32);
  if (err) return err;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((out_cols + tile_n - 1) / tile_n);
  const int pairs = tiles < pairs_room[device] ? tiles : pairs_room[device];
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2 * pairs);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 2;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = chained_launches_enabled() ? 2 : 1;
  const cudaError_t e = cudaLaunchKernelEx(&config, gemm_pair_kernel<BN, EPI, WIDE>, map_x, map_w, map_y, M, N, K, F);
  return e != cudaSuccess ? (int)e : launch_status();
}

template <int EPI>
int launch_width(const void* x, const void* w, void* y, int M, int N, int K, cudaStream_t stream) {
  // The tile width that finishes first by a count of the issuing thread's cycles: rounds over the pairs of SMs (a B200
  // has 74) times what a stage of eight products takes, which is the tensor cores' 131 cycles a product at 256 channels
  // and in proportion for narrower tiles, but never less than the 700 cycles it costs the one thread to issue eight
  // products and their commit. So a tile narrower than 192 channels only pays where it saves a round: measured on
  // [2048 x 6912] . [1536 x 6912]^T, 128-channel tiles (96 tiles, two rounds) took 76 us and 192-channel tiles (64
  // tiles, one round) 49 us (the library: 42 us). Among equals the wider tile wins (it fetches the token rows less often).
  const long long rows = (M + 2 * BM - 1) / (2 * BM);
  const int out_cols = EPI == EPI_SWIGLU ? N / 2 : N;
  const int unit = EPI == EPI_SWIGLU ? 2 : 1;  // a SwiGLU tile of BN stacked rows yields BN / 2 channels
  int device = 0, sms = 148;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const long long pairs = sms / 2 > 0 ? sms / 2 : 1;
  int best = 256;
  long long best_cost = -1;
  for (const int bn : {256, 192, 128, 64}) {
    const long long tiles = rows * ((out_cols * unit + bn - 1) / bn), rounds = (tiles + pairs - 1) / pairs;
    const long long stage = 1048ll * bn / 256 > 700 ? 1048ll * bn / 256 : 700;
    const long long cost = rounds * stage;
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
  }
#define AKAS_PAIR_WIDTH(BN_) \
  case BN_: return K % 64 == 0 ? launch<BN_, EPI, true>(x, w, y, M, N, K, stream) : launch<BN_, EPI, false>(x, w, y, M, N, K, stream);
  switch (best) {
    AKAS_PAIR_WIDTH(256) AKAS_PAIR_WIDTH(192) AKAS_PAIR_WIDTH(128) AKAS_PAIR_WIDTH(64)
  }
#undef AKAS_PAIR_WIDTH
  return (int)cudaErrorInvalidValue;
}

}  // namespace

// x: bfloat16 [M, K]; w: bfloat16 [N, K]; epilogue 0: y bfloat16 [M, N]; 1: y float32 [M, N] +=; 3: y float32 [M, N];
// 2 (swiglu, w the stacked [2F, K] gate and up matrices, N = 2F): y bfloat16 [M, F]. Returns 0, a CUDA error code, or 3000 + a driver
// error from building a tensor map. K and the row pitch of y in bytes must be multiples of 16 bytes' worth of elements
// (K % 8, N % 8 for bfloat16 y, N % 4 for float32 y, F % 8): TMA moves every operand.
AKAS_API int akas_gemm_pair(const void* x, const void* w, void* y, int M, int N, int K, int epilogue, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || (uintptr_t)x % 16 || (uintptr_t)w % 16 || (uintptr_t)y % 16) return (int)cudaErrorInvalidValue;
  if (epilogue == EPI_SWIGLU && (N % 2 || (N / 2) % 8)) return (int)cudaErrorInvalidValue;
  if (epilogue == EPI_BF16 && N % 8) return (int)cudaErrorInvalidValue;
  if ((epilogue == EPI_ACC || epilogue == EPI_F32) && N % 4) return (int)cudaErrorInvalidValue;
  switch (epilogue) {
    case EPI_BF16: return launch_width<EPI_BF16>(x, w, y, M, N, K, stream);
    case EPI_ACC: return launch_width<EPI_ACC>(x, w, y, M, N, K, stream);
    case EPI_SWIGLU: return launch_width<EPI_SWIGLU>(x, w, y, M, N, K, stream);
    case EPI_F32: return launch_width<EPI_F32>(x, w, y, M, N, K, stream);
    default: return (int)cudaErrorInvalidValue;
  }
}

// 0 if no bounded wait of the kernel has ever run out on the current device (1: producer, 2: tensor cores,
// 3: read-out). Synchronises with the device.
AKAS_API int akas_gemm_pair_status() {
  int status = -1;
  const cudaError_t e = cudaMemcpyFromSymbol(&status, g_pair_status, sizeof(int));
  return e == cudaSuccess ? status : -(int)e;
}
