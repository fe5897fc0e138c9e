// bfloat16 matrix product for prompt portions on pairs of SMs: y[M, N] = x[M, K] . W[N, K]^T with
// tcgen05.mma.cta_group::2, float32 accumulation in the tensor memory of both SMs, epilogues fused into the read-out.
//
// A thread-block cluster of two blocks (two SMs) walks output tiles of 256 tokens x 256 channels. Each block stages
// its own 128 token rows of x and HALF of the tile's channels of W (128 rows), 32 KB a step of K instead of the 48 KB a
// lone block needs for a 128 x 256 tile: a product of the pair reads the 256 channels from both blocks' shared
// memory. That halves what a block writes into and reads out of its shared memory per multiply-add, which is what
// bounds the one-block kernel of gemm_tcgen05.cu (its TMA writes and operand reads ask for 192 bytes a cycle of a
// shared memory that gives 128).
//   warp 0   producer, in both blocks: TMA loads of the block's slice of x and of W into a ring of three stages of two
//            64-wide steps of K each. Every load
//            of either block counts its bytes on the LEADER's "full" barrier of the stage (the block of cluster rank
//            0), on which the leader has announced the bytes of both.
//   warp 1   tensor cores: both blocks allocate tensor memory together (two accumulators of 256 columns); one thread
//            of the leader issues, per stage, eight tcgen05.mma.cta_group::2 (M 256, N 256, K 16) and commits them to
//            the stage's "empty" barrier of BOTH blocks (multicast commit); after a tile's last stage it commits to
//            both blocks' "accumulator full" barrier.
//   warps 2-5 epilogue, in both blocks: each warp reads the 32 accumulator lanes (token rows) of its sub-partition of
//            its own block's tensor memory, as in gemm_tcgen05.cu (BF16 and SWIGLU read-outs), and arrives on
//            the leader's "accumulator empty" barrier (the peer does so through the cluster's shared memory window).
// For SWIGLU the leader stages the tile's 128 gate rows and the peer the 128 up rows under them of the stacked
// [2F, K] matrix, so columns 0-127 of an accumulator are gate and 128-255 up, in both blocks.
// No load is multicast. Every wait on an mbarrier is bounded (akas_gemm_pair_status); the cluster meets before any
// block leaves, so that no block writes into or reads from a peer that is gone.
#include <math.h>

#include "tcgen05.cuh"

using namespace akas;
using namespace akas::tc;

namespace {

constexpr int BM = 128;    // token rows a block stages; a pair's tile has 256
constexpr int BN = 256;    // channels of a pair's tile; a block stages half of them
constexpr int STEPS = 2;    // 64-wide steps of K in a stage
constexpr int STAGES = 3;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, HALF_BYTES = A_BYTES + B_BYTES;
constexpr int STAGE_BYTES = STEPS * HALF_BYTES;  // [x, W] of one step of K, then of the next
enum { EPI_BF16 = 0, EPI_SWIGLU = 2 };  // the numbers of gemm_tcgen05.cu's read-outs

__device__ int g_pair_status = 0;  // 0, or which bounded wait ran out last (1 producer, 2 tensor cores, 3 epilogue)

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

template <int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 void* __restrict__ y_, int M, int N, int K, int F) {
  // N: channels of the product (for SWIGLU the stacked height 2F); a tile covers BN of them (SWIGLU: BN/2 gate
  // rows f0.. and BN/2 up rows F + f0..).
  constexpr int TILE_N = EPI == EPI_SWIGLU ? BN / 2 : BN;  // output columns a tile yields
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
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
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(2 * BN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_meet();  // the peer's barriers exist and its tensor memory is allocated before anything arrives there
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_base_s;

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
      unsigned it = 0;
      for (int tile = pair; tile < tiles; tile += pairs) {
        const int m0 = (tile / tiles_n) * 2 * BM + (int)rank * BM, n0 = (tile % tiles_n) * TILE_N;
        // this block's half of the tile's channels: rows of W
        const int w_row = EPI == EPI_SWIGLU ? (rank == 0 ? n0 : F + n0) : n0 + (int)rank * (BN / 2);
        for (int kb = 0; kb < k_blocks; kb += STEPS, ++it) {
          const int s = it % STAGES;
          wait_for(&empty_bar[s], ((it / STAGES) & 1) ^ 1, 1);
          if (*(volatile int*)&abort_s) break;
          unsigned char* a = smem + (size_t)s * STAGE_BYTES;
          const unsigned leader_full = peer_address(&full_bar[s], 0);
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);  // the bytes of both blocks
#pragma unroll
          for (int h = 0; h < STEPS; ++h) {  // a step past the end of K is filled with zeros
            tma_load_2d_for(a + h * HALF_BYTES, &map_x, (kb + h) * BK, m0, leader_full);
            tma_load_2d_for(a + h * HALF_BYTES + A_BYTES, &map_w, (kb + h) * BK, w_row, leader_full);
          }
        }
        if (*(volatile int*)&abort_s) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tensor cores (the leader issues for the pair)
    if (lane == 0 && rank == 0) {
      // instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, N = 256, M = 256 over the pair
      constexpr unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(2 * BM >> 4) << 24);
      unsigned it = 0, t = 0;
      for (int tile = pair; tile < tiles; tile += pairs, ++t) {
        const unsigned acc = t & 1;
        wait_for(&acc_empty[acc], ((t >> 1) & 1) ^ 1, 2);  // both blocks' epilogues have drained this accumulator
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
            const uint64_t a_desc = smem_desc(a + h * HALF_BYTES), b_desc = smem_desc(a + h * HALF_BYTES + A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)  // 32 bytes further along the swizzled row per step
              umma_pair(d, a_desc + (uint64_t)(k * UMMA_K * 2 >> 4), b_desc + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
                        (kb | h | k) != 0 ? 1u : 0u);
          }
          // One commit for eight products: a commit to both blocks costs the issuing thread about as much as four
          // products do, so a stage holds two steps of K.
          umma_commit_pair(&empty_bar[s]);  // the stage is free in both blocks once these products have read it
        }
        if (*(volatile int*)&abort_s) break;
        umma_commit_pair(&acc_full[acc]);  // the tile's sums are complete, in both blocks
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: warps 2..5 (both blocks)
    const int sub = warp & 3;  // the tensor-memory sub-partition (32 lanes) this warp may read
    unsigned t = 0;
    for (int tile = pair; tile < tiles; tile += pairs, ++t) {
      const unsigned acc = t & 1;
      const int m0 = (tile / tiles_n) * 2 * BM + (int)rank * BM, n0 = (tile % tiles_n) * TILE_N;
      wait_for(&acc_full[acc], (t >> 1) & 1, 3);
      if (*(volatile int*)&abort_s) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = m0 + sub * 32 + lane;
      const unsigned taddr = tmem_base + acc * BN + ((unsigned)(sub * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < TILE_N; c += 16) {
        float v[16];
        tmem_load16(taddr + c, v);
        if (EPI == EPI_SWIGLU) {
          float u[16];
          tmem_load16(taddr + BN / 2 + c, u);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = v[i] / (1.f + __expf(-v[i])) * u[i];
        }
        const int col = n0 + c;
        if (row < M && col < out_cols) {
          {
            bf16* dst = (bf16*)y_ + (size_t)row * out_cols + col;
            if (col + 16 <= out_cols && out_cols % 8 == 0) {
              float lo[8], hi[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) { lo[i] = v[i]; hi[i] = v[8 + i]; }
              store_vec(dst, lo);
              store_vec(dst + 8, hi);
            } else {
              for (int i = 0; i < 16 && col + i < out_cols; ++i) dst[i] = __float2bfloat16_rn(v[i]);
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {  // the leader's tensor-core thread waits for all eight warps
        if (rank == 0) mbar_arrive(&acc_empty[acc]);
        else mbar_arrive_at(peer_address(&acc_empty[acc], 0));
      }
    }
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
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN));
  }
}

// ------------------------------------------------------------------------------------------------ host side

template <int EPI>
int launch(const void* x, const void* w, void* y, int M, int N, int K, cudaStream_t stream) {
  constexpr int smem = STAGES * STAGE_BYTES + 1024;
  static int pairs_room = 0;
  if (pairs_room == 0) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    int device = 0, sms = 0;
    cudaGetDevice(&device);
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
    e = cudaOccupancyMaxActiveClusters(&room, gemm_pair_kernel<EPI>, &probe);
    if (e != cudaSuccess) return (int)e;
    if (room < 1) return (int)cudaErrorInvalidConfiguration;
    pairs_room = room < sms / 2 ? room : sms / 2;
  }
  const int F = N / 2;
  CUtensorMap map_x, map_w;
  int err = cached_map(&map_x, x, M, K, BM, false);
  if (err) return err;
  err = cached_map(&map_w, w, N, K, BN / 2, true);
  if (err) return err;
  const int out_cols = EPI == EPI_SWIGLU ? F : N, tile_n = EPI == EPI_SWIGLU ? BN / 2 : BN;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((out_cols + tile_n - 1) / tile_n);
  const int pairs = tiles < pairs_room ? tiles : pairs_room;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2 * pairs);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 2;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&config, gemm_pair_kernel<EPI>, map_x, map_w, y, M, N, K, F);
  return e != cudaSuccess ? (int)e : launch_status();
}

}  // namespace

// x: bfloat16 [M, K]; w: bfloat16 [N, K]; epilogue 0: y bfloat16 [M, N]; 2 (swiglu, w the stacked [2F, K] gate and
// up matrices, N = 2F): y bfloat16 [M, F]. Returns 0, a CUDA error code, or 3000 + a driver error from building a
// tensor map. There is no read-out that adds into a float32 y here: in this kernel its global loads ran at a
// fraction of what the one-block kernel's do (measured; cause not found), and the library serves those products.
AKAS_API int akas_gemm_pair(const void* x, const void* w, void* y, int M, int N, int K, int epilogue, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || (uintptr_t)x % 16 || (uintptr_t)w % 16 || (uintptr_t)y % 16) return (int)cudaErrorInvalidValue;
  if (epilogue == EPI_SWIGLU && (N % 2 || (N / 2) % 8)) return (int)cudaErrorInvalidValue;
  switch (epilogue) {
    case EPI_BF16: return launch<EPI_BF16>(x, w, y, M, N, K, stream);
    case EPI_SWIGLU: return launch<EPI_SWIGLU>(x, w, y, M, N, K, stream);
    default: return (int)cudaErrorInvalidValue;
  }
}

// 0 if no bounded wait of the kernel has ever run out on the current device (1: producer, 2: tensor cores,
// 3: epilogue). Synchronises with the device.
AKAS_API int akas_gemm_pair_status() {
  int status = -1;
  const cudaError_t e = cudaMemcpyFromSymbol(&status, g_pair_status, sizeof(int));
  return e == cudaSuccess ? status : -(int)e;
}
