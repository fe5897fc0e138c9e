// bfloat16 matrix product for prompt portions on Blackwell's tensor cores: y[M, N] = x[M, K] . W[N, K]^T,
// float32 accumulation in tensor memory, epilogues fused into the read-out.
//
// One persistent block per SM walks output tiles of 128 tokens x BN channels (BN = 256, or 128 for narrow
// outputs). Six warps, three roles:
//   warp 0   producer: one thread issues TMA tile loads (cp.async.bulk.tensor, 128-byte swizzle) of the
//            128 x 64 slice of x and the BN x 64 slice of W into a four-stage ring, each stage guarded by a
//            "full" mbarrier (bytes counted) and an "empty" one.
//   warp 1   tensor cores: allocates tensor memory (two accumulators of BN columns), and for every stage one
//            thread issues four tcgen05.mma (M 128, N BN, K 16) on shared-memory descriptors, then commits
//            them to the stage's "empty" barrier; after a tile's last stage it commits to the accumulator's
//            "full" barrier.
//   warps 2-5 epilogue: each warp owns the 32 accumulator lanes (token rows) of its tensor-memory
//            sub-partition; it reads 16 columns at a time with tcgen05.ld and
//              BF16:   rounds and stores y (bfloat16);
//              ACC:    adds into the float32 residual stream y (y += x . W^T);
//              SWIGLU: the tile's B operand is BN/2 gate rows and the BN/2 up rows under them of the stacked
//                      [2F, K] matrix, so a thread holds silu(gate) * up for its token and stores bfloat16
//                      [M, F] - the [M, 2F] intermediate never exists.
//            Two accumulators let the read-out of one tile overlap the products of the next.
// Rows and columns past the edges are zero-filled by TMA on the way in and masked on the way out.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets a status flag (akas_gemm_tcgen05_status),
// all roles fall through to the end, tensor memory is freed and the block returns: no hang, but the
// launch's results are not valid. Needs K % 8 == 0 (16-byte row pitch) and 16-byte aligned operands.
#include <math.h>

#include "tcgen05.cuh"

using namespace akas;
using namespace akas::tc;

namespace {

constexpr int BM = 128, STAGES = 4;
constexpr int THREADS = 192;
enum { EPI_BF16 = 0, EPI_ACC = 1, EPI_SWIGLU = 2 };

__device__ int g_gemm_status = 0;  // 0, or which bounded wait ran out last (1 producer, 2 tensor cores, 3 epilogue)

template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ y_, int M, int N, int K, int F) {
  // N: channels of the product (for SWIGLU the stacked height 2F); a tile covers BN of them (SWIGLU: BN/2 gate
  // rows f0.. and BN/2 up rows F + f0..).
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TILE_N = EPI == EPI_SWIGLU ? BN / 2 : BN;  // output columns a tile yields
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int out_cols = EPI == EPI_SWIGLU ? F : N;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (out_cols + TILE_N - 1) / TILE_N;
  const int tiles = tiles_m * tiles_n, k_blocks = (K + BK - 1) / BK;

  if (tid == 0) {
    abort_s = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory: two accumulators of BN float32 columns, 128 lanes
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(2 * BN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_base_s;

  auto wait_for = [&](uint64_t* bar, unsigned parity, int code) {
    if (*(volatile int*)&abort_s) return;
    if (!mbar_wait(bar, parity)) {
      *(volatile int*)&abort_s = 1;
      atomicExch(&g_gemm_status, code);
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      unsigned it = 0;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * TILE_N;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          wait_for(&empty_bar[s], ((it / STAGES) & 1) ^ 1, 1);
          if (*(volatile int*)&abort_s) break;
          unsigned char* a = smem + (size_t)s * STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          tma_load_2d(a, &map_x, kb * BK, m0, &full_bar[s]);
          if (EPI == EPI_SWIGLU) {
            tma_load_2d(a + A_BYTES, &map_w, kb * BK, n0, &full_bar[s]);
            tma_load_2d(a + A_BYTES + B_BYTES / 2, &map_w, kb * BK, F + n0, &full_bar[s]);
          } else {
            tma_load_2d(a + A_BYTES, &map_w, kb * BK, n0, &full_bar[s]);
          }
        }
        if (*(volatile int*)&abort_s) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tensor cores
    if (lane == 0) {
      // instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, N = BN, M = 128
      constexpr unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
      unsigned it = 0, t = 0;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t) {
        const unsigned acc = t & 1;
        wait_for(&acc_empty[acc], ((t >> 1) & 1) ^ 1, 2);  // the epilogue has drained this accumulator
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          wait_for(&full_bar[s], (it / STAGES) & 1, 2);
          if (*(volatile int*)&abort_s) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned char* a = smem + (size_t)s * STAGE_BYTES;
          const uint64_t a_desc = smem_desc(a), b_desc = smem_desc(a + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)  // 32 bytes further along the swizzled row per step
            umma(d, a_desc + (uint64_t)(k * UMMA_K * 2 >> 4), b_desc + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
                 (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[s]);  // the stage is free once these products have read it
        }
        if (*(volatile int*)&abort_s) break;
        umma_commit(&acc_full[acc]);  // the tile's sums are complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: warps 2..5
    const int sub = warp & 3;  // the tensor-memory sub-partition (32 lanes) this warp may read
    unsigned t = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t) {
      const unsigned acc = t & 1;
      const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * TILE_N;
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
          for (int i = 0; i < 16; ++i) v[i] = __fdividef(v[i], 1.f + __expf(-v[i])) * u[i];  // the fast division: IEEE division cost more than the tile's loads
        }
        const int col = n0 + c;
        if (row < M && col < out_cols) {
          if (EPI == EPI_ACC) {
            float* dst = (float*)y_ + (size_t)row * out_cols + col;
            if (col + 16 <= out_cols && out_cols % 4 == 0) {
#pragma unroll
              for (int i = 0; i < 16; i += 4) {
                float4 h = *reinterpret_cast<float4*>(dst + i);
                h.x += v[i]; h.y += v[i + 1]; h.z += v[i + 2]; h.w += v[i + 3];
                *reinterpret_cast<float4*>(dst + i) = h;
              }
            } else {
              for (int i = 0; i < 16 && col + i < out_cols; ++i) dst[i] += v[i];
            }
          } else {
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
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
  }

  // wind down: everyone meets, then the allocating warp frees tensor memory
  if (*(volatile int*)&abort_s) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // a lost launch: let copies and products in flight finish
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN));
  }
}

// ------------------------------------------------------------------------------------------------ host side

template <int BN, int EPI>
int launch(const void* x, const void* w, void* y, int M, int N, int K, cudaStream_t stream) {
  constexpr int smem = STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
  static int sms_of[64] = {};  // by device ordinal: the launch attribute belongs to a device's copy of the kernel
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  if (sms_of[device] == 0) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    cudaDeviceGetAttribute(&sms_of[device], cudaDevAttrMultiProcessorCount, device);
  }
  const int sms = sms_of[device];
  const int F = N / 2;
  CUtensorMap map_x, map_w;
  int err = cached_map(&map_x, x, M, K, BM, false);
  if (err) return err;
  err = cached_map(&map_w, w, N, K, EPI == EPI_SWIGLU ? BN / 2 : BN, true);
  if (err) return err;
  const int out_cols = EPI == EPI_SWIGLU ? F : N, tile_n = EPI == EPI_SWIGLU ? BN / 2 : BN;
  const int tiles = ((M + BM - 1) / BM) * ((out_cols + tile_n - 1) / tile_n);
  const int grid = tiles < sms ? tiles : sms;
  gemm_tcgen05_kernel<BN, EPI><<<grid, THREADS, smem, stream>>>(map_x, map_w, y, M, N, K, F);
  return launch_status();
}

}  // namespace

// x: bfloat16 [M, K]; w: bfloat16 [N, K]; epilogue 0: y bfloat16 [M, N]; 1: y float32 [M, N] += ; 2 (swiglu, w the
// stacked [2F, K] gate and up matrices, N = 2F): y bfloat16 [M, F]. Returns 0, a CUDA error code, or 3000 + a
// driver error from building a tensor map.
AKAS_API int akas_gemm_tcgen05(const void* x, const void* w, void* y, int M, int N, int K, int epilogue,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || (uintptr_t)x % 16 || (uintptr_t)w % 16 || (uintptr_t)y % 16) return (int)cudaErrorInvalidValue;
  if (epilogue == EPI_SWIGLU && (N % 2 || (N / 2) % 8)) return (int)cudaErrorInvalidValue;
  // 128 x 256 tiles, unless they would leave most SMs without one: then 128 x 128 (measured at 512 and 2,048 tokens:
  // the wide tile wins from about a hundred tiles on)
  const bool narrow = (long long)((M + BM - 1) / BM) * ((N + 255) / 256) <= 64;
  switch (epilogue) {
    case EPI_BF16: return narrow ? launch<128, EPI_BF16>(x, w, y, M, N, K, stream) : launch<256, EPI_BF16>(x, w, y, M, N, K, stream);
    case EPI_ACC: return narrow ? launch<128, EPI_ACC>(x, w, y, M, N, K, stream) : launch<256, EPI_ACC>(x, w, y, M, N, K, stream);
    case EPI_SWIGLU: return launch<256, EPI_SWIGLU>(x, w, y, M, N, K, stream);
    default: return (int)cudaErrorInvalidValue;
  }
}

// 0 if no bounded wait of the kernel has ever run out on the current device (1: producer, 2: tensor cores,
// 3: epilogue). Synchronises with the device.
AKAS_API int akas_gemm_tcgen05_status() {
  int status = -1;
  const cudaError_t e = cudaMemcpyFromSymbol(&status, g_gemm_status, sizeof(int));
  return e == cudaSuccess ? status : -(int)e;
}
