// Matrix products of a decode step on Blackwell's tensor cores: y[M, O] = x[M, K] . W[O, K]^T for a handful of
// tokens (M <= 128). The time of such a product is the time to read W once, so the kernel is built around the
// stream of weights: the weight matrix is the A operand of tcgen05.mma (128 output channels per tile, one per
// accumulator lane), the tokens are its N columns (M rounded up to a multiple of 16), and nothing but TMA and
// the tensor cores ever touches a weight.
//
// Work is cut into tiles of 128 output channels; where there are too few tiles to fill the GPU, K is cut as
// well, into `splits` parts that the blocks of one thread-block cluster take, and their partial sums meet in
// distributed shared memory. Six warps per block, three roles:
//   warp 0    producer: one thread issues TMA loads of 128 x 64 weight tiles (128-byte swizzle) into a ring of
//             up to 12 stages, each with a "full" (bytes counted) and an "empty" mbarrier. Weights are
//             fetched before the kernel waits for its predecessor on the stream (programmatic dependent
//             launch): no kernel writes them. With bfloat16 activations the 64-column slice of x rides in
//             the same stage (fetched after that wait).
//   warp 1    tensor cores: allocates tensor memory (two accumulators of NT float32 columns) and issues four
//             tcgen05.mma (M 128, N NT, K 16) per stage, committed to the stage's "empty" barrier.
//   warps 2-5 activations and read-out. With a fused RMSNorm (x float32, the residual stream) they first write
//             bfloat16(x * norm_weight) for the block's part of K into shared memory in the swizzled
//             K-major layout the tensor cores read, and sum x^2 per token on the way; 1 / rms is applied to
//             the accumulator afterwards, in float32. Then, per tile, each thread reads its channel's NT
//             sums with tcgen05.ld and
//               one part of K:  scales and stores them (bfloat16, float32, added into the float32 residual
//                               stream, or SwiGLU: the tile is 64 gate rows and their 64 up rows of the
//                               stacked [2F, K] matrix, and the two halves meet through shared memory);
//               several parts:  sends them to the block of the cluster that owns the channel (each block
//                               owns 128 / splits channels of the tile) with st.shared::cluster, arrives on
//                               the owner's mbarrier, and every owner adds the parts in rank order (so the
//                               result does not depend on timing) and stores its channels.
// Rows and columns past the edges are zero-filled by TMA and masked on the way out.
//
// Every wait on an mbarrier is bounded; one that runs out sets a status flag (akas_stream_gemm_status), all
// roles fall through, the cluster meets once more, tensor memory is freed and the block returns: no hang, but
// that launch's results are not valid. Needs K % 8 == 0 and 16-byte aligned operands.
#include <math.h>

#include "tcgen05.cuh"

using namespace akas;
using namespace akas::tc;

namespace {

constexpr int BM = 128, THREADS = 192, MAX_STAGES = 12, MAX_SPLITS = 8, MAX_TOKENS = 128;
constexpr int A_BYTES = BM * BK * 2;
constexpr int SMEM_LIMIT = 227 * 1024;  // shared memory a block may have on sm_100, static and dynamic together
enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_ACC = 2, OUT_SWIGLU = 3 };

__device__ int g_stream_status = 0;  // 0, or which bounded wait ran out last (1 producer, 2 tensor cores, 3 read-out, 4 cluster)

__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address of a shared-memory location of block `rank` of this cluster.
__device__ __forceinline__ unsigned peer_address(const void* local, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
  return r;
}
__device__ __forceinline__ void peer_store(unsigned address, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(address), "f"(v) : "memory");
}
__device__ __forceinline__ void peer_arrive(unsigned bar_address) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_address) : "memory");
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
__device__ __forceinline__ void readout_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }  // warps 2-5

template <int OUT>
__device__ __forceinline__ void put(void* y_, size_t at, float v) {
  if (OUT == OUT_F32) ((float*)y_)[at] = v;
  else if (OUT == OUT_ACC) ((float*)y_)[at] += v;
  else ((bf16*)y_)[at] = __float2bfloat16_rn(v);
}

template <bool IN_NORM, int OUT>
__global__ void __launch_bounds__(THREADS)
stream_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const float* __restrict__ x_f32, const int* __restrict__ rows, const float* __restrict__ norm_w, float eps,
                   int zero_centered, void* __restrict__ y_, int M, int O, int K, int NT, int stages, int splits,
                   int tmem_cols) {
  // O: rows of W (for SWIGLU the stacked height 2F). A tile covers 128 of them (SWIGLU: 64 gate rows f0.. and the
  // 64 up rows F + f0..).
  constexpr bool SWIGLU = OUT == OUT_SWIGLU;
  constexpr int TILE_ROWS = SWIGLU ? 64 : BM;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2], b_ready, gathered;
  __shared__ unsigned tmem_base_s;
  __shared__ int abort_s;
  __shared__ float ss_warp[4][MAX_TOKENS];  // sum of x^2 over this block's part of K, by read-out warp
  __shared__ float ss_local[MAX_TOKENS];    // their sum
  __shared__ float inv_s[MAX_TOKENS];       // 1 / rms per token (one part of K)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int out_cols = SWIGLU ? O / 2 : O;
  const int row_tiles = (out_cols + TILE_ROWS - 1) / TILE_ROWS, k_blocks = (K + BK - 1) / BK;
  const unsigned rank = splits > 1 ? cluster_rank() : 0u;
  const int kb_begin = (int)((long long)k_blocks * rank / splits), kb_end = (int)((long long)k_blocks * (rank + 1) / splits);
  const int nk = kb_end - kb_begin;
  const int cluster_id = blockIdx.x / splits, clusters = gridDim.x / splits;
  const int stage_bytes = A_BYTES + (IN_NORM ? 0 : NT * 128);
  const int rows_per = (BM + splits - 1) / splits;  // channels of a tile that one block of the cluster owns
  unsigned char* ring = smem;
  unsigned char* resident = ring + (size_t)stages * stage_bytes;  // IN_NORM: [part's k-blocks][NT][128 bytes]
  float* gather = reinterpret_cast<float*>(resident + (IN_NORM ? (size_t)((k_blocks + splits - 1) / splits) * NT * 128 : 0));
  float* ss_all = gather + (splits > 1 ? splits * M * rows_per : (SWIGLU ? 16 * 64 : 0));  // [splits][M]

  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    if (!IN_NORM) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  if (tid >= 64) {  // warps 2-5 set the barriers up while warp 1 allocates tensor memory
    const int i = tid - 64;
    if (i < stages) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    if (i >= 32 && i < 34) { mbar_init(&acc_full[i - 32], 1); mbar_init(&acc_empty[i - 32], 4); }
    if (i == 34) mbar_init(&b_ready, 128);
    if (i == 35) mbar_init(&gathered, (unsigned)splits);
    if (i == 36) abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(tmem_cols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_base_s;
  if (splits > 1) cluster_meet();  // every block's barriers exist before a peer arrives on them
  chain_release();

  auto wait_for = [&](uint64_t* bar, unsigned parity, int code) {
    if (*(volatile int*)&abort_s) return;
    if (!mbar_wait(bar, parity)) {
      *(volatile int*)&abort_s = 1;
      atomicExch(&g_stream_status, code);
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const int my_tiles = cluster_id < row_tiles ? (row_tiles - cluster_id + clusters - 1) / clusters : 0;
      const int total = my_tiles * nk;
      auto load_w = [&](int i) {
        const int tile = cluster_id + (i / nk) * clusters, kb = kb_begin + i % nk, s = i % stages;
        unsigned char* dst = ring + (size_t)s * stage_bytes;
        mbar_expect_tx(&full_bar[s], stage_bytes);
        if (SWIGLU) {
          tma_load_2d(dst, &map_w, kb * BK, tile * 64, &full_bar[s]);
          tma_load_2d(dst + A_BYTES / 2, &map_w, kb * BK, O / 2 + tile * 64, &full_bar[s]);
        } else {
          tma_load_2d(dst, &map_w, kb * BK, tile * BM, &full_bar[s]);
        }
      };
      auto load_x = [&](int i) {
        const int kb = kb_begin + i % nk, s = i % stages;
        tma_load_2d(ring + (size_t)s * stage_bytes + A_BYTES, &map_x, kb * BK, 0, &full_bar[s]);
      };
      const int head = total < stages ? total : stages;
      for (int i = 0; i < head; ++i) load_w(i);  // weights first: they do not depend on earlier kernels
      chain_wait();
      if (!IN_NORM)
        for (int i = 0; i < head; ++i) load_x(i);
      for (int i = head; i < total; ++i) {
        const int s = i % stages;
        wait_for(&empty_bar[s], ((i / stages) & 1) ^ 1, 1);
        if (*(volatile int*)&abort_s) break;
        load_w(i);
        if (!IN_NORM) load_x(i);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tensor cores
    if (lane == 0) {
      // instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, N = NT, M = 128
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(NT >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
      if (IN_NORM) wait_for(&b_ready, 0, 2);
      unsigned it = 0, t = 0;
      for (int tile = cluster_id; tile < row_tiles; tile += clusters, ++t) {
        const unsigned acc = t & 1;
        wait_for(&acc_empty[acc], ((t >> 1) & 1) ^ 1, 2);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned d = tmem_base + acc * NT;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = it % stages;
          wait_for(&full_bar[s], (it / stages) & 1, 2);
          if (*(volatile int*)&abort_s) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned char* a = ring + (size_t)s * stage_bytes;
          const uint64_t a_desc = smem_desc(a);
          const uint64_t b_desc = smem_desc(IN_NORM ? resident + (size_t)(kb - kb_begin) * NT * 128 : a + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma(d, a_desc + (uint64_t)(k * UMMA_K * 2 >> 4), b_desc + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
                 (kb > kb_begin || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        if (*(volatile int*)&abort_s) break;
        umma_commit(&acc_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ activations and read-out: warps 2..5
    const int e = tid - 64, sub = warp & 3;  // sub: the tensor-memory sub-partition (32 lanes) this warp may read
    const int rho = sub * 32 + lane;         // accumulator lane = channel of the tile
    chain_wait();
    if (IN_NORM) {
      // bfloat16(x * norm_weight) of this block's part of K, 16 bytes (8 elements) at a time, into the layout TMA
      // would have written: row t of k-block b at b * NT * 128 + t * 128, its 16-byte chunks xor-ed with t % 8.
      // Eight tokens at a time share one pass over the chunks. Their loads are issued together, without conditions
      // (rows past M and chunks past K read a valid address and are zeroed afterwards), so that the latencies overlap.
      const float centre = zero_centered ? 1.f : 0.f;
      for (int t0 = 0; t0 < NT; t0 += 8) {
        float ss[8];
        const float* x_row[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ss[j] = 0.f;
          const int t = t0 + j;
          x_row[j] = x_f32 + (size_t)(t < M ? (rows ? rows[t] : t) : 0) * K;
        }
        if (t0 >= M) {  // rows of padding: zeros
          for (int c = e; c < nk * 8; c += 128) {
            unsigned char* slab = resident + (size_t)(c >> 3) * NT * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(slab + (t0 + j) * 128 + (((c & 7) ^ ((t0 + j) & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
          }
          continue;
        }
        for (int c = e; c < nk * 8; c += 128) {
          const int b = c >> 3, ch = c & 7, k0 = (kb_begin + b) * BK + ch * 8;
          const bool inside = k0 < K;
          const int k_safe = inside ? k0 : 0;
          float wv[8], xv[8][8];
          load8(norm_w + k_safe, wv);
#pragma unroll
          for (int j = 0; j < 8; ++j) load8(x_row[j] + k_safe, xv[j]);
          unsigned char* slab = resident + (size_t)b * NT * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int t = t0 + j;
            const bool keep = t < M && inside;
            uint4 packed;
            uint32_t* w32 = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float a0 = keep ? xv[j][2 * i] : 0.f, a1 = keep ? xv[j][2 * i + 1] : 0.f;
              ss[j] += a0 * a0 + a1 * a1;
              const __nv_bfloat162 h = __floats2bfloat162_rn(a0 * (wv[2 * i] + centre), a1 * (wv[2 * i + 1] + centre));
              w32[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(slab + t * 128 + ((ch ^ (t & 7)) << 4)) = packed;
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float total = warp_sum(ss[j]);
          if (lane == 0 && t0 + j < M) ss_warp[warp - 2][t0 + j] = total;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor cores read what these threads wrote
      mbar_arrive(&b_ready);
      readout_barrier();
      if (e < M) {
        const float total = ((ss_warp[0][e] + ss_warp[1][e]) + ss_warp[2][e]) + ss_warp[3][e];
        ss_local[e] = total;
        inv_s[e] = rsqrtf(total / (float)K + eps);
      }
      readout_barrier();
    }

    // Several parts of K, adding into the residual stream: the old values of the (up to two) sums this thread will
    // finish are fetched now, so that their latency hides behind the products.
    const int mine = min(rows_per, BM - (int)rank * rows_per);  // channels of the tile that this block finishes
    float before[2] = {0.f, 0.f};
    if (OUT == OUT_ACC && splits > 1 && cluster_id < row_tiles) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int i = e + j * 128;
        if (i < M * mine) {
          const int o = cluster_id * BM + (int)rank * rows_per + i % mine;
          if (o < O) before[j] = ((const float*)y_)[(size_t)(i / mine) * O + o];
        }
      }
    }

    unsigned t = 0;
    for (int tile = cluster_id; tile < row_tiles; tile += clusters, ++t) {
      const unsigned acc = t & 1;
      wait_for(&acc_full[acc], (t >> 1) & 1, 3);
      if (*(volatile int*)&abort_s) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const unsigned taddr = tmem_base + acc * NT + ((unsigned)(sub * 32) << 16);
      const unsigned owner = (unsigned)(rho / rows_per);
      const unsigned owner_gather = splits > 1 ? peer_address(gather, owner) : 0u;
#pragma unroll 1
      for (int c = 0; c < NT && c < M; c += 16) {
        float v[16];
        tmem_load16(taddr + c, v);
        if (splits > 1) {
          // part of K: send this channel's sums to the block that owns the channel
          const int local = rho % rows_per;
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c + i < M) peer_store(owner_gather + (unsigned)((((int)rank * M + c + i) * rows_per + local) * 4), v[i]);
        } else if (SWIGLU) {
          if (rho >= 64) {
#pragma unroll
            for (int i = 0; i < 16; ++i) gather[i * 64 + rho - 64] = v[i];
          }
          readout_barrier();
          if (rho < 64) {
            const int f = tile * 64 + rho;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int tk = c + i;
              if (tk < M && f < out_cols) {
                const float scale = IN_NORM ? inv_s[tk] : 1.f;
                const float g = v[i] * scale, u = gather[i * 64 + rho] * scale;
                ((bf16*)y_)[(size_t)tk * out_cols + f] = __float2bfloat16_rn(__fdividef(g, 1.f + __expf(-g)) * u);
              }
            }
          }
          readout_barrier();
        } else {
          const int o = tile * BM + rho;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int tk = c + i;
            if (tk < M && o < O) put<OUT>(y_, (size_t)tk * O + o, v[i] * (IN_NORM ? inv_s[tk] : 1.f));
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);

      if (splits > 1) {
        if (IN_NORM && e < M)
          for (int d = 0; d < splits; ++d) peer_store(peer_address(ss_all, d) + (unsigned)(((int)rank * M + e) * 4), ss_local[e]);
        readout_barrier();  // all of this block's parts are written; one thread tells each peer (release, cluster scope)
        if (e < splits) {
          asm volatile("fence.acq_rel.cluster;" ::: "memory");
          peer_arrive(peer_address(&gathered, (unsigned)e));
        }
        if (!*(volatile int*)&abort_s && !mbar_wait_cluster(&gathered, t & 1)) {
          *(volatile int*)&abort_s = 1;
          atomicExch(&g_stream_status, 4);
        }
        if (*(volatile int*)&abort_s) break;
        // this block's channels: the parts added in rank order
        for (int i = e, j = 0; i < M * mine; i += 128, ++j) {
          const int tk = i / mine, local = i % mine;
          float sum = 0.f, ss = 0.f;
          for (int src = 0; src < splits; ++src) {
            sum += gather[(src * M + tk) * rows_per + local];
            if (IN_NORM) ss += ss_all[src * M + tk];
          }
          const int o = tile * BM + (int)rank * rows_per + local;
          const float value = sum * (IN_NORM ? rsqrtf(ss / (float)K + eps) : 1.f);
          if (o < O) {
            if (OUT == OUT_ACC && j < 2) ((float*)y_)[(size_t)tk * O + o] = before[j] + value;
            else put<OUT>(y_, (size_t)tk * O + o, value);
          }
        }
      }
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols));
  }
  if (splits > 1) cluster_meet();  // no block leaves while a peer may still write into its shared memory
}

// ------------------------------------------------------------------------------------------------ host side

struct Plan {
  int nt, row_tiles, k_blocks, splits, stages, smem, tmem_cols, grid;
};

int device_sms(int device) {
  static int sms[64] = {};
  if (sms[device] == 0) cudaDeviceGetAttribute(&sms[device], cudaDevAttrMultiProcessorCount, device);
  return sms[device];
}

// Shared memory of a block with `splits` parts of K; 0 if it does not fit with at least `least` stages.
int layout(int budget, int M, int nt, int k_blocks, bool in_norm, bool swiglu, int splits, int* stages) {
  const int stage = A_BYTES + (in_norm ? 0 : nt * 128);
  const int rows_per = (BM + splits - 1) / splits;
  const long long resident = in_norm ? (long long)((k_blocks + splits - 1) / splits) * nt * 128 : 0;
  const long long gather = splits > 1 ? (long long)splits * M * rows_per * 4 : (swiglu ? 16 * 64 * 4 : 0);
  const long long ss = splits > 1 ? (long long)splits * M * 4 : 0;
  const long long fixed = 1024 + resident + gather + ss + 16;
  const int most = (k_blocks + splits - 1) / splits;  // a block never has more k-blocks in flight than it has
  long long n = (budget - fixed) / stage;
  if (n > MAX_STAGES) n = MAX_STAGES;
  const int least = most < 4 ? most : 4;
  if (n < least || n < 1) return 0;
  *stages = (int)n;
  return (int)(fixed + n * stage);
}

template <bool IN_NORM, int OUT>
int launch(const void* x, const int* rows, const void* norm_w, float eps, int zero_centered, const void* w, void* y, int M,
           int O, int K, bool dry, cudaStream_t stream) {
  constexpr bool SWIGLU = OUT == OUT_SWIGLU;
  auto kernel = stream_gemm_kernel<IN_NORM, OUT>;
  static int budgets[64] = {};  // by device ordinal: dynamic shared memory this kernel may ask for
  static std::map<std::pair<int, int>, int> cluster_room;  // (device, splits) -> clusters of that size resident at once
  static std::mutex mutex;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  int& budget = budgets[device];
  const int sms = device_sms(device);
  Plan p;
  p.nt = (M + 15) / 16 * 16;
  const int out_cols = SWIGLU ? O / 2 : O;
  p.row_tiles = (out_cols + (SWIGLU ? 64 : BM) - 1) / (SWIGLU ? 64 : BM);
  p.k_blocks = (K + BK - 1) / BK;
  p.tmem_cols = 32;
  while (p.tmem_cols < 2 * p.nt) p.tmem_cols *= 2;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (budget == 0) {
      cudaFuncAttributes attributes;
      cudaError_t e = cudaFuncGetAttributes(&attributes, kernel);
      if (e != cudaSuccess) return (int)e;
      const int room = SMEM_LIMIT - (int)attributes.sharedSizeBytes;
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, room);
      if (e != cudaSuccess) return (int)e;
      budget = room;
    }
    int s = 1;
    if (!SWIGLU && p.row_tiles * 2 <= sms) {
      s = sms / p.row_tiles;
      if (s > MAX_SPLITS) s = MAX_SPLITS;
      if (s > p.k_blocks) s = p.k_blocks;
    }
    p.splits = 0;
    for (; s >= 1; --s) {
      const int smem = layout(budget, M, p.nt, p.k_blocks, IN_NORM, SWIGLU, s, &p.stages);
      if (!smem) continue;
      if (s > 1) {
        const auto room_key = std::make_pair(device, s);
        if (!cluster_room.count(room_key)) {
          cudaLaunchConfig_t config = {};
          config.gridDim = dim3(s * 64);
          config.blockDim = dim3(THREADS);
          config.dynamicSmemBytes = budget;
          cudaLaunchAttribute attribute[1];
          attribute[0].id = cudaLaunchAttributeClusterDimension;
          attribute[0].val.clusterDim.x = s;
          attribute[0].val.clusterDim.y = 1;
          attribute[0].val.clusterDim.z = 1;
          config.attrs = attribute;
          config.numAttrs = 1;
          int room = 0;
          if (cudaOccupancyMaxActiveClusters(&room, kernel, &config) != cudaSuccess) { cudaGetLastError(); room = 0; }
          cluster_room[room_key] = room;
        }
        if (cluster_room[room_key] < p.row_tiles) continue;  // all clusters of a launch run at once
      }
      p.splits = s;
      p.smem = smem;
      break;
    }
  }
  if (p.splits == 0) return 3999;
  if (dry) return 0;
  if (p.splits > 1) {
    p.grid = p.row_tiles * p.splits;
  } else {
    const int per = (p.row_tiles + sms - 1) / sms;  // tiles per block, and as few blocks as do it in that many rounds
    p.grid = (p.row_tiles + per - 1) / per;
  }
  CUtensorMap map_w, map_x;
  int err = cached_map(&map_w, w, O, K, SWIGLU ? 64 : BM, true);
  if (err) return err;
  if (IN_NORM) {
    map_x = map_w;
  } else {
    err = cached_map(&map_x, x, M, K, p.nt, false);
    if (err) return err;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(p.grid);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = p.smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  int n = 0;
  if (chained_launches_enabled()) {
    attribute[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (p.splits > 1) {
    attribute[n].id = cudaLaunchAttributeClusterDimension;
    attribute[n].val.clusterDim.x = p.splits;
    attribute[n].val.clusterDim.y = 1;
    attribute[n].val.clusterDim.z = 1;
    ++n;
  }
  config.attrs = attribute;
  config.numAttrs = n;
  return (int)cudaLaunchKernelEx(&config, kernel, map_w, map_x, (const float*)x, rows, (const float*)norm_w, eps, zero_centered,
                                 y, M, O, K, p.nt, p.stages, p.splits, p.tmem_cols);
}

int dispatch(const void* x, const int* rows, const void* norm_w, float eps, int zero_centered, int in_norm, const void* w,
             void* y, int M, int O, int K, int out_mode, bool dry, cudaStream_t stream) {
  if (M <= 0 || O <= 0) return 0;
  if (M > MAX_TOKENS || K <= 0 || K % 8) return 3999;
  if (out_mode == OUT_SWIGLU && O % 2) return 3999;
  if (rows && !in_norm) return (int)cudaErrorInvalidValue;
  if (!dry && ((uintptr_t)x % 16 || (uintptr_t)w % 16 || (in_norm && (uintptr_t)norm_w % 16))) return (int)cudaErrorInvalidValue;
#define AKAS_STREAM_CASE(NORM, MODE) \
  case MODE: return launch<NORM, MODE>(x, rows, norm_w, eps, zero_centered, w, y, M, O, K, dry, stream);
  if (in_norm) {
    switch (out_mode) {
      AKAS_STREAM_CASE(true, OUT_BF16) AKAS_STREAM_CASE(true, OUT_F32) AKAS_STREAM_CASE(true, OUT_ACC)
      AKAS_STREAM_CASE(true, OUT_SWIGLU)
    }
  } else {
    switch (out_mode) {
      AKAS_STREAM_CASE(false, OUT_BF16) AKAS_STREAM_CASE(false, OUT_F32) AKAS_STREAM_CASE(false, OUT_ACC)
      AKAS_STREAM_CASE(false, OUT_SWIGLU)
    }
  }
#undef AKAS_STREAM_CASE
  return (int)cudaErrorInvalidValue;
}

}  // namespace

// y = x . W^T for at most 128 tokens. x: bfloat16 [M, K], or with in_norm float32 [*, K] whose rows `rows` (int32
// [M], or null for rows 0..M-1) are RMS-normalised on the way in (weight norm_w float32 [K], or 1 + norm_w if
// zero_centered; eps). w: bfloat16 [O, K]. out_mode 0: y bfloat16 [M, O]; 1: y float32
// [M, O]; 2: y float32 [M, O] += ; 3 (SwiGLU, w the stacked [2F, K] gate and up matrices, O = 2F): y bfloat16
// [M, F]. Returns 0, a CUDA error code, 3000 + a driver error from building a tensor map, or 3999 if the kernel
// does not take these sizes (nothing was launched).
AKAS_API int akas_stream_gemm(const void* x, const int* rows, const void* norm_w, float eps, int zero_centered, int in_norm,
                              const void* w, void* y, int M, int O, int K, int out_mode, cudaStream_t stream) {
  return dispatch(x, rows, norm_w, eps, zero_centered, in_norm, w, y, M, O, K, out_mode, false, stream);
}

// 1 if akas_stream_gemm takes these sizes on the current device, else 0. Launches nothing.
AKAS_API int akas_stream_gemm_takes(int M, int O, int K, int in_norm, int out_mode) {
  return dispatch(nullptr, nullptr, nullptr, 0.f, 0, in_norm, nullptr, nullptr, M, O, K, out_mode, true, 0) == 0 ? 1 : 0;
}

// 0 if no bounded wait of the kernel has ever run out on the current device (1: producer, 2: tensor cores,
// 3: read-out, 4: waiting for the cluster's parts). Synchronises with the device.
AKAS_API int akas_stream_gemm_status() {
  int status = -1;
  const cudaError_t e = cudaMemcpyFromSymbol(&status, g_stream_status, sizeof(int));
  return e == cudaSuccess ? status : -(int)e;
}
