// Paged GQA attention for prompt portions on Blackwell's tensor cores (tcgen05, accumulators in tensor memory),
// bfloat16, head size 64, pages that hold whole 64-key half tiles (page size a multiple of 64).
//
// One block per (tile of 128 consecutive query tokens of one request, query head). It walks 128-key tiles
// aligned to absolute position 0, from the first key any of its queries may see to its last query's own
// position. Ten warps, three roles:
//   warp 0    producer: TMA loads (128-byte swizzle): the Q tile once, then per key tile two boxes of 64 keys of K
//             and two of V, found through the block table, into a two-stage ring; K and V have "full" and "empty"
//             mbarriers of their own, so the scores can start before V has landed.
//   warp 1    tensor cores: allocates tensor memory (128 columns of scores S, 64 of the output O, 64 of P) and
//             issues S = Q.K^T (four tcgen05.mma, M 128, N 128, K 16, both operands K-major from shared memory)
//             and, once the softmax warps have written P, O += P.V (eight tcgen05.mma, M 128, N 64, K 16: P is the
//             A operand in tensor memory, V is read as it lies in the pages, rows of keys with the head's channels
//             contiguous: an MN-major B operand). The scores of the next tile are issued as soon as the softmax
//             warps hold this tile's in registers, so they run under the exponentials.
//             Both warps walk their loops with all lanes and predicate the one instruction that a single lane
//             issues; an issue costs 70-100 cycles whatever the product's size (measured: one thread issues a
//             128 x 64 x 16 product every 100 cycles, a 128 x 256 x 16 one every 150), so products this small
//             are bound by their issue, not by the tensor cores.
//   warps 2-9 softmax and read-out: two threads per query row (= tensor-memory lane), warps 2-5 for the tile's
//             keys 0-63 and output channels 0-31, warps 6-9 for keys 64-127 and channels 32-63. Per tile a
//             thread reads its half of the row of S (tcgen05.ld) into registers, masks it (causal / window) where
//             the tile needs that, takes the maximum (the two halves meet through shared memory), forms
//             P = exp2(s - reference) with packed float32 pairs, rounds it to bfloat16 and, once P.V of the tile
//             before has run, stores it to tensor memory (tcgen05.st), two keys a column. The output stays in tensor
//             memory over all tiles and is divided by the row's sum at the end. The reference of a row follows its
//             running maximum lazily: only when the maximum has grown by more than 2^8 since the reference was
//             set does the thread rescale its channels of O (tcgen05.ld, multiply, tcgen05.st) and its sum; in
//             between P may exceed 1, which float32 sums and bfloat16's exponent take. Softmax is float32.
// Two blocks fit an SM (84 KB of shared memory and 256 columns of tensor memory each, no static shared memory)
// and fill each other's gaps. The softmax warps set the pace: their exponentials keep the special-function units
// half busy, and their chains of dependent instructions do not fill the issue slots (four such warps a
// scheduler). Measured on the 1.2B shape: 306 TFLOP/s at 2,048 tokens and 589 at 8,192, against 182 and 220 of
// the mma.sync kernel of attention_prefill.cu.
//
// Keys past a query's position are masked by position, not by content: pages past the end of a request are
// not fetched (a valid page stands in), and rows of V past the block's last key are zeroed in shared memory so
// that whatever a page held before cannot meet a zero probability as NaN.
// Every wait on an mbarrier is bounded (akas_prefill_attention_tc_status; see gemm_tcgen05.cu).
#include <math.h>

#include "mma.cuh"
#include "tcgen05.cuh"

using namespace akas;
using namespace akas::tc;

namespace {

constexpr int BQ = 128, BKEYS = 128, D = 64, THREADS = 320, STAGES = 2;
constexpr int TILE_BYTES = 128 * 128;  // 128 rows of 64 bfloat16: Q, one stage of K, one of V
constexpr int SMEM_BYTES = TILE_BYTES * (1 + 2 * STAGES) + 128 + 2048;  // tiles, barriers, exchange
static_assert(2 * (SMEM_BYTES + 1024) <= 228 * 1024, "two blocks an SM");
constexpr int TMEM_COLS = 256;  // S: columns 0..127, O: 128..191, P (bfloat16, two keys a column): 192..255

__device__ int g_attention_status = 0;

// A shared-memory descriptor of an MN-major operand in the 128-byte swizzle: rows of 64 elements along N, one row
// per k, eight rows (1024 bytes) per swizzle atom; atoms follow one another along K.
__device__ __forceinline__ uint64_t smem_desc_mn(const void* tile) {
  return (uint64_t)((smem_u32(tile) >> 4) & 0x3fff) | ((uint64_t)(1024 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
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
// 64 consecutive columns of this thread's lane: two loads in flight, one wait
__device__ __forceinline__ void tmem_load64(unsigned taddr, float (&v)[64]) {
  unsigned r[64];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n"
      "tcgen05.wait::ld.sync.aligned;\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr), "r"(taddr + 32) : "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// 32 columns of this thread's lane from 32 registers
__device__ __forceinline__ void tmem_store32(unsigned taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      "tcgen05.wait::st.sync.aligned;\n" ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory");
}
// The producer and the tensor-core warp walk their loops with all 32 lanes and only predicate the instruction that
// one lane issues: in convergent code the compiler keeps descriptors, coordinates and barrier addresses in uniform
// registers, where TMA and tcgen05.mma want them; inside an "if (lane == 0)" it has to move each of them there
// per instruction, which made the issue of one product cost more than the product.
__device__ __forceinline__ void umma_if(unsigned lead, unsigned tmem_d, uint64_t a_desc, uint64_t b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.b32 p, %4, 0;\n setp.ne.b32 q, %5, 0;\n"
      " @q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(lead) : "memory");
}
// D (tensor memory) (+)= A (tensor memory: lane = row, two bfloat16 of K per column) x B (shared memory)
__device__ __forceinline__ void umma_ts_if(unsigned lead, unsigned tmem_d, unsigned tmem_a, uint64_t b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.b32 p, %4, 0;\n setp.ne.b32 q, %5, 0;\n"
      " @q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(lead) : "memory");
}
__device__ __forceinline__ void umma_commit_if(unsigned lead, uint64_t* bar) {
  asm volatile(
      "{\n .reg .pred q;\n setp.ne.b32 q, %1, 0;\n"
      " @q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n"
      ::"r"(smem_u32(bar)), "r"(lead) : "memory");
}
__device__ __forceinline__ void expect_tx_if(unsigned lead, uint64_t* bar, unsigned bytes) {
  asm volatile(
      "{\n .reg .pred q;\n setp.ne.b32 q, %2, 0;\n @q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n}\n"
      ::"r"(smem_u32(bar)), "r"(bytes), "r"(lead) : "memory");
}
__device__ __forceinline__ void tma_load_2d_if(unsigned lead, void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "{\n .reg .pred q;\n setp.ne.b32 q, %5, 0;\n"
      " @q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n}\n"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)), "r"(lead) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done) : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendNs) : "memory");
  return done != 0;
}
// Two float32 in one 64-bit register: Blackwell's packed fused multiply-add and add halve the instruction count of
// the scale-and-shift before the exponentials and of the row sums after them.
__device__ __forceinline__ uint64_t pair(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpair(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ void tmem_store16(unsigned taddr, const float (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
      "tcgen05.wait::st.sync.aligned;\n" ::"r"(taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
}
// When the running maximum of a row grows by less than this (in powers of two) the output so far is not rescaled:
// the row goes on with its old reference, and its probabilities may reach 2^8 instead of 1 (float32 sums and
// bfloat16's exponent have room for that).
constexpr float RESCALE_STEP = 8.f;

__global__ void __launch_bounds__(THREADS, 2)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                            int max_blocks, const int* __restrict__ cu_seqlens, const int* __restrict__ positions,
                            bf16* __restrict__ out, float scale, int window, int page_size, int H, int KH, int R) {
  // The block has no static shared memory, so the dynamic array starts the block's window, 1024-byte aligned (the
  // swizzled tiles need that; it is checked below): with no bytes lost to alignment, two blocks fit an SM.
  chain_release();  // a kernel after this one that was launched as its programmatic dependent may set itself up meanwhile
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* q_s = smem;                                   // [128 queries][128 bytes]
  unsigned char* k_s = q_s + TILE_BYTES;                       // [STAGES][128 keys][128 bytes]
  unsigned char* v_s = k_s + STAGES * TILE_BYTES;              // [STAGES][128 keys][128 bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + STAGES * TILE_BYTES);
  uint64_t &q_full = bars[0], &s_full = bars[1], &p_full = bars[2], &pv_full = bars[3], &s_empty = bars[14];
  uint64_t *k_full = bars + 4, *k_empty = bars + 6, *v_full = bars + 8, *v_empty = bars + 10;  // STAGES of each
  unsigned& tmem_base_s = *reinterpret_cast<unsigned*>(bars + 12);
  int& abort_s = *reinterpret_cast<int*>(bars + 13);
  float* exchange = reinterpret_cast<float*>(bars + 16);  // [tile parity][2 halves of a row][128 rows]: the maxima meet here

  // which tile of which request: heads are x, tiles y, last tile first (the longest walks start first)
  int tile = (int)gridDim.y - 1 - (int)blockIdx.y, r = 0, n = 0;
  for (; r < R; ++r) {
    n = cu_seqlens[r + 1] - cu_seqlens[r];
    const int tiles = (n + BQ - 1) / BQ;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (r >= R) {  // the grid is sized for 64-token tiles: more blocks than 128-token tiles
    chain_wait();
    return;
  }
  if (smem_u32(smem) & 1023u) {  // never seen; the tiles' swizzle would be wrong
    if (threadIdx.x == 0) atomicExch(&g_attention_status, 9);
    chain_wait();
    return;
  }
  const int head = blockIdx.x, kvh = head / (H / KH);
  const int q0 = cu_seqlens[r] + tile * BQ;
  const int rows = min(BQ, n - tile * BQ);
  const int pos0 = positions[q0];
  const int last_key = pos0 + rows - 1;
  const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int kt0 = first_key / BKEYS, kt1 = last_key / BKEYS, tiles_k = kt1 - kt0 + 1;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    abort_s = 0;
    mbar_init(&q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    mbar_init(&s_full, 1);
    mbar_init(&p_full, 8);  // one arrival per softmax warp
    mbar_init(&s_empty, 8);
    mbar_init(&pv_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_base_s;
  // Up to here the block has read what the host wrote for the step (lengths, positions) and set itself up; the queries
  // and the pages are the work of the kernel ahead.
  chain_wait();

  auto wait_for = [&](uint64_t* bar, unsigned parity, int code) {
    if (*(volatile int*)&abort_s) return;
    if (!mbar_wait(bar, parity)) {
      *(volatile int*)&abort_s = 1;
      atomicExch(&g_attention_status, code);
    }
  };

  // The same for a whole warp in step: every lane polls, and the warp goes on together.
  auto wait_warp = [&](uint64_t* bar, unsigned parity, int code) {
    if (__any_sync(0xffffffffu, *(volatile int*)&abort_s != 0)) return;
    for (unsigned spin = 0; spin < kSpinLimit; ++spin)
      if (__all_sync(0xffffffffu, mbar_try(bar, parity))) return;
    *(volatile int*)&abort_s = 1;
    atomicExch(&g_attention_status, code);
  };
  auto aborted = [&]() { return __any_sync(0xffffffffu, *(volatile int*)&abort_s != 0) != 0; };
  const unsigned lead = lane == 0;  // the lane whose TMA and tcgen05 instructions are not predicated off

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    expect_tx_if(lead, &q_full, TILE_BYTES);
    tma_load_2d_if(lead, q_s, &map_q, head * D, q0, &q_full);
    for (int t = 0; t < tiles_k; ++t) {
      const int s = t % STAGES, kt = kt0 + t;
      // the pool rows of the tile's two halves of 64 keys
      int pool_row[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int key0 = kt * BKEYS + h * 64;
        int page = key0 <= last_key ? block_table[(size_t)r * max_blocks + key0 / page_size] : -1;
        if (page < 0) page = 0;  // nothing of it will be seen: any valid rows will do
        pool_row[h] = __shfl_sync(0xffffffffu, (page * KH + kvh) * page_size + (key0 <= last_key ? key0 % page_size : 0), 0);
      }
      if (t >= STAGES) wait_warp(&k_empty[s], ((t / STAGES) & 1) ^ 1, 1);
      if (aborted()) break;
      expect_tx_if(lead, &k_full[s], TILE_BYTES);
      tma_load_2d_if(lead, k_s + s * TILE_BYTES, &map_k, 0, pool_row[0], &k_full[s]);
      tma_load_2d_if(lead, k_s + s * TILE_BYTES + TILE_BYTES / 2, &map_k, 0, pool_row[1], &k_full[s]);
      if (t >= STAGES) wait_warp(&v_empty[s], ((t / STAGES) & 1) ^ 1, 1);
      if (aborted()) break;
      expect_tx_if(lead, &v_full[s], TILE_BYTES);
      tma_load_2d_if(lead, v_s + s * TILE_BYTES, &map_v, 0, pool_row[0], &v_full[s]);
      tma_load_2d_if(lead, v_s + s * TILE_BYTES + TILE_BYTES / 2, &map_v, 0, pool_row[1], &v_full[s]);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tensor cores
    // float32 accumulate, bfloat16 operands; scores: M 128, N 128, both K-major; P.V: M 128, N 64, B MN-major
    constexpr unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BKEYS >> 3) << 17) | ((unsigned)(BQ >> 4) << 24);
    constexpr unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(D >> 3) << 17) | ((unsigned)(BQ >> 4) << 24);
    const unsigned tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
    const unsigned tmem_s = tmem_u, tmem_pv = tmem_u + 128, tmem_p = tmem_u + 192;
    const uint64_t desc_q = smem_desc(q_s);
    auto scores = [&](int t) {
      const int s = t % STAGES;
      wait_warp(&k_full[s], (t / STAGES) & 1, 2);
      if (aborted()) return;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t b = smem_desc(k_s + s * TILE_BYTES);
#pragma unroll
      for (int k = 0; k < D / UMMA_K; ++k) umma_if(lead, tmem_s, desc_q + (uint64_t)(k * 2), b + (uint64_t)(k * 2), idesc_s, k ? 1u : 0u);
      umma_commit_if(lead, &s_full);      // first what the softmax warps wait for: a commit costs the issuing thread time
      umma_commit_if(lead, &k_empty[s]);
    };
    wait_warp(&q_full, 0, 2);
    scores(0);
    for (int t = 0; t < tiles_k && !aborted(); ++t) {
      const int s = t % STAGES;
      if (t + 1 < tiles_k) {
        wait_warp(&s_empty, t & 1, 2);  // the softmax warps hold S in registers: the next tile's scores may land
        scores(t + 1);
      }
      wait_warp(&p_full, t & 1, 2);  // P is written, and the output so far is rescaled where it had to be
      wait_warp(&v_full[s], (t / STAGES) & 1, 2);
      if (aborted()) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t b = smem_desc_mn(v_s + s * TILE_BYTES);
#pragma unroll
      for (int j = 0; j < BKEYS / UMMA_K; ++j)  // 16 keys a step: P advances by 8 columns, V by 16 rows of 128 bytes
        umma_ts_if(lead, tmem_pv, tmem_p + j * 8, b + (uint64_t)(j * (16 * 128 >> 4)), idesc_pv, (t | j) ? 1u : 0u);
      umma_commit_if(lead, &pv_full);
      umma_commit_if(lead, &v_empty[s]);
    }
  } else {
    // ------------------------------------------------------------------ softmax and read-out: warps 2..9
    const int sub = warp & 3, row = sub * 32 + lane;  // tensor-memory lane = query row of the tile
    const int half = (warp - 2) >> 2;                 // which 64 keys of a tile, which 32 output channels
    const unsigned lane_addr = (unsigned)(sub * 32) << 16;
    const unsigned tmem_s = tmem_base + lane_addr + half * 64, tmem_pv = tmem_base + 128 + lane_addr + half * 32;
    const unsigned tmem_p = tmem_base + 192 + lane_addr + half * 32;
    const int qpos = pos0 + row;
    const float sl2 = scale * 1.4426950408889634f;  // scores in units of log2(e): exp is exp2
    float m_ref = -INFINITY, l_run = 0.f;  // the reference the row's probabilities are taken against, in raw units
    auto meet = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(2 + sub) : "memory"); };  // the two warps of these rows
    for (int t = 0; t < tiles_k; ++t) {
      const int kt = kt0 + t, key_base = kt * BKEYS + half * 64, s = t % STAGES;
      // rows of V past the block's last key: whatever the page held must not meet a zero probability as NaN
      if (kt * BKEYS + BKEYS - 1 > last_key) {
        wait_for(&v_full[s], (t / STAGES) & 1, 3);
        const int first_dead = max(0, last_key + 1 - kt * BKEYS);
        for (int i = (tid - 64) + first_dead * 8; i < BKEYS * 8; i += 256)
          *reinterpret_cast<uint4*>(v_s + s * TILE_BYTES + i * 16) = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      wait_for(&s_full, t & 1, 3);  // after a wait has run out nobody waits any more, but every thread still walks
                                    // all tiles: the two warps of a row meet at a barrier in each
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // This thread's half of the row of S, into registers; tensor memory is then free for the next tile's scores.
      float v[64];
      tmem_load64(tmem_s, v);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty);
      const bool whole = kt * BKEYS + BKEYS - 1 <= pos0 && kt * BKEYS >= first_key &&
                         (window <= 0 || kt * BKEYS > pos0 + rows - 1 - window);  // no query of the tile masks any of it
      if (!whole) {  // all tiles but the last one or two (and the first, under a window) skip this
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int key = key_base + i;
          const bool seen = key <= qpos && key >= first_key && (window <= 0 || key > qpos - window);
          v[i] = seen ? v[i] : -INFINITY;
        }
      }
      float tops[4];  // four chains of three-input maxima, so that one does not wait for the other
#pragma unroll
      for (int c = 0; c < 4; ++c) tops[c] = max3(v[c], v[4 + c], v[8 + c]);
#pragma unroll
      for (int i = 12; i < 60; i += 8) {
#pragma unroll
        for (int c = 0; c < 4; ++c) tops[c] = max3(tops[c], v[i + c], v[i + 4 + c]);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) tops[c] = fmaxf(tops[c], v[60 + c]);
      float top = fmaxf(fmaxf(tops[0], tops[1]), fmaxf(tops[2], tops[3]));
      // The halves' maxima meet through shared memory, in a place of the tile's parity: the other half may still be
      // reading the tile before while this one writes.
      float* mine = exchange + (t & 1) * 256 + half * 128 + row;
      *mine = top;
      meet();
      top = fmaxf(top, exchange[(t & 1) * 256 + (half ^ 1) * 128 + row]);
      const float m_new = fmaxf(m_ref, top);
      // The output so far, O in tensor memory, refers to m_ref. It is brought to the new maximum only when that has
      // grown by more than RESCALE_STEP for some row of this warp (the two warps of a row see the same maxima and
      // decide alike); then every row of the warp moves to its new maximum. (-inf) - (-inf) is NaN: not greater.
      const bool rescale = t > 0 && __any_sync(0xffffffffu, (m_new - m_ref) * sl2 > RESCALE_STEP);
      float corr = 1.f;
      if (t == 0) {
        m_ref = m_new;
      } else if (rescale) {
        corr = m_new == -INFINITY ? 1.f : fast_exp2((m_ref - m_new) * sl2);
        m_ref = m_new;
      }
      const float bias = m_ref == -INFINITY ? 0.f : -m_ref * sl2;  // a row that sees nothing yet: every P is 0
      const uint64_t sl2_2 = pair(sl2, sl2), bias_2 = pair(bias, bias);
      uint64_t sums2[4] = {0ull, 0ull, 0ull, 0ull};  // four chains of pairs of float32 zeros
      uint32_t packed[32];  // P, rounded to bfloat16, two keys a column of tensor memory
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float x0, x1;
        unpair(fma2(pair(v[2 * i], v[2 * i + 1]), sl2_2, bias_2), x0, x1);
        const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
        sums2[i & 3] = add2(sums2[i & 3], pair(p0, p1));
        packed[i] = pack_bf16(p0, p1);
      }
      float sums[4];
      {
        float lo, hi, lo2, hi2;
        unpair(add2(sums2[0], sums2[1]), lo, hi);
        unpair(add2(sums2[2], sums2[3]), lo2, hi2);
        sums[0] = lo; sums[1] = hi; sums[2] = lo2; sums[3] = hi2;
      }
      // Only now does this tile need the product of the tile before: P's columns are free again once it has run,
      // and the output so far is complete. The exponentials above ran while it was issued.
      if (t > 0) {
        wait_for(&pv_full, (t - 1) & 1, 3);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      if (rescale) {
#pragma unroll 1
        for (int c = 0; c < 32; c += 16) {  // in pieces: P is held in registers meanwhile
          float o[16];
          tmem_load16(tmem_pv + c, o);
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] *= corr;
          tmem_store16(tmem_pv + c, o);
        }
      }
      tmem_store32(tmem_p, packed);
      l_run = l_run * corr + ((sums[0] + sums[1]) + (sums[2] + sums[3]));
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full);
    }
    // the output: O of the last product, over the row's sum
    wait_for(&pv_full, (tiles_k - 1) & 1, 3);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    float o[32];
    tmem_load32(tmem_pv, o);
    // the row's sum: both halves, through the Q tile's memory, which no product reads any more
    float* sums = reinterpret_cast<float*>(q_s);
    sums[half * 128 + row] = l_run;
    meet();
    l_run += sums[(half ^ 1) * 128 + row];
    if (row < rows && !*(volatile int*)&abort_s) {
      const float inv = 1.f / l_run;
      bf16* dst = out + ((size_t)(q0 + row) * H + head) * D + half * 32;
#pragma unroll
      for (int c = 0; c < 32; c += 8) {
        float piece[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) piece[i] = o[c + i] * inv;
        store_vec(dst + c, piece);
      }
    }
  }

  if (*(volatile int*)&abort_s) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // a lost launch: let copies and products in flight finish
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

// A tensor map of rows of `row_elems` bfloat16 (row pitch `pitch_elems`), boxes of 64 elements x `box_rows` rows.
int rows_map(CUtensorMap* map, const void* base, long long rows, int row_elems, long long pitch_elems, int box_rows) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return 3001;
  const cuuint64_t dims[2] = {(cuuint64_t)row_elems, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)pitch_elems * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 3000 + (int)r;
}

}  // namespace

// q: bfloat16 [N, H * 64]; pools: bfloat16 [pages, KH, page_size, 64] with page_size a multiple of 64; out: bfloat16
// [N, H * 64]. tiles: an upper bound of the number of 128-token tiles (the sum over requests of ceil(tokens / 64)
// will do). Returns 0, a CUDA error, 3000 + a driver error from building a tensor map, or 3999 if the kernel does
// not take these sizes (nothing was launched).
AKAS_API int akas_prefill_attention_tc(const void* q, const void* k_pool, const void* v_pool, long long pool_rows,
                                       const int* block_table, int max_blocks, const int* cu_seqlens,
                                       const int* positions, void* out, float scale, int window, int page_size, int tiles,
                                       int N, int H, int KH, int head_dim, int R, cudaStream_t stream) {
  if (head_dim != D || page_size % 64 || H % KH || tiles > 65535 || R <= 0 || N <= 0) return 3999;
  if ((uintptr_t)q % 16 || (uintptr_t)k_pool % 16 || (uintptr_t)v_pool % 16 || (uintptr_t)out % 16) return 3999;
  if (tiles <= 0) return 0;
  static bool configured[64] = {};  // by device ordinal: the attribute belongs to a device's copy of the kernel
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  if (!configured[device]) {
    const cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured[device] = true;
  }
  CUtensorMap map_q, map_k, map_v;
  int err = rows_map(&map_q, q, N, H * D, (long long)H * D, 128);
  if (!err) err = rows_map(&map_k, k_pool, pool_rows, D, D, 64);
  if (!err) err = rows_map(&map_v, v_pool, pool_rows, D, D, 64);
  if (err) return err;
  return launch_chained(prefill_attention_tc_kernel, dim3(H, tiles), dim3(THREADS), SMEM_BYTES, stream,
                        map_q, map_k, map_v, block_table, max_blocks, cu_seqlens, positions, (bf16*)out, scale, window, page_size, H, KH, R);
}

// 0 if no bounded wait of the kernel has ever run out on the current device (1: producer, 2: tensor cores,
// 3: softmax). Synchronises with the device.
AKAS_API int akas_prefill_attention_tc_status() {
  int status = -1;
  const cudaError_t e = cudaMemcpyFromSymbol(&status, g_attention_status, sizeof(int));
  return e == cudaSuccess ? status : -(int)e;
}
