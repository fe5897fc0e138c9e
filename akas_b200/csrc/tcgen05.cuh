// Pieces shared by the kernels that drive Blackwell's tensor cores directly: mbarriers with bounded waits,
// TMA tile loads, shared-memory matrix descriptors, tcgen05.mma / commit / ld, and tensor maps of row-major
// bfloat16 matrices (built on the host through the driver's entry point, which is looked up at run time so
// that nothing links against libcuda).
#pragma once

#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace akas {
namespace tc {

constexpr int BK = 64;       // elements of K per tile row: 128 bytes of bfloat16, one swizzle row
constexpr int UMMA_K = 16;   // K of one tcgen05.mma of 16-bit operands
constexpr unsigned kSpinLimit = 1u << 22;
// A waiting thread may be suspended this long (nanoseconds) per try before it polls again, so that waiting does not
// fill the issue slots of the warps that work (a third of all instructions of the attention kernel were polls
// before this). The limit also bounds how late a waiter notices: measured on a B200, a read-out warp that waited
// with a limit of 2,000 ns woke some 0.8 us after its barrier's phase had completed, with 200 ns some 0.2 us.
constexpr unsigned kSuspendNs = 200;

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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
  const unsigned addr = smem_u32(bar);
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity), "r"(kSuspendNs) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bfloat16) in the 128-byte
// swizzle that TMA wrote: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(const void* tile) {
  return (uint64_t)((smem_u32(tile) >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma(unsigned tmem_d, uint64_t a_desc, uint64_t b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_load16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      "tcgen05.wait::ld.sync.aligned;\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}


// ------------------------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled encode_tiled() {
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

// A tensor map of a row-major bfloat16 matrix [rows, K]: boxes of box_rows x 64 elements, 128-byte swizzle,
// zeros outside the matrix.
inline int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return 3001;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 3000 + (int)r;
}

inline std::mutex g_map_mutex;
inline std::map<std::tuple<const void*, int, int, int>, CUtensorMap> g_maps;  // weights keep their maps

inline int cached_map(CUtensorMap* out, const void* base, int rows, int K, int box_rows, bool cache) {
  if (!cache) return make_map(out, base, rows, K, box_rows);
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const auto key = std::make_tuple(base, rows, K, box_rows);
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    CUtensorMap map;
    const int err = make_map(&map, base, rows, K, box_rows);
    if (err) return err;
    it = g_maps.emplace(key, map).first;
  }
  *out = it->second;
  return 0;
}


}  // namespace tc
}  // namespace akas
