// Shared helpers of the sm_100a kernels: element types, conversions, reductions, launch checks.
//
// Every kernel file exports plain C entry points (extern "C") that take raw device pointers,
// sizes and a CUDA stream, launch on that stream, and return the CUDA error code of the launch
// (0 on success). They allocate nothing; the caller owns every buffer.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define AKAS_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
#define AKAS_F32 0
#define AKAS_BF16 1

namespace akas {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  float t = lane < warps ? scratch[lane] : 0.f;
  return warp_sum(t);
}

// Loads `N` consecutive elements (N * sizeof(T) == 16 bytes) as floats. `p` must be 16-byte aligned.
__device__ __forceinline__ void load_vec(const float* p, float (&out)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void load_vec(const bf16* p, float (&out)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// Stores 16 bytes' worth of elements (4 float32 or 8 bfloat16) from floats. `p` must be 16-byte aligned.
__device__ __forceinline__ void store_vec(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store_vec(bf16* p, const float (&v)[8]) {
  uint4 o;
  uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = o;
}
// Stores 8 consecutive elements from floats (two 16-byte stores for float32, one for bfloat16).
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) { store_vec(p, v); }
// Loads 8 consecutive elements as floats.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) { load_vec(p, v); }

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<bf16> { static constexpr int N = 8; };

static inline int launch_status() { return (int)cudaGetLastError(); }

// Programmatic dependent launch. Kernels of a decode step follow one another on one stream; a kernel
// launched with launch_chained may begin while its predecessor is still draining, as soon as every block of
// the predecessor has executed chain_release(). Such a kernel must execute chain_wait() before it touches
// anything an earlier kernel wrote or may still read; what it does before that (fetching weights, which no
// kernel ever writes) overlaps the predecessor's tail. chain_wait() returns when all earlier kernels have
// completed and their writes are visible; in a kernel that was launched the ordinary way both are no-ops.
// Every chained kernel calls chain_wait() in every block before any exit, so that "my predecessor has
// completed" implies "everything before it has completed" along the whole chain.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool chained_launches_enabled();  // AKAS_B200_CHAINED_LAUNCHES=0 turns the attribute off (ordinary launches)

template <typename... Params, typename... Args>
static inline int launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = chained_launches_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&config, kernel, Params(args)...);
}

inline bool chained_launches_enabled() {
  static const bool enabled = [] {
    const char* v = getenv("AKAS_B200_CHAINED_LAUNCHES");
    return !(v && v[0] == '0');
  }();
  return enabled;
}

}  // namespace akas
