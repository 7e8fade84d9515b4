// Shared device helpers for the sm_100a kernels of this engine.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "status.h"

namespace lse {

typedef __nv_bfloat16 bf16;

// Fixed-point sums (LSE_FIXED64 in kernels.h): value * 2^24 in a 64-bit integer.
typedef long long fixed64;
constexpr float kFixedScale = 16777216.f;
constexpr float kFixedInverse = 1.f / 16777216.f;
__device__ __forceinline__ float fixed_to_float(fixed64 v) { return (float)v * kFixedInverse; }

template <typename T>
struct Num;

template <>
struct Num<float> {
  static constexpr int kVec = 4;  // elements in a 16-byte vector
  __device__ __forceinline__ static float to_float(float v) { return v; }
  __device__ __forceinline__ static float from_float(float v) { return v; }
};

template <>
struct Num<bf16> {
  static constexpr int kVec = 8;
  __device__ __forceinline__ static float to_float(bf16 v) { return __bfloat162float(v); }
  __device__ __forceinline__ static bf16 from_float(float v) { return __float2bfloat16_rn(v); }
};

template <>
struct Num<fixed64> {
  static constexpr int kVec = 2;
  __device__ __forceinline__ static float to_float(fixed64 v) { return fixed_to_float(v); }
  __device__ __forceinline__ static fixed64 from_float(float v) { return __float2ll_rn(v * kFixedScale); }
};

// 16-byte vector of T, read and written as one transaction.
template <typename T>
struct alignas(16) Vec16 {
  T v[Num<T>::kVec];
};

template <typename T>
__device__ __forceinline__ Vec16<T> load16(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}

template <typename T>
__device__ __forceinline__ void store16(T* p, const Vec16<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

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

// Sum over a thread block. `scratch` holds at least 32 floats of shared memory. Every thread gets
// the result. The order of the additions depends only on blockDim, never on the data.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  return warp_sum(t);
}

// Page and offset of a token position. page_shift >= 0 when page_tokens is a power of two.
__device__ __forceinline__ void page_of(int pos, int page_tokens, int page_shift, int& idx, int& off) {
  if (page_shift >= 0) {
    idx = pos >> page_shift;
    off = pos & (page_tokens - 1);
  } else {
    idx = pos / page_tokens;
    off = pos - idx * page_tokens;
  }
}

// Programmatic dependent launch. A kernel launched through lse::launch may be scheduled while
// the kernel before it in the stream is still running; it must call pdl_wait() before it touches
// anything that kernel (or any earlier one) wrote, and may do work that depends on nothing first.
// pdl_trigger() lets the *next* kernel in the stream be scheduled early in the same way.
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#ifdef __CUDACC__
inline bool pdl_enabled() {
  static const bool on = (getenv("LSE_NO_PDL") == nullptr);
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

}  // namespace lse
