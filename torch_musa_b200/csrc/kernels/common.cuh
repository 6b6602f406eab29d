// Shared device helpers for the sm_100a kernel library.
#pragma once

#include "b200_kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <stdint.h>

namespace b200k {

constexpr int kSMs = 148;  // B200: 2 dies x 74 SMs

extern std::atomic<int64_t> g_launches;
inline void note_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

#define B200K_LAUNCH_RET()                       \
  do {                                           \
    ::b200k::note_launch();                      \
    return (int)cudaGetLastError();              \
  } while (0)

template <typename T> struct ToF;
template <> struct ToF<float> {
  __device__ __forceinline__ static float to(float v) { return v; }
  __device__ __forceinline__ static float from(float v) { return v; }
};
template <> struct ToF<__nv_bfloat16> {
  __device__ __forceinline__ static float to(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ __forceinline__ static __nv_bfloat16 from(float v) { return __float2bfloat16_rn(v); }
};
template <> struct ToF<__half> {
  __device__ __forceinline__ static float to(__half v) { return __half2float(v); }
  __device__ __forceinline__ static __half from(float v) { return __float2half_rn(v); }
};

// 16-byte vector of T
template <typename T>
struct alignas(16) Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename T>
__device__ __forceinline__ Vec16<T> ld16(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <typename T>
__device__ __forceinline__ void st16(T* p, const Vec16<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}
// streaming (evict-first) variants for data touched once
template <typename T>
__device__ __forceinline__ Vec16<T> ld16_stream(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = __ldcs(reinterpret_cast<const uint4*>(p));
  return r;
}
template <typename T>
__device__ __forceinline__ void st16_stream(T* p, const Vec16<T>& r) {
  __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&r));
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
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reductions; `sh` must hold 32 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* sh) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* sh) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

template <typename T>
inline bool aligned16(const T* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// dtype dispatch over the three floating types the kernels cover
#define B200K_DISPATCH_FLOAT(DTYPE, T, ...)                                   \
  switch (DTYPE) {                                                            \
    case B200_F32: { using T = float; __VA_ARGS__; break; }                   \
    case B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }          \
    case B200_F16: { using T = __half; __VA_ARGS__; break; }                  \
    default: return (int)cudaErrorNotSupported;                               \
  }

}  // namespace b200k
