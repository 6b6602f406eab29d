// Batch normalisation for channels-last activations viewed as a [P, C] matrix (P = N*H*W pixels).
//
// Training forward is two passes over x: per-channel sum / sum of squares (fp32 registers -> shared
// memory -> one atomicAdd per block and channel), then normalise + affine (+ residual add) (+ ReLU)
// fused in the second pass, which also emits save_mean / save_invstd and updates the running
// statistics.  Backward is the mirrored pair: reduce (sum dz, sum dz*xhat) and apply, with the ReLU
// mask recomputed from the saved output so no mask tensor is stored; the gradient that flows to the
// residual branch is written by the same pass.  Every thread owns 8 consecutive channels (one 16-byte
// vector), so loads and stores are coalesced 16-byte accesses along C.
//
// Parity: reference torch_musa/csrc/aten/ops/BatchNorm.cpp (vendor batch norm fwd/bwd) and the
// Conv+BN+activation fused modules in torch_musa/core/ao.
#include "common.cuh"

#include <cstdlib>

namespace b200k {
namespace {

constexpr int kBnThreads = 256;

struct BnGeom {
  int tx;       // threads along channel vectors
  int ty;       // threads along pixels
  int gx, gy;   // grid
};

inline BnGeom bn_geom(int64_t P, int C) {
  const int cv = C / 8;
  BnGeom g;
  g.tx = 1;
  while (g.tx * 2 <= cv && g.tx < 32 && cv % (g.tx * 2) == 0) g.tx *= 2;
  g.ty = kBnThreads / g.tx;
  g.gx = cv / g.tx;
  static const int mult = [] {
    const char* e = std::getenv("B200_BN_GRID_MULT");
    // CTAs per SM that share a channel group.  Every CTA ends with one atomic per channel into the same few cache
    // lines, so more CTAs buy memory-level parallelism and pay contention: measured on a ResNet-50 step (ms):
    // 2 -> 38.3, 4 -> 37.1, 8 -> 40.1, 16 -> 45.5.
    return e ? std::max(1, std::atoi(e)) : 4;
  }();
  int64_t want = (int64_t)kSMs * mult / g.gx;
  if (want < 1) want = 1;
  const int64_t max_y = cdiv(P, (int64_t)g.ty);
  g.gy = (int)std::min<int64_t>(std::max<int64_t>(want, 1), std::max<int64_t>(max_y, 1));
  return g;
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
  Vec16<T> r = ld16(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = ToF<T>::to(r.v[i]);
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]) {
  Vec16<T> r;
#pragma unroll
  for (int i = 0; i < 8; ++i) r.v[i] = ToF<T>::from(v[i]);
  st16(p, r);
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Reduces acc[16] over the ty threads that share a channel vector and adds the result to out0 / out1.
template <int NACC>
__device__ __forceinline__ void reduce_over_y_and_add(float (&acc)[NACC], float* sh, int tx_n, int ty_n, float* out0,
                                                     float* out1, int c0) {
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  // accumulator-major layout: consecutive threads hit consecutive banks (a thread-major layout would put the
  // whole warp on two banks and serialise every access sixteen-fold)
  const int T = tx_n * ty_n, me = ty * tx_n + tx;
#pragma unroll
  for (int i = 0; i < NACC; ++i) sh[i * T + me] = acc[i];
  __syncthreads();
  for (int s = ty_n >> 1; s > 0; s >>= 1) {
    if (ty < s) {
#pragma unroll
      for (int i = 0; i < NACC; ++i) sh[i * T + me] += sh[i * T + me + s * tx_n];
    }
    __syncthreads();
  }
  if (ty == 0) {
    // four floats per reduction message (sm_90+ vector red): a quarter of the traffic on the few cache lines that
    // every CTA of a channel group adds into
    static_assert(NACC == 16, "two groups of eight accumulators");
#pragma unroll
    for (int i = 0; i < 8; i += 4) {
      red_add_v4(out0 + c0 + i, sh[i * T + tx], sh[(i + 1) * T + tx], sh[(i + 2) * T + tx], sh[(i + 3) * T + tx]);
      red_add_v4(out1 + c0 + i, sh[(8 + i) * T + tx], sh[(9 + i) * T + tx], sh[(10 + i) * T + tx], sh[(11 + i) * T + tx]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kBnThreads)
bn_stats_kernel(const T* __restrict__ x, float* __restrict__ sums, int64_t P, int C, int tx_n, int ty_n) {
  extern __shared__ float sh[];
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  const int c0 = (blockIdx.x * tx_n + tx) * 8;
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
  // four independent 16-byte loads in flight per thread: the loop is latency-bound otherwise
  const int64_t step = (int64_t)gridDim.y * ty_n;
  int64_t p = (int64_t)blockIdx.y * ty_n + ty;
  for (; p + 3 * step < P; p += 4 * step) {
    Vec16<T> r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) r[u] = ld16(x + (p + u * step) * C + c0);
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float f = ToF<T>::to(r[u].v[i]);
        acc[i] += f;
        acc[8 + i] = fmaf(f, f, acc[8 + i]);
      }
  }
  for (; p < P; p += step) {
    float v[8];
    load8(x + p * C + c0, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      acc[i] += v[i];
      acc[8 + i] = fmaf(v[i], v[i], acc[8 + i]);
    }
  }
  reduce_over_y_and_add<16>(acc, sh, tx_n, ty_n, sums, sums + C, c0);
}

// stats_mode 0: sums = {sum, sumsq} of this batch (training); 1: use running_mean / running_var (inference)
template <typename T, bool RELU, bool RESID>
__global__ void __launch_bounds__(kBnThreads)
bn_apply_kernel(const T* __restrict__ x, const T* __restrict__ resid, T* __restrict__ y, const float* __restrict__ sums,
                const float* __restrict__ w, const float* __restrict__ b, float* running_mean, float* running_var,
                float* save_mean, float* save_invstd, int64_t P, int C, float eps, float momentum, int stats_mode,
                int tx_n, int ty_n) {
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  const int c0 = (blockIdx.x * tx_n + tx) * 8;
  float scale[8], shift[8];
  const float inv_p = 1.f / (float)P;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float mean, var;
    if (stats_mode == 0) {
      mean = sums[c0 + i] * inv_p;
      var = fmaxf(sums[C + c0 + i] * inv_p - mean * mean, 0.f);
    } else {
      mean = running_mean[c0 + i];
      var = running_var[c0 + i];
    }
    const float invstd = rsqrtf(var + eps);
    const float g = w ? w[c0 + i] : 1.f;
    scale[i] = g * invstd;
    shift[i] = (b ? b[c0 + i] : 0.f) - mean * scale[i];
    if (blockIdx.y == 0 && ty == 0 && stats_mode == 0) {
      if (save_mean) save_mean[c0 + i] = mean;
      if (save_invstd) save_invstd[c0 + i] = invstd;
      if (running_mean) running_mean[c0 + i] = (1.f - momentum) * running_mean[c0 + i] + momentum * mean;
      if (running_var) {
        const float unbiased = P > 1 ? var * ((float)P / (float)(P - 1)) : var;
        running_var[c0 + i] = (1.f - momentum) * running_var[c0 + i] + momentum * unbiased;
      }
    }
  }
  for (int64_t p = (int64_t)blockIdx.y * ty_n + ty; p < P; p += (int64_t)gridDim.y * ty_n) {
    float v[8];
    load8(x + p * C + c0, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = fmaf(v[i], scale[i], shift[i]);
    if constexpr (RESID) {
      float r[8];
      load8(resid + p * C + c0, r);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += r[i];
    }
    if constexpr (RELU) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = fmaxf(v[i], 0.f);
    }
    store8(y + p * C + c0, v);
  }
}

template <typename T, bool RELU>
__global__ void __launch_bounds__(kBnThreads)
bn_bwd_reduce_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ y,
                     const float* __restrict__ mean, const float* __restrict__ invstd, float* __restrict__ sums,
                     int64_t P, int C, int tx_n, int ty_n) {
  extern __shared__ float sh[];
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  const int c0 = (blockIdx.x * tx_n + tx) * 8;
  float mu[8], is[8], acc[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    mu[i] = mean[c0 + i];
    is[i] = invstd[c0 + i];
    acc[i] = acc[8 + i] = 0.f;
  }
  const int64_t step = (int64_t)gridDim.y * ty_n;
  int64_t p = (int64_t)blockIdx.y * ty_n + ty;
  auto consume = [&](const Vec16<T>& rg, const Vec16<T>& rx, const Vec16<T>& ro) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float g = ToF<T>::to(rg.v[i]);
      if constexpr (RELU) g = ToF<T>::to(ro.v[i]) > 0.f ? g : 0.f;
      acc[i] += g;
      acc[8 + i] = fmaf(g, (ToF<T>::to(rx.v[i]) - mu[i]) * is[i], acc[8 + i]);
    }
  };
  // two rows per iteration: four to six independent 16-byte loads in flight per thread
  for (; p + step < P; p += 2 * step) {
    Vec16<T> g0 = ld16(dy + p * C + c0), g1 = ld16(dy + (p + step) * C + c0);
    Vec16<T> x0 = ld16(x + p * C + c0), x1 = ld16(x + (p + step) * C + c0);
    Vec16<T> o0 = g0, o1 = g1;
    if constexpr (RELU) {
      o0 = ld16(y + p * C + c0);
      o1 = ld16(y + (p + step) * C + c0);
    }
    consume(g0, x0, o0);
    consume(g1, x1, o1);
  }
  for (; p < P; p += step) {
    Vec16<T> g0 = ld16(dy + p * C + c0), x0 = ld16(x + p * C + c0), o0 = g0;
    if constexpr (RELU) o0 = ld16(y + p * C + c0);
    consume(g0, x0, o0);
  }
  reduce_over_y_and_add<16>(acc, sh, tx_n, ty_n, sums, sums + C, c0);
}

template <typename T, bool RELU, bool RESID>
__global__ void __launch_bounds__(kBnThreads)
bn_bwd_apply_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ y,
                    const float* __restrict__ mean, const float* __restrict__ invstd, const float* __restrict__ w,
                    const float* __restrict__ sums, T* __restrict__ dx, T* __restrict__ dresid, int64_t P, int C,
                    int tx_n, int ty_n) {
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  const int c0 = (blockIdx.x * tx_n + tx) * 8;
  const float inv_p = 1.f / (float)P;
  float mu[8], is[8], k[8], m_dy[8], m_dyx[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    mu[i] = mean[c0 + i];
    is[i] = invstd[c0 + i];
    k[i] = (w ? w[c0 + i] : 1.f) * is[i];
    m_dy[i] = sums[c0 + i] * inv_p;
    m_dyx[i] = sums[C + c0 + i] * inv_p;
  }
  for (int64_t p = (int64_t)blockIdx.y * ty_n + ty; p < P; p += (int64_t)gridDim.y * ty_n) {
    float g[8], v[8];
    load8(dy + p * C + c0, g);
    load8(x + p * C + c0, v);
    if constexpr (RELU) {
      float o[8];
      load8(y + p * C + c0, o);
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = o[i] > 0.f ? g[i] : 0.f;
    }
    if constexpr (RESID) store8(dresid + p * C + c0, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float xhat = (v[i] - mu[i]) * is[i];
      v[i] = (g[i] - m_dy[i] - xhat * m_dyx[i]) * k[i];
    }
    store8(dx + p * C + c0, v);
  }
}

inline bool bn_ok(int64_t P, int C, const void* a, const void* b) {
  return P > 0 && C > 0 && C % 8 == 0 && aligned16((const char*)a) && (!b || aligned16((const char*)b));
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

int b200_bn_stats(int dtype, const void* x, float* sums, int64_t P, int C, cudaStream_t stream) {
  if (!bn_ok(P, C, x, nullptr)) return (int)cudaErrorNotSupported;
  const BnGeom g = bn_geom(P, C);
  const size_t sh = (size_t)kBnThreads * 16 * sizeof(float);
  cudaError_t e = cudaMemsetAsync(sums, 0, sizeof(float) * 2 * C, stream);
  if (e != cudaSuccess) return (int)e;
  B200K_DISPATCH_FLOAT(dtype, T, {
    if constexpr (std::is_same<T, float>::value) return (int)cudaErrorNotSupported;
    else bn_stats_kernel<T><<<dim3(g.gx, g.gy), kBnThreads, sh, stream>>>((const T*)x, sums, P, C, g.tx, g.ty);
  });
  B200K_LAUNCH_RET();
}

int b200_bn_apply(int dtype, const void* x, const void* resid, void* y, const float* sums, const float* w,
                  const float* b, float* running_mean, float* running_var, float* save_mean, float* save_invstd,
                  int64_t P, int C, float eps, float momentum, int relu, int stats_mode, cudaStream_t stream) {
  if (!bn_ok(P, C, x, y) || (resid && !aligned16((const char*)resid))) return (int)cudaErrorNotSupported;
  if (stats_mode != 0 && (!running_mean || !running_var)) return (int)cudaErrorInvalidValue;
  const BnGeom g = bn_geom(P, C);
#define BN_APPLY(RELU, RESID)                                                                                     \
  bn_apply_kernel<T, RELU, RESID><<<dim3(g.gx, g.gy), kBnThreads, 0, stream>>>(                                   \
      (const T*)x, (const T*)resid, (T*)y, sums, w, b, running_mean, running_var, save_mean, save_invstd, P, C,   \
      eps, momentum, stats_mode, g.tx, g.ty)
  B200K_DISPATCH_FLOAT(dtype, T, {
    if constexpr (std::is_same<T, float>::value) return (int)cudaErrorNotSupported;
    else {
      if (relu && resid) BN_APPLY(true, true);
      else if (relu) BN_APPLY(true, false);
      else if (resid) BN_APPLY(false, true);
      else BN_APPLY(false, false);
    }
  });
#undef BN_APPLY
  B200K_LAUNCH_RET();
}

int b200_bn_bwd_reduce(int dtype, const void* dy, const void* x, const void* y, const float* mean,
                       const float* invstd, float* sums, int64_t P, int C, int relu, cudaStream_t stream) {
  if (!bn_ok(P, C, dy, x) || (relu && !y)) return (int)cudaErrorNotSupported;
  const BnGeom g = bn_geom(P, C);
  const size_t sh = (size_t)kBnThreads * 16 * sizeof(float);
  cudaError_t e = cudaMemsetAsync(sums, 0, sizeof(float) * 2 * C, stream);
  if (e != cudaSuccess) return (int)e;
  B200K_DISPATCH_FLOAT(dtype, T, {
    if constexpr (std::is_same<T, float>::value) return (int)cudaErrorNotSupported;
    else {
      if (relu)
        bn_bwd_reduce_kernel<T, true><<<dim3(g.gx, g.gy), kBnThreads, sh, stream>>>((const T*)dy, (const T*)x,
                                                                                    (const T*)y, mean, invstd, sums,
                                                                                    P, C, g.tx, g.ty);
      else
        bn_bwd_reduce_kernel<T, false><<<dim3(g.gx, g.gy), kBnThreads, sh, stream>>>((const T*)dy, (const T*)x,
                                                                                     (const T*)y, mean, invstd, sums,
                                                                                     P, C, g.tx, g.ty);
    }
  });
  B200K_LAUNCH_RET();
}

int b200_bn_bwd_apply(int dtype, const void* dy, const void* x, const void* y, const float* mean, const float* invstd,
                      const float* w, const float* sums, void* dx, void* dresid, int64_t P, int C, int relu,
                      cudaStream_t stream) {
  if (!bn_ok(P, C, dy, x) || !aligned16((const char*)dx) || (relu && !y)) return (int)cudaErrorNotSupported;
  const BnGeom g = bn_geom(P, C);
#define BN_BWD(RELU, RESID)                                                                                  \
  bn_bwd_apply_kernel<T, RELU, RESID><<<dim3(g.gx, g.gy), kBnThreads, 0, stream>>>(                          \
      (const T*)dy, (const T*)x, (const T*)y, mean, invstd, w, sums, (T*)dx, (T*)dresid, P, C, g.tx, g.ty)
  B200K_DISPATCH_FLOAT(dtype, T, {
    if constexpr (std::is_same<T, float>::value) return (int)cudaErrorNotSupported;
    else {
      if (relu && dresid) BN_BWD(true, true);
      else if (relu) BN_BWD(true, false);
      else if (dresid) BN_BWD(false, true);
      else BN_BWD(false, false);
    }
  });
#undef BN_BWD
  B200K_LAUNCH_RET();
}

}  // extern "C"
