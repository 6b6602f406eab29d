// RMSNorm / LayerNorm forward and backward: one CTA per row (rows of a few
// thousand elements: the row stays in registers between the statistics pass and
// the normalisation pass, so HBM sees exactly one read of x and one write of y),
// fp32 statistics, 128-bit accesses.  Weight gradients are accumulated per CTA
// over a strip of rows and written as [n_strips, cols] fp32 partial sums which
// the caller reduces with the column-sum kernel (deterministic, no atomics).
// Parity: reference torch_musa/csrc/aten/ops/RMSNorm.cpp:113-125,283-306 and
// LayerNorm.cpp:141-147,295-300 (vendor-library calls there).
#include "common.cuh"

namespace b200k {
namespace {


template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS) rmsnorm_fwd_kernel(T* __restrict__ y, float* __restrict__ rstd_out,
                                                              const T* __restrict__ x, const T* __restrict__ w,
                                                              const T* __restrict__ residual, T* __restrict__ res_out,
                                                              int64_t cols, float eps) {
  constexpr int V = Vec16<T>::N;
  __shared__ float sh[32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * cols;
  const T* rr = residual ? residual + row * cols : nullptr;
  T* yr = y + row * cols;
  const int nvec = (int)(cols / V);
  Vec16<T> buf[VPT];
  float ss = 0.f;
  int cnt;
  _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
    Vec16<T> v = ld16_stream(xr + (int64_t)i * V);
    if (rr) {
      Vec16<T> r = ld16_stream(rr + (int64_t)i * V);
#pragma unroll
      for (int k = 0; k < V; ++k) v.v[k] = ToF<T>::from(ToF<T>::to(v.v[k]) + ToF<T>::to(r.v[k]));
      st16(res_out + row * cols + (int64_t)i * V, v);
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float f = ToF<T>::to(v.v[k]);
      ss += f * f;
    }
    if (cnt < VPT) buf[cnt] = v;
  }
  ss = block_sum(ss, sh);
  const float rstd = rsqrtf(ss / (float)cols + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
    Vec16<T> v;
    if (cnt < VPT) v = buf[cnt];
    else v = rr ? ld16(res_out + row * cols + (int64_t)i * V) : ld16(xr + (int64_t)i * V);
    Vec16<T> o;
    if (w) {
      Vec16<T> wv = ld16(w + (int64_t)i * V);
#pragma unroll
      for (int k = 0; k < V; ++k) o.v[k] = ToF<T>::from(ToF<T>::to(v.v[k]) * rstd * ToF<T>::to(wv.v[k]));
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) o.v[k] = ToF<T>::from(ToF<T>::to(v.v[k]) * rstd);
    }
    st16_stream(yr + (int64_t)i * V, o);
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)), xhat = x*rstd. A CTA walks a strip of rows and keeps
// dw partial sums (dy * xhat) for its columns in registers.
template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS) rmsnorm_bwd_kernel(T* __restrict__ dx, float* __restrict__ dw_partial,
                                                              const T* __restrict__ dy, const T* __restrict__ x,
                                                              const T* __restrict__ w, const float* __restrict__ rstd,
                                                              int64_t rows, int64_t cols, int rows_per_cta) {
  constexpr int V = Vec16<T>::N;
  __shared__ float sh[32];
  const int nvec = (int)(cols / V);
  float dwacc[VPT][V];
#pragma unroll
  for (int c = 0; c < VPT; ++c)
#pragma unroll
    for (int k = 0; k < V; ++k) dwacc[c][k] = 0.f;
  Vec16<T> wreg[VPT];
  {
    int cnt;
    _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
      if (w) wreg[cnt] = ld16(w + (int64_t)i * V);
      else {
#pragma unroll
        for (int k = 0; k < V; ++k) wreg[cnt].v[k] = ToF<T>::from(1.f);
      }
    }
  }
  const int64_t r0 = (int64_t)blockIdx.x * rows_per_cta;
  const int64_t r1 = min(r0 + (int64_t)rows_per_cta, rows);
  for (int64_t row = r0; row < r1; ++row) {
    const T* xr = x + row * cols;
    const T* gr = dy + row * cols;
    const float rs = rstd[row];
    Vec16<T> xb[VPT], gb[VPT];
    float dot = 0.f;
    int cnt;
    _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
      xb[cnt] = ld16_stream(xr + (int64_t)i * V);
      gb[cnt] = ld16_stream(gr + (int64_t)i * V);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float xh = ToF<T>::to(xb[cnt].v[k]) * rs;
        float g = ToF<T>::to(gb[cnt].v[k]);
        dot += g * ToF<T>::to(wreg[cnt].v[k]) * xh;
        dwacc[cnt][k] += g * xh;
      }
    }
    dot = block_sum(dot, sh);
    const float m = dot / (float)cols;
      _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
      Vec16<T> o;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float xh = ToF<T>::to(xb[cnt].v[k]) * rs;
        float g = ToF<T>::to(gb[cnt].v[k]) * ToF<T>::to(wreg[cnt].v[k]);
        o.v[k] = ToF<T>::from(rs * (g - xh * m));
      }
      st16_stream(dx + row * cols + (int64_t)i * V, o);
    }
  }
  if (dw_partial) {
    float* out = dw_partial + (int64_t)blockIdx.x * cols;
    int cnt;
    _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
#pragma unroll
      for (int k = 0; k < V; k += 4)
        *reinterpret_cast<float4*>(out + (int64_t)i * V + k) =
            make_float4(dwacc[cnt][k], dwacc[cnt][k + 1], dwacc[cnt][k + 2], dwacc[cnt][k + 3]);
    }
  }
}

template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS) layernorm_fwd_kernel(T* __restrict__ y, float* __restrict__ mean_out,
                                                                float* __restrict__ rstd_out, const T* __restrict__ x,
                                                                const T* __restrict__ w, const T* __restrict__ b,
                                                                int64_t cols, float eps) {
  constexpr int V = Vec16<T>::N;
  __shared__ float sh[32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * cols;
  const int nvec = (int)(cols / V);
  Vec16<T> buf[VPT];
  float s = 0.f;
  int cnt;
  _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
    buf[cnt] = ld16_stream(xr + (int64_t)i * V);
#pragma unroll
    for (int k = 0; k < V; ++k) s += ToF<T>::to(buf[cnt].v[k]);
  }
  const float mean = block_sum(s, sh) / (float)cols;
  float vs = 0.f;
  _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float d = ToF<T>::to(buf[cnt].v[k]) - mean;
      vs += d * d;
    }
  }
  const float rstd = rsqrtf(block_sum(vs, sh) / (float)cols + eps);
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
    Vec16<T> o;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float v = (ToF<T>::to(buf[cnt].v[k]) - mean) * rstd;
      if (w) v *= ToF<T>::to(w[(int64_t)i * V + k]);
      if (b) v += ToF<T>::to(b[(int64_t)i * V + k]);
      o.v[k] = ToF<T>::from(v);
    }
    st16_stream(y + row * cols + (int64_t)i * V, o);
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g*xhat)), g = dy*w
template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS) layernorm_bwd_kernel(T* __restrict__ dx, float* __restrict__ dw_partial,
                                                                float* __restrict__ db_partial,
                                                                const T* __restrict__ dy, const T* __restrict__ x,
                                                                const T* __restrict__ w, const float* __restrict__ mean,
                                                                const float* __restrict__ rstd, int64_t rows,
                                                                int64_t cols, int rows_per_cta) {
  constexpr int V = Vec16<T>::N;
  __shared__ float sh[32];
  const int nvec = (int)(cols / V);
  float dwacc[VPT][V], dbacc[VPT][V];
#pragma unroll
  for (int c = 0; c < VPT; ++c)
#pragma unroll
    for (int k = 0; k < V; ++k) { dwacc[c][k] = 0.f; dbacc[c][k] = 0.f; }
  const int64_t r0 = (int64_t)blockIdx.x * rows_per_cta;
  const int64_t r1 = min(r0 + (int64_t)rows_per_cta, rows);
  for (int64_t row = r0; row < r1; ++row) {
    const float mu = mean[row], rs = rstd[row];
    Vec16<T> xb[VPT], gb[VPT];
    float s1 = 0.f, s2 = 0.f;
    int cnt;
    _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
      xb[cnt] = ld16_stream(x + row * cols + (int64_t)i * V);
      gb[cnt] = ld16_stream(dy + row * cols + (int64_t)i * V);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float xh = (ToF<T>::to(xb[cnt].v[k]) - mu) * rs;
        float g0 = ToF<T>::to(gb[cnt].v[k]);
        float g = w ? g0 * ToF<T>::to(w[(int64_t)i * V + k]) : g0;
        s1 += g;
        s2 += g * xh;
        dwacc[cnt][k] += g0 * xh;
        dbacc[cnt][k] += g0;
      }
    }
    s1 = block_sum(s1, sh) / (float)cols;
    s2 = block_sum(s2, sh) / (float)cols;
      _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
      Vec16<T> o;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float xh = (ToF<T>::to(xb[cnt].v[k]) - mu) * rs;
        float g0 = ToF<T>::to(gb[cnt].v[k]);
        float g = w ? g0 * ToF<T>::to(w[(int64_t)i * V + k]) : g0;
        o.v[k] = ToF<T>::from(rs * (g - s1 - xh * s2));
      }
      st16_stream(dx + row * cols + (int64_t)i * V, o);
    }
  }
  int cnt;
  _Pragma("unroll") for (cnt = 0; cnt < VPT; ++cnt) { const int i = threadIdx.x + cnt * THREADS; if (i >= nvec) break;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      if (dw_partial) dw_partial[(int64_t)blockIdx.x * cols + (int64_t)i * V + k] = dwacc[cnt][k];
      if (db_partial) db_partial[(int64_t)blockIdx.x * cols + (int64_t)i * V + k] = dbacc[cnt][k];
    }
  }
}

// (threads, vectors per thread) for a row of `nvec` 16-byte vectors; rows beyond 512*8 vectors are not covered
#define B200K_ROW_LAUNCH(KERNEL, NVEC, GRID, STREAM, ...)                                        \
  do {                                                                                           \
    /* few threads with several independent 16-byte loads each: more bytes in flight per SM and    \
       more resident CTAs than one vector per thread */                                            \
    if ((NVEC) <= 128) KERNEL<T, 128, 1><<<(GRID), 128, 0, (STREAM)>>>(__VA_ARGS__);             \
    else if ((NVEC) <= 256) KERNEL<T, 128, 2><<<(GRID), 128, 0, (STREAM)>>>(__VA_ARGS__);        \
    else if ((NVEC) <= 512) KERNEL<T, 128, 4><<<(GRID), 128, 0, (STREAM)>>>(__VA_ARGS__);        \
    else if ((NVEC) <= 1024) KERNEL<T, 256, 4><<<(GRID), 256, 0, (STREAM)>>>(__VA_ARGS__);       \
    else if ((NVEC) <= 2048) KERNEL<T, 512, 4><<<(GRID), 512, 0, (STREAM)>>>(__VA_ARGS__);       \
    else KERNEL<T, 512, 8><<<(GRID), 512, 0, (STREAM)>>>(__VA_ARGS__);                           \
  } while (0)

constexpr int64_t kMaxRowVecs = 512 * 8;

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

int b200_rmsnorm_bwd_partial_rows(int64_t rows, int64_t cols) {
  (void)cols;
  // ~2 CTAs per SM, each walking a strip of rows
  int64_t ctas = std::min<int64_t>(rows, (int64_t)kSMs * 2);
  if (ctas < 1) ctas = 1;
  int64_t rpc = cdiv(rows, ctas);
  return (int)cdiv(rows, rpc);
}

int b200_rmsnorm_fwd(int dtype, void* y, float* rstd, const void* x, const void* w, const void* residual,
                     void* res_out, int64_t rows, int64_t cols, float eps, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = Vec16<T>::N;
    int64_t nvec = cols / V;
    if (cols % V != 0 || nvec > kMaxRowVecs || !aligned16((const T*)x) || !aligned16((T*)y) ||
        (w && !aligned16((const T*)w)) || (residual && (!aligned16((const T*)residual) || !aligned16((T*)res_out))))
      return (int)cudaErrorNotSupported;
    B200K_ROW_LAUNCH(rmsnorm_fwd_kernel, nvec, (unsigned)rows, stream, (T*)y, rstd, (const T*)x, (const T*)w,
                     (const T*)residual, (T*)res_out, cols, eps);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_rmsnorm_bwd(int dtype, void* dx, float* dw_partial, int* nblocks_out_host, const void* dy, const void* x,
                     const void* w, const float* rstd, int64_t rows, int64_t cols, cudaStream_t stream) {
  if (rows == 0) return 0;
  int nb = b200_rmsnorm_bwd_partial_rows(rows, cols);
  int rpc = (int)cdiv(rows, nb);
  if (nblocks_out_host) *nblocks_out_host = nb;
  B200K_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = Vec16<T>::N;
    int64_t nvec = cols / V;
    if (cols % V != 0 || nvec > kMaxRowVecs || !aligned16((const T*)x) || !aligned16((const T*)dy) ||
        !aligned16((T*)dx) || (w && !aligned16((const T*)w)))
      return (int)cudaErrorNotSupported;
    B200K_ROW_LAUNCH(rmsnorm_bwd_kernel, nvec, nb, stream, (T*)dx, dw_partial, (const T*)dy, (const T*)x, (const T*)w,
                     rstd, rows, cols, rpc);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_layernorm_fwd(int dtype, void* y, float* mean, float* rstd, const void* x, const void* w, const void* b,
                       int64_t rows, int64_t cols, float eps, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = Vec16<T>::N;
    int64_t nvec = cols / V;
    if (cols % V != 0 || nvec > kMaxRowVecs || !aligned16((const T*)x) || !aligned16((T*)y))
      return (int)cudaErrorNotSupported;
    B200K_ROW_LAUNCH(layernorm_fwd_kernel, nvec, (unsigned)rows, stream, (T*)y, mean, rstd, (const T*)x, (const T*)w,
                     (const T*)b, cols, eps);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_layernorm_bwd(int dtype, void* dx, float* dw_partial, float* db_partial, const void* dy, const void* x,
                       const void* w, const float* mean, const float* rstd, int64_t rows, int64_t cols,
                       cudaStream_t stream) {
  if (rows == 0) return 0;
  int nb = b200_rmsnorm_bwd_partial_rows(rows, cols);
  int rpc = (int)cdiv(rows, nb);
  B200K_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = Vec16<T>::N;
    int64_t nvec = cols / V;
    if (cols % V != 0 || nvec > kMaxRowVecs || !aligned16((const T*)x) || !aligned16((const T*)dy) ||
        !aligned16((T*)dx))
      return (int)cudaErrorNotSupported;
    B200K_ROW_LAUNCH(layernorm_bwd_kernel, nvec, nb, stream, (T*)dx, dw_partial, db_partial, (const T*)dy, (const T*)x,
                     (const T*)w, mean, rstd, rows, cols, rpc);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

}  // extern "C"
