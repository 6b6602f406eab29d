// Softmax / log-softmax (last dim) and fused cross-entropy, one CTA per row with a
// single-pass online (max, sum-exp) reduction: logits are read once for the
// statistics and once more (L2-resident: a 32000-wide bf16 row is 64 KB) to
// produce the output.  The fused cross-entropy never materialises the
// probabilities: forward keeps (loss, lse) per row, backward regenerates
// softmax from lse and may overwrite the logits in place.
// Parity: reference torch_musa/csrc/aten/ops/SoftMax.cpp:28-36,202-285 (vendor
// softmax), Loss.cpp:547-660 (fused 2-D CE) and
// csrc/extension/FusedCrossEntropyLoss.mu:55,160,293 (vocab-parallel pieces).
#include "common.cuh"

namespace b200k {
namespace {

constexpr int kThreads = 512;

struct MaxSum {
  float m, s;
};
__device__ __forceinline__ MaxSum ms_combine(MaxSum a, MaxSum b) {
  float m = fmaxf(a.m, b.m);
  if (m == -INFINITY) return MaxSum{m, 0.f};
  return MaxSum{m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}
__device__ __forceinline__ void ms_push(MaxSum& a, float x) {
  if (x > a.m) {
    a.s = a.s * __expf(a.m - x) + 1.f;
    a.m = x;
  } else if (x != -INFINITY) {
    a.s += __expf(x - a.m);
  }
}
__device__ __forceinline__ MaxSum block_ms(MaxSum v, float* shm, float* shs) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
    v = ms_combine(v, other);
  }
  __syncthreads();
  if (lane == 0) { shm[w] = v.m; shs[w] = v.s; }
  __syncthreads();
  MaxSum r = (lane < nw) ? MaxSum{shm[lane], shs[lane]} : MaxSum{-INFINITY, 0.f};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other{__shfl_xor_sync(0xffffffffu, r.m, o), __shfl_xor_sync(0xffffffffu, r.s, o)};
    r = ms_combine(r, other);
  }
  return r;
}

// Row statistics with optional 16-byte vector loads (VEC requires cols % V == 0 and an aligned base).
template <typename T, bool VEC>
__device__ __forceinline__ MaxSum row_stats(const T* __restrict__ xr, int64_t cols, float* shm, float* shs) {
  constexpr int V = Vec16<T>::N;
  MaxSum acc{-INFINITY, 0.f};
  if constexpr (VEC) {
    const int64_t nvec = cols / V;
    constexpr int U = 4;   // independent 16-byte loads in flight per thread; the max / sum update stays sequential
    for (int64_t i0 = threadIdx.x; i0 < nvec; i0 += (int64_t)blockDim.x * U) {
      Vec16<T> vv[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = i0 + (int64_t)u * blockDim.x;
        if (i < nvec) vv[u] = ld16(xr + i * V);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (i0 + (int64_t)u * blockDim.x >= nvec) break;
        float f[V];
        float lm = -INFINITY;
#pragma unroll
        for (int k = 0; k < V; ++k) { f[k] = ToF<T>::to(vv[u].v[k]); lm = fmaxf(lm, f[k]); }
        if (lm > acc.m) { acc.s *= __expf(acc.m - lm); acc.m = lm; }
        if (acc.m != -INFINITY) {
#pragma unroll
          for (int k = 0; k < V; ++k) acc.s += __expf(f[k] - acc.m);
        }
      }
    }
  } else {
    for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) ms_push(acc, ToF<T>::to(xr[i]));
  }
  return block_ms(acc, shm, shs);
}

template <typename T, bool VEC, bool LOG>
__global__ void __launch_bounds__(kThreads) softmax_fwd_kernel(T* __restrict__ y, const T* __restrict__ x, int64_t cols) {
  constexpr int V = Vec16<T>::N;
  __shared__ float shm[32], shs[32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * cols;
  T* yr = y + row * cols;
  MaxSum st = row_stats<T, VEC>(xr, cols, shm, shs);
  const float lse = st.m + __logf(st.s);
  const float inv = 1.f / st.s;
  if constexpr (VEC) {
    int64_t nvec = cols / V;
    for (int64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
      Vec16<T> v = ld16(xr + i * V), o;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float f = ToF<T>::to(v.v[k]);
        o.v[k] = ToF<T>::from(LOG ? f - lse : __expf(f - st.m) * inv);
      }
      st16_stream(yr + i * V, o);
    }
  } else {
    for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
      float f = ToF<T>::to(xr[i]);
      yr[i] = ToF<T>::from(LOG ? f - lse : __expf(f - st.m) * inv);
    }
  }
}

// softmax: dx = y * (dy - sum(dy*y)); log-softmax: dx = dy - exp(y) * sum(dy)
template <typename T, bool LOG>
__global__ void __launch_bounds__(kThreads) softmax_bwd_kernel(T* __restrict__ dx, const T* __restrict__ dy,
                                                               const T* __restrict__ y, int64_t cols) {
  __shared__ float sh[32];
  const int64_t row = blockIdx.x;
  const T* gr = dy + row * cols;
  const T* yr = y + row * cols;
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float g = ToF<T>::to(gr[i]);
    s += LOG ? g : g * ToF<T>::to(yr[i]);
  }
  s = block_sum(s, sh);
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float g = ToF<T>::to(gr[i]), yy = ToF<T>::to(yr[i]);
    dx[row * cols + i] = ToF<T>::from(LOG ? g - __expf(yy) * s : yy * (g - s));
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) ce_fwd_kernel(float* __restrict__ loss, float* __restrict__ lse_out,
                                                          const T* __restrict__ logits,
                                                          const int64_t* __restrict__ target, int64_t cols,
                                                          int64_t ignore_index, float smoothing) {
  __shared__ float shm[32], shs[32], sh[32];
  const int64_t row = blockIdx.x;
  const T* xr = logits + row * cols;
  MaxSum st = row_stats<T, VEC>(xr, cols, shm, shs);
  const float lse = st.m + __logf(st.s);
  float sum_logits = 0.f;
  if (smoothing > 0.f) {
    for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) sum_logits += ToF<T>::to(xr[i]);
    sum_logits = block_sum(sum_logits, sh);
  }
  if (threadIdx.x == 0) {
    const int64_t t = target[row];
    lse_out[row] = lse;
    if (t == ignore_index || t < 0 || t >= cols) {
      loss[row] = 0.f;
    } else {
      float nll = lse - ToF<T>::to(xr[t]);
      if (smoothing > 0.f) {
        float smooth = lse - sum_logits / (float)cols;  // mean over classes of -log p
        loss[row] = (1.f - smoothing) * nll + smoothing * smooth;
      } else {
        loss[row] = nll;
      }
    }
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) ce_bwd_kernel(T* __restrict__ dlogits, const T* __restrict__ logits,
                                                          const float* __restrict__ lse,
                                                          const int64_t* __restrict__ target,
                                                          const float* __restrict__ grad_loss, int grad_is_scalar,
                                                          float scale, int64_t cols, int64_t ignore_index,
                                                          float smoothing) {
  constexpr int V = Vec16<T>::N;
  const int64_t row = blockIdx.x;
  const int64_t t = target[row];
  const bool ignored = (t == ignore_index || t < 0 || t >= cols);
  const float g = ignored ? 0.f : scale * (grad_loss ? (grad_is_scalar ? grad_loss[0] : grad_loss[row]) : 1.f);
  const float l = lse[row];
  const T* xr = logits + row * cols;
  T* dr = dlogits + row * cols;
  const float on = 1.f - smoothing, off = smoothing / (float)cols;
  if constexpr (VEC) {
    const int64_t nvec = cols / V;
    constexpr int U = 4;   // independent 16-byte loads in flight per thread
    for (int64_t i0 = threadIdx.x; i0 < nvec; i0 += (int64_t)blockDim.x * U) {
      Vec16<T> v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = i0 + (int64_t)u * blockDim.x;
        if (i < nvec) v[u] = ld16(xr + i * V);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = i0 + (int64_t)u * blockDim.x;
        if (i < nvec) {
          Vec16<T> o;
#pragma unroll
          for (int k = 0; k < V; ++k) {
            const float p = __expf(ToF<T>::to(v[u].v[k]) - l);
            const float y = ((i * V + k) == t ? on : 0.f) + off;
            o.v[k] = ToF<T>::from(g * (p - y));
          }
          st16(dr + i * V, o);
        }
      }
    }
  } else {
    for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
      float p = __expf(ToF<T>::to(xr[i]) - l);
      float y = (i == t ? on : 0.f) + off;
      dr[i] = ToF<T>::from(g * (p - y));
    }
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) online_stats_kernel(float* __restrict__ stats3,
                                                                const T* __restrict__ logits,
                                                                const int64_t* __restrict__ target, int64_t cols,
                                                                int64_t vocab_start) {
  __shared__ float shm[32], shs[32];
  const int64_t row = blockIdx.x;
  const T* xr = logits + row * cols;
  MaxSum st = row_stats<T, VEC>(xr, cols, shm, shs);
  if (threadIdx.x == 0) {
    int64_t t = target[row] - vocab_start;
    stats3[row * 3 + 0] = st.m;
    stats3[row * 3 + 1] = st.s;
    stats3[row * 3 + 2] = (t >= 0 && t < cols) ? ToF<T>::to(xr[t]) : 0.f;  // summed across shards
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) vp_ce_finish_kernel(float* __restrict__ loss, T* __restrict__ logits,
                                                                const float* __restrict__ all_stats, int world,
                                                                const int64_t* __restrict__ target, int64_t rows,
                                                                int64_t cols, int64_t vocab_start,
                                                                int64_t ignore_index) {
  const int64_t row = blockIdx.x;
  // all_stats layout: [world, rows, 3]
  MaxSum g{-INFINITY, 0.f};
  float tl = 0.f;
  for (int r = 0; r < world; ++r) {
    const float* s = all_stats + ((int64_t)r * rows + row) * 3;
    g = ms_combine(g, MaxSum{s[0], s[1]});
    tl += s[2];
  }
  const float lse = g.m + __logf(g.s);
  const int64_t tg = target[row];
  const bool ignored = (tg == ignore_index);
  if (threadIdx.x == 0 && loss) loss[row] = ignored ? 0.f : lse - tl;
  const int64_t t = tg - vocab_start;
  T* xr = logits + row * cols;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float p = __expf(ToF<T>::to(xr[i]) - lse);
    xr[i] = ToF<T>::from(ignored ? 0.f : (p - (i == t ? 1.f : 0.f)));
  }
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

int b200_softmax_fwd(int dtype, void* y, const void* x, int64_t rows, int64_t cols, int log_softmax,
                     cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    bool vec = cols % Vec16<T>::N == 0 && aligned16((const T*)x) && aligned16((T*)y);
    dim3 grid((unsigned)rows);
    if (vec) {
      if (log_softmax) softmax_fwd_kernel<T, true, true><<<grid, kThreads, 0, stream>>>((T*)y, (const T*)x, cols);
      else softmax_fwd_kernel<T, true, false><<<grid, kThreads, 0, stream>>>((T*)y, (const T*)x, cols);
    } else {
      if (log_softmax) softmax_fwd_kernel<T, false, true><<<grid, kThreads, 0, stream>>>((T*)y, (const T*)x, cols);
      else softmax_fwd_kernel<T, false, false><<<grid, kThreads, 0, stream>>>((T*)y, (const T*)x, cols);
    }
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_softmax_bwd(int dtype, void* dx, const void* dy, const void* y, int64_t rows, int64_t cols, int log_softmax,
                     cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    dim3 grid((unsigned)rows);
    if (log_softmax) softmax_bwd_kernel<T, true><<<grid, kThreads, 0, stream>>>((T*)dx, (const T*)dy, (const T*)y, cols);
    else softmax_bwd_kernel<T, false><<<grid, kThreads, 0, stream>>>((T*)dx, (const T*)dy, (const T*)y, cols);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_cross_entropy_fwd(int dtype, float* loss, float* lse, const void* logits, const int64_t* target, int64_t rows,
                           int64_t cols, int64_t ignore_index, float label_smoothing, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    bool vec = cols % Vec16<T>::N == 0 && aligned16((const T*)logits);
    dim3 grid((unsigned)rows);
    if (vec) ce_fwd_kernel<T, true><<<grid, kThreads, 0, stream>>>(loss, lse, (const T*)logits, target, cols, ignore_index, label_smoothing);
    else ce_fwd_kernel<T, false><<<grid, kThreads, 0, stream>>>(loss, lse, (const T*)logits, target, cols, ignore_index, label_smoothing);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_cross_entropy_bwd(int dtype, void* dlogits, const void* logits, const float* lse, const int64_t* target,
                           const float* grad_loss, int grad_is_scalar, float scale, int64_t rows, int64_t cols,
                           int64_t ignore_index, float label_smoothing, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    bool vec = cols % Vec16<T>::N == 0 && aligned16((const T*)logits) && aligned16((T*)dlogits);
    dim3 grid((unsigned)rows);
    if (vec) ce_bwd_kernel<T, true><<<grid, kThreads, 0, stream>>>((T*)dlogits, (const T*)logits, lse, target, grad_loss, grad_is_scalar, scale, cols, ignore_index, label_smoothing);
    else ce_bwd_kernel<T, false><<<grid, kThreads, 0, stream>>>((T*)dlogits, (const T*)logits, lse, target, grad_loss, grad_is_scalar, scale, cols, ignore_index, label_smoothing);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_online_softmax_stats(int dtype, float* stats3, const void* logits, const int64_t* target, int64_t rows,
                              int64_t cols, int64_t vocab_start, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    bool vec = cols % Vec16<T>::N == 0 && aligned16((const T*)logits);
    dim3 grid((unsigned)rows);
    if (vec) online_stats_kernel<T, true><<<grid, kThreads, 0, stream>>>(stats3, (const T*)logits, target, cols, vocab_start);
    else online_stats_kernel<T, false><<<grid, kThreads, 0, stream>>>(stats3, (const T*)logits, target, cols, vocab_start);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_vocab_parallel_ce_finish(int dtype, float* loss, void* logits_inout, const float* all_stats, int world,
                                  const int64_t* target, int64_t rows, int64_t cols, int64_t vocab_start,
                                  int64_t ignore_index, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    vp_ce_finish_kernel<T><<<(unsigned)rows, kThreads, 0, stream>>>(loss, (T*)logits_inout, all_stats, world, target, rows, cols, vocab_start, ignore_index);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

}  // extern "C"
