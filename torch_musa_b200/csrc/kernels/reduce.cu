// Reductions: last-dim (row) reductions, full reductions (two-stage, deterministic)
// and column sums (used to finish the norm weight gradients and bias gradients).
// Parity: reference torch_musa/csrc/aten/ops/musa/Reduce.muh:92-227 (block
// reduce + multi-CTA second stage).
#include "common.cuh"

namespace b200k {
namespace {

constexpr int kThreads = 256;

template <int OP>
__device__ __forceinline__ float ident() {
  if constexpr (OP == B200_RED_MAX) return -INFINITY;
  else if constexpr (OP == B200_RED_MIN) return INFINITY;
  else return 0.f;
}
template <int OP>
__device__ __forceinline__ float pre(float x) {
  if constexpr (OP == B200_RED_SUMSQ) return x * x;
  else if constexpr (OP == B200_RED_ABSMAX) return fabsf(x);
  else return x;
}
template <int OP>
__device__ __forceinline__ float comb(float a, float b) {
  if constexpr (OP == B200_RED_MAX || OP == B200_RED_ABSMAX) return (a != a || b != b) ? NAN : fmaxf(a, b);
  else if constexpr (OP == B200_RED_MIN) return (a != a || b != b) ? NAN : fminf(a, b);
  else return a + b;
}
template <int OP>
__device__ __forceinline__ float block_red(float v, float* sh) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = comb<OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : ident<OP>();
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = comb<OP>(r, __shfl_xor_sync(0xffffffffu, r, o));
  return r;
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads) reduce_rows_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                               int64_t cols) {
  __shared__ float sh[32];
  const int64_t row = blockIdx.x;
  const T* p = in + row * cols;
  float acc = ident<OP>();
  constexpr int V = Vec16<T>::N;
  if (cols % V == 0 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
    for (int64_t i = threadIdx.x; i < cols / V; i += blockDim.x) {
      Vec16<T> v = ld16(p + i * V);
#pragma unroll
      for (int k = 0; k < V; ++k) acc = comb<OP>(acc, pre<OP>(ToF<T>::to(v.v[k])));
    }
  } else {
    for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) acc = comb<OP>(acc, pre<OP>(ToF<T>::to(p[i])));
  }
  acc = block_red<OP>(acc, sh);
  if (threadIdx.x == 0) {
    if constexpr (OP == B200_RED_MEAN) acc /= (float)cols;
    out[row] = ToF<T>::from(acc);
  }
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads) reduce_all_stage1(float* __restrict__ partial, const T* __restrict__ in,
                                                              int64_t n) {
  __shared__ float sh[32];
  float acc = ident<OP>();
  constexpr int V = Vec16<T>::N;
  int64_t nvec = ((reinterpret_cast<uintptr_t>(in) & 15) == 0) ? n / V : 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    Vec16<T> v = ld16(in + i * V);
#pragma unroll
    for (int k = 0; k < V; ++k) acc = comb<OP>(acc, pre<OP>(ToF<T>::to(v.v[k])));
  }
  for (int64_t i = nvec * V + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    acc = comb<OP>(acc, pre<OP>(ToF<T>::to(in[i])));
  acc = block_red<OP>(acc, sh);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads) reduce_all_stage2(void* __restrict__ out, int out_f32,
                                                              const float* __restrict__ partial, int np, int64_t n) {
  __shared__ float sh[32];
  float acc = ident<OP>();
  for (int i = threadIdx.x; i < np; i += blockDim.x) acc = comb<OP>(acc, partial[i]);
  acc = block_red<OP>(acc, sh);
  if (threadIdx.x == 0) {
    if constexpr (OP == B200_RED_MEAN) acc /= (float)n;
    if (out_f32) *reinterpret_cast<float*>(out) = acc;
    else *reinterpret_cast<T*>(out) = ToF<T>::from(acc);
  }
}

// Column sums of a [rows, cols] matrix: a CTA owns a strip of 32*VT columns and 8 warps split the rows.
template <typename T, typename O>
__global__ void __launch_bounds__(256) reduce_cols_kernel(O* __restrict__ out, const T* __restrict__ in, int64_t rows,
                                                          int64_t cols) {
  __shared__ float sh[8][33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t c = (int64_t)blockIdx.x * 32 + lane;
  float acc = 0.f;
  if (c < cols)
    for (int64_t r = w; r < rows; r += 8) acc += ToF<T>::to(in[r * cols + c]);
  sh[w][lane] = acc;
  __syncthreads();
  if (w == 0 && c < cols) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += sh[k][lane];
    out[c] = ToF<O>::from(s);
  }
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

#define RED_CASE(OPC, CALL) case OPC: { constexpr int OP = OPC; CALL; break; }
#define RED_SWITCH(op, CALL)                                                                      \
  switch (op) {                                                                                   \
    RED_CASE(B200_RED_SUM, CALL) RED_CASE(B200_RED_MEAN, CALL) RED_CASE(B200_RED_MAX, CALL)       \
    RED_CASE(B200_RED_MIN, CALL) RED_CASE(B200_RED_SUMSQ, CALL) RED_CASE(B200_RED_ABSMAX, CALL)   \
    default: return (int)cudaErrorNotSupported;                                                   \
  }

int b200_reduce_rows(int op, int dtype, void* out, const void* in, int64_t rows, int64_t cols, cudaStream_t stream) {
  if (rows == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    RED_SWITCH(op, (reduce_rows_kernel<T, OP><<<(unsigned)rows, kThreads, 0, stream>>>((T*)out, (const T*)in, cols)));
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_reduce_all(int op, int dtype, void* out, int out_f32, const void* in, int64_t n, float* scratch,
                    cudaStream_t stream) {
  int np = (int)std::min<int64_t>(std::max<int64_t>(cdiv(n, (int64_t)kThreads * 16), 1), 1024);
  B200K_DISPATCH_FLOAT(dtype, T, {
    RED_SWITCH(op, (reduce_all_stage1<T, OP><<<np, kThreads, 0, stream>>>(scratch, (const T*)in, n)));
    note_launch();
    RED_SWITCH(op, (reduce_all_stage2<T, OP><<<1, kThreads, 0, stream>>>(out, out_f32, scratch, np, n)));
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_reduce_cols_sum(int dtype, void* out, int out_dtype, const void* in, int64_t rows, int64_t cols,
                         cudaStream_t stream) {
  if (cols == 0) return 0;
  unsigned grid = (unsigned)cdiv(cols, 32);
  B200K_DISPATCH_FLOAT(dtype, T, {
    B200K_DISPATCH_FLOAT(out_dtype, O, (reduce_cols_kernel<T, O><<<grid, 256, 0, stream>>>((O*)out, (const T*)in, rows, cols)));
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

}  // extern "C"
