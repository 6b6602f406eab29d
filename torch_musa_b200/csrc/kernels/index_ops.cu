// Indexing, scan and selection kernels:
//   index_select / index_put over a [outer, dim, inner] view (byte movers: rows are copied in the widest unit that
//   divides them; accumulation uses native atomics), gather / scatter / scatter_add along a dimension, triangular
//   masks, arange, inclusive cumulative sums along rows, top-k of short rows (one thread per row, the k best kept
//   in registers) and full row sorts (CUB segmented radix sort, stable, with the original positions as values).
// Parity: reference torch_musa/csrc/aten/ops/musa/{IndexKernel,Indexing,IndexSelect,ScatterGatherKernel,CumsumKernel,
// Tril,Range}.mu and ops/Topk.cpp, Sort.cpp (ports of ATen kernels plus vendor-library sort / top-k).
#include "common.cuh"

#include <cub/cub.cuh>

namespace b200k {
namespace {

constexpr int kIdxThreads = 256;

template <typename T, typename A> struct ToAcc {
  static __device__ __forceinline__ A get(T v) { return (A)v; }
  static __device__ __forceinline__ T put(A v) { return (T)v; }
};
template <> struct ToAcc<__nv_bfloat16, float> {
  static __device__ __forceinline__ float get(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 put(float v) { return __float2bfloat16_rn(v); }
};
template <> struct ToAcc<__half, float> {
  static __device__ __forceinline__ float get(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half put(float v) { return __float2half_rn(v); }
};

template <typename T> inline T from_double(double v) { return (T)v; }
template <> inline __nv_bfloat16 from_double<__nv_bfloat16>(double v) { return __float2bfloat16_rn((float)v); }
template <> inline __half from_double<__half>(double v) { return __float2half_rn((float)v); }

inline unsigned blocks_for(int64_t n, int per_block = kIdxThreads) {
  int64_t b = cdiv(n, per_block);
  if (b < 1) b = 1;
  return (unsigned)std::min<int64_t>(b, 2147483647ll);
}

template <typename I>
__device__ __forceinline__ int64_t wrap_index(I v, int64_t size, int* status) {
  int64_t i = (int64_t)v;
  if (i < 0) i += size;
  if (i < 0 || i >= size) {          // out of range: record it and clamp (never a wild address)
    if (status) atomicExch(status, 1);
    i = i < 0 ? 0 : size - 1;
  }
  return i;
}

// ------------------------------------------------------------------ index_select: out[o, j, i] = in[o, idx[j], i]
template <typename U, typename I>
__global__ void __launch_bounds__(kIdxThreads) index_select_kernel(U* __restrict__ out, const U* __restrict__ in,
                                                                   const I* __restrict__ idx, int64_t outer, int64_t D,
                                                                   int64_t inner, int64_t J, int* status) {
  const int64_t total = outer * J * inner;
  for (int64_t t = (int64_t)blockIdx.x * kIdxThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kIdxThreads) {
    const int64_t i = t % inner, j = (t / inner) % J, o = t / (inner * J);
    const int64_t src = wrap_index(idx[j], D, status);
    out[t] = in[(o * D + src) * inner + i];
  }
}

// ------------------------------------------------------------------ index_put: self[o, idx[j], i] (+)= val[o, j, i]
template <typename T> __device__ __forceinline__ void atomic_add_any(T* p, T v) { atomicAdd(p, v); }
template <> __device__ __forceinline__ void atomic_add_any<int64_t>(int64_t* p, int64_t v) {
  atomicAdd(reinterpret_cast<unsigned long long*>(p), (unsigned long long)v);
}
template <> __device__ __forceinline__ void atomic_add_any<int16_t>(int16_t* p, int16_t v) {
  unsigned short* a = reinterpret_cast<unsigned short*>(p);
  unsigned short old = *a, assumed;
  do { assumed = old; old = atomicCAS(a, assumed, (unsigned short)((int16_t)assumed + v)); } while (old != assumed);
}
template <> __device__ __forceinline__ void atomic_add_any<uint8_t>(uint8_t* p, uint8_t v) {
  unsigned int* base = reinterpret_cast<unsigned int*>(reinterpret_cast<uintptr_t>(p) & ~(uintptr_t)3);
  const unsigned shift = (unsigned)((reinterpret_cast<uintptr_t>(p) & 3) * 8);
  unsigned int old = *base, assumed;
  do {
    assumed = old;
    const unsigned int byte = ((assumed >> shift) + v) & 0xffu;
    old = atomicCAS(base, assumed, (assumed & ~(0xffu << shift)) | (byte << shift));
  } while (old != assumed);
}
template <> __device__ __forceinline__ void atomic_add_any<int8_t>(int8_t* p, int8_t v) {
  atomic_add_any<uint8_t>(reinterpret_cast<uint8_t*>(p), (uint8_t)v);
}

template <typename T, typename I, bool ACC>
__global__ void __launch_bounds__(kIdxThreads) index_put_kernel(T* __restrict__ self, const T* __restrict__ val,
                                                                const I* __restrict__ idx, int64_t outer, int64_t D,
                                                                int64_t inner, int64_t J, int64_t val_stride_j,
                                                                int64_t val_stride_o, int* status) {
  const int64_t total = outer * J * inner;
  for (int64_t t = (int64_t)blockIdx.x * kIdxThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kIdxThreads) {
    const int64_t i = t % inner, j = (t / inner) % J, o = t / (inner * J);
    const int64_t dst = wrap_index(idx[j], D, status);
    const T v = val[o * val_stride_o + j * val_stride_j + i];
    T* p = self + (o * D + dst) * inner + i;
    if constexpr (ACC) atomic_add_any<T>(p, v);
    else *p = v;
  }
}

// ------------------------------------------------------------------ gather / scatter along a dimension
// index [outer, J, inner]; the other tensor [outer, D, inner]
template <typename U, typename I>
__global__ void __launch_bounds__(kIdxThreads) gather_kernel(U* __restrict__ out, const U* __restrict__ in,
                                                             const I* __restrict__ idx, int64_t outer, int64_t D,
                                                             int64_t inner, int64_t J, int* status) {
  const int64_t total = outer * J * inner;
  for (int64_t t = (int64_t)blockIdx.x * kIdxThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kIdxThreads) {
    const int64_t i = t % inner, o = t / (inner * J);
    const int64_t src = wrap_index(idx[t], D, status);
    out[t] = in[(o * D + src) * inner + i];
  }
}
template <typename T, typename I, int MODE>   // 0 assign from src, 1 add from src, 2 assign scalar
__global__ void __launch_bounds__(kIdxThreads) scatter_kernel(T* __restrict__ self, const T* __restrict__ src, T value,
                                                              const I* __restrict__ idx, int64_t outer, int64_t D,
                                                              int64_t inner, int64_t J, int* status) {
  const int64_t total = outer * J * inner;
  for (int64_t t = (int64_t)blockIdx.x * kIdxThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kIdxThreads) {
    const int64_t i = t % inner, o = t / (inner * J);
    const int64_t dst = wrap_index(idx[t], D, status);
    T* p = self + (o * D + dst) * inner + i;
    if constexpr (MODE == 1) atomic_add_any<T>(p, src[t]);
    else if constexpr (MODE == 0) *p = src[t];
    else *p = value;
  }
}

// ------------------------------------------------------------------ triangular masks, arange
template <typename U>
__global__ void __launch_bounds__(kIdxThreads) tri_kernel(U* __restrict__ out, const U* __restrict__ in, int64_t batch,
                                                          int64_t rows, int64_t cols, int64_t diagonal, int upper) {
  const int64_t total = batch * rows * cols;
  for (int64_t t = (int64_t)blockIdx.x * kIdxThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kIdxThreads) {
    const int64_t c = t % cols, r = (t / cols) % rows;
    const bool keep = upper ? (c - r >= diagonal) : (c - r <= diagonal);
    U z;
    memset(&z, 0, sizeof(U));
    out[t] = keep ? in[t] : z;
  }
}
template <typename T>
__global__ void __launch_bounds__(kIdxThreads) arange_kernel(T* __restrict__ out, double start, double step, int64_t n) {
  for (int64_t t = (int64_t)blockIdx.x * kIdxThreads + threadIdx.x; t < n; t += (int64_t)gridDim.x * kIdxThreads)
    out[t] = ToF<T>::from((float)(start + step * (double)t));
}
template <> __global__ void __launch_bounds__(kIdxThreads) arange_kernel<double>(double* __restrict__ out, double start, double step, int64_t n) {
  for (int64_t t = (int64_t)blockIdx.x * kIdxThreads + threadIdx.x; t < n; t += (int64_t)gridDim.x * kIdxThreads)
    out[t] = start + step * (double)t;
}
template <typename T>
__global__ void __launch_bounds__(kIdxThreads) arange_int_kernel(T* __restrict__ out, int64_t start, int64_t step, int64_t n) {
  for (int64_t t = (int64_t)blockIdx.x * kIdxThreads + threadIdx.x; t < n; t += (int64_t)gridDim.x * kIdxThreads)
    out[t] = (T)(start + step * t);
}

// ------------------------------------------------------------------ inclusive cumulative sum along rows
template <typename T, typename A>
__global__ void __launch_bounds__(kIdxThreads) cumsum_rows_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t rows,
                                                                  int64_t cols) {
  using Scan = cub::BlockScan<A, kIdxThreads>;
  __shared__ typename Scan::TempStorage tmp;
  __shared__ A carry_sh;
  constexpr int PER = 4;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    A carry = (A)0;
    for (int64_t c0 = 0; c0 < cols; c0 += (int64_t)kIdxThreads * PER) {
      A v[PER];
#pragma unroll
      for (int k = 0; k < PER; ++k) {
        const int64_t c = c0 + (int64_t)threadIdx.x * PER + k;
        v[k] = c < cols ? (A)ToAcc<T, A>::get(in[row * cols + c]) : (A)0;
      }
      A total;
      Scan(tmp).InclusiveSum(v, v, total);
#pragma unroll
      for (int k = 0; k < PER; ++k) {
        const int64_t c = c0 + (int64_t)threadIdx.x * PER + k;
        if (c < cols) out[row * cols + c] = ToAcc<T, A>::put(v[k] + carry);
      }
      __syncthreads();
      if (threadIdx.x == 0) carry_sh = carry + total;
      __syncthreads();
      carry = carry_sh;
    }
  }
}

// ------------------------------------------------------------------ top-k of short rows: one thread per row
template <typename T, int KMAX>
__global__ void __launch_bounds__(128) topk_small_kernel(T* __restrict__ vals, int64_t* __restrict__ idxs,
                                                         const T* __restrict__ in, int64_t rows, int cols, int k,
                                                         int largest) {
  const int64_t row = (int64_t)blockIdx.x * 128 + threadIdx.x;
  if (row >= rows) return;
  float best[KMAX];
  int where[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) { best[j] = largest ? -INFINITY : INFINITY; where[j] = -1; }
  const T* src = in + row * cols;
  for (int c = 0; c < cols; ++c) {
    float v = ToF<T>::to(src[c]);
    const bool vnan = v != v;
    // insertion into the sorted list of the k best; NaN counts as the largest value, earlier positions win ties
    int pos = k;
#pragma unroll
    for (int j = KMAX - 1; j >= 0; --j) {
      if (j < k) {
        const float b = best[j];
        const bool bnan = b != b;
        bool better;
        if (where[j] < 0) better = true;
        else if (largest) better = (vnan && !bnan) || (!vnan && !bnan && v > b);
        else better = (!vnan && bnan) || (!vnan && !bnan && v < b);
        if (better) pos = j;
      }
    }
    if (pos < k) {
#pragma unroll
      for (int j = KMAX - 1; j > 0; --j)
        if (j > pos && j < k) { best[j] = best[j - 1]; where[j] = where[j - 1]; }
#pragma unroll
      for (int j = 0; j < KMAX; ++j)
        if (j == pos) { best[j] = v; where[j] = c; }
    }
  }
  for (int j = 0; j < k; ++j) {
    vals[row * k + j] = src[where[j] < 0 ? 0 : where[j]];
    idxs[row * k + j] = where[j] < 0 ? 0 : where[j];
  }
}

__global__ void iota_rows_kernel(int64_t* __restrict__ out, int64_t rows, int64_t cols) {
  const int64_t total = rows * cols;
  for (int64_t t = (int64_t)blockIdx.x * kIdxThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kIdxThreads)
    out[t] = t % cols;
}
__global__ void segment_offsets_kernel(int64_t* __restrict__ off, int64_t rows, int64_t cols) {
  const int64_t t = (int64_t)blockIdx.x * kIdxThreads + threadIdx.x;
  if (t <= rows) off[t] = t * cols;
}

template <typename K>
int sort_rows_impl(void* temp, size_t* temp_bytes, const K* keys_in, K* keys_out, const int64_t* vals_in, int64_t* vals_out,
                   int64_t rows, int64_t cols, int descending, const int64_t* offsets, cudaStream_t stream) {
  if (rows * cols > 2147483647ll) return (int)cudaErrorNotSupported;
  cudaError_t e;
  if (rows == 1) {
    e = descending ? cub::DeviceRadixSort::SortPairsDescending(temp, *temp_bytes, keys_in, keys_out, vals_in, vals_out, (int)cols, 0, (int)sizeof(K) * 8, stream)
                   : cub::DeviceRadixSort::SortPairs(temp, *temp_bytes, keys_in, keys_out, vals_in, vals_out, (int)cols, 0, (int)sizeof(K) * 8, stream);
  } else {
    e = descending ? cub::DeviceSegmentedRadixSort::SortPairsDescending(temp, *temp_bytes, keys_in, keys_out, vals_in, vals_out, (int)(rows * cols), (int)rows, offsets, offsets + 1, 0, (int)sizeof(K) * 8, stream)
                   : cub::DeviceSegmentedRadixSort::SortPairs(temp, *temp_bytes, keys_in, keys_out, vals_in, vals_out, (int)(rows * cols), (int)rows, offsets, offsets + 1, 0, (int)sizeof(K) * 8, stream);
  }
  return (int)e;
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

#define IDX_DISPATCH(IDT, I, ...)                                     \
  if (IDT == B200_I64) { using I = int64_t; __VA_ARGS__; }            \
  else if (IDT == B200_I32) { using I = int32_t; __VA_ARGS__; }       \
  else return (int)cudaErrorNotSupported;

#define UNIT_DISPATCH(BYTES, U, ...)                                  \
  switch (BYTES) {                                                    \
    case 1: { using U = uint8_t; __VA_ARGS__; break; }                \
    case 2: { using U = uint16_t; __VA_ARGS__; break; }               \
    case 4: { using U = uint32_t; __VA_ARGS__; break; }               \
    case 8: { using U = uint64_t; __VA_ARGS__; break; }               \
    case 16: { using U = uint4; __VA_ARGS__; break; }                 \
    default: return (int)cudaErrorNotSupported;                       \
  }

// widest unit (bytes) that divides a row of `inner` elements of `eb` bytes and both base addresses
static int widest_unit(int64_t inner, int eb, const void* a, const void* b) {
  const int64_t row = inner * eb;
  const uintptr_t m = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | (uintptr_t)row;
  int u = eb;
  while (u < 16 && (m % (uintptr_t)(u * 2)) == 0) u *= 2;
  return u;
}

int b200_index_select(void* out, const void* in, const void* idx, int idx_dtype, int elem_bytes, int64_t outer, int64_t D,
                      int64_t inner, int64_t J, int* status, cudaStream_t stream) {
  if (outer * J * inner == 0) return 0;
  const int unit = widest_unit(inner, elem_bytes, out, in);
  const int64_t inner_u = inner * elem_bytes / unit;
  IDX_DISPATCH(idx_dtype, I, UNIT_DISPATCH(unit, U,
      (index_select_kernel<U, I><<<blocks_for(outer * J * inner_u), kIdxThreads, 0, stream>>>(
          (U*)out, (const U*)in, (const I*)idx, outer, D, inner_u, J, status))));
  B200K_LAUNCH_RET();
}

int b200_gather(void* out, const void* in, const void* idx, int idx_dtype, int elem_bytes, int64_t outer, int64_t D,
                int64_t inner, int64_t J, int* status, cudaStream_t stream) {
  if (outer * J * inner == 0) return 0;
  IDX_DISPATCH(idx_dtype, I, UNIT_DISPATCH(elem_bytes, U,
      (gather_kernel<U, I><<<blocks_for(outer * J * inner), kIdxThreads, 0, stream>>>(
          (U*)out, (const U*)in, (const I*)idx, outer, D, inner, J, status))));
  B200K_LAUNCH_RET();
}

#define VAL_DISPATCH(DT, T, ...)                                      \
  switch (DT) {                                                       \
    case B200_F32: { using T = float; __VA_ARGS__; break; }           \
    case B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }  \
    case B200_F16: { using T = __half; __VA_ARGS__; break; }          \
    case B200_F64: { using T = double; __VA_ARGS__; break; }          \
    case B200_I32: { using T = int32_t; __VA_ARGS__; break; }         \
    case B200_I64: { using T = int64_t; __VA_ARGS__; break; }         \
    case B200_I16: { using T = int16_t; __VA_ARGS__; break; }         \
    case B200_I8: { using T = int8_t; __VA_ARGS__; break; }           \
    case B200_U8: case B200_BOOL: { using T = uint8_t; __VA_ARGS__; break; } \
    default: return (int)cudaErrorNotSupported;                       \
  }

int b200_index_put(void* self, const void* val, const void* idx, int idx_dtype, int dtype, int accumulate, int64_t outer,
                   int64_t D, int64_t inner, int64_t J, int64_t val_stride_j, int64_t val_stride_o, int* status,
                   cudaStream_t stream) {
  if (outer * J * inner == 0) return 0;
  const unsigned grid = blocks_for(outer * J * inner);
  IDX_DISPATCH(idx_dtype, I, VAL_DISPATCH(dtype, T, {
    if (accumulate)
      index_put_kernel<T, I, true><<<grid, kIdxThreads, 0, stream>>>((T*)self, (const T*)val, (const I*)idx, outer, D, inner, J, val_stride_j, val_stride_o, status);
    else
      index_put_kernel<T, I, false><<<grid, kIdxThreads, 0, stream>>>((T*)self, (const T*)val, (const I*)idx, outer, D, inner, J, val_stride_j, val_stride_o, status);
  }));
  B200K_LAUNCH_RET();
}

int b200_scatter(void* self, const void* src, double value, const void* idx, int idx_dtype, int dtype, int mode,
                 int64_t outer, int64_t D, int64_t inner, int64_t J, int* status, cudaStream_t stream) {
  if (outer * J * inner == 0) return 0;
  const unsigned grid = blocks_for(outer * J * inner);
  IDX_DISPATCH(idx_dtype, I, VAL_DISPATCH(dtype, T, {
    const T v = from_double<T>(value);
    if (mode == 0) scatter_kernel<T, I, 0><<<grid, kIdxThreads, 0, stream>>>((T*)self, (const T*)src, v, (const I*)idx, outer, D, inner, J, status);
    else if (mode == 1) scatter_kernel<T, I, 1><<<grid, kIdxThreads, 0, stream>>>((T*)self, (const T*)src, v, (const I*)idx, outer, D, inner, J, status);
    else scatter_kernel<T, I, 2><<<grid, kIdxThreads, 0, stream>>>((T*)self, (const T*)src, v, (const I*)idx, outer, D, inner, J, status);
  }));
  B200K_LAUNCH_RET();
}

int b200_tri(void* out, const void* in, int elem_bytes, int64_t batch, int64_t rows, int64_t cols, int64_t diagonal, int upper,
             cudaStream_t stream) {
  if (batch * rows * cols == 0) return 0;
  UNIT_DISPATCH(elem_bytes, U, (tri_kernel<U><<<blocks_for(batch * rows * cols), kIdxThreads, 0, stream>>>(
      (U*)out, (const U*)in, batch, rows, cols, diagonal, upper)));
  B200K_LAUNCH_RET();
}

int b200_arange(void* out, int dtype, double start, double step, int64_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  const unsigned grid = blocks_for(n);
  switch (dtype) {
    case B200_F32: arange_kernel<float><<<grid, kIdxThreads, 0, stream>>>((float*)out, start, step, n); break;
    case B200_BF16: arange_kernel<__nv_bfloat16><<<grid, kIdxThreads, 0, stream>>>((__nv_bfloat16*)out, start, step, n); break;
    case B200_F16: arange_kernel<__half><<<grid, kIdxThreads, 0, stream>>>((__half*)out, start, step, n); break;
    case B200_F64: arange_kernel<double><<<grid, kIdxThreads, 0, stream>>>((double*)out, start, step, n); break;
    case B200_I64: arange_int_kernel<int64_t><<<grid, kIdxThreads, 0, stream>>>((int64_t*)out, (int64_t)start, (int64_t)step, n); break;
    case B200_I32: arange_int_kernel<int32_t><<<grid, kIdxThreads, 0, stream>>>((int32_t*)out, (int64_t)start, (int64_t)step, n); break;
    case B200_I16: arange_int_kernel<int16_t><<<grid, kIdxThreads, 0, stream>>>((int16_t*)out, (int64_t)start, (int64_t)step, n); break;
    case B200_I8: arange_int_kernel<int8_t><<<grid, kIdxThreads, 0, stream>>>((int8_t*)out, (int64_t)start, (int64_t)step, n); break;
    case B200_U8: arange_int_kernel<uint8_t><<<grid, kIdxThreads, 0, stream>>>((uint8_t*)out, (int64_t)start, (int64_t)step, n); break;
    default: return (int)cudaErrorNotSupported;
  }
  B200K_LAUNCH_RET();
}

int b200_cumsum_rows(void* out, const void* in, int dtype, int64_t rows, int64_t cols, cudaStream_t stream) {
  if (rows * cols == 0) return 0;
  const unsigned grid = (unsigned)std::min<int64_t>(rows, (int64_t)kSMs * 8);
  switch (dtype) {
    case B200_F32: cumsum_rows_kernel<float, float><<<grid, kIdxThreads, 0, stream>>>((float*)out, (const float*)in, rows, cols); break;
    case B200_BF16: cumsum_rows_kernel<__nv_bfloat16, float><<<grid, kIdxThreads, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)in, rows, cols); break;
    case B200_F16: cumsum_rows_kernel<__half, float><<<grid, kIdxThreads, 0, stream>>>((__half*)out, (const __half*)in, rows, cols); break;
    case B200_F64: cumsum_rows_kernel<double, double><<<grid, kIdxThreads, 0, stream>>>((double*)out, (const double*)in, rows, cols); break;
    case B200_I64: cumsum_rows_kernel<int64_t, int64_t><<<grid, kIdxThreads, 0, stream>>>((int64_t*)out, (const int64_t*)in, rows, cols); break;
    case B200_I32: cumsum_rows_kernel<int32_t, int64_t><<<grid, kIdxThreads, 0, stream>>>((int32_t*)out, (const int32_t*)in, rows, cols); break;
    default: return (int)cudaErrorNotSupported;
  }
  B200K_LAUNCH_RET();
}

int b200_topk_small(void* vals, int64_t* idxs, const void* in, int dtype, int64_t rows, int cols, int k, int largest,
                    cudaStream_t stream) {
  if (rows == 0 || k == 0) return 0;
  if (k > 16 || cols > 1024 || k > cols) return (int)cudaErrorNotSupported;
  const unsigned grid = blocks_for(rows, 128);
#define TOPK(T)                                                                                                   \
  if (k <= 4) topk_small_kernel<T, 4><<<grid, 128, 0, stream>>>((T*)vals, idxs, (const T*)in, rows, cols, k, largest); \
  else if (k <= 8) topk_small_kernel<T, 8><<<grid, 128, 0, stream>>>((T*)vals, idxs, (const T*)in, rows, cols, k, largest); \
  else topk_small_kernel<T, 16><<<grid, 128, 0, stream>>>((T*)vals, idxs, (const T*)in, rows, cols, k, largest);
  switch (dtype) {
    case B200_F32: TOPK(float) break;
    case B200_BF16: TOPK(__nv_bfloat16) break;
    case B200_F16: TOPK(__half) break;
    default: return (int)cudaErrorNotSupported;
  }
#undef TOPK
  B200K_LAUNCH_RET();
}

/* Sorts every row of keys_in [rows, cols] (stable); vals_out receives the original column of every sorted key.
 * scratch layout is private: call with temp == NULL to get the required size in *temp_bytes. */
int b200_sort_rows(void* temp, size_t* temp_bytes, const void* keys_in, void* keys_out, int64_t* vals_out, int dtype,
                   int64_t rows, int64_t cols, int descending, cudaStream_t stream) {
  if (rows * cols == 0) { if (!temp) *temp_bytes = 16; return 0; }
  // private scratch: [iota rows*cols int64][offsets rows+1 int64][cub temp]
  const size_t iota_bytes = ((size_t)(rows * cols) * 8 + 255) / 256 * 256;
  const size_t off_bytes = ((size_t)(rows + 1) * 8 + 255) / 256 * 256;
  int64_t* iota = temp ? static_cast<int64_t*>(temp) : nullptr;
  int64_t* offs = temp ? reinterpret_cast<int64_t*>(static_cast<char*>(temp) + iota_bytes) : nullptr;
  void* cub_temp = temp ? static_cast<char*>(temp) + iota_bytes + off_bytes : nullptr;
  size_t cub_bytes = temp ? (*temp_bytes - iota_bytes - off_bytes) : 0;
  if (temp) {
    iota_rows_kernel<<<blocks_for(rows * cols), kIdxThreads, 0, stream>>>(iota, rows, cols);
    segment_offsets_kernel<<<blocks_for(rows + 1), kIdxThreads, 0, stream>>>(offs, rows, cols);
    note_launch(2);
  }
  int e;
  switch (dtype) {
    case B200_F32: e = sort_rows_impl<float>(cub_temp, &cub_bytes, (const float*)keys_in, (float*)keys_out, iota, vals_out, rows, cols, descending, offs, stream); break;
    case B200_BF16: e = sort_rows_impl<__nv_bfloat16>(cub_temp, &cub_bytes, (const __nv_bfloat16*)keys_in, (__nv_bfloat16*)keys_out, iota, vals_out, rows, cols, descending, offs, stream); break;
    case B200_F16: e = sort_rows_impl<__half>(cub_temp, &cub_bytes, (const __half*)keys_in, (__half*)keys_out, iota, vals_out, rows, cols, descending, offs, stream); break;
    case B200_F64: e = sort_rows_impl<double>(cub_temp, &cub_bytes, (const double*)keys_in, (double*)keys_out, iota, vals_out, rows, cols, descending, offs, stream); break;
    case B200_I64: e = sort_rows_impl<int64_t>(cub_temp, &cub_bytes, (const int64_t*)keys_in, (int64_t*)keys_out, iota, vals_out, rows, cols, descending, offs, stream); break;
    case B200_I32: e = sort_rows_impl<int32_t>(cub_temp, &cub_bytes, (const int32_t*)keys_in, (int32_t*)keys_out, iota, vals_out, rows, cols, descending, offs, stream); break;
    case B200_I16: e = sort_rows_impl<int16_t>(cub_temp, &cub_bytes, (const int16_t*)keys_in, (int16_t*)keys_out, iota, vals_out, rows, cols, descending, offs, stream); break;
    case B200_U8: e = sort_rows_impl<uint8_t>(cub_temp, &cub_bytes, (const uint8_t*)keys_in, (uint8_t*)keys_out, iota, vals_out, rows, cols, descending, offs, stream); break;
    case B200_I8: e = sort_rows_impl<int8_t>(cub_temp, &cub_bytes, (const int8_t*)keys_in, (int8_t*)keys_out, iota, vals_out, rows, cols, descending, offs, stream); break;
    default: return (int)cudaErrorNotSupported;
  }
  if (!temp) {
    *temp_bytes = iota_bytes + off_bytes + cub_bytes + 256;
    return e;
  }
  if (e != 0) return e;
  B200K_LAUNCH_RET();
}

}  // extern "C"
