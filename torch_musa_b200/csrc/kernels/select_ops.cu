// Selection kernels: searchsorted / bucketize (binary search per element), histc (shared-memory bins merged
// with atomics), nonzero (flag compaction + coordinate expansion) and the pieces of unique over sorted keys
// (run-length encoding, run ids for the inverse map).  CUB device primitives do the scans and compactions;
// every entry point follows the two-call convention for temporary storage (temp == NULL: size query).
// Parity: reference torch_musa/csrc/aten/ops/musa/{Bucketize,Unique,Histc}.mu and Nonzero.cpp.
#include "common.cuh"

#include <cub/cub.cuh>

namespace b200k {
namespace {

constexpr int kThreads = 256;
inline unsigned blocks_for(int64_t n) { return (unsigned)std::min<int64_t>(cdiv(std::max<int64_t>(n, 1), kThreads), 148 * 16); }

// boundaries: [rows_b, nb] (rows_b == 1: shared by every row); values: [rows, nv]
template <typename T, typename OutT>
__global__ void __launch_bounds__(kThreads) searchsorted_kernel(OutT* __restrict__ out, const T* __restrict__ bounds,
                                                                const T* __restrict__ vals,
                                                                const int64_t* __restrict__ sorter, int64_t rows,
                                                                int64_t nv, int64_t nb, int shared_bounds, int right) {
  const int64_t total = rows * nv;
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kThreads) {
    const int64_t r = t / nv;
    const T* b = bounds + (shared_bounds ? 0 : r * nb);
    const int64_t* so = sorter ? sorter + (shared_bounds ? 0 : r * nb) : nullptr;
    const float v = ToF<T>::to(vals[t]);
    int64_t lo = 0, hi = nb;
    while (lo < hi) {
      const int64_t mid = lo + ((hi - lo) >> 1);
      const float m = ToF<T>::to(b[so ? so[mid] : mid]);
      const bool go_right = right ? !(v < m) : (m < v);   // right: first element > v; left: first element >= v
      if (go_right) lo = mid + 1; else hi = mid;
    }
    out[t] = (OutT)lo;
  }
}
template <typename OutT>
__global__ void __launch_bounds__(kThreads) searchsorted_i64_kernel(OutT* __restrict__ out, const int64_t* __restrict__ bounds,
                                                                    const int64_t* __restrict__ vals,
                                                                    const int64_t* __restrict__ sorter, int64_t rows,
                                                                    int64_t nv, int64_t nb, int shared_bounds, int right) {
  const int64_t total = rows * nv;
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kThreads) {
    const int64_t r = t / nv;
    const int64_t* b = bounds + (shared_bounds ? 0 : r * nb);
    const int64_t* so = sorter ? sorter + (shared_bounds ? 0 : r * nb) : nullptr;
    const int64_t v = vals[t];
    int64_t lo = 0, hi = nb;
    while (lo < hi) {
      const int64_t mid = lo + ((hi - lo) >> 1);
      const int64_t m = b[so ? so[mid] : mid];
      const bool go_right = right ? !(v < m) : (m < v);
      if (go_right) lo = mid + 1; else hi = mid;
    }
    out[t] = (OutT)lo;
  }
}

// counts[bins] (fp32) += histogram of x over [lo, hi]; values outside the range are ignored
template <typename T>
__global__ void __launch_bounds__(kThreads) histc_kernel(float* __restrict__ counts, const T* __restrict__ x, int64_t n,
                                                         int bins, float lo, float hi) {
  extern __shared__ unsigned int sh_bins[];
  const bool use_sh = bins <= 8192;
  if (use_sh) {
    for (int i = threadIdx.x; i < bins; i += kThreads) sh_bins[i] = 0;
    __syncthreads();
  }
  const float scale = (float)bins / (hi - lo);
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < n; t += (int64_t)gridDim.x * kThreads) {
    const float v = ToF<T>::to(x[t]);
    if (!(v >= lo && v <= hi)) continue;
    int b = (int)((v - lo) * scale);
    if (b >= bins) b = bins - 1;   // v == hi falls into the last bin
    if (use_sh) atomicAdd(&sh_bins[b], 1u); else atomicAdd(&counts[b], 1.f);
  }
  if (use_sh) {
    __syncthreads();
    for (int i = threadIdx.x; i < bins; i += kThreads)
      if (sh_bins[i]) atomicAdd(&counts[i], (float)sh_bins[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) nonzero_flags_kernel(unsigned char* __restrict__ flags, const T* __restrict__ x,
                                                                 int64_t n) {
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < n; t += (int64_t)gridDim.x * kThreads)
    flags[t] = x[t] != T(0) ? 1 : 0;
}
template <>
__global__ void __launch_bounds__(kThreads) nonzero_flags_kernel<__nv_bfloat16>(unsigned char* __restrict__ flags,
                                                                                const __nv_bfloat16* __restrict__ x, int64_t n) {
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < n; t += (int64_t)gridDim.x * kThreads)
    flags[t] = __bfloat162float(x[t]) != 0.f ? 1 : 0;
}
template <>
__global__ void __launch_bounds__(kThreads) nonzero_flags_kernel<__half>(unsigned char* __restrict__ flags,
                                                                        const __half* __restrict__ x, int64_t n) {
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < n; t += (int64_t)gridDim.x * kThreads)
    flags[t] = __half2float(x[t]) != 0.f ? 1 : 0;
}

struct Dims { int64_t size[8]; int nd; };
// linear[nnz] -> coords[nnz, nd] (row-major coordinates)
__global__ void __launch_bounds__(kThreads) unravel_kernel(int64_t* __restrict__ coords, const int64_t* __restrict__ linear,
                                                           const int64_t* __restrict__ count, Dims d) {
  const int64_t nnz = *count;
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < nnz; t += (int64_t)gridDim.x * kThreads) {
    int64_t r = linear[t];
    for (int k = d.nd - 1; k >= 0; --k) {
      coords[t * d.nd + k] = r % d.size[k];
      r /= d.size[k];
    }
  }
}

// run id of every element of a sorted key array (0 for the first run), scattered through perm: the inverse map
template <typename T>
__global__ void __launch_bounds__(kThreads) run_heads_kernel(int64_t* __restrict__ head, const T* __restrict__ keys, int64_t n) {
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < n; t += (int64_t)gridDim.x * kThreads)
    head[t] = (t > 0 && !(keys[t] == keys[t - 1])) ? 1 : 0;
}
__global__ void __launch_bounds__(kThreads) scatter_inverse_kernel(int64_t* __restrict__ inverse, const int64_t* __restrict__ run_id,
                                                                   const int64_t* __restrict__ perm, int64_t n) {
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < n; t += (int64_t)gridDim.x * kThreads)
    inverse[perm[t]] = run_id[t];
}

template <typename T>
int unique_sorted_impl(void* temp, size_t* temp_bytes, const T* keys, T* uniq, int64_t* counts, int64_t* num_runs,
                       int64_t* run_id, int64_t n, cudaStream_t stream) {
  size_t rle = 0, scan = 0;
  cudaError_t e = cub::DeviceRunLengthEncode::Encode(nullptr, rle, keys, uniq, counts, num_runs, (int)n, stream);
  if (e != cudaSuccess) return (int)e;
  e = cub::DeviceScan::InclusiveSum(nullptr, scan, run_id, run_id, (int)n, stream);
  if (e != cudaSuccess) return (int)e;
  const size_t need = std::max(rle, scan) + 256;
  if (!temp) { *temp_bytes = need; return 0; }
  if (*temp_bytes < need) return (int)cudaErrorInvalidValue;
  e = cub::DeviceRunLengthEncode::Encode(temp, rle, keys, uniq, counts, num_runs, (int)n, stream);
  if (e != cudaSuccess) return (int)e;
  if (run_id) {
    run_heads_kernel<T><<<blocks_for(n), kThreads, 0, stream>>>(run_id, keys, n);
    e = cub::DeviceScan::InclusiveSum(temp, scan, run_id, run_id, (int)n, stream);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cudaGetLastError();
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

int b200_searchsorted(void* out, int out_i32, const void* bounds, const void* vals, const int64_t* sorter, int dtype,
                      int64_t rows, int64_t nv, int64_t nb, int shared_bounds, int right, cudaStream_t stream) {
  const int64_t total = rows * nv;
  if (total == 0) return 0;
#define SS(T)                                                                                                          \
  do {                                                                                                                 \
    if (out_i32) searchsorted_kernel<T, int><<<blocks_for(total), kThreads, 0, stream>>>((int*)out, (const T*)bounds, (const T*)vals, sorter, rows, nv, nb, shared_bounds, right); \
    else searchsorted_kernel<T, int64_t><<<blocks_for(total), kThreads, 0, stream>>>((int64_t*)out, (const T*)bounds, (const T*)vals, sorter, rows, nv, nb, shared_bounds, right); \
  } while (0)
  switch (dtype) {
    case B200_F32: SS(float); break;
    case B200_BF16: SS(__nv_bfloat16); break;
    case B200_F16: SS(__half); break;
    case B200_I64:
      if (out_i32) searchsorted_i64_kernel<int><<<blocks_for(total), kThreads, 0, stream>>>((int*)out, (const int64_t*)bounds, (const int64_t*)vals, sorter, rows, nv, nb, shared_bounds, right);
      else searchsorted_i64_kernel<int64_t><<<blocks_for(total), kThreads, 0, stream>>>((int64_t*)out, (const int64_t*)bounds, (const int64_t*)vals, sorter, rows, nv, nb, shared_bounds, right);
      break;
    default: return (int)cudaErrorNotSupported;
  }
#undef SS
  B200K_LAUNCH_RET();
}

int b200_histc(float* counts, const void* x, int dtype, int64_t n, int bins, float lo, float hi, cudaStream_t stream) {
  if (n == 0 || bins <= 0) return 0;
  const size_t sh = bins <= 8192 ? (size_t)bins * sizeof(unsigned int) : 0;
  switch (dtype) {
    case B200_F32: histc_kernel<float><<<blocks_for(n), kThreads, sh, stream>>>(counts, (const float*)x, n, bins, lo, hi); break;
    case B200_BF16: histc_kernel<__nv_bfloat16><<<blocks_for(n), kThreads, sh, stream>>>(counts, (const __nv_bfloat16*)x, n, bins, lo, hi); break;
    case B200_F16: histc_kernel<__half><<<blocks_for(n), kThreads, sh, stream>>>(counts, (const __half*)x, n, bins, lo, hi); break;
    default: return (int)cudaErrorNotSupported;
  }
  B200K_LAUNCH_RET();
}

/* linear[n] (capacity), count[1]: indices of the non-zero elements of x in order.  temp == NULL: size query. */
int b200_nonzero_linear(void* temp, size_t* temp_bytes, int64_t* linear, int64_t* count, const void* x, int dtype, int64_t n,
                        cudaStream_t stream) {
  size_t cub_bytes = 0;
  cub::CountingInputIterator<int64_t> iota(0);
  cudaError_t e = cub::DeviceSelect::Flagged(nullptr, cub_bytes, iota, (unsigned char*)nullptr, linear, count, (int)n, stream);
  if (e != cudaSuccess) return (int)e;
  const size_t flag_bytes = ((size_t)n + 255) / 256 * 256;
  if (!temp) { *temp_bytes = flag_bytes + cub_bytes + 256; return 0; }
  if (n == 0) return (int)cudaMemsetAsync(count, 0, sizeof(int64_t), stream);
  unsigned char* flags = static_cast<unsigned char*>(temp);
  void* cub_temp = flags + flag_bytes;
  switch (dtype) {
    case B200_F32: nonzero_flags_kernel<float><<<blocks_for(n), kThreads, 0, stream>>>(flags, (const float*)x, n); break;
    case B200_BF16: nonzero_flags_kernel<__nv_bfloat16><<<blocks_for(n), kThreads, 0, stream>>>(flags, (const __nv_bfloat16*)x, n); break;
    case B200_F16: nonzero_flags_kernel<__half><<<blocks_for(n), kThreads, 0, stream>>>(flags, (const __half*)x, n); break;
    case B200_I64: nonzero_flags_kernel<int64_t><<<blocks_for(n), kThreads, 0, stream>>>(flags, (const int64_t*)x, n); break;
    case B200_I32: nonzero_flags_kernel<int><<<blocks_for(n), kThreads, 0, stream>>>(flags, (const int*)x, n); break;
    case B200_BOOL:
    case B200_U8: nonzero_flags_kernel<unsigned char><<<blocks_for(n), kThreads, 0, stream>>>(flags, (const unsigned char*)x, n); break;
    default: return (int)cudaErrorNotSupported;
  }
  e = cub::DeviceSelect::Flagged(cub_temp, cub_bytes, iota, flags, linear, count, (int)n, stream);
  return (int)e;
}

int b200_unravel(int64_t* coords, const int64_t* linear, const int64_t* count, int64_t capacity, const int64_t* sizes, int nd,
                 cudaStream_t stream) {
  if (capacity == 0 || nd == 0) return 0;
  if (nd > 8) return (int)cudaErrorNotSupported;
  Dims d;
  d.nd = nd;
  for (int i = 0; i < nd; ++i) d.size[i] = sizes[i];
  unravel_kernel<<<blocks_for(capacity), kThreads, 0, stream>>>(coords, linear, count, d);
  B200K_LAUNCH_RET();
}

/* keys sorted ascending: uniq[<=n], counts[<=n], num_runs[1]; run_id[n] (may be NULL) = index of each key's run */
int b200_unique_sorted(void* temp, size_t* temp_bytes, const void* keys, void* uniq, int64_t* counts, int64_t* num_runs,
                       int64_t* run_id, int dtype, int64_t n, cudaStream_t stream) {
  switch (dtype) {
    case B200_F32: return unique_sorted_impl<float>(temp, temp_bytes, (const float*)keys, (float*)uniq, counts, num_runs, run_id, n, stream);
    case B200_I64: return unique_sorted_impl<int64_t>(temp, temp_bytes, (const int64_t*)keys, (int64_t*)uniq, counts, num_runs, run_id, n, stream);
    case B200_I32: return unique_sorted_impl<int>(temp, temp_bytes, (const int*)keys, (int*)uniq, counts, num_runs, run_id, n, stream);
    default: return (int)cudaErrorNotSupported;
  }
}

int b200_scatter_inverse(int64_t* inverse, const int64_t* run_id, const int64_t* perm, int64_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  scatter_inverse_kernel<<<blocks_for(n), kThreads, 0, stream>>>(inverse, run_id, perm, n);
  B200K_LAUNCH_RET();
}

}  // extern "C"
