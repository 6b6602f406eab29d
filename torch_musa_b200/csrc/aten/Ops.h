// Shared declarations for the ATen operator layer.
#pragma once

#include "core/Device.h"
#include "core/Stream.h"
#include "kernels/b200_kernels.h"

#include <ATen/core/Tensor.h>

namespace b200 {
namespace ops {

inline bool on_device(const at::Tensor& t) { return t.defined() && t.device().type() == kDeviceType; }

// Every tensor argument whose pointer goes to a kernel must live on the device of the first one: a host pointer
// dereferenced on the GPU is a memory fault, not an exception.  Undefined / absent tensors are skipped.
inline void check_one_device(const char* op, const at::Tensor& ref, const at::Tensor& t) {
  TORCH_CHECK(!t.defined() || t.device() == ref.device(), "Expected all tensors to be on the same device, but found at "
              "least two devices, ", ref.device(), " and ", t.device(), "! (when checking arguments of ", op, ")");
}
inline void check_one_device(const char* op, const at::Tensor& ref, const std::optional<at::Tensor>& t) {
  if (t.has_value()) check_one_device(op, ref, *t);
}
template <class... Ts>
inline void check_devices(const char* op, const at::Tensor& ref, const Ts&... ts) {
  (check_one_device(op, ref, ts), ...);
}

// dtype code shared with the kernel library, or -1 if the kernels do not cover the type
inline int kdtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return B200_F32;
    case at::kBFloat16: return B200_BF16;
    case at::kHalf: return B200_F16;
    default: return -1;
  }
}

// Strided and/or dtype-converting same-device copy on our own kernels. Returns false when the
// configuration is not covered (caller then uses the generic route).
bool try_native_cast_copy(const at::Tensor& src, const at::Tensor& dst, cudaStream_t stream);

inline cudaStream_t current_raw_stream(const at::Tensor& t) { return get_current_stream(t.device().index()).stream(); }

// Kernels that take an epoch, a sequence number or an arena half as a launch argument must not be recorded into a
// graph: a replay would repeat the recorded value and skip the cross-rank ordering.
inline void check_not_capturing(cudaStream_t s, const char* what) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &st) != cudaSuccess) {
    (void)cudaGetLastError();
    return;
  }
  TORCH_CHECK(st == cudaStreamCaptureStatusNone, what, ": peer-memory kernels cannot be captured into a graph");
}

// Switch the tcgen05 GEMM off/on (off: every matmul goes to the library GEMM through the fallback).
B200_EXPORT void set_tensor_core_gemm(bool on);
B200_EXPORT bool tensor_core_gemm_enabled();

// Fused scaled-dot-product attention on/off (off: the math decomposition is always chosen).
B200_EXPORT void set_fused_sdp(bool on);
B200_EXPORT bool fused_sdp_enabled();
B200_EXPORT void set_sdp_impl(int impl);  // 0 library flash, 1 library cuDNN, 2 hand-written tcgen05 forward and backward (default)
B200_EXPORT int sdp_impl();
B200_EXPORT int64_t native_sdp_forward_calls();  // launches of the hand-written attention forward
B200_EXPORT int64_t native_sdp_backward_calls();

// 1x1 convolutions as GEMMs over the channels-last matrix view (off: every convolution uses the library route).
B200_EXPORT void set_pointwise_conv_gemm(bool on);
B200_EXPORT int64_t pointwise_conv_hits();
B200_EXPORT void set_implicit_conv_gemm(bool on);
B200_EXPORT int64_t implicit_conv_hits();

// Counter of hand-written kernel launches (reported by the benchmark as its own-kernel launch count).
B200_EXPORT void count_launch(int n = 1);
B200_EXPORT int64_t launch_count();
B200_EXPORT void reset_launch_count();

}  // namespace ops
}  // namespace b200
