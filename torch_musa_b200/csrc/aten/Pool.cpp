// max_pool2d_with_indices / avg_pool2d forward and backward on the pooling kernels (kernels/pool.cu) for floating
// activations in channels-last or contiguous NCHW layout.  ceil_mode and 3-D inputs keep the library route.
// Parity: reference torch_musa/csrc/aten/ops/Pool.cpp.
#include "aten/FallbackCall.h"
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {

int64_t pair_at(at::IntArrayRef v, int i, int64_t dflt) {
  if (v.empty()) return dflt;
  return v.size() == 1 ? v[0] : v[i];
}

struct PoolPlan {
  bool ok = false;
  bool nhwc = false;
  b200_pool_t g{};
  int64_t N = 0, C = 0;
};

PoolPlan plan(const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef stride, at::IntArrayRef padding,
              at::IntArrayRef dilation, bool ceil_mode) {
  PoolPlan p;
  if (!on_device(self) || self.dim() != 4 || kdtype(self.scalar_type()) < 0 || ceil_mode || self.numel() == 0) return p;
  const bool cl = self.is_contiguous(at::MemoryFormat::ChannelsLast) && !self.is_contiguous();
  if (!cl && !self.is_contiguous()) return p;
  const int64_t N = self.size(0), C = self.size(1), H = self.size(2), W = self.size(3);
  b200_pool_t& g = p.g;
  g.kh = (int)pair_at(kernel, 0, 1); g.kw = (int)pair_at(kernel, 1, 1);
  g.sh = (int)pair_at(stride, 0, g.kh); g.sw = (int)pair_at(stride, 1, g.kw);
  g.ph = (int)pair_at(padding, 0, 0); g.pw = (int)pair_at(padding, 1, 0);
  g.dh = (int)pair_at(dilation, 0, 1); g.dw = (int)pair_at(dilation, 1, 1);
  if (g.sh <= 0 || g.sw <= 0 || g.ph * 2 > g.kh || g.pw * 2 > g.kw) return p;
  g.H = H; g.W = W;
  g.Ho = (H + 2 * g.ph - g.dh * (g.kh - 1) - 1) / g.sh + 1;
  g.Wo = (W + 2 * g.pw - g.dw * (g.kw - 1) - 1) / g.sw + 1;
  if (g.Ho <= 0 || g.Wo <= 0) return p;
  p.nhwc = cl;
  g.N = cl ? N : N * C;
  g.C = cl ? C : 1;
  p.N = N; p.C = C;
  p.ok = true;
  return p;
}

at::Tensor out_like(const at::Tensor& self, const PoolPlan& p, int64_t Ho, int64_t Wo, at::ScalarType dt) {
  return at::empty({p.N, p.C, Ho, Wo}, self.options().dtype(dt),
                   p.nhwc ? at::MemoryFormat::ChannelsLast : at::MemoryFormat::Contiguous);
}

std::tuple<at::Tensor, at::Tensor> max_pool2d_with_indices(const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef stride,
                                                           at::IntArrayRef padding, at::IntArrayRef dilation, bool ceil_mode) {
  PoolPlan p = plan(self, kernel, stride, padding, dilation, ceil_mode);
  if (p.ok) {
    at::Tensor out = out_like(self, p, p.g.Ho, p.g.Wo, self.scalar_type());
    at::Tensor idx = out_like(self, p, p.g.Ho, p.g.Wo, at::kLong);
    DeviceSwitch sw(self.device().index());
    int e = b200_maxpool2d_fwd(&p.g, kdtype(self.scalar_type()), out.mutable_data_ptr(), idx.data_ptr<int64_t>(),
                               self.const_data_ptr(), current_raw_stream(self));
    if (e == 0) return {out, idx};
    if (e != (int)cudaErrorNotSupported) B200_KERNEL_CALL(e);
  }
  auto st = run_fallback(B200_OP_HANDLE("aten::max_pool2d_with_indices", ""), self, kernel, stride, padding, dilation, ceil_mode);
  return {st[0].toTensor(), st[1].toTensor()};
}

at::Tensor max_pool2d_with_indices_backward(const at::Tensor& grad, const at::Tensor& self, at::IntArrayRef kernel,
                                            at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                                            bool ceil_mode, const at::Tensor& indices) {
  PoolPlan p = plan(self, kernel, stride, padding, dilation, ceil_mode);
  if (p.ok && on_device(grad) && grad.scalar_type() == self.scalar_type() && on_device(indices) &&
      indices.scalar_type() == at::kLong) {
    const auto fmt = p.nhwc ? at::MemoryFormat::ChannelsLast : at::MemoryFormat::Contiguous;
    at::Tensor g = grad.contiguous(fmt), idx = indices.contiguous(fmt);
    at::Tensor gin = at::empty(self.sizes(), self.options(), fmt);
    DeviceSwitch sw(self.device().index());
    int e = b200_maxpool2d_bwd(&p.g, kdtype(self.scalar_type()), gin.mutable_data_ptr(), g.const_data_ptr(),
                               idx.data_ptr<int64_t>(), current_raw_stream(self));
    if (e == 0) return gin;
    if (e != (int)cudaErrorNotSupported) B200_KERNEL_CALL(e);
  }
  return fallback_tensor(B200_OP_HANDLE("aten::max_pool2d_with_indices_backward", ""), grad, self, kernel, stride, padding,
                         dilation, ceil_mode, indices);
}

int divisor_mode(bool count_include_pad, const std::optional<int64_t>& override_) {
  if (override_.has_value()) return (int)*override_;
  return count_include_pad ? 0 : -1;
}

at::Tensor avg_pool2d(const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef stride, at::IntArrayRef padding,
                      bool ceil_mode, bool count_include_pad, std::optional<int64_t> divisor_override) {
  PoolPlan p = plan(self, kernel, stride, padding, {}, ceil_mode);
  if (p.ok && (!divisor_override || *divisor_override > 0)) {
    at::Tensor out = out_like(self, p, p.g.Ho, p.g.Wo, self.scalar_type());
    DeviceSwitch sw(self.device().index());
    int e = b200_avgpool2d_fwd(&p.g, kdtype(self.scalar_type()), out.mutable_data_ptr(), self.const_data_ptr(),
                               divisor_mode(count_include_pad, divisor_override), current_raw_stream(self));
    if (e == 0) return out;
    if (e != (int)cudaErrorNotSupported) B200_KERNEL_CALL(e);
  }
  return fallback_tensor(B200_OP_HANDLE("aten::avg_pool2d", ""), self, kernel, stride, padding, ceil_mode, count_include_pad,
                         divisor_override);
}

at::Tensor avg_pool2d_backward(const at::Tensor& grad, const at::Tensor& self, at::IntArrayRef kernel, at::IntArrayRef stride,
                               at::IntArrayRef padding, bool ceil_mode, bool count_include_pad,
                               std::optional<int64_t> divisor_override) {
  PoolPlan p = plan(self, kernel, stride, padding, {}, ceil_mode);
  if (p.ok && on_device(grad) && grad.scalar_type() == self.scalar_type() && (!divisor_override || *divisor_override > 0)) {
    const auto fmt = p.nhwc ? at::MemoryFormat::ChannelsLast : at::MemoryFormat::Contiguous;
    at::Tensor g = grad.contiguous(fmt);
    at::Tensor gin = at::empty(self.sizes(), self.options(), fmt);
    DeviceSwitch sw(self.device().index());
    int e = b200_avgpool2d_bwd(&p.g, kdtype(self.scalar_type()), gin.mutable_data_ptr(), g.const_data_ptr(),
                               divisor_mode(count_include_pad, divisor_override), current_raw_stream(self));
    if (e == 0) return gin;
    if (e != (int)cudaErrorNotSupported) B200_KERNEL_CALL(e);
  }
  return fallback_tensor(B200_OP_HANDLE("aten::avg_pool2d_backward", ""), grad, self, kernel, stride, padding, ceil_mode,
                         count_include_pad, divisor_override);
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("max_pool2d_with_indices", TORCH_FN(max_pool2d_with_indices));
  m.impl("max_pool2d_with_indices_backward", TORCH_FN(max_pool2d_with_indices_backward));
  m.impl("avg_pool2d", TORCH_FN(avg_pool2d));
  m.impl("avg_pool2d_backward", TORCH_FN(avg_pool2d_backward));
}

}  // namespace
}  // namespace ops
}  // namespace b200
