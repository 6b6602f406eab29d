// Convolution for the blackwell device.
//
// ATen sends every convolution on a PrivateUse1 tensor to `convolution_overrideable` /
// `convolution_backward_overrideable`.  Two routes:
//   * pointwise (1x1, stride 1, no padding, groups 1) convolutions on channels-last bf16/fp16 tensors are
//     plain matrix products over the [N*H*W, C] view of the activation: forward, data-gradient and
//     weight-gradient each run as ONE launch of the tcgen05 GEMM with no copy or transpose (the GEMM takes
//     K-major and MN-major operands straight from the strides).  That is 36 of ResNet-50's 53 convolutions.
//   * everything else runs the library convolution on the same memory through the CUDA-alias bridge.
// Parity: reference torch_musa/csrc/aten/ops/Convolution.cpp (vendor-library convolution fwd/dgrad/wgrad).
#include "aten/FallbackCall.h"
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <torch/library.h>

#include <atomic>

namespace b200 {
namespace ops {

namespace {

std::atomic<bool> g_pointwise_gemm{true};
std::atomic<int64_t> g_pointwise_hits{0};

bool all_eq(at::IntArrayRef v, int64_t x) {
  for (auto e : v)
    if (e != x) return false;
  return true;
}

// [N, C, H, W] with channels-last strides -> [N*H*W, C] view (no copy), or an undefined tensor.
at::Tensor nhwc_matrix(const at::Tensor& t) {
  if (t.dim() != 4) return {};
  const int64_t N = t.size(0), C = t.size(1), H = t.size(2), W = t.size(3);
  if (t.stride(1) != 1 && C != 1) return {};
  if (W > 1 && t.stride(3) != C) return {};
  if (H > 1 && t.stride(2) != W * C) return {};
  if (N > 1 && t.stride(0) != H * W * C) return {};
  return t.as_strided({N * H * W, C}, {C, 1});
}

bool pointwise_eligible(const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride,
                        at::IntArrayRef padding, at::IntArrayRef dilation, bool transposed, int64_t groups) {
  if (!g_pointwise_gemm.load(std::memory_order_relaxed)) return false;
  if (transposed || groups != 1 || input.dim() != 4 || weight.dim() != 4) return false;
  if (weight.size(2) != 1 || weight.size(3) != 1) return false;
  if (!all_eq(stride, 1) || !all_eq(padding, 0) || !all_eq(dilation, 1)) return false;
  const auto dt = input.scalar_type();
  if ((dt != at::kBFloat16 && dt != at::kHalf) || weight.scalar_type() != dt) return false;
  if (input.size(1) % 8 != 0 || weight.size(0) % 8 != 0 || input.numel() == 0) return false;
  // a [N, C, 1, 1] tensor is ambiguous between the two memory formats; both give the same matrix
  return nhwc_matrix(input).defined();
}

at::Tensor weight_matrix(const at::Tensor& weight) {  // [Cout, Cin, 1, 1] -> [Cout, Cin], any memory format
  return weight.reshape({weight.size(0), weight.size(1)});
}

at::Tensor nhwc_from_matrix(const at::Tensor& m, int64_t N, int64_t H, int64_t W) {
  const int64_t C = m.size(1);
  return m.as_strided({N, C, H, W}, {H * W * C, 1, W * C, C});
}

at::Tensor convolution_overrideable(const at::Tensor& input, const at::Tensor& weight,
                                    const std::optional<at::Tensor>& bias, at::IntArrayRef stride,
                                    at::IntArrayRef padding, at::IntArrayRef dilation, bool transposed,
                                    at::IntArrayRef output_padding, int64_t groups) {
  if (pointwise_eligible(input, weight, stride, padding, dilation, transposed, groups)) {
    g_pointwise_hits.fetch_add(1, std::memory_order_relaxed);
    const at::Tensor x = nhwc_matrix(input);
    const at::Tensor w = weight_matrix(weight);
    at::Tensor y = (bias.has_value() && bias->defined()) ? at::addmm(*bias, x, w.t()) : at::mm(x, w.t());
    return nhwc_from_matrix(y, input.size(0), input.size(2), input.size(3));
  }
  return fallback_tensor(B200_OP_HANDLE("aten::convolution", ""), input, weight, bias, stride, padding, dilation,
                         transposed, output_padding, groups);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> convolution_backward_overrideable(
    const at::Tensor& grad_output, const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride,
    at::IntArrayRef padding, at::IntArrayRef dilation, bool transposed, at::IntArrayRef output_padding,
    int64_t groups, std::array<bool, 3> output_mask) {
  if (pointwise_eligible(input, weight, stride, padding, dilation, transposed, groups) &&
      grad_output.scalar_type() == input.scalar_type()) {
    at::Tensor gy = nhwc_matrix(grad_output);
    if (!gy.defined()) gy = nhwc_matrix(grad_output.contiguous(at::MemoryFormat::ChannelsLast));
    const at::Tensor x = nhwc_matrix(input);
    const at::Tensor w = weight_matrix(weight);
    at::Tensor gx, gw, gb;
    if (output_mask[0]) gx = nhwc_from_matrix(at::mm(gy, w), input.size(0), input.size(2), input.size(3));
    if (output_mask[1]) {
      gw = at::mm(gy.t(), x).reshape(weight.sizes());
      if (weight.is_contiguous(at::MemoryFormat::ChannelsLast) && !weight.is_contiguous())
        gw = gw.contiguous(at::MemoryFormat::ChannelsLast);
    }
    if (output_mask[2]) gb = gy.sum(0);
    g_pointwise_hits.fetch_add(1, std::memory_order_relaxed);
    return {gx, gw, gb};
  }
  std::optional<std::vector<int64_t>> bias_sizes;
  if (output_mask[2]) bias_sizes = std::vector<int64_t>{weight.size(transposed ? 1 : 0) * (transposed ? groups : 1)};
  c10::List<bool> mask;
  mask.push_back(output_mask[0]);
  mask.push_back(output_mask[1]);
  mask.push_back(output_mask[2]);
  auto st = run_fallback(B200_OP_HANDLE("aten::convolution_backward", ""), grad_output, input, weight,
                         bias_sizes ? c10::IValue(*bias_sizes) : c10::IValue(), stride, padding, dilation, transposed,
                         output_padding, groups, mask);
  auto pick = [&](size_t i) { return st[i].isTensor() ? st[i].toTensor() : at::Tensor(); };
  return {pick(0), pick(1), pick(2)};
}

}  // namespace

void set_pointwise_conv_gemm(bool on) { g_pointwise_gemm.store(on); }
int64_t pointwise_conv_hits() { return g_pointwise_hits.load(); }

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("convolution_overrideable", TORCH_FN(convolution_overrideable));
  m.impl("convolution_backward_overrideable", TORCH_FN(convolution_backward_overrideable));
}

}  // namespace ops
}  // namespace b200
