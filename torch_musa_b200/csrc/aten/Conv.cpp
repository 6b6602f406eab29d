// Convolution for the blackwell device.
//
// ATen sends every convolution on a PrivateUse1 tensor to `convolution_overrideable` /
// `convolution_backward_overrideable`.  Two routes:
//   * pointwise (1x1, stride 1, no padding, groups 1) convolutions on channels-last bf16/fp16 tensors are
//     plain matrix products over the [N*H*W, C] view of the activation: forward, data-gradient and
//     weight-gradient each run as ONE launch of the tcgen05 GEMM with no copy or transpose (the GEMM takes
//     K-major and MN-major operands straight from the strides).  That is 36 of ResNet-50's 53 convolutions.
//   * every other 2-D convolution of 16-bit tensors with stride 1 or 2, no dilation and groups 1 (3x3, 7x7, strided
//     1x1 ...) runs the implicit-GEMM tcgen05 kernels of kernels/conv_tcgen05.cu: forward, data gradient and weight
//     gradient read the channels-last activation through shifted TMA boxes, no im2col buffer is built.  A filter
//     with fewer than 8 input channels (the RGB stem) is zero-padded to 8 channels first.
//   * what is left (dilation, groups, 1-D/3-D, fp32) runs the library convolution on the same memory through the
//     CUDA-alias bridge.
// Parity: reference torch_musa/csrc/aten/ops/Convolution.cpp (vendor-library convolution fwd/dgrad/wgrad).
#include "aten/FallbackCall.h"
#include "aten/Ops.h"

#include <ATen/Context.h>
#include <ATen/Functions.h>
#include <torch/library.h>

#include <atomic>
#include <mutex>

namespace b200 {
namespace ops {

namespace {

std::atomic<bool> g_pointwise_gemm{true};
std::atomic<int64_t> g_pointwise_hits{0};
std::atomic<bool> g_implicit_gemm{true};
std::atomic<int64_t> g_implicit_hits{0};

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

// ---------------------------------------------------------------- implicit GEMM route
bool implicit_eligible(const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride,
                       at::IntArrayRef padding, at::IntArrayRef dilation, bool transposed, int64_t groups) {
  if (!g_implicit_gemm.load(std::memory_order_relaxed)) return false;
  if (transposed || groups != 1 || input.dim() != 4 || weight.dim() != 4) return false;
  if (stride.size() != 2 || padding.size() != 2 || !all_eq(dilation, 1)) return false;
  const auto dt = input.scalar_type();
  if ((dt != at::kBFloat16 && dt != at::kHalf) || weight.scalar_type() != dt) return false;
  if (stride[0] < 1 || stride[0] > 2 || stride[1] < 1 || stride[1] > 2) return false;
  if (weight.size(2) * weight.size(3) > 49 || weight.size(0) % 8 != 0 || input.numel() == 0) return false;
  if (input.size(1) != weight.size(1)) return false;
  if (input.size(1) % 8 != 0 && input.size(1) > 8) return false;
  return true;
}

b200_conv_t conv_desc(const at::Tensor& x, const at::Tensor& w, at::IntArrayRef stride, at::IntArrayRef padding) {
  b200_conv_t d{};
  d.N = x.size(0), d.C = x.size(1), d.H = x.size(2), d.W = x.size(3);
  d.K = w.size(0), d.R = (int)w.size(2), d.S = (int)w.size(3);
  d.sh = (int)stride[0], d.sw = (int)stride[1], d.ph = (int)padding[0], d.pw = (int)padding[1];
  d.Ho = (d.H + 2 * d.ph - d.R) / d.sh + 1;
  d.Wo = (d.W + 2 * d.pw - d.S) / d.sw + 1;
  d.dtype = kdtype(x.scalar_type());
  return d;
}

// Channels-last dense tensor with the channel dimension zero-padded up to a multiple of 8.
at::Tensor nhwc_padded(const at::Tensor& t) {
  const int64_t C = t.size(1), Cp = (C + 7) / 8 * 8;
  if (Cp == C) return t.contiguous(at::MemoryFormat::ChannelsLast);
  // (at::zeros drops the memory format of its options)
  at::Tensor out = at::empty({t.size(0), Cp, t.size(2), t.size(3)}, t.options().memory_format(at::MemoryFormat::ChannelsLast));
  out.zero_();
  out.narrow(1, 0, C).copy_(t);
  return out;
}

// ---- few-channel first layer: the image is written out with its zero border and 8 channels, filters row-packed
bool stem_eligible(const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride, at::IntArrayRef padding,
                   b200_conv_t* d) {
  if (input.size(1) > 8 || weight.size(3) * 8 > 64) return false;
  *d = b200_conv_t{};
  d->N = input.size(0), d->C = 8, d->H = input.size(2), d->W = input.size(3);
  d->K = weight.size(0), d->R = (int)weight.size(2), d->S = (int)weight.size(3);
  d->sh = (int)stride[0], d->sw = (int)stride[1], d->ph = (int)padding[0], d->pw = (int)padding[1];
  d->Ho = (d->H + 2 * d->ph - d->R) / d->sh + 1;
  d->Wo = (d->W + 2 * d->pw - d->S) / d->sw + 1;
  d->dtype = kdtype(input.scalar_type());
  return d->Ho > 0 && d->Wo > 0 && b200_conv_stem_supported(d) != 0;
}

// The forward's padded image is kept for the backward of the same input (same storage, same version counter,
// same geometry) and dropped when the backward has used it.
struct StemCache {
  const void* ptr = nullptr;
  uint32_t version = 0;
  int64_t N = 0, H = 0, W = 0, C = 0;
  int ph = 0, pw = 0;
  at::Tensor xp;
};
std::mutex g_stem_mu;
StemCache g_stem_cache;  // backward runs on the autograd thread

bool stem_cache_matches(const StemCache& c, const at::Tensor& input, const b200_conv_t& d) {
  return c.xp.defined() && c.ptr == input.const_data_ptr() && c.version == input._version() && c.N == d.N &&
         c.H == d.H && c.W == d.W && c.C == input.size(1) && c.ph == d.ph && c.pw == d.pw;
}

at::Tensor stem_padded_image(const at::Tensor& input, const b200_conv_t& d, bool forward) {
  {
    std::lock_guard<std::mutex> g(g_stem_mu);
    if (!forward && stem_cache_matches(g_stem_cache, input, d)) {
      at::Tensor xp = std::move(g_stem_cache.xp);
      g_stem_cache = StemCache{};
      return xp;
    }
  }
  at::Tensor xp = at::empty({d.N, d.H + 2 * d.ph, d.W + 2 * d.pw, 8}, input.options());
  xp.zero_();
  xp.narrow(1, d.ph, d.H).narrow(2, d.pw, d.W).narrow(3, 0, input.size(1)).copy_(input.permute({0, 2, 3, 1}));
  if (forward && at::GradMode::is_enabled()) {
    std::lock_guard<std::mutex> g(g_stem_mu);
    g_stem_cache = StemCache{input.const_data_ptr(), input._version(), d.N, d.H, d.W, input.size(1), d.ph, d.pw, xp};
  }
  return xp;
}

at::Tensor stem_packed_filter(const at::Tensor& weight, const b200_conv_t& d) {
  at::Tensor wp = at::empty({d.K, d.R, 8, 8}, weight.options());
  wp.zero_();
  wp.narrow(2, 0, d.S).narrow(3, 0, weight.size(1)).copy_(weight.permute({0, 2, 3, 1}));
  return wp;
}

at::Tensor implicit_forward(const at::Tensor& input, const at::Tensor& weight, const std::optional<at::Tensor>& bias,
                            at::IntArrayRef stride, at::IntArrayRef padding) {
  b200_conv_t sd;
  if (stem_eligible(input, weight, stride, padding, &sd)) {
    const at::Tensor xp = stem_padded_image(input, sd, /*forward=*/true);
    const at::Tensor wp = stem_packed_filter(weight, sd);
    at::Tensor y = at::empty({sd.N, sd.K, sd.Ho, sd.Wo}, input.options().memory_format(at::MemoryFormat::ChannelsLast));
    at::Tensor b;
    if (bias.has_value() && bias->defined()) b = bias->to(input.scalar_type()).contiguous();
    B200_KERNEL_CALL(b200_conv_stem_fwd(&sd, y.data_ptr(), xp.const_data_ptr(), wp.const_data_ptr(),
                                        b.defined() ? b.const_data_ptr() : nullptr, 0, current_raw_stream(input)));
    g_implicit_hits.fetch_add(1, std::memory_order_relaxed);
    return y;
  }
  const at::Tensor x = nhwc_padded(input);
  const at::Tensor w = nhwc_padded(weight);
  b200_conv_t d = conv_desc(x, w, stride, padding);
  TORCH_CHECK(d.Ho > 0 && d.Wo > 0, "convolution: the filter does not fit the padded input");
  at::Tensor y = at::empty({d.N, d.K, d.Ho, d.Wo}, x.options().memory_format(at::MemoryFormat::ChannelsLast));
  at::Tensor b;
  if (bias.has_value() && bias->defined()) b = bias->to(x.scalar_type()).contiguous();
  auto stream = current_raw_stream(x);
  B200_KERNEL_CALL(b200_conv_fwd(&d, y.data_ptr(), x.const_data_ptr(), w.const_data_ptr(),
                                 b.defined() ? b.const_data_ptr() : nullptr, 0, stream));
  g_implicit_hits.fetch_add(1, std::memory_order_relaxed);
  return y;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> implicit_backward(const at::Tensor& grad_output, const at::Tensor& input,
                                                                 const at::Tensor& weight, at::IntArrayRef stride,
                                                                 at::IntArrayRef padding, std::array<bool, 3> mask) {
  const at::Tensor gy = grad_output.contiguous(at::MemoryFormat::ChannelsLast);
  const int64_t C = input.size(1);
  at::Tensor gx, gw, gb;
  b200_conv_t sd0;
  const bool stem_only = !mask[0] && stem_eligible(input, weight, stride, padding, &sd0);
  const at::Tensor x = stem_only ? input : nhwc_padded(input);
  const at::Tensor w = stem_only ? weight : nhwc_padded(weight);
  b200_conv_t d = conv_desc(x, w, stride, padding);
  auto stream = current_raw_stream(input);
  if (mask[0]) {
    gx = at::empty(x.sizes(), x.options().memory_format(at::MemoryFormat::ChannelsLast));
    B200_KERNEL_CALL(b200_conv_dgrad(&d, gx.data_ptr(), gy.const_data_ptr(), w.const_data_ptr(), stream));
    if (x.size(1) != C) gx = gx.narrow(1, 0, C).contiguous(at::MemoryFormat::ChannelsLast);
  }
  b200_conv_t sd;
  if (mask[1] && stem_eligible(input, weight, stride, padding, &sd)) {
    const at::Tensor xp = stem_padded_image(input, sd, /*forward=*/false);
    at::Tensor acc = at::zeros({sd.K, sd.R, 8, 8}, input.options().dtype(at::kFloat));
    if (at::globalContext().deterministicAlgorithms())
      at::globalContext().alertNotDeterministic("the row-packed first-layer weight gradient (fp32 atomics over pixel splits)");
    B200_KERNEL_CALL(b200_conv_stem_wgrad(&sd, acc.data_ptr<float>(), gy.const_data_ptr(), xp.const_data_ptr(), stream));
    gw = acc.narrow(2, 0, sd.S).narrow(3, 0, C).permute({0, 3, 1, 2}).to(weight.scalar_type());  // [K, C, R, S]
    const bool cl = weight.is_contiguous(at::MemoryFormat::ChannelsLast) && !weight.is_contiguous();
    gw = gw.contiguous(cl ? at::MemoryFormat::ChannelsLast : at::MemoryFormat::Contiguous);
  } else if (mask[1]) {
    at::Tensor acc = at::zeros({d.K, d.R, d.S, d.C}, x.options().dtype(at::kFloat));
    b200_conv_set_deterministic(at::globalContext().deterministicAlgorithms() ? 1 : 0);
    B200_KERNEL_CALL(b200_conv_wgrad(&d, acc.data_ptr<float>(), gy.const_data_ptr(), x.const_data_ptr(), stream));
    gw = acc.to(weight.scalar_type()).permute({0, 3, 1, 2});  // [K, C, R, S] with channels-last strides
    if (x.size(1) != C) gw = gw.narrow(1, 0, C);
    const bool cl = weight.is_contiguous(at::MemoryFormat::ChannelsLast) && !weight.is_contiguous();
    gw = gw.contiguous(cl ? at::MemoryFormat::ChannelsLast : at::MemoryFormat::Contiguous);
  }
  if (mask[2]) gb = gy.sum({0, 2, 3});
  g_implicit_hits.fetch_add(1, std::memory_order_relaxed);
  return {gx, gw, gb};
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
  if (implicit_eligible(input, weight, stride, padding, dilation, transposed, groups))
    return implicit_forward(input, weight, bias, stride, padding);
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
  if (implicit_eligible(input, weight, stride, padding, dilation, transposed, groups) &&
      grad_output.scalar_type() == input.scalar_type())
    return implicit_backward(grad_output, input, weight, stride, padding, output_mask);
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
void set_implicit_conv_gemm(bool on) { g_implicit_gemm.store(on); }
int64_t implicit_conv_hits() { return g_implicit_hits.load(); }

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("convolution_overrideable", TORCH_FN(convolution_overrideable));
  m.impl("convolution_backward_overrideable", TORCH_FN(convolution_backward_overrideable));
}

}  // namespace ops
}  // namespace b200
