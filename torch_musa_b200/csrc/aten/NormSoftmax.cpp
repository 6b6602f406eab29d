// RMSNorm / LayerNorm / softmax / log-softmax / embedding / dropout registered for
// the stock ATen operators, so torch.nn modules hit the hand-written kernels with
// no model changes (torch.rms_norm -> aten::_fused_rms_norm, F.layer_norm ->
// native_layer_norm, F.softmax -> _softmax, nn.Embedding -> embedding, ...).
// Parity: reference torch_musa/csrc/aten/ops/RMSNorm.cpp, LayerNorm.cpp, SoftMax.cpp,
// Embedding.cpp, Dropout.cpp.
#include "aten/FallbackCall.h"
#include "aten/Ops.h"
#include "core/Generator.h"

#include <ATen/Functions.h>
#include <ATen/core/Generator.h>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {

inline bool fast(const at::Tensor& t) { return on_device(t) && kdtype(t.scalar_type()) >= 0; }

int64_t prod(at::IntArrayRef v) {
  int64_t p = 1;
  for (auto x : v) p *= x;
  return p;
}

// --------------------------------------------------------------------- RMSNorm
std::tuple<at::Tensor, at::Tensor> fused_rms_norm(const at::Tensor& input, at::IntArrayRef normalized_shape,
                                                  const std::optional<at::Tensor>& weight, std::optional<double> eps) {
  check_devices("rms_norm", input, weight);
  const int64_t cols = prod(normalized_shape);
  const bool w_ok = !weight.has_value() || !weight->defined() ||
                    (weight->scalar_type() == input.scalar_type() && weight->is_contiguous());
  if (fast(input) && w_ok && cols > 0 && input.numel() > 0) {
    at::Tensor x = input.contiguous();
    const int64_t rows = x.numel() / cols;
    at::Tensor y = at::empty_like(x);
    std::vector<int64_t> stat_shape(input.sizes().begin(), input.sizes().end());
    for (size_t i = 0; i < normalized_shape.size(); ++i) stat_shape[stat_shape.size() - 1 - i] = 1;
    at::Tensor rstd = at::empty(stat_shape, x.options().dtype(at::kFloat));
    double e = eps.has_value() ? *eps : (double)std::numeric_limits<float>::epsilon();
    if (input.scalar_type() == at::kBFloat16 && !eps.has_value()) e = 0.0078125;   // bf16 epsilon
    if (input.scalar_type() == at::kHalf && !eps.has_value()) e = 0.0009765625;     // fp16 epsilon
    DeviceSwitch sw(x.device().index());
    const void* wp = (weight.has_value() && weight->defined()) ? weight->const_data_ptr() : nullptr;
    int err = b200_rmsnorm_fwd(kdtype(x.scalar_type()), y.mutable_data_ptr(), rstd.data_ptr<float>(),
                               x.const_data_ptr(), wp, nullptr, nullptr, rows, cols, (float)e, current_raw_stream(x));
    if (err == 0) return {y, rstd};
    if (err != (int)cudaErrorNotSupported) B200_KERNEL_CALL(err);
  }
  auto st = run_fallback(B200_OP_HANDLE("aten::_fused_rms_norm", ""), input, normalized_shape, weight, eps);
  return {st[0].toTensor(), st[1].toTensor()};
}

std::tuple<at::Tensor, at::Tensor> fused_rms_norm_backward(const at::Tensor& grad_out, const at::Tensor& input,
                                                           at::IntArrayRef normalized_shape, const at::Tensor& rstd,
                                                           const std::optional<at::Tensor>& weight,
                                                           std::array<bool, 2> mask) {
  check_devices("rms_norm_backward", input, grad_out, rstd, weight);
  const int64_t cols = prod(normalized_shape);
  const bool has_w = weight.has_value() && weight->defined();
  const bool w_ok = !has_w || (weight->scalar_type() == input.scalar_type() && weight->is_contiguous());
  if (fast(input) && w_ok && grad_out.scalar_type() == input.scalar_type() && rstd.scalar_type() == at::kFloat &&
      cols > 0 && input.numel() > 0) {
    at::Tensor x = input.contiguous(), dy = grad_out.contiguous(), rs = rstd.contiguous();
    const int64_t rows = x.numel() / cols;
    at::Tensor dx = at::empty_like(x);
    const bool need_dw = mask[1] && has_w;
    const int nb = b200_rmsnorm_bwd_partial_rows(rows, cols);
    at::Tensor partial;
    if (need_dw) partial = at::empty({nb, cols}, x.options().dtype(at::kFloat));
    DeviceSwitch sw(x.device().index());
    cudaStream_t s = current_raw_stream(x);
    int err = b200_rmsnorm_bwd(kdtype(x.scalar_type()), dx.mutable_data_ptr(),
                               need_dw ? partial.data_ptr<float>() : nullptr, nullptr, dy.const_data_ptr(),
                               x.const_data_ptr(), has_w ? weight->const_data_ptr() : nullptr, rs.data_ptr<float>(),
                               rows, cols, s);
    if (err == 0) {
      at::Tensor dw;
      if (need_dw) {
        dw = at::empty_like(*weight);
        B200_KERNEL_CALL(b200_reduce_cols_sum(B200_F32, dw.mutable_data_ptr(), kdtype(dw.scalar_type()),
                                              partial.const_data_ptr(), nb, cols, s));
      }
      return {mask[0] ? dx : at::Tensor(), dw};
    }
    if (err != (int)cudaErrorNotSupported) B200_KERNEL_CALL(err);
  }
  auto st = run_fallback(B200_OP_HANDLE("aten::_fused_rms_norm_backward", ""), grad_out, input, normalized_shape, rstd,
                         weight, mask);
  return {st[0].toTensor(), st[1].toTensor()};
}

// --------------------------------------------------------------------- LayerNorm
std::tuple<at::Tensor, at::Tensor, at::Tensor> native_layer_norm(const at::Tensor& input,
                                                                 c10::SymIntArrayRef normalized_shape_,
                                                                 const std::optional<at::Tensor>& weight,
                                                                 const std::optional<at::Tensor>& bias, double eps) {
  check_devices("layer_norm", input, weight, bias);
  auto normalized_shape = C10_AS_INTARRAYREF_SLOW(normalized_shape_);
  const int64_t cols = prod(normalized_shape);
  const bool has_w = weight.has_value() && weight->defined(), has_b = bias.has_value() && bias->defined();
  const bool ok = (!has_w || (weight->scalar_type() == input.scalar_type() && weight->is_contiguous())) &&
                  (!has_b || (bias->scalar_type() == input.scalar_type() && bias->is_contiguous()));
  if (fast(input) && ok && cols > 0 && input.numel() > 0) {
    at::Tensor x = input.contiguous();
    const int64_t rows = x.numel() / cols;
    at::Tensor y = at::empty_like(x);
    std::vector<int64_t> stat_shape(input.sizes().begin(), input.sizes().end());
    for (size_t i = 0; i < normalized_shape.size(); ++i) stat_shape[stat_shape.size() - 1 - i] = 1;
    // statistics are returned in fp32 for reduced-precision inputs, like the CUDA backend
    at::Tensor mean = at::empty(stat_shape, x.options().dtype(at::kFloat));
    at::Tensor rstd = at::empty(stat_shape, x.options().dtype(at::kFloat));
    DeviceSwitch sw(x.device().index());
    int err = b200_layernorm_fwd(kdtype(x.scalar_type()), y.mutable_data_ptr(), mean.data_ptr<float>(),
                                 rstd.data_ptr<float>(), x.const_data_ptr(), has_w ? weight->const_data_ptr() : nullptr,
                                 has_b ? bias->const_data_ptr() : nullptr, rows, cols, (float)eps, current_raw_stream(x));
    if (err == 0) return {y, mean, rstd};
    if (err != (int)cudaErrorNotSupported) B200_KERNEL_CALL(err);
  }
  auto st = run_fallback(B200_OP_HANDLE("aten::native_layer_norm", ""), input, normalized_shape_, weight, bias, eps);
  return {st[0].toTensor(), st[1].toTensor(), st[2].toTensor()};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> native_layer_norm_backward(
    const at::Tensor& grad_out, const at::Tensor& input, c10::SymIntArrayRef normalized_shape_, const at::Tensor& mean,
    const at::Tensor& rstd, const std::optional<at::Tensor>& weight, const std::optional<at::Tensor>& bias,
    std::array<bool, 3> mask) {
  auto normalized_shape = C10_AS_INTARRAYREF_SLOW(normalized_shape_);
  check_devices("layer_norm_backward", input, grad_out, mean, rstd, weight, bias);
  const int64_t cols = prod(normalized_shape);
  const bool has_w = weight.has_value() && weight->defined();
  const bool ok = (!has_w || (weight->scalar_type() == input.scalar_type() && weight->is_contiguous())) &&
                  mean.scalar_type() == at::kFloat && rstd.scalar_type() == at::kFloat &&
                  grad_out.scalar_type() == input.scalar_type();
  if (fast(input) && ok && cols > 0 && input.numel() > 0) {
    at::Tensor x = input.contiguous(), dy = grad_out.contiguous(), mu = mean.contiguous(), rs = rstd.contiguous();
    const int64_t rows = x.numel() / cols;
    at::Tensor dx = at::empty_like(x);
    const int nb = b200_rmsnorm_bwd_partial_rows(rows, cols);
    const bool need_dw = mask[1], need_db = mask[2];
    at::Tensor pw, pb;
    if (need_dw) pw = at::empty({nb, cols}, x.options().dtype(at::kFloat));
    if (need_db) pb = at::empty({nb, cols}, x.options().dtype(at::kFloat));
    DeviceSwitch sw(x.device().index());
    cudaStream_t s = current_raw_stream(x);
    int err = b200_layernorm_bwd(kdtype(x.scalar_type()), dx.mutable_data_ptr(), need_dw ? pw.data_ptr<float>() : nullptr,
                                 need_db ? pb.data_ptr<float>() : nullptr, dy.const_data_ptr(), x.const_data_ptr(),
                                 has_w ? weight->const_data_ptr() : nullptr, mu.data_ptr<float>(), rs.data_ptr<float>(),
                                 rows, cols, s);
    if (err == 0) {
      at::Tensor dw, db;
      auto wopt = x.options();
      std::vector<int64_t> wshape(normalized_shape.begin(), normalized_shape.end());
      if (need_dw) {
        dw = at::empty(wshape, wopt);
        B200_KERNEL_CALL(b200_reduce_cols_sum(B200_F32, dw.mutable_data_ptr(), kdtype(dw.scalar_type()),
                                              pw.const_data_ptr(), nb, cols, s));
      }
      if (need_db) {
        db = at::empty(wshape, wopt);
        B200_KERNEL_CALL(b200_reduce_cols_sum(B200_F32, db.mutable_data_ptr(), kdtype(db.scalar_type()),
                                              pb.const_data_ptr(), nb, cols, s));
      }
      return {mask[0] ? dx : at::Tensor(), dw, db};
    }
    if (err != (int)cudaErrorNotSupported) B200_KERNEL_CALL(err);
  }
  auto st = run_fallback(B200_OP_HANDLE("aten::native_layer_norm_backward", ""), grad_out, input, normalized_shape_,
                         mean, rstd, weight, bias, mask);
  return {st[0].toTensor(), st[1].toTensor(), st[2].toTensor()};
}

// --------------------------------------------------------------------- softmax
at::Tensor softmax_common(const at::Tensor& self, int64_t dim, bool half_to_float, bool log) {
  const int64_t d = at::maybe_wrap_dim(dim, self.dim());
  if (fast(self) && !half_to_float && self.dim() > 0 && d == self.dim() - 1 && self.numel() > 0) {
    at::Tensor x = self.contiguous();
    at::Tensor y = at::empty_like(x);
    const int64_t cols = x.size(-1), rows = x.numel() / cols;
    DeviceSwitch sw(x.device().index());
    int err = b200_softmax_fwd(kdtype(x.scalar_type()), y.mutable_data_ptr(), x.const_data_ptr(), rows, cols, log ? 1 : 0,
                               current_raw_stream(x));
    if (err == 0) return y;
    if (err != (int)cudaErrorNotSupported) B200_KERNEL_CALL(err);
  }
  if (log) return fallback_tensor(B200_OP_HANDLE("aten::_log_softmax", ""), self, dim, half_to_float);
  return fallback_tensor(B200_OP_HANDLE("aten::_softmax", ""), self, dim, half_to_float);
}
at::Tensor _softmax(const at::Tensor& self, int64_t dim, bool h2f) { return softmax_common(self, dim, h2f, false); }
at::Tensor _log_softmax(const at::Tensor& self, int64_t dim, bool h2f) { return softmax_common(self, dim, h2f, true); }

at::Tensor softmax_bwd_common(const at::Tensor& grad, const at::Tensor& out, int64_t dim, at::ScalarType in_dtype,
                              bool log) {
  check_devices("softmax_backward", out, grad);
  const int64_t d = at::maybe_wrap_dim(dim, out.dim());
  if (fast(out) && grad.scalar_type() == out.scalar_type() && in_dtype == out.scalar_type() && out.dim() > 0 &&
      d == out.dim() - 1 && out.numel() > 0) {
    at::Tensor y = out.contiguous(), g = grad.contiguous();
    at::Tensor dx = at::empty_like(y);
    const int64_t cols = y.size(-1), rows = y.numel() / cols;
    DeviceSwitch sw(y.device().index());
    int err = b200_softmax_bwd(kdtype(y.scalar_type()), dx.mutable_data_ptr(), g.const_data_ptr(), y.const_data_ptr(), rows,
                               cols, log ? 1 : 0, current_raw_stream(y));
    if (err == 0) return dx;
    if (err != (int)cudaErrorNotSupported) B200_KERNEL_CALL(err);
  }
  if (log) return fallback_tensor(B200_OP_HANDLE("aten::_log_softmax_backward_data", ""), grad, out, dim, in_dtype);
  return fallback_tensor(B200_OP_HANDLE("aten::_softmax_backward_data", ""), grad, out, dim, in_dtype);
}
at::Tensor _softmax_backward_data(const at::Tensor& g, const at::Tensor& o, int64_t dim, at::ScalarType t) {
  return softmax_bwd_common(g, o, dim, t, false);
}
at::Tensor _log_softmax_backward_data(const at::Tensor& g, const at::Tensor& o, int64_t dim, at::ScalarType t) {
  return softmax_bwd_common(g, o, dim, t, true);
}

// --------------------------------------------------------------------- embedding
at::Tensor embedding(const at::Tensor& weight, const at::Tensor& indices, c10::SymInt padding_idx,
                     bool scale_grad_by_freq, bool sparse) {
  if (fast(weight) && weight.dim() == 2 && weight.is_contiguous() && on_device(indices) &&
      indices.scalar_type() == at::kLong && indices.numel() > 0) {
    at::Tensor idx = indices.contiguous();
    std::vector<int64_t> shape(idx.sizes().begin(), idx.sizes().end());
    shape.push_back(weight.size(1));
    at::Tensor out = at::empty(shape, weight.options());
    DeviceSwitch sw(weight.device().index());
    int err = b200_embedding_fwd(kdtype(weight.scalar_type()), out.mutable_data_ptr(), weight.const_data_ptr(),
                                 idx.data_ptr<int64_t>(), idx.numel(), weight.size(1), weight.size(0),
                                 current_raw_stream(weight));
    if (err == 0) return out;
    if (err != (int)cudaErrorNotSupported) B200_KERNEL_CALL(err);
  }
  return fallback_tensor(B200_OP_HANDLE("aten::embedding", ""), weight, indices, padding_idx, scale_grad_by_freq, sparse);
}

at::Tensor embedding_dense_backward(const at::Tensor& grad, const at::Tensor& indices, c10::SymInt num_weights,
                                    c10::SymInt padding_idx, bool scale_grad_by_freq) {
  if (fast(grad) && !scale_grad_by_freq && on_device(indices) && indices.scalar_type() == at::kLong &&
      indices.numel() > 0) {
    const int64_t vocab = num_weights.expect_int(), dim = grad.size(-1);
    at::Tensor g = grad.contiguous().view({-1, dim});
    at::Tensor idx = indices.contiguous().view({-1});
    DeviceSwitch sw(grad.device().index());
    cudaStream_t s = current_raw_stream(grad);
    if (at::globalContext().deterministicAlgorithms()) {
      auto sorted = idx.sort();
      at::Tensor gw = at::zeros({vocab, dim}, grad.options());
      int err = b200_embedding_bwd_sorted(kdtype(g.scalar_type()), gw.mutable_data_ptr(), g.const_data_ptr(),
                                          std::get<0>(sorted).data_ptr<int64_t>(), std::get<1>(sorted).data_ptr<int64_t>(),
                                          idx.numel(), dim, vocab, padding_idx.expect_int(), s);
      if (err == 0) return gw;
      if (err != (int)cudaErrorNotSupported) B200_KERNEL_CALL(err);
    } else {
      at::Tensor acc = at::zeros({vocab, dim}, grad.options().dtype(at::kFloat));
      int err = b200_embedding_bwd_atomic(kdtype(g.scalar_type()), acc.data_ptr<float>(), g.const_data_ptr(),
                                          idx.data_ptr<int64_t>(), idx.numel(), dim, vocab, padding_idx.expect_int(), s);
      if (err == 0) return grad.scalar_type() == at::kFloat ? acc : acc.to(grad.scalar_type());
      if (err != (int)cudaErrorNotSupported) B200_KERNEL_CALL(err);
    }
  }
  return fallback_tensor(B200_OP_HANDLE("aten::embedding_dense_backward", ""), grad, indices, num_weights, padding_idx,
                         scale_grad_by_freq);
}

// --------------------------------------------------------------------- dropout / random fills
b200_philox_t philox_for(const at::Tensor& t, std::optional<at::Generator> gen, int64_t n) {
  at::Generator g = (gen.has_value() && gen->defined()) ? *gen : default_generator(t.device().index());
  auto* impl = at::check_generator<GeneratorImpl>(g);
  std::lock_guard<std::mutex> lock(impl->mutex_);
  PhiloxArgs a = impl->philox_args(b200_philox_increment(n));
  b200_philox_t r;
  r.seed = a.seed; r.offset = a.offset; r.seed_ptr = a.seed_ptr; r.offset_ptr = a.offset_ptr;
  r.offset_intragraph = a.offset_intragraph; r.captured = a.captured;
  return r;
}

std::tuple<at::Tensor, at::Tensor> native_dropout(const at::Tensor& input, double p, std::optional<bool> train) {
  if (fast(input) && input.is_non_overlapping_and_dense() && train.value_or(true) && p > 0.0 && p < 1.0 &&
      input.numel() > 0) {
    at::Tensor out = at::empty_strided(input.sizes(), input.strides(), input.options());
    at::Tensor mask = at::empty_strided(input.sizes(), input.strides(), input.options().dtype(at::kBool));
    DeviceSwitch sw(input.device().index());
    B200_KERNEL_CALL(b200_dropout_fwd(kdtype(input.scalar_type()), out.mutable_data_ptr(),
                                      reinterpret_cast<uint8_t*>(mask.mutable_data_ptr()), input.const_data_ptr(),
                                      input.numel(), (float)p, philox_for(input, std::nullopt, input.numel()),
                                      current_raw_stream(input)));
    return {out, mask};
  }
  auto st = run_fallback(B200_OP_HANDLE("aten::native_dropout", ""), input, p, train);
  return {st[0].toTensor(), st[1].toTensor()};
}

at::Tensor native_dropout_backward(const at::Tensor& grad, const at::Tensor& mask, double scale) {
  check_devices("native_dropout_backward", grad, mask);
  if (fast(grad) && grad.is_non_overlapping_and_dense() && mask.scalar_type() == at::kBool &&
      mask.sizes() == grad.sizes() && mask.strides() == grad.strides() && grad.numel() > 0) {
    at::Tensor dx = at::empty_strided(grad.sizes(), grad.strides(), grad.options());
    DeviceSwitch sw(grad.device().index());
    B200_KERNEL_CALL(b200_dropout_bwd(kdtype(grad.scalar_type()), dx.mutable_data_ptr(), grad.const_data_ptr(),
                                      reinterpret_cast<const uint8_t*>(mask.const_data_ptr()), grad.numel(),
                                      (float)scale, current_raw_stream(grad)));
    return dx;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::native_dropout_backward", ""), grad, mask, scale);
}

at::Tensor& uniform_(at::Tensor& self, double from, double to, std::optional<at::Generator> gen) {
  bool ours = !gen.has_value() || !gen->defined() || gen->device().type() == kDeviceType;
  if (fast(self) && self.is_non_overlapping_and_dense() && ours) {
    if (self.numel() == 0) return self;
    DeviceSwitch sw(self.device().index());
    B200_KERNEL_CALL(b200_uniform(kdtype(self.scalar_type()), self.mutable_data_ptr(), self.numel(), from, to,
                                  philox_for(self, gen, self.numel()), current_raw_stream(self)));
    return self;
  }
  run_fallback(B200_OP_HANDLE("aten::uniform_", ""), self, from, to, gen);
  return self;
}

at::Tensor& normal_(at::Tensor& self, double mean, double std, std::optional<at::Generator> gen) {
  bool ours = !gen.has_value() || !gen->defined() || gen->device().type() == kDeviceType;
  if (fast(self) && self.is_non_overlapping_and_dense() && ours) {
    TORCH_CHECK(std >= 0.0, "normal expects std >= 0.0, but found std ", std);
    if (self.numel() == 0) return self;
    DeviceSwitch sw(self.device().index());
    B200_KERNEL_CALL(b200_normal(kdtype(self.scalar_type()), self.mutable_data_ptr(), self.numel(), mean, std,
                                 philox_for(self, gen, self.numel()), current_raw_stream(self)));
    return self;
  }
  run_fallback(B200_OP_HANDLE("aten::normal_", ""), self, mean, std, gen);
  return self;
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("_fused_rms_norm", TORCH_FN(fused_rms_norm));
  m.impl("_fused_rms_norm_backward", TORCH_FN(fused_rms_norm_backward));
  m.impl("native_layer_norm", TORCH_FN(native_layer_norm));
  m.impl("native_layer_norm_backward", TORCH_FN(native_layer_norm_backward));
  m.impl("_softmax", TORCH_FN(_softmax));
  m.impl("_log_softmax", TORCH_FN(_log_softmax));
  m.impl("_softmax_backward_data", TORCH_FN(_softmax_backward_data));
  m.impl("_log_softmax_backward_data", TORCH_FN(_log_softmax_backward_data));
  m.impl("embedding", TORCH_FN(embedding));
  m.impl("embedding_dense_backward", TORCH_FN(embedding_dense_backward));
  m.impl("native_dropout", TORCH_FN(native_dropout));
  m.impl("native_dropout_backward", TORCH_FN(native_dropout_backward));
  m.impl("uniform_", TORCH_FN(uniform_));
  m.impl("normal_", TORCH_FN(normal_));
}

}  // namespace ops
}  // namespace b200
