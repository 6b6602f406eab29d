// Fused optimizers and gradient-scaler operators on the multi_tensor_apply kernels:
// aten::_fused_adam_/_fused_adamw_/_fused_sgd_ (float and tensor learning rates,
// grad_scale / found_inf aware) so torch.optim.*(fused=True) works on the device,
// aten::_amp_foreach_non_finite_check_and_unscale_ / _amp_update_scale_ for
// GradScaler, aten::_foreach_norm (2-norm) for clip_grad_norm_, and the backend's own
// multi-tensor L2-norm / scale / axpby / LAMB entry points.
// Parity: reference torch_musa/csrc/aten/ops/FusedAdam.cpp, musa/FusedSgdKernel.mu:147-425,
// Amp.cpp, musa/Amp.mu, musa/ForeachReduceOp.mu, csrc/extension/FusedAdam.mu:348-472,
// csrc/extension/apex/*.
#include "aten/FallbackCall.h"
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {

struct Lists {
  std::vector<void*> p;
  std::vector<int64_t> n;
};

bool dense_list(at::TensorList l) {
  for (const auto& t : l)
    if (!on_device(t) || !t.is_non_overlapping_and_dense() || kdtype(t.scalar_type()) < 0) return false;
  return true;
}
bool same_dtype(at::TensorList l) {
  for (const auto& t : l)
    if (t.scalar_type() != l[0].scalar_type()) return false;
  return true;
}
std::vector<void*> ptrs(at::TensorList l) {
  std::vector<void*> v;
  v.reserve(l.size());
  for (const auto& t : l) v.push_back(t.data_ptr());
  return v;
}
std::vector<int64_t> numels(at::TensorList l) {
  std::vector<int64_t> v;
  v.reserve(l.size());
  for (const auto& t : l) v.push_back(t.numel());
  return v;
}
const float* opt_scalar(const std::optional<at::Tensor>& t, const char* what) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(on_device(*t) && t->scalar_type() == at::kFloat && t->numel() == 1, what,
              " must be a float32 scalar tensor on the device");
  return t->data_ptr<float>();
}

// Same element order in memory: strides agree on every dimension that has more than one element (a
// [C_out, C_in, 1, 1] weight is the same memory in the contiguous and the channels-last format).
bool same_layout(const at::Tensor& a, const at::Tensor& b) {
  if (a.sizes() != b.sizes()) return false;
  for (int64_t d = 0; d < a.dim(); ++d)
    if (a.size(d) > 1 && a.stride(d) != b.stride(d)) return false;
  return true;
}

bool adam_fast(at::TensorList params, at::TensorList grads, at::TensorList ea, at::TensorList es, at::TensorList mx,
               at::TensorList steps, bool amsgrad) {
  if (params.empty()) return true;
  if (!dense_list(params) || !dense_list(grads) || !dense_list(ea) || !dense_list(es)) return false;
  if (amsgrad && !dense_list(mx)) return false;
  if (!same_dtype(params) || !same_dtype(grads) || !same_dtype(ea) || !same_dtype(es)) return false;
  if (ea[0].scalar_type() != es[0].scalar_type()) return false;
  for (const auto& s : steps)
    if (!on_device(s) || s.scalar_type() != at::kFloat || s.numel() != 1) return false;
  for (size_t i = 0; i < params.size(); ++i) {
    if (!same_layout(params[i], grads[i]) || !same_layout(params[i], ea[i]) || !same_layout(params[i], es[i]))
      return false;
  }
  return true;
}

void fused_adam_common(at::TensorList params, at::TensorList grads, at::TensorList ea, at::TensorList es,
                       at::TensorList mx, at::TensorList steps, double lr, const at::Tensor* lr_t, double beta1,
                       double beta2, double wd, double eps, bool amsgrad, bool maximize,
                       const std::optional<at::Tensor>& grad_scale, const std::optional<at::Tensor>& found_inf,
                       bool adamw) {
  if (params.empty()) return;
  b200_adam_args_t a{};
  a.lr = (float)lr;
  a.beta1 = (float)beta1;
  a.beta2 = (float)beta2;
  a.eps = (float)eps;
  a.weight_decay = (float)wd;
  a.adamw = adamw;
  a.amsgrad = amsgrad;
  a.maximize = maximize;
  a.lr_ptr = nullptr;
  if (lr_t) {
    if (lr_t->device().is_cpu()) a.lr = lr_t->item<float>();
    else {
      TORCH_CHECK(lr_t->scalar_type() == at::kFloat && lr_t->numel() == 1, "lr tensor must be a float32 scalar");
      a.lr_ptr = lr_t->data_ptr<float>();
    }
  }
  a.grad_scale = opt_scalar(grad_scale, "grad_scale");
  a.found_inf = opt_scalar(found_inf, "found_inf");
  auto P = ptrs(params), G = ptrs(grads), M = ptrs(ea), V = ptrs(es), X = amsgrad ? ptrs(mx) : std::vector<void*>();
  std::vector<float*> S;
  for (const auto& s : steps) S.push_back(s.data_ptr<float>());
  auto N = numels(params);
  DeviceSwitch sw(params[0].device().index());
  B200_KERNEL_CALL(b200_multi_tensor_adam((int)P.size(), kdtype(params[0].scalar_type()), kdtype(grads[0].scalar_type()),
                                          kdtype(ea[0].scalar_type()), P.data(), G.data(), M.data(), V.data(),
                                          amsgrad ? X.data() : nullptr, S.data(), N.data(), a,
                                          current_raw_stream(params[0])));
}

#define B200_ADAM_OP(FN, NAME, OVERLOAD, ADAMW, LR_DECL, LR_VAL, LR_PTR)                                              \
  void FN(at::TensorList self, at::TensorList grads, at::TensorList exp_avgs, at::TensorList exp_avg_sqs,             \
          at::TensorList max_exp_avg_sqs, at::TensorList state_steps, LR_DECL, double beta1, double beta2,             \
          double weight_decay, double eps, bool amsgrad, bool maximize, const std::optional<at::Tensor>& grad_scale,  \
          const std::optional<at::Tensor>& found_inf) {                                                               \
    if (adam_fast(self, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps, amsgrad)) {                       \
      fused_adam_common(self, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps, LR_VAL, LR_PTR, beta1,      \
                        beta2, weight_decay, eps, amsgrad, maximize, grad_scale, found_inf, ADAMW);                   \
      return;                                                                                                         \
    }                                                                                                                 \
    run_fallback(B200_OP_HANDLE(NAME, OVERLOAD), self, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps,    \
                 lr, beta1, beta2, weight_decay, eps, amsgrad, maximize, grad_scale, found_inf);                      \
  }

B200_ADAM_OP(fused_adamw_, "aten::_fused_adamw_", "", true, double lr, lr, nullptr)
B200_ADAM_OP(fused_adam_, "aten::_fused_adam_", "", false, double lr, lr, nullptr)
B200_ADAM_OP(fused_adamw_tensor_lr_, "aten::_fused_adamw_", "tensor_lr", true, const at::Tensor& lr, 0.0, &lr)
B200_ADAM_OP(fused_adam_tensor_lr_, "aten::_fused_adam_", "tensor_lr", false, const at::Tensor& lr, 0.0, &lr)

bool sgd_fast(at::TensorList params, at::TensorList grads, at::TensorList bufs, double momentum) {
  if (params.empty()) return true;
  if (!dense_list(params) || !dense_list(grads) || !same_dtype(params) || !same_dtype(grads)) return false;
  if (momentum != 0.0) {
    if (bufs.size() != params.size() || !dense_list(bufs)) return false;
    for (size_t i = 0; i < params.size(); ++i)
      if (bufs[i].scalar_type() != params[i].scalar_type() || !same_layout(bufs[i], params[i])) return false;
  }
  for (size_t i = 0; i < params.size(); ++i)
    if (!same_layout(params[i], grads[i])) return false;
  return true;
}

void fused_sgd_common(at::TensorList params, at::TensorList grads, at::TensorList bufs, double wd, double momentum,
                      double lr, const at::Tensor* lr_t, double dampening, bool nesterov, bool maximize, bool first,
                      const std::optional<at::Tensor>& grad_scale, const std::optional<at::Tensor>& found_inf) {
  if (params.empty()) return;
  b200_sgd_args_t a{};
  a.lr = (float)lr;
  a.momentum = (float)momentum;
  a.dampening = (float)dampening;
  a.weight_decay = (float)wd;
  a.nesterov = nesterov;
  a.maximize = maximize;
  a.first_step = first;
  if (lr_t) {
    if (lr_t->device().is_cpu()) a.lr = lr_t->item<float>();
    else a.lr_ptr = lr_t->data_ptr<float>();
  }
  a.grad_scale = opt_scalar(grad_scale, "grad_scale");
  a.found_inf = opt_scalar(found_inf, "found_inf");
  auto P = ptrs(params), G = ptrs(grads);
  std::vector<void*> B = momentum != 0.0 ? ptrs(bufs) : std::vector<void*>();
  auto N = numels(params);
  DeviceSwitch sw(params[0].device().index());
  B200_KERNEL_CALL(b200_multi_tensor_sgd((int)P.size(), kdtype(params[0].scalar_type()), kdtype(grads[0].scalar_type()),
                                         P.data(), G.data(), momentum != 0.0 ? B.data() : nullptr, N.data(), a,
                                         current_raw_stream(params[0])));
}

void fused_sgd_(at::TensorList self, at::TensorList grads, at::TensorList bufs, double weight_decay, double momentum,
                double lr, double dampening, bool nesterov, bool maximize, bool is_first_step,
                const std::optional<at::Tensor>& grad_scale, const std::optional<at::Tensor>& found_inf) {
  if (sgd_fast(self, grads, bufs, momentum)) {
    fused_sgd_common(self, grads, bufs, weight_decay, momentum, lr, nullptr, dampening, nesterov, maximize,
                     is_first_step, grad_scale, found_inf);
    return;
  }
  run_fallback(B200_OP_HANDLE("aten::_fused_sgd_", ""), self, grads, bufs, weight_decay, momentum, lr, dampening,
               nesterov, maximize, is_first_step, grad_scale, found_inf);
}

void fused_sgd_tensor_lr_(at::TensorList self, at::TensorList grads, at::TensorList bufs, double weight_decay,
                          double momentum, const at::Tensor& lr, double dampening, bool nesterov, bool maximize,
                          bool is_first_step, const std::optional<at::Tensor>& grad_scale,
                          const std::optional<at::Tensor>& found_inf) {
  if (sgd_fast(self, grads, bufs, momentum)) {
    fused_sgd_common(self, grads, bufs, weight_decay, momentum, 0.0, &lr, dampening, nesterov, maximize, is_first_step,
                     grad_scale, found_inf);
    return;
  }
  run_fallback(B200_OP_HANDLE("aten::_fused_sgd_", "tensor_lr"), self, grads, bufs, weight_decay, momentum, lr,
               dampening, nesterov, maximize, is_first_step, grad_scale, found_inf);
}

// ------------------------------------------------------------------ AMP
void amp_unscale_(at::TensorList self, at::Tensor& found_inf, const at::Tensor& inv_scale) {
  if (self.empty()) return;
  if (dense_list(self) && on_device(found_inf) && found_inf.scalar_type() == at::kFloat &&
      on_device(inv_scale) && inv_scale.scalar_type() == at::kFloat) {
    // group by dtype: the kernel takes one dtype per launch
    for (auto dt : {at::kFloat, at::kBFloat16, at::kHalf}) {
      std::vector<void*> P;
      std::vector<int64_t> N;
      for (const auto& t : self)
        if (t.scalar_type() == dt) { P.push_back(t.data_ptr()); N.push_back(t.numel()); }
      if (P.empty()) continue;
      DeviceSwitch sw(self[0].device().index());
      B200_KERNEL_CALL(b200_multi_tensor_scale((int)P.size(), kdtype(dt), P.data(), N.data(), inv_scale.data_ptr<float>(),
                                               1.f, found_inf.data_ptr<float>(), current_raw_stream(self[0])));
    }
    return;
  }
  run_fallback(B200_OP_HANDLE("aten::_amp_foreach_non_finite_check_and_unscale_", ""), self, found_inf, inv_scale);
}

at::Tensor& amp_update_scale_(at::Tensor& self, at::Tensor& growth_tracker, const at::Tensor& found_inf,
                              double growth, double backoff, int64_t interval) {
  TORCH_CHECK(on_device(self) && on_device(growth_tracker) && on_device(found_inf), "_amp_update_scale_: device mismatch");
  TORCH_CHECK(self.scalar_type() == at::kFloat && found_inf.scalar_type() == at::kFloat &&
                  growth_tracker.scalar_type() == at::kInt && self.numel() == 1 && growth_tracker.numel() == 1,
              "_amp_update_scale_: expected float32 scale/found_inf and int32 growth_tracker scalars");
  DeviceSwitch sw(self.device().index());
  B200_KERNEL_CALL(b200_amp_update_scale(self.data_ptr<float>(), growth_tracker.data_ptr<int>(),
                                         found_inf.data_ptr<float>(), (float)growth, (float)backoff, (int)interval,
                                         current_raw_stream(self)));
  return self;
}

// ------------------------------------------------------------------ L2 norm
std::tuple<at::Tensor, at::Tensor> multi_tensor_l2norm(at::TensorList tensors, bool per_tensor) {
  TORCH_CHECK(!tensors.empty(), "multi_tensor_l2norm: empty tensor list");
  TORCH_CHECK(dense_list(tensors) && same_dtype(tensors),
              "multi_tensor_l2norm: tensors must be dense blackwell tensors of one floating dtype");
  const int n = (int)tensors.size();
  auto opts = tensors[0].options().dtype(at::kFloat);
  at::Tensor total = at::empty({1}, opts);
  at::Tensor per = per_tensor ? at::empty({n}, opts) : at::Tensor();
  at::Tensor scratch = at::empty({(int64_t)b200_multi_tensor_l2norm_scratch_floats(n)}, opts);
  auto P = ptrs(tensors);
  auto N = numels(tensors);
  DeviceSwitch sw(tensors[0].device().index());
  B200_KERNEL_CALL(b200_multi_tensor_l2norm(n, kdtype(tensors[0].scalar_type()), P.data(), N.data(),
                                            total.data_ptr<float>(), per_tensor ? per.data_ptr<float>() : nullptr,
                                            scratch.data_ptr<float>(), current_raw_stream(tensors[0])));
  return {total, per_tensor ? per : at::empty({0}, opts)};
}

std::vector<at::Tensor> foreach_norm(at::TensorList self, const at::Scalar& ord, std::optional<at::ScalarType> dtype) {
  bool two = (ord.isIntegral(false) && ord.toLong() == 2) || (ord.isFloatingPoint() && ord.toDouble() == 2.0);
  if (two && !self.empty() && dense_list(self) && same_dtype(self) && (!dtype.has_value() || *dtype == at::kFloat ||
                                                                       *dtype == self[0].scalar_type())) {
    auto r = multi_tensor_l2norm(self, true);
    at::Tensor per = std::get<1>(r);
    at::ScalarType odt = dtype.value_or(self[0].scalar_type());
    if (odt != at::kFloat) per = per.to(odt);
    std::vector<at::Tensor> out;
    out.reserve(self.size());
    for (int64_t i = 0; i < (int64_t)self.size(); ++i) out.push_back(per.select(0, i));
    return out;
  }
  auto st = run_fallback(B200_OP_HANDLE("aten::_foreach_norm", "Scalar"), self, ord, dtype);
  return st.back().toTensorVector();
}

void multi_tensor_scale_(at::TensorList tensors, const std::optional<at::Tensor>& inv_scale, double scale,
                         at::Tensor& found_inf) {
  if (tensors.empty()) return;
  TORCH_CHECK(dense_list(tensors) && same_dtype(tensors), "multi_tensor_scale_: dense blackwell tensors of one dtype");
  auto P = ptrs(tensors);
  auto N = numels(tensors);
  DeviceSwitch sw(tensors[0].device().index());
  B200_KERNEL_CALL(b200_multi_tensor_scale((int)P.size(), kdtype(tensors[0].scalar_type()), P.data(), N.data(),
                                           opt_scalar(inv_scale, "inv_scale"), (float)scale,
                                           found_inf.defined() ? found_inf.data_ptr<float>() : nullptr,
                                           current_raw_stream(tensors[0])));
}

void multi_tensor_axpby_(at::TensorList out, at::TensorList x, at::TensorList y, double a, double b) {
  if (out.empty()) return;
  TORCH_CHECK(dense_list(out) && dense_list(x) && same_dtype(out) && x.size() == out.size() &&
                  (y.empty() || y.size() == out.size()),
              "multi_tensor_axpby_: list mismatch");
  auto O = ptrs(out), X = ptrs(x);
  std::vector<void*> Y = y.empty() ? std::vector<void*>() : ptrs(y);
  auto N = numels(out);
  DeviceSwitch sw(out[0].device().index());
  B200_KERNEL_CALL(b200_multi_tensor_axpby((int)O.size(), kdtype(out[0].scalar_type()), O.data(), X.data(),
                                           y.empty() ? nullptr : Y.data(), N.data(), (float)a, (float)b,
                                           current_raw_stream(out[0])));
}

void multi_tensor_lamb_(at::TensorList params, at::TensorList grads, at::TensorList ea, at::TensorList es, double lr,
                        double beta1, double beta2, double eps, double wd, int64_t step, bool bias_correction,
                        bool grad_averaging, bool adam_w_mode, double max_grad_norm, bool use_nvlamb,
                        const std::optional<at::Tensor>& global_grad_norm) {
  if (params.empty()) return;
  TORCH_CHECK(dense_list(params) && dense_list(grads) && dense_list(ea) && dense_list(es) && same_dtype(params) &&
                  grads[0].scalar_type() == params[0].scalar_type() && ea[0].scalar_type() == params[0].scalar_type(),
              "multi_tensor_lamb_: params, grads and moments must be dense blackwell tensors of one dtype");
  b200_lamb_args_t a{};
  a.lr = (float)lr; a.beta1 = (float)beta1; a.beta2 = (float)beta2; a.eps = (float)eps; a.weight_decay = (float)wd;
  a.max_grad_norm = (float)max_grad_norm; a.step = (int)step; a.bias_correction = bias_correction;
  a.grad_averaging = grad_averaging; a.adam_w_mode = adam_w_mode; a.use_nvlamb = use_nvlamb;
  a.global_grad_norm = opt_scalar(global_grad_norm, "global_grad_norm");
  auto P = ptrs(params), G = ptrs(grads), M = ptrs(ea), V = ptrs(es);
  auto N = numels(params);
  at::Tensor scratch = at::empty({(int64_t)b200_multi_tensor_lamb_scratch_floats((int)P.size(), N.data())},
                                 params[0].options().dtype(at::kFloat));
  DeviceSwitch sw(params[0].device().index());
  B200_KERNEL_CALL(b200_multi_tensor_lamb((int)P.size(), kdtype(params[0].scalar_type()), P.data(), G.data(), M.data(),
                                          V.data(), N.data(), a, scratch.data_ptr<float>(),
                                          current_raw_stream(params[0])));
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("_fused_adamw_", TORCH_FN(fused_adamw_));
  m.impl("_fused_adamw_.tensor_lr", TORCH_FN(fused_adamw_tensor_lr_));
  m.impl("_fused_adam_", TORCH_FN(fused_adam_));
  m.impl("_fused_adam_.tensor_lr", TORCH_FN(fused_adam_tensor_lr_));
  m.impl("_fused_sgd_", TORCH_FN(fused_sgd_));
  m.impl("_fused_sgd_.tensor_lr", TORCH_FN(fused_sgd_tensor_lr_));
  m.impl("_amp_foreach_non_finite_check_and_unscale_", TORCH_FN(amp_unscale_));
  m.impl("_amp_update_scale_", TORCH_FN(amp_update_scale_));
  m.impl("_foreach_norm.Scalar", TORCH_FN(foreach_norm));
}

TORCH_LIBRARY_IMPL(blackwell, PrivateUse1, m) {
  m.impl("multi_tensor_l2norm", TORCH_FN(multi_tensor_l2norm));
  m.impl("multi_tensor_scale_", TORCH_FN(multi_tensor_scale_));
  m.impl("multi_tensor_axpby_", TORCH_FN(multi_tensor_axpby_));
  m.impl("multi_tensor_lamb_", TORCH_FN(multi_tensor_lamb_));
}

}  // namespace ops
}  // namespace b200
