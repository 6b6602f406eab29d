// Loss functions composed from the backend's own pointwise, gather / scatter and reduce kernels: mean squared error,
// negative log likelihood (class weights, ignore_index, 2-D inputs) and binary cross entropy, forward and backward.
// (Cross entropy over logits has its own fused online-softmax kernels: kernels/softmax_loss.cu.)  KL divergence,
// L1 and BCE-with-logits are composite in ATen and reach the same kernels without help.
// Parity: reference torch_musa/csrc/aten/ops/Loss.cpp (vendor-library NLL / MSE / BCE / KL kernels).
#include "aten/FallbackCall.h"
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <ATen/TensorOperators.h>
#include <ATen/core/Reduction.h>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {

bool floaty(const at::Tensor& t) {
  return on_device(t) && t.layout() == c10::kStrided && c10::isFloatingType(t.scalar_type()) && !t.is_quantized();
}

at::Tensor reduce_loss(const at::Tensor& per_elem, int64_t reduction) {
  if (reduction == at::Reduction::Mean) return per_elem.mean();
  if (reduction == at::Reduction::Sum) return per_elem.sum();
  return per_elem;
}

// ------------------------------------------------------------------------------------------------ MSE
at::Tensor mse_loss(const at::Tensor& self, const at::Tensor& target, int64_t reduction) {
  if (floaty(self) && floaty(target) && self.device() == target.device()) {
    at::Tensor d = at::sub(self, target);
    return reduce_loss(at::mul(d, d), reduction);
  }
  return fallback_tensor(B200_OP_HANDLE("aten::mse_loss", ""), self, target, reduction);
}
at::Tensor mse_loss_backward(const at::Tensor& grad, const at::Tensor& self, const at::Tensor& target, int64_t reduction) {
  if (floaty(self) && floaty(target) && floaty(grad) && self.device() == target.device()) {
    const double norm = reduction == at::Reduction::Mean ? 2.0 / (double)std::max<int64_t>(self.numel(), 1) : 2.0;
    return at::mul(at::mul(at::sub(self, target), norm), grad);
  }
  return fallback_tensor(B200_OP_HANDLE("aten::mse_loss_backward", ""), grad, self, target, reduction);
}

// ------------------------------------------------------------------------------------------------ NLL
// self [N, C] (or [C]) log-probabilities, target [N] (or scalar) class indices
std::tuple<at::Tensor, at::Tensor> nll_loss_forward(const at::Tensor& self, const at::Tensor& target,
                                                    const std::optional<at::Tensor>& weight, int64_t reduction,
                                                    c10::SymInt ignore_index_) {
  const int64_t ignore_index = ignore_index_.expect_int();
  if (floaty(self) && on_device(target) && target.scalar_type() == at::kLong && self.dim() >= 1 && self.dim() <= 2 &&
      (!weight || !weight->defined() || floaty(*weight))) {
    at::Tensor x = self.dim() == 1 ? self.unsqueeze(0) : self;
    at::Tensor t = target.dim() == 0 ? target.unsqueeze(0) : target;
    at::Tensor keep = at::ne(t, ignore_index);
    at::Tensor safe = at::where(keep, t, at::zeros_like(t));
    at::Tensor picked = at::neg(at::gather(x, 1, safe.unsqueeze(1)).squeeze(1));
    at::Tensor w = (weight && weight->defined()) ? at::index_select(*weight, 0, safe).to(x.scalar_type())
                                                 : at::ones_like(picked);
    w = at::mul(w, keep.to(w.scalar_type()));
    at::Tensor per = at::mul(picked, w);
    at::Tensor total = w.sum();
    if (reduction == at::Reduction::None) return {self.dim() == 1 ? per.squeeze(0) : per, total};
    at::Tensor s = per.sum();
    if (reduction == at::Reduction::Mean) s = at::div(s, total);
    return {s, total};
  }
  auto st = run_fallback(B200_OP_HANDLE("aten::nll_loss_forward", ""), self, target, weight, reduction, ignore_index_);
  return {st[0].toTensor(), st[1].toTensor()};
}
at::Tensor nll_loss_backward(const at::Tensor& grad, const at::Tensor& self, const at::Tensor& target,
                             const std::optional<at::Tensor>& weight, int64_t reduction, c10::SymInt ignore_index_,
                             const at::Tensor& total_weight) {
  const int64_t ignore_index = ignore_index_.expect_int();
  if (floaty(self) && floaty(grad) && on_device(target) && target.scalar_type() == at::kLong && self.dim() >= 1 &&
      self.dim() <= 2 && (!weight || !weight->defined() || floaty(*weight))) {
    at::Tensor x = self.dim() == 1 ? self.unsqueeze(0) : self;
    at::Tensor t = target.dim() == 0 ? target.unsqueeze(0) : target;
    at::Tensor keep = at::ne(t, ignore_index);
    at::Tensor safe = at::where(keep, t, at::zeros_like(t));
    at::Tensor w = (weight && weight->defined()) ? at::index_select(*weight, 0, safe).to(x.scalar_type())
                                                 : at::ones({t.size(0)}, x.options());
    w = at::neg(at::mul(w, keep.to(w.scalar_type())));
    at::Tensor g = grad.to(x.scalar_type());
    if (reduction == at::Reduction::None) w = at::mul(w, g.dim() == 0 ? g.unsqueeze(0) : g);
    else if (reduction == at::Reduction::Mean) w = at::mul(w, at::div(g, total_weight.to(x.scalar_type())));
    else w = at::mul(w, g);
    at::Tensor gi = at::zeros_like(x, at::MemoryFormat::Contiguous);
    gi.scatter_(1, safe.unsqueeze(1), w.unsqueeze(1));
    return self.dim() == 1 ? gi.squeeze(0) : gi;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::nll_loss_backward", ""), grad, self, target, weight, reduction,
                         ignore_index_, total_weight);
}

// ------------------------------------------------------------------------------------------------ BCE
at::Tensor binary_cross_entropy(const at::Tensor& self, const at::Tensor& target, const std::optional<at::Tensor>& weight,
                                int64_t reduction) {
  if (floaty(self) && floaty(target) && (!weight || !weight->defined() || floaty(*weight))) {
    // -(t * max(log x, -100) + (1 - t) * max(log(1 - x), -100))
    at::Tensor lx = at::clamp_min(at::log(self), -100.0);
    at::Tensor l1x = at::clamp_min(at::log(at::rsub(self, 1.0)), -100.0);
    at::Tensor per = at::neg(at::add(at::mul(target, lx), at::mul(at::rsub(target, 1.0), l1x)));
    if (weight && weight->defined()) per = at::mul(per, *weight);
    return reduce_loss(per, reduction);
  }
  return fallback_tensor(B200_OP_HANDLE("aten::binary_cross_entropy", ""), self, target, weight, reduction);
}
at::Tensor binary_cross_entropy_backward(const at::Tensor& grad, const at::Tensor& self, const at::Tensor& target,
                                         const std::optional<at::Tensor>& weight, int64_t reduction) {
  if (floaty(self) && floaty(target) && floaty(grad) && (!weight || !weight->defined() || floaty(*weight))) {
    // (x - t) / max(x (1 - x), eps) * grad
    at::Tensor denom = at::clamp_min(at::mul(self, at::rsub(self, 1.0)), 1e-12);
    at::Tensor gi = at::mul(at::div(at::sub(self, target), denom), grad);
    if (weight && weight->defined()) gi = at::mul(gi, *weight);
    if (reduction == at::Reduction::Mean) gi = at::div(gi, (double)std::max<int64_t>(self.numel(), 1));
    return gi;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::binary_cross_entropy_backward", ""), grad, self, target, weight, reduction);
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("mse_loss", TORCH_FN(mse_loss));
  m.impl("mse_loss_backward", TORCH_FN(mse_loss_backward));
  m.impl("nll_loss_forward", TORCH_FN(nll_loss_forward));
  m.impl("nll_loss_backward", TORCH_FN(nll_loss_backward));
  m.impl("binary_cross_entropy", TORCH_FN(binary_cross_entropy));
  m.impl("binary_cross_entropy_backward", TORCH_FN(binary_cross_entropy_backward));
}

}  // namespace
}  // namespace ops
}  // namespace b200
