// Batch normalisation on the hand-written channels-last kernels.
//
// `native_batch_norm` (+ the `_native_batch_norm_legit` spellings) and `native_batch_norm_backward` take the
// fast path for bf16/fp16 activations that are a [P, C] matrix in memory (4-D channels-last, or 2-D) with
// fp32 affine parameters and statistics -- the autocast training setup -- and the library kernels otherwise.
// `blackwell::batch_norm_act(+_backward)` is the fused form: normalise + affine (+ residual add) (+ ReLU) in
// the same pass, backward recomputing the ReLU mask from the saved output and emitting the residual gradient.
// Parity: reference torch_musa/csrc/aten/ops/BatchNorm.cpp; fused Conv+BN+activation modules in
// torch_musa/core/ao.
#include "aten/FallbackCall.h"
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {

using Opt = std::optional<at::Tensor>;

bool defined(const Opt& t) { return t.has_value() && t->defined(); }

// The [P, C] matrix behind `t` (no copy), or P = 0 when the layout does not allow it.
struct Mat { int64_t P = 0; int64_t C = 0; };
Mat as_matrix(const at::Tensor& t) {
  Mat m;
  if (t.dim() == 2 && t.is_contiguous()) { m.P = t.size(0); m.C = t.size(1); return m; }
  if (t.dim() != 4) return m;
  const int64_t N = t.size(0), C = t.size(1), H = t.size(2), W = t.size(3);
  if ((C > 1 && t.stride(1) != 1) || (W > 1 && t.stride(3) != C) || (H > 1 && t.stride(2) != W * C) ||
      (N > 1 && t.stride(0) != H * W * C))
    return m;
  m.P = N * H * W;
  m.C = C;
  return m;
}

bool f32_vec(const Opt& t, int64_t C) {
  return !defined(t) || (on_device(*t) && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == C);
}

bool bn_fast(const at::Tensor& x, const Opt& w, const Opt& b, const Opt& rm, const Opt& rv) {
  if (!on_device(x) || (x.scalar_type() != at::kBFloat16 && x.scalar_type() != at::kHalf)) return false;
  const Mat m = as_matrix(x);
  if (m.P == 0 || m.C % 8 != 0) return false;
  return f32_vec(w, m.C) && f32_vec(b, m.C) && f32_vec(rm, m.C) && f32_vec(rv, m.C);
}

const float* fptr(const Opt& t) { return defined(t) ? t->const_data_ptr<float>() : nullptr; }
float* fptr_mut(const Opt& t) { return defined(t) ? t->data_ptr<float>() : nullptr; }

std::tuple<at::Tensor, at::Tensor, at::Tensor> bn_forward(const at::Tensor& x, const Opt& w, const Opt& b, const Opt& rm,
                                                          const Opt& rv, const Opt& resid, bool training,
                                                          double momentum, double eps, bool relu) {
  const Mat m = as_matrix(x);
  auto stream = current_raw_stream(x);
  const int dt = kdtype(x.scalar_type());
  at::Tensor y = at::empty_like(x);
  auto fopt = x.options().dtype(at::kFloat);
  at::Tensor save_mean, save_invstd, sums;
  const void* rp = nullptr;
  if (defined(resid)) {
    check_devices("batch_norm_act", x, *resid);
    TORCH_CHECK(resid->sizes() == x.sizes() && resid->strides() == x.strides() && resid->scalar_type() == x.scalar_type(),
                "batch_norm_act: the residual must have the layout and dtype of the input");
    rp = resid->const_data_ptr();
  }
  if (training) {
    sums = at::empty({2 * m.C}, fopt);
    save_mean = at::empty({m.C}, fopt);
    save_invstd = at::empty({m.C}, fopt);
    B200_KERNEL_CALL(b200_bn_stats(dt, x.const_data_ptr(), sums.data_ptr<float>(), m.P, (int)m.C, stream));
    B200_KERNEL_CALL(b200_bn_apply(dt, x.const_data_ptr(), rp, y.mutable_data_ptr(), sums.data_ptr<float>(), fptr(w),
                                   fptr(b), fptr_mut(rm), fptr_mut(rv), save_mean.data_ptr<float>(),
                                   save_invstd.data_ptr<float>(), m.P, (int)m.C, (float)eps, (float)momentum,
                                   relu ? 1 : 0, 0, stream));
  } else {
    TORCH_CHECK(defined(rm) && defined(rv), "batch_norm in evaluation mode needs running statistics");
    save_mean = at::empty({0}, fopt);
    save_invstd = at::empty({0}, fopt);
    B200_KERNEL_CALL(b200_bn_apply(dt, x.const_data_ptr(), rp, y.mutable_data_ptr(), nullptr, fptr(w), fptr(b),
                                   fptr_mut(rm), fptr_mut(rv), nullptr, nullptr, m.P, (int)m.C, (float)eps,
                                   (float)momentum, relu ? 1 : 0, 1, stream));
  }
  return {y, save_mean, save_invstd};
}

// returns (dx, dweight, dbias, dresidual)
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> bn_backward(const at::Tensor& dy_in, const at::Tensor& x,
                                                                       const Opt& y, const Opt& w,
                                                                       const at::Tensor& mean, const at::Tensor& invstd,
                                                                       bool relu, bool want_resid) {
  const Mat m = as_matrix(x);
  auto stream = current_raw_stream(x);
  const int dt = kdtype(x.scalar_type());
  check_devices("batch_norm_backward", x, dy_in, y, w, mean, invstd);
  at::Tensor dy = dy_in;
  if (dy.scalar_type() != x.scalar_type()) dy = dy.to(x.scalar_type());
  if (dy.strides() != x.strides()) {
    at::Tensor t = at::empty_like(x);
    t.copy_(dy);
    dy = t;
  }
  const void* yp = nullptr;
  if (relu) {
    TORCH_CHECK(defined(y) && y->strides() == x.strides(), "batch_norm_act_backward needs the saved output");
    yp = y->const_data_ptr();
  }
  at::Tensor sums = at::empty({2 * m.C}, x.options().dtype(at::kFloat));
  at::Tensor dx = at::empty_like(x);
  at::Tensor dres = want_resid ? at::empty_like(x) : at::Tensor();
  B200_KERNEL_CALL(b200_bn_bwd_reduce(dt, dy.const_data_ptr(), x.const_data_ptr(), yp, mean.const_data_ptr<float>(),
                                      invstd.const_data_ptr<float>(), sums.data_ptr<float>(), m.P, (int)m.C,
                                      relu ? 1 : 0, stream));
  B200_KERNEL_CALL(b200_bn_bwd_apply(dt, dy.const_data_ptr(), x.const_data_ptr(), yp, mean.const_data_ptr<float>(),
                                     invstd.const_data_ptr<float>(), fptr(w), sums.data_ptr<float>(),
                                     dx.mutable_data_ptr(), want_resid ? dres.mutable_data_ptr() : nullptr, m.P,
                                     (int)m.C, relu ? 1 : 0, stream));
  return {dx, sums.narrow(0, m.C, m.C), sums.narrow(0, 0, m.C), dres};
}

// ------------------------------------------------------------------ aten entry points
std::tuple<at::Tensor, at::Tensor, at::Tensor> bn_native(const at::Tensor& x, const Opt& w, const Opt& b,
                                                                 const Opt& rm, const Opt& rv, bool training,
                                                                 double momentum, double eps) {
  if (bn_fast(x, w, b, rm, rv) && (training || (defined(rm) && defined(rv))))
    return bn_forward(x, w, b, rm, rv, std::nullopt, training, momentum, eps, false);
  auto st = run_fallback(B200_OP_HANDLE("aten::native_batch_norm", ""), x, w, b, rm, rv, training, momentum, eps);
  return {st[0].toTensor(), st[1].toTensor(), st[2].toTensor()};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> legit(const at::Tensor& x, const Opt& w, const Opt& b, at::Tensor& rm,
                                                     at::Tensor& rv, bool training, double momentum, double eps) {
  return bn_native(x, w, b, Opt(rm), Opt(rv), training, momentum, eps);
}
std::tuple<at::Tensor, at::Tensor, at::Tensor> legit_no_stats(const at::Tensor& x, const Opt& w, const Opt& b,
                                                              bool training, double momentum, double eps) {
  return bn_native(x, w, b, Opt(), Opt(), training, momentum, eps);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> bn_native_backward(const at::Tensor& dy, const at::Tensor& x,
                                                                          const Opt& w, const Opt& rm, const Opt& rv,
                                                                          const Opt& save_mean, const Opt& save_invstd,
                                                                          bool train, double eps,
                                                                          std::array<bool, 3> mask) {
  if (train && defined(save_mean) && defined(save_invstd) && save_mean->numel() > 0 &&
      bn_fast(x, w, std::nullopt, std::nullopt, std::nullopt) && save_mean->scalar_type() == at::kFloat &&
      save_invstd->scalar_type() == at::kFloat) {
    auto [dx, dw, db, dres] = bn_backward(dy, x, std::nullopt, w, *save_mean, *save_invstd, false, false);
    (void)dres;
    return {mask[0] ? dx : at::Tensor(), (mask[1] && defined(w)) ? dw : at::Tensor(), mask[2] ? db : at::Tensor()};
  }
  c10::List<bool> m;
  m.push_back(mask[0]); m.push_back(mask[1]); m.push_back(mask[2]);
  auto st = run_fallback(B200_OP_HANDLE("aten::native_batch_norm_backward", ""), dy, x, w, rm, rv, save_mean,
                         save_invstd, train, eps, m);
  auto pick = [&](size_t i) { return st[i].isTensor() ? st[i].toTensor() : at::Tensor(); };
  return {pick(0), pick(1), pick(2)};
}

// ------------------------------------------------------------------ fused custom ops
std::tuple<at::Tensor, at::Tensor, at::Tensor> batch_norm_act(const at::Tensor& x, const Opt& w, const Opt& b,
                                                              const Opt& rm, const Opt& rv, const Opt& resid,
                                                              bool training, double momentum, double eps, bool relu) {
  TORCH_CHECK(bn_fast(x, w, b, rm, rv),
              "blackwell::batch_norm_act needs bf16/fp16 channels-last (or 2-D) input with C % 8 == 0 and fp32 "
              "parameters / statistics");
  return bn_forward(x, w, b, rm, rv, resid, training, momentum, eps, relu);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> batch_norm_act_backward(
    const at::Tensor& dy, const at::Tensor& x, const Opt& y, const Opt& w, const at::Tensor& save_mean,
    const at::Tensor& save_invstd, bool relu, bool has_residual) {
  auto [dx, dw, db, dres] = bn_backward(dy, x, y, w, save_mean, save_invstd, relu, has_residual);
  if (!has_residual) dres = at::empty({0}, x.options());
  return {dx, dw, db, dres};
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("native_batch_norm", TORCH_FN(bn_native));
  m.impl("_native_batch_norm_legit", TORCH_FN(legit));
  m.impl("_native_batch_norm_legit.no_stats", TORCH_FN(legit_no_stats));
  m.impl("native_batch_norm_backward", TORCH_FN(bn_native_backward));
}

TORCH_LIBRARY_FRAGMENT(blackwell, m) {
  m.def("batch_norm_act(Tensor input, Tensor? weight, Tensor? bias, Tensor(a!)? running_mean, Tensor(b!)? running_var, "
        "Tensor? residual, bool training, float momentum, float eps, bool relu) -> (Tensor, Tensor, Tensor)");
  m.def("batch_norm_act_backward(Tensor grad_out, Tensor input, Tensor? out, Tensor? weight, Tensor save_mean, "
        "Tensor save_invstd, bool relu, bool has_residual) -> (Tensor, Tensor, Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(blackwell, PrivateUse1, m) {
  m.impl("batch_norm_act", TORCH_FN(batch_norm_act));
  m.impl("batch_norm_act_backward", TORCH_FN(batch_norm_act_backward));
}

}  // namespace ops
}  // namespace b200
