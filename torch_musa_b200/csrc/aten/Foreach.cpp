// The _foreach_* pointwise family on the multi-tensor-apply kernel: a whole parameter list per launch instead of one
// launch per tensor.  Lists that the kernel does not cover (mixed dtypes, strided views, integer tensors, another
// device among them) run tensor by tensor on the general pointwise loops.
// Parity: reference torch_musa/csrc/aten/ops/musa/ForeachBinaryOpScalar.mu, ForeachBinaryOpList.mu,
// ForeachPointwiseOp.mu, ForeachUnaryOp.mu (ports of ATen's foreach kernels).
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {

bool fast_list(at::TensorList l, const at::Tensor& ref) {
  for (const auto& t : l)
    if (!on_device(t) || t.device() != ref.device() || t.scalar_type() != ref.scalar_type() || kdtype(t.scalar_type()) < 0 ||
        !t.is_non_overlapping_and_dense() || t.is_conj() || t.is_neg())
      return false;
  return true;
}
bool same_layout(at::TensorList a, at::TensorList b) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i)
    if (a[i].sizes() != b[i].sizes() || a[i].strides() != b[i].strides()) return false;
  return true;
}
std::vector<void*> ptrs_of(at::TensorList l) {
  std::vector<void*> v;
  v.reserve(l.size());
  for (const auto& t : l) v.push_back(t.data_ptr());
  return v;
}

// out = f(a[, b[, c]]); returns false when the lists are not covered
bool run_lists(int op, at::TensorList out, at::TensorList a, at::TensorList b, at::TensorList c, double s0, double s1) {
  if (out.empty()) return true;
  const at::Tensor& ref = out[0];
  if (!fast_list(out, ref) || !fast_list(a, ref) || !same_layout(out, a)) return false;
  if (!b.empty() && (!fast_list(b, ref) || !same_layout(out, b))) return false;
  if (!c.empty() && (!fast_list(c, ref) || !same_layout(out, c))) return false;
  auto O = ptrs_of(out), A = ptrs_of(a);
  std::vector<void*> B = b.empty() ? std::vector<void*>() : ptrs_of(b);
  std::vector<void*> C = c.empty() ? std::vector<void*>() : ptrs_of(c);
  std::vector<int64_t> N;
  for (const auto& t : out) N.push_back(t.numel());
  DeviceSwitch sw(ref.device().index());
  int e = b200_multi_tensor_pointwise(op, (int)O.size(), kdtype(ref.scalar_type()), O.data(), A.data(),
                                      b.empty() ? nullptr : B.data(), c.empty() ? nullptr : C.data(), N.data(), (float)s0,
                                      (float)s1, current_raw_stream(ref));
  if (e == (int)cudaErrorNotSupported) return false;
  B200_KERNEL_CALL(e);
  return true;
}

std::vector<at::Tensor> like_list(at::TensorList l) {
  std::vector<at::Tensor> v;
  v.reserve(l.size());
  for (const auto& t : l) v.push_back(at::empty_strided(t.sizes(), t.strides(), t.options()));
  return v;
}

// ---- in-place and functional forms built from one description ---------------------------------------------
#define FE_SCALAR(NAME, OP, SLOW)                                                                         \
  void NAME##_scalar_(at::TensorList self, const at::Scalar& s) {                                         \
    if (!s.isComplex() && run_lists(OP, self, self, {}, {}, s.toDouble(), 0.0)) return;                   \
    for (auto& t : self) { at::Tensor x = t; SLOW; }                                                      \
  }                                                                                                       \
  std::vector<at::Tensor> NAME##_scalar(at::TensorList self, const at::Scalar& s) {                       \
    std::vector<at::Tensor> out = like_list(self);                                                        \
    if (!s.isComplex() && run_lists(OP, out, self, {}, {}, s.toDouble(), 0.0)) return out;                \
    out.clear();                                                                                          \
    for (const auto& t : self) { at::Tensor x = t.clone(); SLOW; out.push_back(x); }                      \
    return out;                                                                                           \
  }
FE_SCALAR(fe_add, B200_FE_ADD_SCALAR, x.add_(s))
FE_SCALAR(fe_mul, B200_FE_MUL_SCALAR, x.mul_(s))
FE_SCALAR(fe_div, B200_FE_DIV_SCALAR, x.div_(s))

void fe_add_list_(at::TensorList self, at::TensorList other, const at::Scalar& alpha) {
  TORCH_CHECK(self.size() == other.size(), "Tensor lists must have the same number of tensors");
  if (!alpha.isComplex() && run_lists(B200_FE_ADD, self, self, other, {}, alpha.toDouble(), 0.0)) return;
  for (size_t i = 0; i < self.size(); ++i) { at::Tensor x = self[i]; x.add_(other[i], alpha); }
}
std::vector<at::Tensor> fe_add_list(at::TensorList self, at::TensorList other, const at::Scalar& alpha) {
  TORCH_CHECK(self.size() == other.size(), "Tensor lists must have the same number of tensors");
  std::vector<at::Tensor> out = like_list(self);
  if (!alpha.isComplex() && run_lists(B200_FE_ADD, out, self, other, {}, alpha.toDouble(), 0.0)) return out;
  out.clear();
  for (size_t i = 0; i < self.size(); ++i) out.push_back(at::add(self[i], other[i], alpha));
  return out;
}
void fe_sub_list_(at::TensorList self, at::TensorList other, const at::Scalar& alpha) {
  TORCH_CHECK(self.size() == other.size(), "Tensor lists must have the same number of tensors");
  if (!alpha.isComplex() && run_lists(B200_FE_ADD, self, self, other, {}, -alpha.toDouble(), 0.0)) return;
  for (size_t i = 0; i < self.size(); ++i) { at::Tensor x = self[i]; x.sub_(other[i], alpha); }
}

#define FE_LIST(NAME, OP, SLOW_INPLACE, SLOW_FN)                                                          \
  void NAME##_list_(at::TensorList self, at::TensorList other) {                                          \
    TORCH_CHECK(self.size() == other.size(), "Tensor lists must have the same number of tensors");        \
    if (run_lists(OP, self, self, other, {}, 1.0, 0.0)) return;                                           \
    for (size_t i = 0; i < self.size(); ++i) { at::Tensor x = self[i]; const at::Tensor& y = other[i]; SLOW_INPLACE; } \
  }                                                                                                       \
  std::vector<at::Tensor> NAME##_list(at::TensorList self, at::TensorList other) {                        \
    TORCH_CHECK(self.size() == other.size(), "Tensor lists must have the same number of tensors");        \
    std::vector<at::Tensor> out = like_list(self);                                                        \
    if (run_lists(OP, out, self, other, {}, 1.0, 0.0)) return out;                                        \
    out.clear();                                                                                          \
    for (size_t i = 0; i < self.size(); ++i) { const at::Tensor& x = self[i]; const at::Tensor& y = other[i]; out.push_back(SLOW_FN); } \
    return out;                                                                                           \
  }
FE_LIST(fe_mul, B200_FE_MUL, x.mul_(y), at::mul(x, y))
FE_LIST(fe_div, B200_FE_DIV, x.div_(y), at::div(x, y))
FE_LIST(fe_maximum, B200_FE_MAXIMUM, x.copy_(at::maximum(x, y)), at::maximum(x, y))
FE_LIST(fe_minimum, B200_FE_MINIMUM, x.copy_(at::minimum(x, y)), at::minimum(x, y))

#define FE_UNARY(NAME, OP, SLOW_INPLACE, SLOW_FN)                                                         \
  void NAME##_(at::TensorList self) {                                                                     \
    if (run_lists(OP, self, self, {}, {}, 0.0, 0.0)) return;                                              \
    for (auto& t : self) { at::Tensor x = t; SLOW_INPLACE; }                                              \
  }                                                                                                       \
  std::vector<at::Tensor> NAME(at::TensorList self) {                                                     \
    std::vector<at::Tensor> out = like_list(self);                                                        \
    if (run_lists(OP, out, self, {}, {}, 0.0, 0.0)) return out;                                           \
    out.clear();                                                                                          \
    for (const auto& x : self) out.push_back(SLOW_FN);                                                    \
    return out;                                                                                           \
  }
FE_UNARY(fe_sqrt, B200_FE_SQRT, x.sqrt_(), at::sqrt(x))
FE_UNARY(fe_neg, B200_FE_NEG, x.neg_(), at::neg(x))
FE_UNARY(fe_reciprocal, B200_FE_RECIPROCAL, x.reciprocal_(), at::reciprocal(x))
FE_UNARY(fe_abs, B200_FE_ABS, x.abs_(), at::abs(x))

void fe_zero_(at::TensorList self) {
  if (run_lists(B200_FE_ZERO, self, self, {}, {}, 0.0, 0.0)) return;
  for (auto& t : self) { at::Tensor x = t; x.zero_(); }
}

#define FE_ADDC(NAME, OP, SLOW)                                                                           \
  void NAME##_scalar_(at::TensorList self, at::TensorList t1, at::TensorList t2, const at::Scalar& v) {   \
    TORCH_CHECK(self.size() == t1.size() && self.size() == t2.size(), "Tensor lists must have the same number of tensors"); \
    if (!v.isComplex() && run_lists(OP, self, self, t1, t2, v.toDouble(), 0.0)) return;                   \
    for (size_t i = 0; i < self.size(); ++i) { at::Tensor x = self[i]; SLOW; }                            \
  }
FE_ADDC(fe_addcmul, B200_FE_ADDCMUL, x.addcmul_(t1[i], t2[i], v))
FE_ADDC(fe_addcdiv, B200_FE_ADDCDIV, x.addcdiv_(t1[i], t2[i], v))

void fe_lerp_scalar_(at::TensorList self, at::TensorList end, const at::Scalar& w) {
  TORCH_CHECK(self.size() == end.size(), "Tensor lists must have the same number of tensors");
  if (!w.isComplex() && run_lists(B200_FE_LERP, self, self, end, {}, w.toDouble(), 0.0)) return;
  for (size_t i = 0; i < self.size(); ++i) { at::Tensor x = self[i]; x.lerp_(end[i], w); }
}

void fe_copy_(at::TensorList self, at::TensorList src, bool non_blocking) {
  TORCH_CHECK(self.size() == src.size(), "Tensor lists must have the same number of tensors");
  if (run_lists(B200_FE_COPY, self, src, {}, {}, 0.0, 0.0)) return;
  for (size_t i = 0; i < self.size(); ++i) { at::Tensor x = self[i]; x.copy_(src[i], non_blocking); }
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("_foreach_add_.Scalar", TORCH_FN(fe_add_scalar_));
  m.impl("_foreach_add.Scalar", TORCH_FN(fe_add_scalar));
  m.impl("_foreach_mul_.Scalar", TORCH_FN(fe_mul_scalar_));
  m.impl("_foreach_mul.Scalar", TORCH_FN(fe_mul_scalar));
  m.impl("_foreach_div_.Scalar", TORCH_FN(fe_div_scalar_));
  m.impl("_foreach_div.Scalar", TORCH_FN(fe_div_scalar));
  m.impl("_foreach_add_.List", TORCH_FN(fe_add_list_));
  m.impl("_foreach_add.List", TORCH_FN(fe_add_list));
  m.impl("_foreach_sub_.List", TORCH_FN(fe_sub_list_));
  m.impl("_foreach_mul_.List", TORCH_FN(fe_mul_list_));
  m.impl("_foreach_mul.List", TORCH_FN(fe_mul_list));
  m.impl("_foreach_div_.List", TORCH_FN(fe_div_list_));
  m.impl("_foreach_div.List", TORCH_FN(fe_div_list));
  m.impl("_foreach_maximum_.List", TORCH_FN(fe_maximum_list_));
  m.impl("_foreach_maximum.List", TORCH_FN(fe_maximum_list));
  m.impl("_foreach_minimum_.List", TORCH_FN(fe_minimum_list_));
  m.impl("_foreach_minimum.List", TORCH_FN(fe_minimum_list));
  m.impl("_foreach_sqrt_", TORCH_FN(fe_sqrt_));
  m.impl("_foreach_sqrt", TORCH_FN(fe_sqrt));
  m.impl("_foreach_neg_", TORCH_FN(fe_neg_));
  m.impl("_foreach_neg", TORCH_FN(fe_neg));
  m.impl("_foreach_reciprocal_", TORCH_FN(fe_reciprocal_));
  m.impl("_foreach_reciprocal", TORCH_FN(fe_reciprocal));
  m.impl("_foreach_abs_", TORCH_FN(fe_abs_));
  m.impl("_foreach_abs", TORCH_FN(fe_abs));
  m.impl("_foreach_zero_", TORCH_FN(fe_zero_));
  m.impl("_foreach_addcmul_.Scalar", TORCH_FN(fe_addcmul_scalar_));
  m.impl("_foreach_addcdiv_.Scalar", TORCH_FN(fe_addcdiv_scalar_));
  m.impl("_foreach_lerp_.Scalar", TORCH_FN(fe_lerp_scalar_));
  m.impl("_foreach_copy_", TORCH_FN(fe_copy_));
}

}  // namespace
}  // namespace ops
}  // namespace b200
