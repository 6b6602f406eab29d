// Pointwise operators on the general loops (aten/Loops.h, kernels/ew_generic.cu): broadcasting, strided views,
// type promotion, Scalars and 0-dim host tensors, all ten element types.  Elementwise.cpp keeps the vectorised
// same-layout fast paths of the hot training operators and falls through to these loops; only what neither covers
// (complex numbers, quantized tensors) reaches the library fallback.
// Parity: reference torch_musa/csrc/aten/ops/{Binary,Unary,Compare,TensorCompare,PointwiseOps,Lerp,Activation}.cpp.
#include "aten/FallbackCall.h"
#include "aten/Loops.h"

#include <ATen/Functions.h>
#include <ATen/native/Resize.h>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {
using loops::In;

enum Rule { kSame, kBool, kFloat };

// out = op(a[, b[, c]]).  `out` undefined: allocated with the promoted dtype; defined: used as is (in-place and
// out= variants; out= is resized to the broadcast shape first).
bool pointwise_into(int op, Rule rule, at::Tensor& out, const In& a, const In& b = In(), const In& c = In(),
                    double p0 = 0.0, double p1 = 0.0, bool resize_out = false,
                    std::optional<at::ScalarType> fixed_dtype = std::nullopt) {
  const at::Tensor* dev = loops::device_operand(a, b, c);
  if (!dev) return false;
  for (const In* i : {&a, &b, &c})
    if (i->present && i->t && (i->t->is_complex() || i->t->is_quantized() || i->t->layout() != c10::kStrided)) return false;
  at::ScalarType common = op == B200_EW_WHERE ? loops::result_type(b, c) : loops::result_type(a, b, c);
  if (op == B200_EW_MASKED_FILL) common = a.t->scalar_type();
  if (c10::isComplexType(common) || loops::any_dtype(common) < 0) return false;
  at::ScalarType dt = common;
  if (rule == kBool) dt = at::kBool;
  else if (rule == kFloat && c10::isIntegralType(common, /*includeBool=*/true)) dt = c10::get_default_dtype_as_scalartype();
  if (fixed_dtype) dt = *fixed_dtype;
  const std::vector<int64_t> shape = loops::broadcast_shape(a, b, c);
  if (!out.defined()) {
    out = loops::make_out(shape, dt, *dev);
  } else if (resize_out) {
    if (out.sizes() != at::IntArrayRef(shape)) at::native::resize_output(out, shape);
  } else if (out.sizes() != at::IntArrayRef(shape)) {
    TORCH_CHECK(false, "output with shape ", out.sizes(), " doesn't match the broadcast shape ", at::IntArrayRef(shape));
  }
  // floating compute although no tensor input is floating: true division of integers, int tensor with a
  // floating Scalar, floating functions of integers
  bool any_float_in = false;
  for (const In* i : {&a, &b, &c})
    if (i->present && !i->scalar && i->t && c10::isFloatingType(i->t->scalar_type())) any_float_in = true;
  const bool float_compute = !any_float_in && (c10::isFloatingType(common) || c10::isFloatingType(dt));
  return loops::run(op, out, a, b, c, p0, p1, float_compute);
}

}  // namespace

// exported for Elementwise.cpp: the general path behind its fast paths
bool generic_binary(int op, at::Tensor& out, const at::Tensor& a, const at::Tensor& b, double alpha, bool float_result,
                    bool resize_out) {
  return pointwise_into(op, float_result ? kFloat : kSame, out, In(a), In(b), In(), alpha, 0.0, resize_out);
}
bool generic_binary_scalar(int op, at::Tensor& out, const at::Tensor& a, const at::Scalar& s, double alpha) {
  return pointwise_into(op, kSame, out, In(a), In(s), In(), alpha);
}
bool generic_unary(int op, at::Tensor& out, const at::Tensor& a, bool float_result, bool resize_out) {
  return pointwise_into(op, float_result ? kFloat : kSame, out, In(a), In(), In(), 0.0, 0.0, resize_out);
}
bool generic_binary_same(int op, at::Tensor& out, const at::Tensor& a, const at::Tensor& b, double p0, double p1) {
  return pointwise_into(op, kSame, out, In(a), In(b), In(), p0, p1);
}

namespace {

// ------------------------------------------------------------------------------------------------ binary
#define B200_PW_BINARY(CNAME, ATEN, OV_F, OV_I, OV_O, OP, RULE)                                              \
  at::Tensor CNAME(const at::Tensor& a, const at::Tensor& b) {                                               \
    at::Tensor out;                                                                                          \
    if (pointwise_into(OP, RULE, out, In(a), In(b))) return out;                                             \
    return fallback_tensor(B200_OP_HANDLE("aten::" ATEN, OV_F), a, b);                                       \
  }                                                                                                          \
  at::Tensor& CNAME##_(at::Tensor& a, const at::Tensor& b) {                                                 \
    if (pointwise_into(OP, RULE, a, In(a), In(b))) return a;                                                 \
    run_fallback(B200_OP_HANDLE("aten::" ATEN "_", OV_I), a, b);                                             \
    return a;                                                                                                \
  }                                                                                                          \
  at::Tensor& CNAME##_out(const at::Tensor& a, const at::Tensor& b, at::Tensor& out) {                       \
    if (pointwise_into(OP, RULE, out, In(a), In(b), In(), 0.0, 0.0, true)) return out;                       \
    run_fallback(B200_OP_HANDLE("aten::" ATEN, OV_O), a, b, out);                                            \
    return out;                                                                                              \
  }
#define B200_PW_BINARY_SCALAR(CNAME, ATEN, OV_F, OV_I, OV_O, OP, RULE)                                       \
  at::Tensor CNAME(const at::Tensor& a, const at::Scalar& b) {                                               \
    at::Tensor out;                                                                                          \
    if (pointwise_into(OP, RULE, out, In(a), In(b))) return out;                                             \
    return fallback_tensor(B200_OP_HANDLE("aten::" ATEN, OV_F), a, b);                                       \
  }                                                                                                          \
  at::Tensor& CNAME##_(at::Tensor& a, const at::Scalar& b) {                                                 \
    if (pointwise_into(OP, RULE, a, In(a), In(b))) return a;                                                 \
    run_fallback(B200_OP_HANDLE("aten::" ATEN "_", OV_I), a, b);                                             \
    return a;                                                                                                \
  }                                                                                                          \
  at::Tensor& CNAME##_out(const at::Tensor& a, const at::Scalar& b, at::Tensor& out) {                       \
    if (pointwise_into(OP, RULE, out, In(a), In(b), In(), 0.0, 0.0, true)) return out;                       \
    run_fallback(B200_OP_HANDLE("aten::" ATEN, OV_O), a, b, out);                                            \
    return out;                                                                                              \
  }

B200_PW_BINARY(maximum, "maximum", "", "", "out", B200_EW_MAXIMUM, kSame)
B200_PW_BINARY(minimum, "minimum", "", "", "out", B200_EW_MINIMUM, kSame)
B200_PW_BINARY(eq_t, "eq", "Tensor", "Tensor", "Tensor_out", B200_EW_EQ, kBool)
B200_PW_BINARY(ne_t, "ne", "Tensor", "Tensor", "Tensor_out", B200_EW_NE, kBool)
B200_PW_BINARY(lt_t, "lt", "Tensor", "Tensor", "Tensor_out", B200_EW_LT, kBool)
B200_PW_BINARY(le_t, "le", "Tensor", "Tensor", "Tensor_out", B200_EW_LE, kBool)
B200_PW_BINARY(gt_t, "gt", "Tensor", "Tensor", "Tensor_out", B200_EW_GT, kBool)
B200_PW_BINARY(ge_t, "ge", "Tensor", "Tensor", "Tensor_out", B200_EW_GE, kBool)
B200_PW_BINARY_SCALAR(eq_s, "eq", "Scalar", "Scalar", "Scalar_out", B200_EW_EQ, kBool)
B200_PW_BINARY_SCALAR(ne_s, "ne", "Scalar", "Scalar", "Scalar_out", B200_EW_NE, kBool)
B200_PW_BINARY_SCALAR(lt_s, "lt", "Scalar", "Scalar", "Scalar_out", B200_EW_LT, kBool)
B200_PW_BINARY_SCALAR(le_s, "le", "Scalar", "Scalar", "Scalar_out", B200_EW_LE, kBool)
B200_PW_BINARY_SCALAR(gt_s, "gt", "Scalar", "Scalar", "Scalar_out", B200_EW_GT, kBool)
B200_PW_BINARY_SCALAR(ge_s, "ge", "Scalar", "Scalar", "Scalar_out", B200_EW_GE, kBool)
B200_PW_BINARY(logical_and, "logical_and", "", "", "out", B200_EW_LOGICAL_AND, kBool)
B200_PW_BINARY(logical_or, "logical_or", "", "", "out", B200_EW_LOGICAL_OR, kBool)
B200_PW_BINARY(logical_xor, "logical_xor", "", "", "out", B200_EW_LOGICAL_XOR, kBool)
B200_PW_BINARY(bitwise_and, "bitwise_and", "Tensor", "Tensor", "Tensor_out", B200_EW_BITWISE_AND, kSame)
B200_PW_BINARY(bitwise_or, "bitwise_or", "Tensor", "Tensor", "Tensor_out", B200_EW_BITWISE_OR, kSame)
B200_PW_BINARY(bitwise_xor, "bitwise_xor", "Tensor", "Tensor", "Tensor_out", B200_EW_BITWISE_XOR, kSame)
B200_PW_BINARY(pow_tt, "pow", "Tensor_Tensor", "Tensor", "Tensor_Tensor_out", B200_EW_POW, kSame)
B200_PW_BINARY_SCALAR(pow_ts, "pow", "Tensor_Scalar", "Scalar", "Tensor_Scalar_out", B200_EW_POW, kSame)
B200_PW_BINARY(remainder_t, "remainder", "Tensor", "Tensor", "Tensor_out", B200_EW_REMAINDER, kSame)
B200_PW_BINARY(fmod_t, "fmod", "Tensor", "Tensor", "Tensor_out", B200_EW_FMOD, kSame)
B200_PW_BINARY(atan2, "atan2", "", "", "out", B200_EW_ATAN2, kFloat)
B200_PW_BINARY(xlogy_t, "xlogy", "Tensor", "Tensor", "OutTensor", B200_EW_XLOGY, kFloat)

at::Tensor rsub_scalar(const at::Tensor& a, const at::Scalar& other, const at::Scalar& alpha) {
  at::Tensor out;
  if (!alpha.isComplex() && pointwise_into(B200_EW_RSUB, kSame, out, In(a), In(other), In(), alpha.toDouble())) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::rsub", "Scalar"), a, other, alpha);
}
at::Tensor rsub_tensor(const at::Tensor& a, const at::Tensor& other, const at::Scalar& alpha) {
  at::Tensor out;
  if (!alpha.isComplex() && pointwise_into(B200_EW_RSUB, kSame, out, In(a), In(other), In(), alpha.toDouble())) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::rsub", "Tensor"), a, other, alpha);
}

at::Tensor pow_scalar_base(const at::Scalar& base, const at::Tensor& e) {
  at::Tensor out;
  if (pointwise_into(B200_EW_POW, kSame, out, In(base), In(e))) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::pow", "Scalar"), base, e);
}

int div_op(const std::optional<c10::string_view>& mode, Rule* rule) {
  if (!mode.has_value()) { *rule = kFloat; return B200_EW_DIV; }
  *rule = kSame;
  if (*mode == "floor") return B200_EW_DIV_FLOOR;
  if (*mode == "trunc") return B200_EW_DIV_TRUNC;
  TORCH_CHECK(false, "div expected rounding_mode to be one of None, 'trunc', or 'floor' but found '", *mode, "'");
}
at::Tensor div_mode(const at::Tensor& a, const at::Tensor& b, std::optional<c10::string_view> mode) {
  Rule r;
  const int op = div_op(mode, &r);
  at::Tensor out;
  if (pointwise_into(op, r, out, In(a), In(b))) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::div", "Tensor_mode"), a, b, mode);
}
at::Tensor& div_mode_(at::Tensor& a, const at::Tensor& b, std::optional<c10::string_view> mode) {
  Rule r;
  const int op = div_op(mode, &r);
  if (pointwise_into(op, r, a, In(a), In(b))) return a;
  run_fallback(B200_OP_HANDLE("aten::div_", "Tensor_mode"), a, b, mode);
  return a;
}
at::Tensor& div_mode_out(const at::Tensor& a, const at::Tensor& b, std::optional<c10::string_view> mode, at::Tensor& out) {
  Rule r;
  const int op = div_op(mode, &r);
  if (pointwise_into(op, r, out, In(a), In(b), In(), 0.0, 0.0, true)) return out;
  run_fallback(B200_OP_HANDLE("aten::div", "out_mode"), a, b, mode, out);
  return out;
}
at::Tensor floor_divide(const at::Tensor& a, const at::Tensor& b) {
  at::Tensor out;
  if (pointwise_into(B200_EW_DIV_FLOOR, kSame, out, In(a), In(b))) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::floor_divide", ""), a, b);
}

// ------------------------------------------------------------------------------------------------ unary
#define B200_PW_UNARY(CNAME, ATEN, OP, RULE)                                                                 \
  at::Tensor CNAME(const at::Tensor& a) {                                                                    \
    at::Tensor out;                                                                                          \
    if (pointwise_into(OP, RULE, out, In(a))) return out;                                                    \
    return fallback_tensor(B200_OP_HANDLE("aten::" ATEN, ""), a);                                            \
  }                                                                                                          \
  at::Tensor& CNAME##_(at::Tensor& a) {                                                                      \
    if (pointwise_into(OP, RULE, a, In(a))) return a;                                                        \
    run_fallback(B200_OP_HANDLE("aten::" ATEN "_", ""), a);                                                  \
    return a;                                                                                                \
  }                                                                                                          \
  at::Tensor& CNAME##_out(const at::Tensor& a, at::Tensor& out) {                                            \
    if (pointwise_into(OP, RULE, out, In(a), In(), In(), 0.0, 0.0, true)) return out;                        \
    run_fallback(B200_OP_HANDLE("aten::" ATEN, "out"), a, out);                                              \
    return out;                                                                                              \
  }

B200_PW_UNARY(floor, "floor", B200_EW_FLOOR, kSame)
B200_PW_UNARY(ceil, "ceil", B200_EW_CEIL, kSame)
B200_PW_UNARY(round, "round", B200_EW_ROUND, kSame)
B200_PW_UNARY(trunc, "trunc", B200_EW_TRUNC, kSame)
B200_PW_UNARY(frac, "frac", B200_EW_FRAC, kSame)
B200_PW_UNARY(sign, "sign", B200_EW_SIGN, kSame)
B200_PW_UNARY(sgn, "sgn", B200_EW_SIGN, kSame)
B200_PW_UNARY(exp2, "exp2", B200_EW_EXP2, kFloat)
B200_PW_UNARY(expm1, "expm1", B200_EW_EXPM1, kFloat)
B200_PW_UNARY(log, "log", B200_EW_LOG, kFloat)
B200_PW_UNARY(log2, "log2", B200_EW_LOG2, kFloat)
B200_PW_UNARY(log10, "log10", B200_EW_LOG10, kFloat)
B200_PW_UNARY(log1p, "log1p", B200_EW_LOG1P, kFloat)
B200_PW_UNARY(sin, "sin", B200_EW_SIN, kFloat)
B200_PW_UNARY(cos, "cos", B200_EW_COS, kFloat)
B200_PW_UNARY(tan, "tan", B200_EW_TAN, kFloat)
B200_PW_UNARY(erf, "erf", B200_EW_ERF, kFloat)
B200_PW_UNARY(asin, "asin", B200_EW_ASIN, kFloat)
B200_PW_UNARY(acos, "acos", B200_EW_ACOS, kFloat)
B200_PW_UNARY(atan, "atan", B200_EW_ATAN, kFloat)
B200_PW_UNARY(sinh, "sinh", B200_EW_SINH, kFloat)
B200_PW_UNARY(cosh, "cosh", B200_EW_COSH, kFloat)
B200_PW_UNARY(asinh, "asinh", B200_EW_ASINH, kFloat)
B200_PW_UNARY(acosh, "acosh", B200_EW_ACOSH, kFloat)
B200_PW_UNARY(atanh, "atanh", B200_EW_ATANH, kFloat)
B200_PW_UNARY(erfc, "erfc", B200_EW_ERFC, kFloat)
B200_PW_UNARY(bitwise_not, "bitwise_not", B200_EW_BITWISE_NOT, kSame)
// .out forms of the operators whose functional / in-place forms live in Elementwise.cpp
B200_PW_UNARY(exp_g, "exp", B200_EW_EXP, kFloat)
B200_PW_UNARY(sqrt_g, "sqrt", B200_EW_SQRT, kFloat)
B200_PW_UNARY(rsqrt_g, "rsqrt", B200_EW_RSQRT, kFloat)
B200_PW_UNARY(reciprocal_g, "reciprocal", B200_EW_RECIPROCAL, kFloat)
B200_PW_UNARY(sigmoid_g, "sigmoid", B200_EW_SIGMOID, kFloat)
B200_PW_UNARY(tanh_g, "tanh", B200_EW_TANH, kFloat)
B200_PW_UNARY(neg_g, "neg", B200_EW_NEG, kSame)
B200_PW_UNARY(abs_g, "abs", B200_EW_ABS, kSame)

at::Tensor isnan(const at::Tensor& a) {
  at::Tensor out;
  if (pointwise_into(B200_EW_ISNAN, kBool, out, In(a))) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::isnan", ""), a);
}
at::Tensor logical_not(const at::Tensor& a) {
  at::Tensor out;
  if (pointwise_into(B200_EW_LOGICAL_NOT, kBool, out, In(a))) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::logical_not", ""), a);
}
at::Tensor& logical_not_out(const at::Tensor& a, at::Tensor& out) {
  if (pointwise_into(B200_EW_LOGICAL_NOT, kBool, out, In(a), In(), In(), 0.0, 0.0, true)) return out;
  run_fallback(B200_OP_HANDLE("aten::logical_not", "out"), a, out);
  return out;
}

// ------------------------------------------------------------------------------------------------ ternary & parametrised
at::Tensor where_self(const at::Tensor& cond, const at::Tensor& a, const at::Tensor& b) {
  at::Tensor out;
  if (cond.scalar_type() == at::kBool || cond.scalar_type() == at::kByte)
    if (pointwise_into(B200_EW_WHERE, kSame, out, In(cond), In(a), In(b))) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::where", "self"), cond, a, b);
}
at::Tensor& where_self_out(const at::Tensor& cond, const at::Tensor& a, const at::Tensor& b, at::Tensor& out) {
  if (cond.scalar_type() == at::kBool || cond.scalar_type() == at::kByte)
    if (pointwise_into(B200_EW_WHERE, kSame, out, In(cond), In(a), In(b), 0.0, 0.0, true)) return out;
  run_fallback(B200_OP_HANDLE("aten::where", "self_out"), cond, a, b, out);
  return out;
}

at::Tensor& masked_fill_scalar_(at::Tensor& self, const at::Tensor& mask, const at::Scalar& value) {
  if (!value.isComplex() && mask.scalar_type() == at::kBool &&
      pointwise_into(B200_EW_MASKED_FILL, kSame, self, In(self), In(mask), In(), value.toDouble()))
    return self;
  run_fallback(B200_OP_HANDLE("aten::masked_fill_", "Scalar"), self, mask, value);
  return self;
}
at::Tensor& masked_fill_tensor_(at::Tensor& self, const at::Tensor& mask, const at::Tensor& value) {
  // a 0-dim host value folds into the launch; a device value is read with a WHERE over (mask, value, self)
  if (mask.scalar_type() == at::kBool && value.dim() == 0 && !value.is_complex()) {
    if (value.device().is_cpu()) {
      if (pointwise_into(B200_EW_MASKED_FILL, kSame, self, In(self), In(mask), In(), value.item<double>())) return self;
    } else if (pointwise_into(B200_EW_WHERE, kSame, self, In(mask), In(value), In(self), 0.0, 0.0, false,
                              self.scalar_type())) {
      return self;
    }
  }
  run_fallback(B200_OP_HANDLE("aten::masked_fill_", "Tensor"), self, mask, value);
  return self;
}

bool clamp_into(at::Tensor& out, const at::Tensor& a, const std::optional<at::Scalar>& lo,
                const std::optional<at::Scalar>& hi, bool resize) {
  TORCH_CHECK(lo.has_value() || hi.has_value(), "torch.clamp: At least one of 'min' or 'max' must not be None");
  const double l = lo ? lo->toDouble() : -std::numeric_limits<double>::infinity();
  const double h = hi ? hi->toDouble() : std::numeric_limits<double>::infinity();
  In b = lo ? In(*lo) : In(), c = In();
  // the bounds take part in type promotion (clamp of an int tensor with a float bound is float)
  at::ScalarType dt = a.scalar_type();
  if (lo) dt = at::native::result_type(a, *lo);
  if (hi) dt = c10::promoteTypes(dt, at::native::result_type(a, *hi));
  (void)b; (void)c;
  return pointwise_into(B200_EW_CLAMP, kSame, out, In(a), In(), In(), l, h, resize, out.defined() ? std::nullopt : std::optional<at::ScalarType>(dt));
}
at::Tensor pw_clamp(const at::Tensor& a, const std::optional<at::Scalar>& lo, const std::optional<at::Scalar>& hi) {
  at::Tensor out;
  if (clamp_into(out, a, lo, hi, false)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::clamp", ""), a, lo, hi);
}
at::Tensor& pw_clamp_(at::Tensor& a, const std::optional<at::Scalar>& lo, const std::optional<at::Scalar>& hi) {
  if (clamp_into(a, a, lo, hi, false)) return a;
  run_fallback(B200_OP_HANDLE("aten::clamp_", ""), a, lo, hi);
  return a;
}
at::Tensor& clamp_out(const at::Tensor& a, const std::optional<at::Scalar>& lo, const std::optional<at::Scalar>& hi,
                      at::Tensor& out) {
  if (clamp_into(out, a, lo, hi, true)) return out;
  run_fallback(B200_OP_HANDLE("aten::clamp", "out"), a, lo, hi, out);
  return out;
}
at::Tensor clamp_min(const at::Tensor& a, const at::Scalar& lo) { return pw_clamp(a, std::optional<at::Scalar>(lo), std::optional<at::Scalar>()); }
at::Tensor& clamp_min_(at::Tensor& a, const at::Scalar& lo) { return pw_clamp_(a, std::optional<at::Scalar>(lo), std::optional<at::Scalar>()); }
at::Tensor clamp_max(const at::Tensor& a, const at::Scalar& hi) { return pw_clamp(a, std::optional<at::Scalar>(), std::optional<at::Scalar>(hi)); }
at::Tensor& clamp_max_(at::Tensor& a, const at::Scalar& hi) { return pw_clamp_(a, std::optional<at::Scalar>(), std::optional<at::Scalar>(hi)); }
at::Tensor hardtanh(const at::Tensor& a, const at::Scalar& lo, const at::Scalar& hi) { return pw_clamp(a, std::optional<at::Scalar>(lo), std::optional<at::Scalar>(hi)); }
at::Tensor& hardtanh_(at::Tensor& a, const at::Scalar& lo, const at::Scalar& hi) { return pw_clamp_(a, std::optional<at::Scalar>(lo), std::optional<at::Scalar>(hi)); }
at::Tensor hardtanh_backward(const at::Tensor& g, const at::Tensor& x, const at::Scalar& lo, const at::Scalar& hi) {
  at::Tensor out;
  if (pointwise_into(B200_EW_HARDTANH_BWD, kSame, out, In(g), In(x), In(), lo.toDouble(), hi.toDouble())) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::hardtanh_backward", ""), g, x, lo, hi);
}

#define B200_PW_ADDC(CNAME, ATEN, OP)                                                                        \
  at::Tensor CNAME(const at::Tensor& a, const at::Tensor& t1, const at::Tensor& t2, const at::Scalar& v) {   \
    at::Tensor out;                                                                                          \
    if (pointwise_into(OP, kSame, out, In(a), In(t1), In(t2), v.toDouble())) return out;                     \
    return fallback_tensor(B200_OP_HANDLE("aten::" ATEN, ""), a, t1, t2, v);                                 \
  }                                                                                                          \
  at::Tensor& CNAME##_(at::Tensor& a, const at::Tensor& t1, const at::Tensor& t2, const at::Scalar& v) {     \
    if (pointwise_into(OP, kSame, a, In(a), In(t1), In(t2), v.toDouble())) return a;                         \
    run_fallback(B200_OP_HANDLE("aten::" ATEN "_", ""), a, t1, t2, v);                                       \
    return a;                                                                                                \
  }                                                                                                          \
  at::Tensor& CNAME##_out(const at::Tensor& a, const at::Tensor& t1, const at::Tensor& t2, const at::Scalar& v, \
                          at::Tensor& out) {                                                                 \
    if (pointwise_into(OP, kSame, out, In(a), In(t1), In(t2), v.toDouble(), 0.0, true)) return out;          \
    run_fallback(B200_OP_HANDLE("aten::" ATEN, "out"), a, t1, t2, v, out);                                   \
    return out;                                                                                              \
  }
B200_PW_ADDC(addcmul, "addcmul", B200_EW_ADDCMUL)
B200_PW_ADDC(addcdiv, "addcdiv", B200_EW_ADDCDIV)

at::Tensor lerp_scalar(const at::Tensor& a, const at::Tensor& end, const at::Scalar& w) {
  at::Tensor out;
  if (pointwise_into(B200_EW_LERP, kSame, out, In(a), In(end), In(), w.toDouble())) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::lerp", "Scalar"), a, end, w);
}
at::Tensor& lerp_scalar_(at::Tensor& a, const at::Tensor& end, const at::Scalar& w) {
  if (pointwise_into(B200_EW_LERP, kSame, a, In(a), In(end), In(), w.toDouble())) return a;
  run_fallback(B200_OP_HANDLE("aten::lerp_", "Scalar"), a, end, w);
  return a;
}
at::Tensor lerp_tensor(const at::Tensor& a, const at::Tensor& end, const at::Tensor& w) {
  at::Tensor out;
  if (pointwise_into(B200_EW_LERP_TENSOR, kSame, out, In(a), In(end), In(w))) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::lerp", "Tensor"), a, end, w);
}
at::Tensor& lerp_tensor_(at::Tensor& a, const at::Tensor& end, const at::Tensor& w) {
  if (pointwise_into(B200_EW_LERP_TENSOR, kSame, a, In(a), In(end), In(w))) return a;
  run_fallback(B200_OP_HANDLE("aten::lerp_", "Tensor"), a, end, w);
  return a;
}

at::Tensor leaky_relu(const at::Tensor& a, const at::Scalar& slope) {
  at::Tensor out;
  if (pointwise_into(B200_EW_LEAKY_RELU, kSame, out, In(a), In(), In(), slope.toDouble())) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::leaky_relu", ""), a, slope);
}
at::Tensor& leaky_relu_(at::Tensor& a, const at::Scalar& slope) {
  if (pointwise_into(B200_EW_LEAKY_RELU, kSame, a, In(a), In(), In(), slope.toDouble())) return a;
  run_fallback(B200_OP_HANDLE("aten::leaky_relu_", ""), a, slope);
  return a;
}
at::Tensor leaky_relu_backward(const at::Tensor& g, const at::Tensor& x, const at::Scalar& slope, bool is_result) {
  at::Tensor out;
  if (pointwise_into(B200_EW_LEAKY_RELU_BWD, kSame, out, In(g), In(x), In(), slope.toDouble())) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::leaky_relu_backward", ""), g, x, slope, is_result);
}
at::Tensor elu(const at::Tensor& a, const at::Scalar& alpha, const at::Scalar& scale, const at::Scalar& input_scale) {
  at::Tensor out;
  if (input_scale.toDouble() == 1.0 &&
      pointwise_into(B200_EW_ELU, kSame, out, In(a), In(), In(), alpha.toDouble(), scale.toDouble()))
    return out;
  return fallback_tensor(B200_OP_HANDLE("aten::elu", ""), a, alpha, scale, input_scale);
}
std::tuple<at::Tensor, at::Tensor> log_sigmoid_forward(const at::Tensor& a) {
  at::Tensor out;
  if (pointwise_into(B200_EW_LOG_SIGMOID, kSame, out, In(a))) return {out, at::empty({0}, a.options())};
  auto st = run_fallback(B200_OP_HANDLE("aten::log_sigmoid_forward", ""), a);
  return {st[0].toTensor(), st[1].toTensor()};
}
at::Tensor log_sigmoid_backward(const at::Tensor& g, const at::Tensor& x, const at::Tensor& buffer) {
  at::Tensor out;
  if (pointwise_into(B200_EW_LOG_SIGMOID_BWD, kSame, out, In(g), In(x))) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::log_sigmoid_backward", ""), g, x, buffer);
}
at::Tensor softplus(const at::Tensor& a, const at::Scalar& beta, const at::Scalar& threshold) {
  at::Tensor out;
  if (pointwise_into(B200_EW_SOFTPLUS, kSame, out, In(a), In(), In(), beta.toDouble(), threshold.toDouble())) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::softplus", ""), a, beta, threshold);
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
#define REG3(CNAME, ATEN, OV_F, OV_I, OV_O)                 \
  m.impl(ATEN OV_F, TORCH_FN(CNAME));                       \
  m.impl(ATEN "_" OV_I, TORCH_FN(CNAME##_));                \
  m.impl(ATEN OV_O, TORCH_FN(CNAME##_out));
  REG3(maximum, "maximum", "", "", ".out")
  REG3(minimum, "minimum", "", "", ".out")
  REG3(eq_t, "eq", ".Tensor", ".Tensor", ".Tensor_out")
  REG3(ne_t, "ne", ".Tensor", ".Tensor", ".Tensor_out")
  REG3(lt_t, "lt", ".Tensor", ".Tensor", ".Tensor_out")
  REG3(le_t, "le", ".Tensor", ".Tensor", ".Tensor_out")
  REG3(gt_t, "gt", ".Tensor", ".Tensor", ".Tensor_out")
  REG3(ge_t, "ge", ".Tensor", ".Tensor", ".Tensor_out")
  REG3(eq_s, "eq", ".Scalar", ".Scalar", ".Scalar_out")
  REG3(ne_s, "ne", ".Scalar", ".Scalar", ".Scalar_out")
  REG3(lt_s, "lt", ".Scalar", ".Scalar", ".Scalar_out")
  REG3(le_s, "le", ".Scalar", ".Scalar", ".Scalar_out")
  REG3(gt_s, "gt", ".Scalar", ".Scalar", ".Scalar_out")
  REG3(ge_s, "ge", ".Scalar", ".Scalar", ".Scalar_out")
  REG3(logical_and, "logical_and", "", "", ".out")
  REG3(logical_or, "logical_or", "", "", ".out")
  REG3(logical_xor, "logical_xor", "", "", ".out")
  REG3(bitwise_and, "bitwise_and", ".Tensor", ".Tensor", ".Tensor_out")
  REG3(bitwise_or, "bitwise_or", ".Tensor", ".Tensor", ".Tensor_out")
  REG3(bitwise_xor, "bitwise_xor", ".Tensor", ".Tensor", ".Tensor_out")
  REG3(pow_tt, "pow", ".Tensor_Tensor", ".Tensor", ".Tensor_Tensor_out")
  REG3(pow_ts, "pow", ".Tensor_Scalar", ".Scalar", ".Tensor_Scalar_out")
  REG3(remainder_t, "remainder", ".Tensor", ".Tensor", ".Tensor_out")
  REG3(fmod_t, "fmod", ".Tensor", ".Tensor", ".Tensor_out")
  REG3(atan2, "atan2", "", "", ".out")
  REG3(xlogy_t, "xlogy", ".Tensor", ".Tensor", ".OutTensor")
  m.impl("log_sigmoid_forward", TORCH_FN(log_sigmoid_forward));
  m.impl("log_sigmoid_backward", TORCH_FN(log_sigmoid_backward));
  m.impl("pow.Scalar", TORCH_FN(pow_scalar_base));
  m.impl("rsub.Scalar", TORCH_FN(rsub_scalar));
  m.impl("rsub.Tensor", TORCH_FN(rsub_tensor));
  m.impl("div.Tensor_mode", TORCH_FN(div_mode));
  m.impl("div_.Tensor_mode", TORCH_FN(div_mode_));
  m.impl("div.out_mode", TORCH_FN(div_mode_out));
  m.impl("floor_divide", TORCH_FN(floor_divide));
  REG3(floor, "floor", "", "", ".out")
  REG3(ceil, "ceil", "", "", ".out")
  REG3(round, "round", "", "", ".out")
  REG3(trunc, "trunc", "", "", ".out")
  REG3(frac, "frac", "", "", ".out")
  REG3(sign, "sign", "", "", ".out")
  REG3(sgn, "sgn", "", "", ".out")
  REG3(exp2, "exp2", "", "", ".out")
  REG3(expm1, "expm1", "", "", ".out")
  REG3(log, "log", "", "", ".out")
  REG3(log2, "log2", "", "", ".out")
  REG3(log10, "log10", "", "", ".out")
  REG3(log1p, "log1p", "", "", ".out")
  REG3(sin, "sin", "", "", ".out")
  REG3(cos, "cos", "", "", ".out")
  REG3(tan, "tan", "", "", ".out")
  REG3(erf, "erf", "", "", ".out")
  REG3(asin, "asin", "", "", ".out")
  REG3(acos, "acos", "", "", ".out")
  REG3(atan, "atan", "", "", ".out")
  REG3(sinh, "sinh", "", "", ".out")
  REG3(cosh, "cosh", "", "", ".out")
  REG3(asinh, "asinh", "", "", ".out")
  REG3(acosh, "acosh", "", "", ".out")
  REG3(atanh, "atanh", "", "", ".out")
  REG3(erfc, "erfc", "", "", ".out")
  REG3(bitwise_not, "bitwise_not", "", "", ".out")
  m.impl("exp.out", TORCH_FN(exp_g_out));
  m.impl("sqrt.out", TORCH_FN(sqrt_g_out));
  m.impl("rsqrt.out", TORCH_FN(rsqrt_g_out));
  m.impl("reciprocal.out", TORCH_FN(reciprocal_g_out));
  m.impl("sigmoid.out", TORCH_FN(sigmoid_g_out));
  m.impl("tanh.out", TORCH_FN(tanh_g_out));
  m.impl("neg.out", TORCH_FN(neg_g_out));
  m.impl("abs.out", TORCH_FN(abs_g_out));
  m.impl("isnan", TORCH_FN(isnan));
  m.impl("logical_not", TORCH_FN(logical_not));
  m.impl("logical_not.out", TORCH_FN(logical_not_out));
  m.impl("where.self", TORCH_FN(where_self));
  m.impl("where.self_out", TORCH_FN(where_self_out));
  m.impl("masked_fill_.Scalar", TORCH_FN(masked_fill_scalar_));
  m.impl("masked_fill_.Tensor", TORCH_FN(masked_fill_tensor_));
  m.impl("clamp", TORCH_FN(pw_clamp));
  m.impl("clamp_", TORCH_FN(pw_clamp_));
  m.impl("clamp.out", TORCH_FN(clamp_out));
  m.impl("clamp_min", TORCH_FN(clamp_min));
  m.impl("clamp_min_", TORCH_FN(clamp_min_));
  m.impl("clamp_max", TORCH_FN(clamp_max));
  m.impl("clamp_max_", TORCH_FN(clamp_max_));
  m.impl("hardtanh", TORCH_FN(hardtanh));
  m.impl("hardtanh_", TORCH_FN(hardtanh_));
  m.impl("hardtanh_backward", TORCH_FN(hardtanh_backward));
  REG3(addcmul, "addcmul", "", "", ".out")
  REG3(addcdiv, "addcdiv", "", "", ".out")
  m.impl("lerp.Scalar", TORCH_FN(lerp_scalar));
  m.impl("lerp_.Scalar", TORCH_FN(lerp_scalar_));
  m.impl("lerp.Tensor", TORCH_FN(lerp_tensor));
  m.impl("lerp_.Tensor", TORCH_FN(lerp_tensor_));
  m.impl("leaky_relu", TORCH_FN(leaky_relu));
  m.impl("leaky_relu_", TORCH_FN(leaky_relu_));
  m.impl("leaky_relu_backward", TORCH_FN(leaky_relu_backward));
  m.impl("elu", TORCH_FN(elu));
  m.impl("softplus", TORCH_FN(softplus));
#undef REG3
}

}  // namespace
}  // namespace ops
}  // namespace b200
