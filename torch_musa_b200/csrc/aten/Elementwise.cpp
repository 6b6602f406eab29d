// Pointwise operators on the hand-written elementwise substrate.  The fast path
// covers what training loops actually issue (same-shape, same-dtype, densely laid
// out fp32/bf16/fp16 operands, tensor-scalar forms); broadcasting, type promotion
// and exotic dtypes are forwarded to the CUDA-alias fallback.
// Parity: reference torch_musa/csrc/aten/ops/{Binary,Unary,Activation,Fill}.cpp and
// musa/{Add,Mul,Div,Fill}.mu.
#include "aten/FallbackCall.h"
#include "aten/Loops.h"
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <torch/library.h>

#include <atomic>

namespace b200 {
namespace ops {

// the general loops behind the fast paths (aten/Pointwise.cpp)
bool generic_binary(int op, at::Tensor& out, const at::Tensor& a, const at::Tensor& b, double alpha, bool float_result,
                    bool resize_out);
bool generic_binary_scalar(int op, at::Tensor& out, const at::Tensor& a, const at::Scalar& s, double alpha);
bool generic_unary(int op, at::Tensor& out, const at::Tensor& a, bool float_result, bool resize_out);
bool generic_binary_same(int op, at::Tensor& out, const at::Tensor& a, const at::Tensor& b, double p0, double p1);

namespace {
std::atomic<int64_t> g_unused{0};

inline bool fast_dtype(const at::Tensor& t) { return kdtype(t.scalar_type()) >= 0; }

// Same sizes and strides, no gaps: element i of one is element i of the other in memory.
inline bool same_dense(const at::Tensor& a, const at::Tensor& b) {
  return a.sizes() == b.sizes() && a.strides() == b.strides() && a.is_non_overlapping_and_dense();
}
inline bool plain(const at::Tensor& t) { return !t.is_conj() && !t.is_neg(); }

bool binary_fast(int op, const at::Tensor& out, const at::Tensor& a, const at::Tensor& b, double alpha) {
  if (!on_device(a) || !on_device(b) || !fast_dtype(a) || a.scalar_type() != b.scalar_type() ||
      out.scalar_type() != a.scalar_type() || !same_dense(a, b) || !same_dense(a, out) || !plain(a) || !plain(b))
    return false;
  if (a.numel() == 0) return true;
  DeviceSwitch sw(a.device().index());
  int e = b200_binary(op, kdtype(a.scalar_type()), out.mutable_data_ptr(), a.const_data_ptr(), b.const_data_ptr(), 0.0,
                      alpha, a.numel(), current_raw_stream(a));
  if (e == (int)cudaErrorNotSupported) return false;
  B200_KERNEL_CALL(e);
  return true;
}

bool binary_scalar_fast(int op, const at::Tensor& out, const at::Tensor& a, double s, double alpha) {
  if (!on_device(a) || !fast_dtype(a) || out.scalar_type() != a.scalar_type() || !same_dense(a, out) || !plain(a))
    return false;
  if (a.numel() == 0) return true;
  DeviceSwitch sw(a.device().index());
  int e = b200_binary(op, kdtype(a.scalar_type()), out.mutable_data_ptr(), a.const_data_ptr(), nullptr, s, alpha,
                      a.numel(), current_raw_stream(a));
  if (e == (int)cudaErrorNotSupported) return false;
  B200_KERNEL_CALL(e);
  return true;
}

bool unary_fast(int op, const at::Tensor& out, const at::Tensor& a) {
  if (!on_device(a) || !fast_dtype(a) || out.scalar_type() != a.scalar_type() || !same_dense(a, out) || !plain(a))
    return false;
  if (a.numel() == 0) return true;
  DeviceSwitch sw(a.device().index());
  int e = b200_unary(op, kdtype(a.scalar_type()), out.mutable_data_ptr(), a.const_data_ptr(), a.numel(),
                     current_raw_stream(a));
  if (e == (int)cudaErrorNotSupported) return false;
  B200_KERNEL_CALL(e);
  return true;
}

inline at::Tensor like(const at::Tensor& a) { return at::empty_strided(a.sizes(), a.strides(), a.options()); }

// ----------------------------------------------------------------- binary (Tensor, Tensor[, alpha])
#define B200_BINARY_ALPHA(NAME, OPC, OPG)                                                                  \
  at::Tensor NAME##_tensor(const at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha) {            \
    if (a.dim() > 0 && b.dim() > 0 && fast_dtype(a) && a.is_non_overlapping_and_dense()) {                 \
      at::Tensor out = like(a);                                                                            \
      if (binary_fast(OPC, out, a, b, alpha.toDouble())) return out;                                       \
    }                                                                                                      \
    if (!alpha.isComplex()) {                                                                              \
      at::Tensor out;                                                                                      \
      if (generic_binary(OPG, out, a, b, alpha.toDouble(), false, false)) return out;                      \
    }                                                                                                      \
    return fallback_tensor(B200_OP_HANDLE("aten::" #NAME, "Tensor"), a, b, alpha);                         \
  }                                                                                                        \
  at::Tensor& NAME##_tensor_(at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha) {                \
    if (a.dim() > 0 && b.dim() > 0 && binary_fast(OPC, a, a, b, alpha.toDouble())) return a;               \
    if (!alpha.isComplex() && generic_binary(OPG, a, a, b, alpha.toDouble(), false, false)) return a;      \
    run_fallback(B200_OP_HANDLE("aten::" #NAME "_", "Tensor"), a, b, alpha);                               \
    return a;                                                                                              \
  }                                                                                                        \
  at::Tensor& NAME##_tensor_out(const at::Tensor& a, const at::Tensor& b, const at::Scalar& alpha,         \
                                at::Tensor& out) {                                                         \
    if (a.dim() > 0 && b.dim() > 0 && out.sizes() == a.sizes() && binary_fast(OPC, out, a, b, alpha.toDouble())) \
      return out;                                                                                          \
    if (!alpha.isComplex() && generic_binary(OPG, out, a, b, alpha.toDouble(), false, true)) return out;   \
    run_fallback(B200_OP_HANDLE("aten::" #NAME, "out"), a, b, alpha, out);                                 \
    return out;                                                                                            \
  }

B200_BINARY_ALPHA(add, B200_OP_ADD, B200_EW_ADD)
B200_BINARY_ALPHA(sub, B200_OP_SUB, B200_EW_SUB)

#define B200_BINARY(NAME, OPC, OPG, FLOATRES)                                                              \
  at::Tensor NAME##_tensor(const at::Tensor& a, const at::Tensor& b) {                                     \
    if (a.dim() > 0 && b.dim() > 0 && fast_dtype(a) && a.is_non_overlapping_and_dense()) {                 \
      at::Tensor out = like(a);                                                                            \
      if (binary_fast(OPC, out, a, b, 1.0)) return out;                                                    \
    }                                                                                                      \
    if (a.dim() > 0 && b.dim() == 0 && b.device().is_cpu() && fast_dtype(a) &&                             \
        a.is_non_overlapping_and_dense() && b.is_floating_point()) {                                       \
      at::Tensor out = like(a);                                                                            \
      if (binary_scalar_fast(OPC, out, a, b.item<double>(), 1.0)) return out;                              \
    }                                                                                                      \
    {                                                                                                      \
      at::Tensor out;                                                                                      \
      if (generic_binary(OPG, out, a, b, 1.0, FLOATRES, false)) return out;                                \
    }                                                                                                      \
    return fallback_tensor(B200_OP_HANDLE("aten::" #NAME, "Tensor"), a, b);                                \
  }                                                                                                        \
  at::Tensor& NAME##_tensor_out(const at::Tensor& a, const at::Tensor& b, at::Tensor& out) {               \
    if (a.dim() > 0 && b.dim() > 0 && out.sizes() == a.sizes() && binary_fast(OPC, out, a, b, 1.0)) return out; \
    if (generic_binary(OPG, out, a, b, 1.0, FLOATRES, true)) return out;                                   \
    run_fallback(B200_OP_HANDLE("aten::" #NAME, "out"), a, b, out);                                        \
    return out;                                                                                            \
  }                                                                                                        \
  at::Tensor& NAME##_tensor_(at::Tensor& a, const at::Tensor& b) {                                         \
    if (a.dim() > 0 && b.dim() > 0 && binary_fast(OPC, a, a, b, 1.0)) return a;                            \
    if (a.dim() > 0 && b.dim() == 0 && b.device().is_cpu() && b.is_floating_point() &&                     \
        binary_scalar_fast(OPC, a, a, b.item<double>(), 1.0))                                              \
      return a;                                                                                            \
    if (generic_binary(OPG, a, a, b, 1.0, FLOATRES, false)) return a;                                      \
    run_fallback(B200_OP_HANDLE("aten::" #NAME "_", "Tensor"), a, b);                                      \
    return a;                                                                                              \
  }

B200_BINARY(mul, B200_OP_MUL, B200_EW_MUL, false)
B200_BINARY(div, B200_OP_DIV, B200_EW_DIV, true)

// ----------------------------------------------------------------- unary
#define B200_UNARY(NAME, OPC, OPG, FLOATRES)                                                               \
  at::Tensor NAME(const at::Tensor& a) {                                                                   \
    if (fast_dtype(a) && a.is_non_overlapping_and_dense()) {                                               \
      at::Tensor out = like(a);                                                                            \
      if (unary_fast(OPC, out, a)) return out;                                                             \
    }                                                                                                      \
    {                                                                                                      \
      at::Tensor out;                                                                                      \
      if (generic_unary(OPG, out, a, FLOATRES, false)) return out;                                         \
    }                                                                                                      \
    return fallback_tensor(B200_OP_HANDLE("aten::" #NAME, ""), a);                                         \
  }                                                                                                        \
  at::Tensor& NAME##_(at::Tensor& a) {                                                                     \
    if (unary_fast(OPC, a, a)) return a;                                                                   \
    if (generic_unary(OPG, a, a, FLOATRES, false)) return a;                                               \
    run_fallback(B200_OP_HANDLE("aten::" #NAME "_", ""), a);                                               \
    return a;                                                                                              \
  }

B200_UNARY(relu, B200_OP_RELU, B200_EW_RELU, false)
B200_UNARY(silu, B200_OP_SILU, B200_EW_SILU, true)
B200_UNARY(sigmoid, B200_OP_SIGMOID, B200_EW_SIGMOID, true)
B200_UNARY(tanh, B200_OP_TANH, B200_EW_TANH, true)
B200_UNARY(exp, B200_OP_EXP, B200_EW_EXP, true)
B200_UNARY(neg, B200_OP_NEG, B200_EW_NEG, false)
B200_UNARY(abs, B200_OP_ABS, B200_EW_ABS, false)
B200_UNARY(sqrt, B200_OP_SQRT, B200_EW_SQRT, true)
B200_UNARY(rsqrt, B200_OP_RSQRT, B200_EW_RSQRT, true)
B200_UNARY(reciprocal, B200_OP_RECIPROCAL, B200_EW_RECIPROCAL, true)

at::Tensor gelu(const at::Tensor& a, c10::string_view approximate) {
  if (fast_dtype(a) && a.is_non_overlapping_and_dense()) {
    at::Tensor out = like(a);
    if (unary_fast(approximate == "tanh" ? B200_OP_GELU_TANH : B200_OP_GELU_ERF, out, a)) return out;
  }
  {
    at::Tensor out;
    if (generic_unary(approximate == "tanh" ? B200_EW_GELU_TANH : B200_EW_GELU_ERF, out, a, true, false)) return out;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::gelu", ""), a, approximate);
}
at::Tensor gelu_backward(const at::Tensor& grad, const at::Tensor& a, c10::string_view approximate) {
  if (fast_dtype(a) && a.is_non_overlapping_and_dense()) {
    at::Tensor out = like(a);
    if (binary_fast(approximate == "tanh" ? B200_OP_GELU_TANH_BWD : B200_OP_GELU_ERF_BWD, out, grad, a, 1.0)) return out;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::gelu_backward", ""), grad, a, approximate);
}
at::Tensor silu_backward(const at::Tensor& grad, const at::Tensor& a) {
  if (fast_dtype(a) && a.is_non_overlapping_and_dense()) {
    at::Tensor out = like(a);
    if (binary_fast(B200_OP_SILU_BWD, out, grad, a, 1.0)) return out;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::silu_backward", ""), grad, a);
}
at::Tensor threshold_backward(const at::Tensor& grad, const at::Tensor& a, const at::Scalar& threshold) {
  if (threshold.toDouble() == 0.0 && fast_dtype(a) && a.is_non_overlapping_and_dense()) {
    at::Tensor out = like(a);
    if (binary_fast(B200_OP_RELU_BWD, out, grad, a, 1.0)) return out;
  }
  {
    at::Tensor out;
    if (generic_binary_same(B200_EW_THRESHOLD_BWD, out, grad, a, threshold.toDouble(), 0.0)) return out;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::threshold_backward", ""), grad, a, threshold);
}
at::Tensor sigmoid_backward(const at::Tensor& grad, const at::Tensor& y) {
  if (fast_dtype(y) && y.is_non_overlapping_and_dense()) {
    at::Tensor out = like(y);
    if (binary_fast(B200_OP_SIGMOID_BWD, out, grad, y, 1.0)) return out;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::sigmoid_backward", ""), grad, y);
}
at::Tensor tanh_backward(const at::Tensor& grad, const at::Tensor& y) {
  if (fast_dtype(y) && y.is_non_overlapping_and_dense()) {
    at::Tensor out = like(y);
    if (binary_fast(B200_OP_TANH_BWD, out, grad, y, 1.0)) return out;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::tanh_backward", ""), grad, y);
}

// ----------------------------------------------------------------- scalar forms
at::Tensor mul_scalar(const at::Tensor& a, const at::Scalar& s) {
  if (fast_dtype(a) && a.is_non_overlapping_and_dense() && !s.isComplex()) {
    at::Tensor out = like(a);
    if (binary_scalar_fast(B200_OP_MUL, out, a, s.toDouble(), 1.0)) return out;
  }
  if (!s.isComplex()) {
    at::Tensor out;
    if (generic_binary_scalar(B200_EW_MUL, out, a, s, 1.0)) return out;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::mul", "Scalar"), a, s);
}
at::Tensor& mul_scalar_(at::Tensor& a, const at::Scalar& s) {
  if (!s.isComplex() && binary_scalar_fast(B200_OP_MUL, a, a, s.toDouble(), 1.0)) return a;
  if (!s.isComplex() && generic_binary_scalar(B200_EW_MUL, a, a, s, 1.0)) return a;
  run_fallback(B200_OP_HANDLE("aten::mul_", "Scalar"), a, s);
  return a;
}
at::Tensor add_scalar(const at::Tensor& a, const at::Scalar& s, const at::Scalar& alpha) {
  if (fast_dtype(a) && a.is_non_overlapping_and_dense() && !s.isComplex()) {
    at::Tensor out = like(a);
    if (binary_scalar_fast(B200_OP_ADD, out, a, s.toDouble(), alpha.toDouble())) return out;
  }
  if (!s.isComplex() && !alpha.isComplex()) {
    at::Tensor out;
    if (generic_binary_scalar(B200_EW_ADD, out, a, s, alpha.toDouble())) return out;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::add", "Scalar"), a, s, alpha);
}

// ----------------------------------------------------------------- fill
at::Tensor& fill_scalar_(at::Tensor& self, const at::Scalar& v) {
  if (on_device(self) && fast_dtype(self) && self.is_non_overlapping_and_dense() && !v.isComplex() && plain(self)) {
    if (self.numel() == 0) return self;
    DeviceSwitch sw(self.device().index());
    cudaStream_t s = current_raw_stream(self);
    double d = v.toDouble();
    if (d == 0.0) {
      B200_CUDA_CHECK(cudaMemsetAsync(self.mutable_data_ptr(), 0, (size_t)self.numel() * self.dtype().itemsize(), s));
      return self;
    }
    int e = b200_fill(self.mutable_data_ptr(), kdtype(self.scalar_type()), d, self.numel(), s);
    if (e == 0) return self;
    if (e != (int)cudaErrorNotSupported) B200_KERNEL_CALL(e);
  }
  if (on_device(self) && !v.isComplex() && !self.is_complex() &&
      loops::run(B200_EW_FILL, self, loops::In(), loops::In(), loops::In(), v.toDouble()))
    return self;
  run_fallback(B200_OP_HANDLE("aten::fill_", "Scalar"), self, v);
  return self;
}

at::Tensor& zero_(at::Tensor& self) {
  if (on_device(self) && self.is_non_overlapping_and_dense() && plain(self) && self.layout() == c10::kStrided) {
    if (self.numel() == 0) return self;
    DeviceSwitch sw(self.device().index());
    B200_CUDA_CHECK(cudaMemsetAsync(self.mutable_data_ptr(), 0, (size_t)self.numel() * self.dtype().itemsize(),
                                    current_raw_stream(self)));
    return self;
  }
  run_fallback(B200_OP_HANDLE("aten::zero_", ""), self);
  return self;
}

}  // namespace

bool try_native_cast_copy(const at::Tensor& src, const at::Tensor& dst, cudaStream_t stream) {
  int sd = kdtype(src.scalar_type()), dd = kdtype(dst.scalar_type());
  if (sd < 0 || dd < 0 || src.dim() > 8 || src.sizes() != dst.sizes() || !plain(src) || !plain(dst)) return false;
  if (src.numel() == 0) return true;
  // the kernel walks dst with its own strides: overlapping destinations are not allowed here
  int e = b200_cast_copy(dst.mutable_data_ptr(), dd, src.const_data_ptr(), sd, (int)src.dim(), src.sizes().data(),
                         dst.strides().data(), src.strides().data(), stream);
  if (e == (int)cudaErrorNotSupported) return false;
  B200_KERNEL_CALL(e);
  return true;
}

void count_launch(int) {}
int64_t launch_count() { return b200_launch_count(); }
void reset_launch_count() { b200_reset_launch_count(); }

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("add.Tensor", TORCH_FN(add_tensor));
  m.impl("add_.Tensor", TORCH_FN(add_tensor_));
  m.impl("add.out", TORCH_FN(add_tensor_out));
  m.impl("sub.Tensor", TORCH_FN(sub_tensor));
  m.impl("sub_.Tensor", TORCH_FN(sub_tensor_));
  m.impl("sub.out", TORCH_FN(sub_tensor_out));
  m.impl("mul.Tensor", TORCH_FN(mul_tensor));
  m.impl("mul_.Tensor", TORCH_FN(mul_tensor_));
  m.impl("mul.out", TORCH_FN(mul_tensor_out));
  m.impl("div.Tensor", TORCH_FN(div_tensor));
  m.impl("div_.Tensor", TORCH_FN(div_tensor_));
  m.impl("div.out", TORCH_FN(div_tensor_out));
  m.impl("relu", TORCH_FN(relu));
  m.impl("relu_", TORCH_FN(relu_));
  m.impl("silu", TORCH_FN(silu));
  m.impl("silu_", TORCH_FN(silu_));
  m.impl("sigmoid", TORCH_FN(sigmoid));
  m.impl("sigmoid_", TORCH_FN(sigmoid_));
  m.impl("tanh", TORCH_FN(tanh));
  m.impl("tanh_", TORCH_FN(tanh_));
  m.impl("exp", TORCH_FN(exp));
  m.impl("exp_", TORCH_FN(exp_));
  m.impl("neg", TORCH_FN(neg));
  m.impl("neg_", TORCH_FN(neg_));
  m.impl("abs", TORCH_FN(abs));
  m.impl("abs_", TORCH_FN(abs_));
  m.impl("sqrt", TORCH_FN(sqrt));
  m.impl("sqrt_", TORCH_FN(sqrt_));
  m.impl("rsqrt", TORCH_FN(rsqrt));
  m.impl("rsqrt_", TORCH_FN(rsqrt_));
  m.impl("reciprocal", TORCH_FN(reciprocal));
  m.impl("reciprocal_", TORCH_FN(reciprocal_));
  m.impl("gelu", TORCH_FN(gelu));
  m.impl("gelu_backward", TORCH_FN(gelu_backward));
  m.impl("silu_backward", TORCH_FN(silu_backward));
  m.impl("threshold_backward", TORCH_FN(threshold_backward));
  m.impl("sigmoid_backward", TORCH_FN(sigmoid_backward));
  m.impl("tanh_backward", TORCH_FN(tanh_backward));
  m.impl("fill_.Scalar", TORCH_FN(fill_scalar_));
  m.impl("zero_", TORCH_FN(zero_));
}

// mul.Scalar / add.Scalar are CompositeExplicitAutograd in ATen (they wrap the scalar and call the
// Tensor overload); overriding them on this key keeps the scalar out of a 0-dim tensor round trip.
TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("mul.Scalar", TORCH_FN(mul_scalar));
  m.impl("mul_.Scalar", TORCH_FN(mul_scalar_));
  m.impl("add.Scalar", TORCH_FN(add_scalar));
}

}  // namespace ops
}  // namespace b200
