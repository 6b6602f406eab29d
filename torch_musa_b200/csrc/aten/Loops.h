// Host side of the general pointwise loops (kernels/ew_generic.cu): broadcasts the operands to the output shape,
// folds 0-dim host tensors and Scalars into the launch, coalesces the iteration space and launches.
// Parity: reference torch_musa/csrc/aten/utils/TensorIterator.h:14-171 (the reference configures ATen's
// TensorIterator and hands it to ported loops; here the plan is a small struct built directly from the tensors).
#pragma once

#include "aten/Ops.h"

#include <c10/core/Scalar.h>

#include <optional>

namespace b200 {
namespace ops {
namespace loops {

// dtype code of the kernel library for any of the ten element types, -1 otherwise
int any_dtype(at::ScalarType t);

struct In {
  const at::Tensor* t = nullptr;
  double value = 0.0;
  bool scalar = false;
  bool present = false;
  std::optional<at::Scalar> sc;     // the original Scalar: integer Scalars promote differently from floating ones
  In() = default;
  In(const at::Tensor& x);          // NOLINT: implicit on purpose; 0-dim host tensors become scalars
  In(const at::Scalar& s);          // NOLINT
  In(double v) : value(v), scalar(true), present(true), sc(at::Scalar(v)) {}   // NOLINT
};

// out = op(a[, b[, c]]) with broadcasting; out must already have the broadcast shape.  Returns false when the
// operands are not covered (unsupported dtype, another device, complex / conjugated views): the caller falls back.
bool run(int op, const at::Tensor& out, const In& a, const In& b = In(), const In& c = In(), double p0 = 0.0,
         double p1 = 0.0, bool float_compute = false);

// Broadcast shape of the tensor operands.
std::vector<int64_t> broadcast_shape(const In& a, const In& b = In(), const In& c = In());

// Result type under torch's promotion rules for the given operands (Scalars take part as wrapped numbers).
at::ScalarType result_type(const In& a, const In& b = In(), const In& c = In());

// A fresh output for (shape, dtype): keeps the layout of `like` when the shapes match and it is dense.
at::Tensor make_out(const std::vector<int64_t>& shape, at::ScalarType dtype, const at::Tensor& like);

// Device tensor among the operands (first one), or nullptr.
const at::Tensor* device_operand(const In& a, const In& b = In(), const In& c = In());

}  // namespace loops
}  // namespace ops
}  // namespace b200
