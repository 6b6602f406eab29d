#include "aten/Loops.h"

#include <ATen/ExpandUtils.h>
#include <ATen/Functions.h>
#include <ATen/native/TypeProperties.h>

namespace b200 {
namespace ops {
namespace loops {

int any_dtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return B200_F32;
    case at::kBFloat16: return B200_BF16;
    case at::kHalf: return B200_F16;
    case at::kDouble: return B200_F64;
    case at::kInt: return B200_I32;
    case at::kLong: return B200_I64;
    case at::kByte: return B200_U8;
    case at::kBool: return B200_BOOL;
    case at::kChar: return B200_I8;
    case at::kShort: return B200_I16;
    default: return -1;
  }
}

In::In(const at::Tensor& x) : present(x.defined()) {
  if (!present) return;
  if (x.dim() == 0 && x.device().is_cpu() && !x.is_complex()) {
    scalar = true;
    value = x.item<double>();
    t = &x;          // kept for type promotion (wrapped numbers promote differently from tensors)
  } else {
    t = &x;
  }
}
In::In(const at::Scalar& s) : present(true), sc(s) {
  scalar = true;
  value = s.isComplex() ? s.toComplexDouble().real() : s.toDouble();
}

const at::Tensor* device_operand(const In& a, const In& b, const In& c) {
  for (const In* i : {&a, &b, &c})
    if (i->present && !i->scalar && i->t && on_device(*i->t)) return i->t;
  return nullptr;
}

std::vector<int64_t> broadcast_shape(const In& a, const In& b, const In& c) {
  std::vector<int64_t> shape;
  bool first = true;
  for (const In* i : {&a, &b, &c}) {
    if (!i->present || i->scalar) continue;
    if (first) {
      shape = i->t->sizes().vec();
      first = false;
    } else {
      shape = at::infer_size(shape, i->t->sizes());
    }
  }
  return shape;
}

at::ScalarType result_type(const In& a, const In& b, const In& c) {
  at::native::ResultTypeState st{};
  for (const In* i : {&a, &b, &c}) {
    if (!i->present) continue;
    if (i->t) st = at::native::update_result_type_state(*i->t, st);
    else st = at::native::update_result_type_state(i->sc.value_or(at::Scalar(i->value)), st);
  }
  return at::native::result_type(st);
}

at::Tensor make_out(const std::vector<int64_t>& shape, at::ScalarType dtype, const at::Tensor& like) {
  if (like.sizes() == at::IntArrayRef(shape) && like.is_non_overlapping_and_dense() && like.dim() > 1)
    return at::empty_strided(like.sizes(), like.strides(), like.options().dtype(dtype));
  return at::empty(shape, like.options().dtype(dtype));
}

bool run(int op, const at::Tensor& out, const In& a, const In& b, const In& c, double p0, double p1, bool float_compute) {
  if (!on_device(out) || out.is_conj() || out.is_neg() || out.layout() != c10::kStrided) return false;
  b200_ew_t d{};
  d.dtype[0] = any_dtype(out.scalar_type());
  if (d.dtype[0] < 0) return false;
  const In* ins[3] = {&a, &b, &c};
  int n_in = 0;
  for (int k = 0; k < 3; ++k)
    if (ins[k]->present) n_in = k + 1;
  for (int k = 0; k < n_in; ++k)
    if (!ins[k]->present) return false;
  const int64_t nd = out.dim();
  if (nd > 8) return false;
  // broadcast strides (elements), outermost first
  int64_t sizes[8], st[4][8];
  const int64_t ndim = nd == 0 ? 1 : nd;
  for (int64_t i = 0; i < ndim; ++i) {
    sizes[i] = nd == 0 ? 1 : out.size(i);
    st[0][i] = nd == 0 ? 0 : out.stride(i);
  }
  d.ptr[0] = out.numel() ? out.mutable_data_ptr() : nullptr;
  for (int k = 0; k < n_in; ++k) {
    const In& in = *ins[k];
    if (in.scalar) {
      d.scalar_mask |= 1 << k;
      d.scalar[k] = in.value;
      for (int64_t i = 0; i < ndim; ++i) st[k + 1][i] = 0;
      continue;
    }
    const at::Tensor& t = *in.t;
    if (!on_device(t) || t.device() != out.device() || t.is_conj() || t.is_neg() || t.layout() != c10::kStrided) return false;
    d.dtype[k + 1] = any_dtype(t.scalar_type());
    if (d.dtype[k + 1] < 0) return false;
    const int64_t td = t.dim();
    if (td > nd) return false;
    for (int64_t i = 0; i < ndim; ++i) {
      const int64_t ti = i - (ndim - (td == 0 ? 0 : td));      // right-aligned
      if (td == 0 || ti < 0) { st[k + 1][i] = 0; continue; }
      const int64_t tsz = t.size(ti);
      if (tsz == sizes[i]) st[k + 1][i] = t.stride(ti);
      else if (tsz == 1) st[k + 1][i] = 0;
      else return false;
    }
    d.ptr[k + 1] = t.numel() ? const_cast<void*>(t.const_data_ptr()) : nullptr;
  }
  if (out.numel() == 0) return true;
  // an output that overlaps itself cannot be written elementwise
  for (int64_t i = 0; i < ndim; ++i)
    if (sizes[i] > 1 && st[0][i] == 0) return false;
  // coalesce: innermost first, drop size-1 dimensions, merge neighbours that are contiguous for every operand
  int out_nd = 0;
  for (int64_t i = ndim - 1; i >= 0; --i) {
    if (sizes[i] == 1) continue;
    bool merged = false;
    if (out_nd > 0) {
      const int p = out_nd - 1;
      bool can = true;
      for (int t = 0; t <= n_in; ++t)
        if (st[t][i] != d.strides[t][p] * d.sizes[p]) { can = false; break; }
      if (can) {
        d.sizes[p] *= sizes[i];
        merged = true;
      }
    }
    if (!merged) {
      d.sizes[out_nd] = sizes[i];
      for (int t = 0; t <= n_in; ++t) d.strides[t][out_nd] = st[t][i];
      ++out_nd;
    }
  }
  if (out_nd == 0) {
    d.sizes[0] = 1;
    for (int t = 0; t <= n_in; ++t) d.strides[t][0] = 0;
    out_nd = 1;
  }
  d.ndim = out_nd;
  d.n_in = n_in;
  d.p0 = p0;
  d.p1 = p1;
  d.float_compute = float_compute ? 1 : 0;
  DeviceSwitch sw(out.device().index());
  int e = b200_ew(op, &d, current_raw_stream(out));
  if (e == (int)cudaErrorNotSupported) return false;
  B200_KERNEL_CALL(e);
  return true;
}

}  // namespace loops
}  // namespace ops
}  // namespace b200
