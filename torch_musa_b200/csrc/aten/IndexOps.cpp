// Indexing, scan, selection and shape helpers on the kernels of kernels/index_ops.cu: index_select, gather,
// scatter / scatter_add, advanced indexing (index.Tensor, _index_put_impl_) through a flattened index over the
// indexed block of dimensions, tril / triu, arange, cumsum, topk, sort, split_with_sizes_copy.
// An index out of range is clamped by the kernel and reported at the next synchronisation (core/DeviceAssert.h).
// Parity: reference torch_musa/csrc/aten/ops/{Indexing,IndexSelect,ScatterGather,Tril,Range,Cumsum,Topk,Sort,
// TensorShape}.cpp.
#include "aten/FallbackCall.h"
#include "aten/Loops.h"
#include "core/DeviceAssert.h"

#include <ATen/Context.h>
#include <ATen/ExpandUtils.h>
#include <ATen/Functions.h>
#include <ATen/TensorOperators.h>
#include <ATen/WrapDimUtils.h>
#include <ATen/native/Resize.h>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {

bool data_ok(const at::Tensor& t) {
  return on_device(t) && t.layout() == c10::kStrided && !t.is_quantized() && !t.is_conj() && !t.is_neg();
}
bool index_ok(const at::Tensor& t) {
  return data_ok(t) && (t.scalar_type() == at::kLong || t.scalar_type() == at::kInt);
}
int idx_code(const at::Tensor& t) { return t.scalar_type() == at::kLong ? B200_I64 : B200_I32; }

struct View3 { int64_t outer = 1, D = 1, inner = 1; };
View3 view3(at::IntArrayRef sizes, int64_t dim) {
  View3 v;
  for (int64_t i = 0; i < (int64_t)sizes.size(); ++i) {
    if (i < dim) v.outer *= sizes[i];
    else if (i == dim) v.D = sizes[i];
    else v.inner *= sizes[i];
  }
  return v;
}

// Uses `out` when it is a defined contiguous tensor of the right dtype (after resizing), else a temporary.
at::Tensor work_out(at::Tensor* out, at::IntArrayRef shape, const at::TensorOptions& opt) {
  if (!out || !out->defined()) {
    at::Tensor t = at::empty(shape, opt);
    if (out) *out = t;
    return t;
  }
  if (out->sizes() != shape) at::native::resize_output(*out, shape);
  if (out->is_contiguous() && out->scalar_type() == c10::typeMetaToScalarType(opt.dtype())) return *out;
  return at::empty(shape, opt);
}

// ------------------------------------------------------------------------------------------------ index_select
bool index_select_into(const at::Tensor& self, int64_t dim, const at::Tensor& index, at::Tensor* out) {
  if (!data_ok(self) || !index_ok(index) || index.dim() > 1 || self.device() != index.device()) return false;
  const int64_t nd = self.dim();
  const int64_t d = at::maybe_wrap_dim(dim, nd == 0 ? 1 : nd);
  at::Tensor in = self.contiguous(), idx = index.contiguous();
  std::vector<int64_t> shape = self.sizes().vec();
  const int64_t J = idx.numel();
  if (nd == 0) shape = {};
  else shape[d] = J;
  const View3 v = nd == 0 ? View3{1, 1, 1} : view3(self.sizes(), d);
  at::Tensor w = work_out(out, shape, self.options());
  if (w.numel()) {
    DeviceSwitch sw(self.device().index());
    int e = b200_index_select(w.mutable_data_ptr(), in.const_data_ptr(), idx.const_data_ptr(), idx_code(idx),
                              (int)self.element_size(), v.outer, v.D, v.inner, nd == 0 ? 1 : J,
                              device_assert_word(self.device().index()), current_raw_stream(self));
    if (e == (int)cudaErrorNotSupported) return false;
    B200_KERNEL_CALL(e);
  }
  if (out && !w.is_same(*out)) out->copy_(w);
  return true;
}
at::Tensor index_select(const at::Tensor& self, int64_t dim, const at::Tensor& index) {
  at::Tensor out;
  if (index_select_into(self, dim, index, &out)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::index_select", ""), self, dim, index);
}
at::Tensor& index_select_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, at::Tensor& out) {
  if (index_select_into(self, dim, index, &out)) return out;
  run_fallback(B200_OP_HANDLE("aten::index_select", "out"), self, dim, index, out);
  return out;
}

// ------------------------------------------------------------------------------------------------ gather / scatter
// Brings (data, index) to contiguous [outer, D, inner] / [outer, J, inner] views; the data tensor is narrowed to the
// index's extent in every other dimension, as the operators' semantics allow a smaller index there.
bool gather_into(const at::Tensor& self, int64_t dim, const at::Tensor& index, at::Tensor* out) {
  if (!data_ok(self) || !index_ok(index) || self.device() != index.device()) return false;
  const int64_t nd = std::max<int64_t>(self.dim(), 1);
  if (index.dim() != self.dim() && !(self.dim() == 0 && index.dim() <= 1)) return false;
  const int64_t d = at::maybe_wrap_dim(dim, nd);
  at::Tensor in = self.dim() == 0 ? self.reshape({1}) : self;
  at::Tensor idx = index.dim() == 0 ? index.reshape({1}) : index;
  for (int64_t i = 0; i < nd; ++i) {
    if (i == d) continue;
    if (idx.size(i) > in.size(i)) return false;
    if (idx.size(i) < in.size(i)) in = in.narrow(i, 0, idx.size(i));
  }
  in = in.contiguous();
  idx = idx.contiguous();
  const View3 v = view3(in.sizes(), d);
  at::Tensor w = work_out(out, index.sizes(), self.options());
  if (w.numel()) {
    DeviceSwitch sw(self.device().index());
    int e = b200_gather(w.mutable_data_ptr(), in.const_data_ptr(), idx.const_data_ptr(), idx_code(idx),
                        (int)self.element_size(), v.outer, v.D, v.inner, idx.size(d),
                        device_assert_word(self.device().index()), current_raw_stream(self));
    if (e == (int)cudaErrorNotSupported) return false;
    B200_KERNEL_CALL(e);
  }
  if (out && !w.is_same(*out)) out->copy_(w);
  return true;
}
at::Tensor gather(const at::Tensor& self, int64_t dim, const at::Tensor& index, bool sparse_grad) {
  at::Tensor out;
  if (gather_into(self, dim, index, &out)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::gather", ""), self, dim, index, sparse_grad);
}
at::Tensor& gather_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, bool sparse_grad, at::Tensor& out) {
  if (gather_into(self, dim, index, &out)) return out;
  run_fallback(B200_OP_HANDLE("aten::gather", "out"), self, dim, index, sparse_grad, out);
  return out;
}

// mode 0 assign, 1 add, 2 scalar.  `self` is updated in place (it must be contiguous in the narrowed window, which a
// contiguous tensor with a full-extent index is; otherwise a contiguous copy is scattered into and copied back).
bool scatter_inplace(at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor* src, double value, int mode) {
  if (!data_ok(self) || !index_ok(index) || self.device() != index.device() || loops::any_dtype(self.scalar_type()) < 0)
    return false;
  if (src && (!data_ok(*src) || src->scalar_type() != self.scalar_type() || src->device() != self.device())) return false;
  if (self.dim() == 0 || index.dim() != self.dim() || (src && src->dim() != index.dim())) return false;
  const int64_t nd = self.dim();
  const int64_t d = at::maybe_wrap_dim(dim, nd);
  // the kernel walks [outer, J, inner] of the index against [outer, D, inner] of self: every other dimension of the
  // index must span self completely, else go through the narrowed window
  bool full = true;
  for (int64_t i = 0; i < nd; ++i)
    if (i != d && index.size(i) != self.size(i)) { if (index.size(i) > self.size(i)) return false; full = false; }
  at::Tensor idx = index.contiguous();
  at::Tensor s;
  if (src) {
    s = *src;
    for (int64_t i = 0; i < nd; ++i) {
      if (s.size(i) < index.size(i)) return false;
      if (s.size(i) > index.size(i)) s = s.narrow(i, 0, index.size(i));
    }
    s = s.contiguous();
  }
  at::Tensor window = self;
  if (!full)
    for (int64_t i = 0; i < nd; ++i)
      if (i != d && index.size(i) < self.size(i)) window = window.narrow(i, 0, index.size(i));
  at::Tensor target = window.is_contiguous() ? window : window.contiguous();
  const View3 v = view3(target.sizes(), d);
  if (idx.numel()) {
    DeviceSwitch sw(self.device().index());
    int e = b200_scatter(target.mutable_data_ptr(), src ? s.const_data_ptr() : nullptr, value, idx.const_data_ptr(),
                         idx_code(idx), loops::any_dtype(self.scalar_type()), mode, v.outer, v.D, v.inner, idx.size(d),
                         device_assert_word(self.device().index()), current_raw_stream(self));
    if (e == (int)cudaErrorNotSupported) return false;
    B200_KERNEL_CALL(e);
  }
  if (!target.is_same(window)) window.copy_(target);
  return true;
}

#define B200_SCATTER_SRC(CNAME, ATEN, OV, OV_O, MODE)                                                       \
  at::Tensor& CNAME##_(at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& src) {     \
    if (scatter_inplace(self, dim, index, &src, 0.0, MODE)) return self;                                    \
    run_fallback(B200_OP_HANDLE("aten::" ATEN "_", OV), self, dim, index, src);                             \
    return self;                                                                                            \
  }                                                                                                         \
  at::Tensor CNAME(const at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& src) {   \
    at::Tensor out = self.clone(at::MemoryFormat::Contiguous);                                              \
    return CNAME##_(out, dim, index, src);                                                                  \
  }                                                                                                         \
  at::Tensor& CNAME##_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& src, \
                          at::Tensor& out) {                                                                \
    if (!out.is_same(self)) {                                                                               \
      if (out.sizes() != self.sizes()) at::native::resize_output(out, self.sizes());                        \
      out.copy_(self);                                                                                      \
    }                                                                                                       \
    return CNAME##_(out, dim, index, src);                                                                  \
  }
B200_SCATTER_SRC(scatter_src, "scatter", "src", "src_out", 0)
B200_SCATTER_SRC(scatter_add, "scatter_add", "", "out", 1)

at::Tensor& scatter_value_(at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Scalar& value) {
  if (!value.isComplex() && scatter_inplace(self, dim, index, nullptr, value.toDouble(), 2)) return self;
  run_fallback(B200_OP_HANDLE("aten::scatter_", "value"), self, dim, index, value);
  return self;
}
at::Tensor scatter_value(const at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Scalar& value) {
  at::Tensor out = self.clone(at::MemoryFormat::Contiguous);
  return scatter_value_(out, dim, index, value);
}

// ------------------------------------------------------------------------------------------------ advanced indexing
// The index tensors must sit on one block of adjacent dimensions [first, first + k).  They are broadcast, wrapped
// and combined into one flat index over the block viewed as a single dimension; index.Tensor then is an
// index_select and _index_put_impl_ an index_put over that view.
struct Adv {
  bool ok = false;
  int64_t first = 0, k = 0;
  at::Tensor flat;                     // int64 [n]
  std::vector<int64_t> index_shape;    // broadcast shape of the index tensors
};
Adv plan_advanced(const at::Tensor& self, const c10::List<std::optional<at::Tensor>>& indices) {
  Adv a;
  if (!data_ok(self) || (int64_t)indices.size() > self.dim()) return a;
  std::vector<at::Tensor> idx;
  int64_t first = -1, last = -1;
  for (int64_t i = 0; i < (int64_t)indices.size(); ++i) {
    const std::optional<at::Tensor> t = indices.get(i);
    if (t.has_value() && t->defined()) {
      if (!index_ok(*t) || t->device() != self.device()) return a;   // boolean masks and host indices: fallback
      if (first < 0) first = i;
      if (last >= 0 && i != last + 1) return a;                      // not adjacent
      last = i;
      idx.push_back(*t);
    }
  }
  if (idx.empty()) return a;
  auto expanded = at::expand_outplace(idx);
  a.index_shape = expanded[0].sizes().vec();
  a.first = first;
  a.k = (int64_t)idx.size();
  // flat = sum_k wrap(idx_k) * stride_k, strides of the block as if it were contiguous
  int64_t stride = 1;
  at::Tensor flat;
  for (int64_t j = a.k - 1; j >= 0; --j) {
    const int64_t size = self.size(first + j);
    at::Tensor t = expanded[j].to(at::kLong);
    t = at::where(at::lt(t, 0), at::add(t, size), t);
    at::Tensor scaled = stride == 1 ? t : at::mul(t, stride);
    flat = flat.defined() ? at::add(flat, scaled) : scaled;
    stride *= size;
  }
  a.flat = flat.reshape({-1}).contiguous();
  a.ok = true;
  return a;
}

at::Tensor index_tensor(const at::Tensor& self, const c10::List<std::optional<at::Tensor>>& indices) {
  Adv a = plan_advanced(self, indices);
  if (a.ok) {
    std::vector<int64_t> viewshape;
    int64_t block = 1;
    for (int64_t i = 0; i < self.dim(); ++i) {
      if (i < a.first || i >= a.first + a.k) viewshape.push_back(self.size(i));
      else {
        block *= self.size(i);
        if (i == a.first + a.k - 1) viewshape.push_back(block);
      }
    }
    at::Tensor in = self.contiguous().view(viewshape);
    at::Tensor sel;
    if (index_select_into(in, a.first, a.flat, &sel)) {
      std::vector<int64_t> shape;
      for (int64_t i = 0; i < a.first; ++i) shape.push_back(self.size(i));
      shape.insert(shape.end(), a.index_shape.begin(), a.index_shape.end());
      for (int64_t i = a.first + a.k; i < self.dim(); ++i) shape.push_back(self.size(i));
      return sel.view(shape);
    }
  }
  return fallback_tensor(B200_OP_HANDLE("aten::index", "Tensor"), self, indices);
}

at::Tensor& index_put_impl_(at::Tensor& self, const c10::List<std::optional<at::Tensor>>& indices, const at::Tensor& values,
                            bool accumulate, bool unsafe) {
  Adv a = plan_advanced(self, indices);
  if (a.ok && data_ok(values) && values.device() == self.device() && loops::any_dtype(self.scalar_type()) >= 0) {
    int64_t outer = 1, block = 1, inner = 1;
    for (int64_t i = 0; i < self.dim(); ++i) {
      if (i < a.first) outer *= self.size(i);
      else if (i < a.first + a.k) block *= self.size(i);
      else inner *= self.size(i);
    }
    // values broadcast to [outer dims..., index shape..., inner dims...]
    std::vector<int64_t> vshape;
    for (int64_t i = 0; i < a.first; ++i) vshape.push_back(self.size(i));
    vshape.insert(vshape.end(), a.index_shape.begin(), a.index_shape.end());
    for (int64_t i = a.first + a.k; i < self.dim(); ++i) vshape.push_back(self.size(i));
    at::Tensor v = values.scalar_type() == self.scalar_type() ? values : values.to(self.scalar_type());
    bool shapes_ok = true;
    try {
      v = v.expand(vshape).contiguous();
    } catch (const c10::Error&) {
      shapes_ok = false;
    }
    if (shapes_ok) {
      at::Tensor target = self.is_contiguous() ? self : self.contiguous();
      const int64_t J = a.flat.numel();
      // accumulating floating-point values with atomics adds in an order that varies between runs: with
      // deterministic algorithms requested the sort-based library path below runs instead
      const bool atomics_unwanted = accumulate && at::isFloatingType(self.scalar_type()) &&
                                    at::globalContext().deterministicAlgorithms();
      if (J > 0 && outer * inner > 0 && !atomics_unwanted) {
        DeviceSwitch sw(self.device().index());
        int e = b200_index_put(target.mutable_data_ptr(), v.const_data_ptr(), a.flat.const_data_ptr(), B200_I64,
                               loops::any_dtype(self.scalar_type()), accumulate ? 1 : 0, outer, block, inner, J, inner,
                               J * inner, device_assert_word(self.device().index()), current_raw_stream(self));
        if (e != (int)cudaErrorNotSupported) {
          B200_KERNEL_CALL(e);
          if (!target.is_same(self)) self.copy_(target);
          return self;
        }
      } else if (!atomics_unwanted) {
        return self;
      }
    }
  }
  run_fallback(B200_OP_HANDLE("aten::_index_put_impl_", ""), self, indices, values, accumulate, unsafe);
  return self;
}

// ------------------------------------------------------------------------------------------------ tril / triu
bool tri_into(const at::Tensor& self, int64_t diagonal, bool upper, at::Tensor* out) {
  if (!data_ok(self) || self.dim() < 2) return false;
  const int eb = (int)self.element_size();
  if (eb != 1 && eb != 2 && eb != 4 && eb != 8 && eb != 16) return false;
  at::Tensor in = self.contiguous();
  at::Tensor w = work_out(out, self.sizes(), self.options());
  const int64_t rows = self.size(-2), cols = self.size(-1);
  const int64_t batch = rows * cols ? self.numel() / (rows * cols) : 0;
  if (w.numel()) {
    DeviceSwitch sw(self.device().index());
    int e = b200_tri(w.mutable_data_ptr(), in.const_data_ptr(), eb, batch, rows, cols, diagonal, upper ? 1 : 0,
                     current_raw_stream(self));
    if (e == (int)cudaErrorNotSupported) return false;
    B200_KERNEL_CALL(e);
  }
  if (out && !w.is_same(*out)) out->copy_(w);
  return true;
}
at::Tensor tril(const at::Tensor& self, int64_t diagonal) {
  at::Tensor out;
  if (tri_into(self, diagonal, false, &out)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::tril", ""), self, diagonal);
}
at::Tensor triu(const at::Tensor& self, int64_t diagonal) {
  at::Tensor out;
  if (tri_into(self, diagonal, true, &out)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::triu", ""), self, diagonal);
}
at::Tensor& tril_(at::Tensor& self, int64_t diagonal) {
  at::Tensor out;
  if (tri_into(self, diagonal, false, &out)) { self.copy_(out); return self; }
  run_fallback(B200_OP_HANDLE("aten::tril_", ""), self, diagonal);
  return self;
}
at::Tensor& triu_(at::Tensor& self, int64_t diagonal) {
  at::Tensor out;
  if (tri_into(self, diagonal, true, &out)) { self.copy_(out); return self; }
  run_fallback(B200_OP_HANDLE("aten::triu_", ""), self, diagonal);
  return self;
}
at::Tensor& tril_out(const at::Tensor& self, int64_t diagonal, at::Tensor& out) {
  if (tri_into(self, diagonal, false, &out)) return out;
  run_fallback(B200_OP_HANDLE("aten::tril", "out"), self, diagonal, out);
  return out;
}
at::Tensor& triu_out(const at::Tensor& self, int64_t diagonal, at::Tensor& out) {
  if (tri_into(self, diagonal, true, &out)) return out;
  run_fallback(B200_OP_HANDLE("aten::triu", "out"), self, diagonal, out);
  return out;
}

// ------------------------------------------------------------------------------------------------ arange
at::Tensor& arange_start_out(const at::Scalar& start, const at::Scalar& end, const at::Scalar& step, at::Tensor& out) {
  const int code = loops::any_dtype(out.scalar_type());
  if (data_ok(out) && code >= 0 && code != B200_BOOL && !start.isComplex() && !end.isComplex() && !step.isComplex()) {
    const double s = start.toDouble(), e = end.toDouble(), st = step.toDouble();
    TORCH_CHECK(st != 0.0, "step must be nonzero");
    TORCH_CHECK((st > 0 && e >= s) || (st < 0 && e <= s), "upper bound and lower bound inconsistent with step sign");
    int64_t n;
    if (start.isIntegral(false) && end.isIntegral(false) && step.isIntegral(false)) {
      const int64_t is = start.toLong(), ie = end.toLong(), ist = step.toLong();
      n = (std::abs(ie - is) + std::abs(ist) - 1) / std::abs(ist);
    } else {
      n = (int64_t)std::ceil((e - s) / st);
    }
    if (out.numel() != n) at::native::resize_output(out, {n});
    at::Tensor w = out.is_contiguous() ? out : at::empty({n}, out.options());
    if (n > 0) {
      DeviceSwitch sw(out.device().index());
      int err = b200_arange(w.mutable_data_ptr(), code, s, st, n, current_raw_stream(out));
      if (err != (int)cudaErrorNotSupported) {
        B200_KERNEL_CALL(err);
        if (!w.is_same(out)) out.copy_(w);
        return out;
      }
    } else {
      return out;
    }
  }
  run_fallback(B200_OP_HANDLE("aten::arange", "start_out"), start, end, step, out);
  return out;
}

// ------------------------------------------------------------------------------------------------ cumsum
bool cumsum_into(const at::Tensor& self, int64_t dim, std::optional<at::ScalarType> dtype, at::Tensor* out) {
  if (!data_ok(self)) return false;
  at::ScalarType dt = dtype.value_or(c10::isIntegralType(self.scalar_type(), true) ? at::kLong : self.scalar_type());
  if (out && out->defined() && !dtype) dt = out->scalar_type();
  const int code = loops::any_dtype(dt);
  if (code != B200_F32 && code != B200_BF16 && code != B200_F16 && code != B200_F64 && code != B200_I64 && code != B200_I32)
    return false;
  const int64_t nd = std::max<int64_t>(self.dim(), 1);
  const int64_t d = at::maybe_wrap_dim(dim, nd);
  at::Tensor in = self.scalar_type() == dt ? self : self.to(dt);
  if (self.dim() == 0) in = in.reshape({1});
  // the scan runs along rows: bring `dim` last
  at::Tensor rows = d == nd - 1 ? in.contiguous() : in.transpose(d, nd - 1).contiguous();
  const int64_t cols = rows.size(-1);
  at::Tensor res = at::empty_like(rows);
  if (rows.numel()) {
    DeviceSwitch sw(self.device().index());
    int e = b200_cumsum_rows(res.mutable_data_ptr(), rows.const_data_ptr(), code, rows.numel() / cols, cols,
                             current_raw_stream(self));
    if (e == (int)cudaErrorNotSupported) return false;
    B200_KERNEL_CALL(e);
  }
  if (d != nd - 1) res = res.transpose(d, nd - 1);
  if (self.dim() == 0) res = res.reshape({});
  if (out->defined()) {
    if (out->sizes() != res.sizes()) at::native::resize_output(*out, res.sizes());
    out->copy_(res);
  } else {
    *out = res.contiguous();
  }
  return true;
}
at::Tensor cumsum(const at::Tensor& self, int64_t dim, std::optional<at::ScalarType> dtype) {
  at::Tensor out;
  if (cumsum_into(self, dim, dtype, &out)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::cumsum", ""), self, dim, dtype);
}
at::Tensor& cumsum_(at::Tensor& self, int64_t dim, std::optional<at::ScalarType> dtype) {
  if (cumsum_into(self, dim, dtype, &self)) return self;
  run_fallback(B200_OP_HANDLE("aten::cumsum_", ""), self, dim, dtype);
  return self;
}
at::Tensor& cumsum_out(const at::Tensor& self, int64_t dim, std::optional<at::ScalarType> dtype, at::Tensor& out) {
  if (cumsum_into(self, dim, dtype, &out)) return out;
  run_fallback(B200_OP_HANDLE("aten::cumsum", "out"), self, dim, dtype, out);
  return out;
}

// ------------------------------------------------------------------------------------------------ sort / topk
bool sort_into(const at::Tensor& self, int64_t dim, bool descending, at::Tensor* values, at::Tensor* indices) {
  if (!data_ok(self)) return false;
  const int code = loops::any_dtype(self.scalar_type());
  if (code < 0 || code == B200_BOOL) return false;
  const int64_t nd = std::max<int64_t>(self.dim(), 1);
  const int64_t d = at::maybe_wrap_dim(dim, nd);
  at::Tensor in = self.dim() == 0 ? self.reshape({1}) : self;
  at::Tensor rows = d == nd - 1 ? in.contiguous() : in.transpose(d, nd - 1).contiguous();
  const int64_t cols = rows.size(-1);
  const int64_t nrows = cols ? rows.numel() / cols : 0;
  at::Tensor v = at::empty_like(rows), i = at::empty(rows.sizes(), rows.options().dtype(at::kLong));
  if (rows.numel()) {
    DeviceSwitch sw(self.device().index());
    cudaStream_t s = current_raw_stream(self);
    size_t bytes = 0;
    int e = b200_sort_rows(nullptr, &bytes, rows.const_data_ptr(), v.mutable_data_ptr(), i.data_ptr<int64_t>(), code, nrows,
                           cols, descending ? 1 : 0, s);
    if (e == (int)cudaErrorNotSupported) return false;
    B200_KERNEL_CALL(e);
    at::Tensor temp = at::empty({(int64_t)bytes}, self.options().dtype(at::kByte));
    e = b200_sort_rows(temp.mutable_data_ptr(), &bytes, rows.const_data_ptr(), v.mutable_data_ptr(), i.data_ptr<int64_t>(),
                       code, nrows, cols, descending ? 1 : 0, s);
    if (e == (int)cudaErrorNotSupported) return false;
    B200_KERNEL_CALL(e);
  }
  if (d != nd - 1) { v = v.transpose(d, nd - 1); i = i.transpose(d, nd - 1); }
  if (self.dim() == 0) { v = v.reshape({}); i = i.reshape({}); }
  auto give = [](at::Tensor* dst, const at::Tensor& src) {
    if (dst->defined()) {
      if (dst->sizes() != src.sizes()) at::native::resize_output(*dst, src.sizes());
      dst->copy_(src);
    } else {
      *dst = src;
    }
  };
  give(values, v);
  give(indices, i);
  return true;
}
std::tuple<at::Tensor, at::Tensor> sort_stable(const at::Tensor& self, std::optional<bool> stable, int64_t dim, bool descending) {
  at::Tensor v, i;
  if (sort_into(self, dim, descending, &v, &i)) return {v, i};
  auto st = run_fallback(B200_OP_HANDLE("aten::sort", "stable"), self, stable, dim, descending);
  return {st[0].toTensor(), st[1].toTensor()};
}
std::tuple<at::Tensor&, at::Tensor&> sort_values_stable(const at::Tensor& self, std::optional<bool> stable, int64_t dim,
                                                        bool descending, at::Tensor& values, at::Tensor& indices) {
  if (sort_into(self, dim, descending, &values, &indices)) return {values, indices};
  run_fallback(B200_OP_HANDLE("aten::sort", "values_stable"), self, stable, dim, descending, values, indices);
  return {values, indices};
}

std::tuple<at::Tensor, at::Tensor> topk(const at::Tensor& self, c10::SymInt k_, int64_t dim, bool largest, bool sorted) {
  const int64_t k = k_.expect_int();
  if (data_ok(self) && self.dim() > 0) {
    const int64_t nd = self.dim();
    const int64_t d = at::maybe_wrap_dim(dim, nd);
    TORCH_CHECK(k >= 0 && k <= self.size(d), "selected index k out of range");
    const int code = loops::any_dtype(self.scalar_type());
    if ((code == B200_F32 || code == B200_BF16 || code == B200_F16) && k <= 16 && self.size(d) <= 1024 && k > 0) {
      at::Tensor rows = d == nd - 1 ? self.contiguous() : self.transpose(d, nd - 1).contiguous();
      const int64_t cols = rows.size(-1), nrows = rows.numel() / std::max<int64_t>(cols, 1);
      std::vector<int64_t> shape = rows.sizes().vec();
      shape.back() = k;
      at::Tensor v = at::empty(shape, rows.options()), i = at::empty(shape, rows.options().dtype(at::kLong));
      DeviceSwitch sw(self.device().index());
      int e = b200_topk_small(v.mutable_data_ptr(), i.data_ptr<int64_t>(), rows.const_data_ptr(), code, nrows, (int)cols,
                              (int)k, largest ? 1 : 0, current_raw_stream(self));
      if (e == 0) {
        if (d != nd - 1) return {v.transpose(d, nd - 1).contiguous(), i.transpose(d, nd - 1).contiguous()};
        return {v, i};
      }
      if (e != (int)cudaErrorNotSupported) B200_KERNEL_CALL(e);
    }
    at::Tensor v, i;
    if (sort_into(self, d, largest, &v, &i)) return {v.narrow(d, 0, k).contiguous(), i.narrow(d, 0, k).contiguous()};
  }
  auto st = run_fallback(B200_OP_HANDLE("aten::topk", ""), self, k_, dim, largest, sorted);
  return {st[0].toTensor(), st[1].toTensor()};
}

// ------------------------------------------------------------------------------------------------ split_with_sizes_copy
void split_with_sizes_copy_out(const at::Tensor& self, at::IntArrayRef split_sizes, int64_t dim, at::TensorList out) {
  // every piece is one strided copy on the copy kernel (views of self, no library call)
  const int64_t d = at::maybe_wrap_dim(dim, self.dim());
  TORCH_CHECK(out.size() == split_sizes.size(), "split_with_sizes_copy: expected ", split_sizes.size(), " outputs");
  int64_t start = 0;
  for (size_t i = 0; i < split_sizes.size(); ++i) {
    at::Tensor piece = self.narrow(d, start, split_sizes[i]);
    at::Tensor o = out[i];
    if (o.sizes() != piece.sizes()) at::native::resize_output(o, piece.sizes());
    o.copy_(piece);
    start += split_sizes[i];
  }
  TORCH_CHECK(start == self.size(d), "split_with_sizes_copy: the sizes do not add up to the dimension");
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("index_select", TORCH_FN(index_select));
  m.impl("index_select.out", TORCH_FN(index_select_out));
  m.impl("gather", TORCH_FN(gather));
  m.impl("gather.out", TORCH_FN(gather_out));
  m.impl("scatter.src", TORCH_FN(scatter_src));
  m.impl("scatter_.src", TORCH_FN(scatter_src_));
  m.impl("scatter.src_out", TORCH_FN(scatter_src_out));
  m.impl("scatter_add", TORCH_FN(scatter_add));
  m.impl("scatter_add_", TORCH_FN(scatter_add_));
  m.impl("scatter_add.out", TORCH_FN(scatter_add_out));
  m.impl("scatter.value", TORCH_FN(scatter_value));
  m.impl("scatter_.value", TORCH_FN(scatter_value_));
  m.impl("index.Tensor", TORCH_FN(index_tensor));
  m.impl("_index_put_impl_", TORCH_FN(index_put_impl_));
  m.impl("tril", TORCH_FN(tril));
  m.impl("triu", TORCH_FN(triu));
  m.impl("tril_", TORCH_FN(tril_));
  m.impl("triu_", TORCH_FN(triu_));
  m.impl("tril.out", TORCH_FN(tril_out));
  m.impl("triu.out", TORCH_FN(triu_out));
  m.impl("arange.start_out", TORCH_FN(arange_start_out));
  m.impl("cumsum", TORCH_FN(cumsum));
  m.impl("cumsum_", TORCH_FN(cumsum_));
  m.impl("cumsum.out", TORCH_FN(cumsum_out));
  m.impl("sort.stable", TORCH_FN(sort_stable));
  m.impl("sort.values_stable", TORCH_FN(sort_values_stable));
  m.impl("topk", TORCH_FN(topk));
  m.impl("split_with_sizes_copy.out", TORCH_FN(split_with_sizes_copy_out));
}

}  // namespace
}  // namespace ops
}  // namespace b200
