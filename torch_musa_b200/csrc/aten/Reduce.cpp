// Reductions on the general reduce kernels (kernels/reduce_generic.cu): sum / mean / prod / amax / amin / max / min
// (with indices) / argmax / argmin / any / all / var / std / vector norms over any set of dimensions of any layout.
// The input is brought to a contiguous [outer, reduce, inner] view: for one run of adjacent reduced dimensions of
// a contiguous tensor that is free, otherwise the kept dimensions are permuted in front (one strided copy).
// Parity: reference torch_musa/csrc/aten/ops/{Reduce,ReduceOps}.cpp (vendor-library reductions plus ported
// ATen kernels).
#include "aten/FallbackCall.h"
#include "aten/Loops.h"

#include <ATen/Functions.h>
#include <ATen/WrapDimUtilsMulti.h>
#include <ATen/native/Resize.h>
#include <torch/library.h>

#include <bitset>

namespace b200 {
namespace ops {

namespace {

struct Plan {
  at::Tensor in;                       // contiguous
  int64_t outer = 1, reduce = 1, inner = 1;
  std::vector<int64_t> out_shape;
};

bool eligible(const at::Tensor& t) {
  return on_device(t) && t.layout() == c10::kStrided && !t.is_complex() && !t.is_quantized() && !t.is_conj() &&
         !t.is_neg() && loops::any_dtype(t.scalar_type()) >= 0 && t.dim() <= 64;
}

Plan make_plan(const at::Tensor& self, at::OptionalIntArrayRef dims, bool keepdim) {
  Plan p;
  const int64_t nd = self.dim();
  std::bitset<64> red;
  if (!dims.has_value() || dims->empty()) red.set();
  else red = at::dim_list_to_bitset(*dims, nd == 0 ? 1 : nd);
  for (int64_t i = 0; i < nd; ++i) {
    if (red[i]) { if (keepdim) p.out_shape.push_back(1); }
    else p.out_shape.push_back(self.size(i));
  }
  // runs of kept / reduced dimensions, size-1 dimensions ignored
  std::vector<std::pair<bool, int64_t>> runs;
  for (int64_t i = 0; i < nd; ++i) {
    if (self.size(i) == 1) continue;
    if (!runs.empty() && runs.back().first == (bool)red[i]) runs.back().second *= self.size(i);
    else runs.emplace_back((bool)red[i], self.size(i));
  }
  int reduced_runs = 0;
  for (auto& r : runs) reduced_runs += r.first ? 1 : 0;
  if (reduced_runs <= 1) {
    p.in = self.contiguous();
    bool seen = false;
    for (auto& r : runs) {
      if (r.first) { p.reduce = r.second; seen = true; }
      else if (!seen) p.outer *= r.second;
      else p.inner *= r.second;
    }
    if (self.numel() == 0) {   // keep the products consistent with empty tensors
      p.outer = 1; p.inner = 1; p.reduce = 1;
      for (int64_t i = 0; i < nd; ++i) (red[i] ? p.reduce : p.outer) *= self.size(i);
    }
  } else {
    std::vector<int64_t> perm;
    for (int64_t i = 0; i < nd; ++i) if (!red[i]) perm.push_back(i);
    for (int64_t i = 0; i < nd; ++i) if (red[i]) perm.push_back(i);
    p.in = self.permute(perm).contiguous();
    for (int64_t i = 0; i < nd; ++i) (red[i] ? p.reduce : p.outer) *= self.size(i);
  }
  return p;
}

// out (and / or out_index) = reduction of self.  `out` undefined: allocated with out_dtype.
bool reduce_into(int op, const at::Tensor& self, at::OptionalIntArrayRef dims, bool keepdim, at::ScalarType out_dtype,
                 at::Tensor* out, at::Tensor* out_index, double p0 = 0.0) {
  if (!eligible(self)) return false;
  const int in_code = loops::any_dtype(self.scalar_type());
  const int out_code = loops::any_dtype(out_dtype);
  if (out_code < 0) return false;
  Plan p = make_plan(self, dims, keepdim);
  const bool arg = op == B200_RD_ARGMAX || op == B200_RD_ARGMIN;
  if (p.reduce == 0) {
    // identity of the operator over an empty range; the arg operators and max / min have none
    TORCH_CHECK(!arg && op != B200_RD_AMAX && op != B200_RD_AMIN,
                "reduction over an empty dimension has no identity for this operator");
  }
  at::Tensor val, idx;
  auto prepare = [&](at::Tensor* user, at::ScalarType dt, at::Tensor& work) {
    if (!user) return;
    if (!user->defined()) {
      *user = at::empty(p.out_shape, self.options().dtype(dt));
      work = *user;
    } else {
      if (user->sizes() != at::IntArrayRef(p.out_shape)) at::native::resize_output(*user, p.out_shape);
      work = (user->is_contiguous() && user->scalar_type() == dt) ? *user : at::empty(p.out_shape, self.options().dtype(dt));
    }
  };
  prepare(out, out_dtype, val);
  prepare(out_index, at::kLong, idx);
  b200_reduce_t d{};
  d.op = op;
  d.in_dtype = in_code;
  d.out_dtype = out_code;
  d.outer = p.outer; d.reduce = p.reduce; d.inner = p.inner;
  d.p0 = p0;
  d.in = p.in.numel() ? p.in.const_data_ptr() : nullptr;
  d.out = val.defined() && val.numel() ? val.mutable_data_ptr() : nullptr;
  d.out_index = idx.defined() && idx.numel() ? idx.data_ptr<int64_t>() : nullptr;
  at::Tensor scratch;
  if (p.outer * p.inner < (int64_t)2 * 148 * 256 && p.reduce >= 64) {
    const int64_t per = (int64_t)b200_reduce_state_bytes();
    const int64_t want = std::min<int64_t>(per * std::max<int64_t>(p.outer * p.inner, 1) * 1024, (int64_t)64 << 20);
    scratch = at::empty({std::max<int64_t>(want, per * 4096)}, self.options().dtype(at::kByte));
    d.scratch = scratch.mutable_data_ptr();
    d.scratch_bytes = (size_t)scratch.numel();
  }
  if (p.outer * p.inner > 0) {
    DeviceSwitch sw(self.device().index());
    int e = b200_reduce(&d, current_raw_stream(self));
    if (e == (int)cudaErrorNotSupported) return false;
    B200_KERNEL_CALL(e);
  }
  if (out && !val.is_same(*out)) out->copy_(val);
  if (out_index && !idx.is_same(*out_index)) out_index->copy_(idx);
  return true;
}

at::ScalarType sum_dtype(const at::Tensor& self, std::optional<at::ScalarType> dtype) {
  if (dtype) return *dtype;
  return c10::isIntegralType(self.scalar_type(), true) ? at::kLong : self.scalar_type();
}

// sum / prod / mean honour an explicit dtype by converting the input first when the kernel has no direct pair
at::Tensor cast_for(const at::Tensor& self, at::ScalarType out_dt) {
  const auto in = self.scalar_type();
  if (in == out_dt) return self;
  if (c10::isIntegralType(in, true) && out_dt == at::kLong) return self;
  if ((in == at::kBFloat16 || in == at::kHalf) && out_dt == at::kFloat) return self;
  return self.to(out_dt);
}

// ------------------------------------------------------------------------------------------------ sum / mean / prod
at::Tensor sum_dim(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, std::optional<at::ScalarType> dtype) {
  const auto dt = sum_dtype(self, dtype);
  at::Tensor out;
  if (eligible(self) && reduce_into(B200_RD_SUM, cast_for(self, dt), dim, keepdim, dt, &out, nullptr)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::sum", "dim_IntList"), self, dim, keepdim, dtype);
}
at::Tensor& sum_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, std::optional<at::ScalarType> dtype,
                    at::Tensor& out) {
  const auto dt = dtype.value_or(out.scalar_type());
  if (eligible(self) && reduce_into(B200_RD_SUM, cast_for(self, dt), dim, keepdim, dt, &out, nullptr)) return out;
  run_fallback(B200_OP_HANDLE("aten::sum", "IntList_out"), self, dim, keepdim, dtype, out);
  return out;
}
at::Tensor mean_dim(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, std::optional<at::ScalarType> dtype) {
  const auto dt = dtype.value_or(self.scalar_type());
  if (eligible(self) && c10::isFloatingType(dt)) {
    at::Tensor in = cast_for(self, dt), out;
    Plan p = make_plan(in, dim, keepdim);
    if (reduce_into(B200_RD_MEAN, in, dim, keepdim, dt, &out, nullptr, p.reduce ? 1.0 / (double)p.reduce : NAN)) return out;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::mean", "dim"), self, dim, keepdim, dtype);
}
at::Tensor& mean_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, std::optional<at::ScalarType> dtype,
                     at::Tensor& out) {
  const auto dt = dtype.value_or(out.scalar_type());
  if (eligible(self) && c10::isFloatingType(dt)) {
    at::Tensor in = cast_for(self, dt);
    Plan p = make_plan(in, dim, keepdim);
    if (reduce_into(B200_RD_MEAN, in, dim, keepdim, dt, &out, nullptr, p.reduce ? 1.0 / (double)p.reduce : NAN)) return out;
  }
  run_fallback(B200_OP_HANDLE("aten::mean", "out"), self, dim, keepdim, dtype, out);
  return out;
}
at::Tensor prod_all(const at::Tensor& self, std::optional<at::ScalarType> dtype) {
  const auto dt = sum_dtype(self, dtype);
  at::Tensor out;
  if (eligible(self) && reduce_into(B200_RD_PROD, cast_for(self, dt), std::nullopt, false, dt, &out, nullptr)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::prod", ""), self, dtype);
}
at::Tensor prod_dim(const at::Tensor& self, int64_t dim, bool keepdim, std::optional<at::ScalarType> dtype) {
  const auto dt = sum_dtype(self, dtype);
  at::Tensor out;
  const int64_t dims[1] = {dim};
  if (eligible(self) && self.dim() > 0 &&
      reduce_into(B200_RD_PROD, cast_for(self, dt), at::IntArrayRef(dims, 1), keepdim, dt, &out, nullptr))
    return out;
  return fallback_tensor(B200_OP_HANDLE("aten::prod", "dim_int"), self, dim, keepdim, dtype);
}

// ------------------------------------------------------------------------------------------------ max / min family
at::Tensor amax(const at::Tensor& self, at::IntArrayRef dim, bool keepdim) {
  at::Tensor out;
  if (eligible(self) && reduce_into(B200_RD_AMAX, self, dim, keepdim, self.scalar_type(), &out, nullptr)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::amax", ""), self, dim, keepdim);
}
at::Tensor& amax_out(const at::Tensor& self, at::IntArrayRef dim, bool keepdim, at::Tensor& out) {
  if (eligible(self) && reduce_into(B200_RD_AMAX, self, dim, keepdim, self.scalar_type(), &out, nullptr)) return out;
  run_fallback(B200_OP_HANDLE("aten::amax", "out"), self, dim, keepdim, out);
  return out;
}
at::Tensor amin(const at::Tensor& self, at::IntArrayRef dim, bool keepdim) {
  at::Tensor out;
  if (eligible(self) && reduce_into(B200_RD_AMIN, self, dim, keepdim, self.scalar_type(), &out, nullptr)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::amin", ""), self, dim, keepdim);
}
at::Tensor& amin_out(const at::Tensor& self, at::IntArrayRef dim, bool keepdim, at::Tensor& out) {
  if (eligible(self) && reduce_into(B200_RD_AMIN, self, dim, keepdim, self.scalar_type(), &out, nullptr)) return out;
  run_fallback(B200_OP_HANDLE("aten::amin", "out"), self, dim, keepdim, out);
  return out;
}
at::Tensor max_all(const at::Tensor& self) {
  at::Tensor out;
  if (eligible(self) && self.numel() > 0 && reduce_into(B200_RD_AMAX, self, std::nullopt, false, self.scalar_type(), &out, nullptr))
    return out;
  return fallback_tensor(B200_OP_HANDLE("aten::max", ""), self);
}
at::Tensor min_all(const at::Tensor& self) {
  at::Tensor out;
  if (eligible(self) && self.numel() > 0 && reduce_into(B200_RD_AMIN, self, std::nullopt, false, self.scalar_type(), &out, nullptr))
    return out;
  return fallback_tensor(B200_OP_HANDLE("aten::min", ""), self);
}
std::tuple<at::Tensor, at::Tensor> max_dim(const at::Tensor& self, int64_t dim, bool keepdim) {
  at::Tensor v, i;
  const int64_t dims[1] = {dim};
  if (eligible(self) && self.dim() > 0 && self.numel() > 0 &&
      reduce_into(B200_RD_ARGMAX, self, at::IntArrayRef(dims, 1), keepdim, self.scalar_type(), &v, &i))
    return {v, i};
  auto st = run_fallback(B200_OP_HANDLE("aten::max", "dim"), self, dim, keepdim);
  return {st[0].toTensor(), st[1].toTensor()};
}
std::tuple<at::Tensor&, at::Tensor&> max_dim_out(const at::Tensor& self, int64_t dim, bool keepdim, at::Tensor& v, at::Tensor& i) {
  const int64_t dims[1] = {dim};
  if (eligible(self) && self.dim() > 0 && self.numel() > 0 &&
      reduce_into(B200_RD_ARGMAX, self, at::IntArrayRef(dims, 1), keepdim, self.scalar_type(), &v, &i))
    return {v, i};
  run_fallback(B200_OP_HANDLE("aten::max", "dim_max"), self, dim, keepdim, v, i);
  return {v, i};
}
std::tuple<at::Tensor, at::Tensor> min_dim(const at::Tensor& self, int64_t dim, bool keepdim) {
  at::Tensor v, i;
  const int64_t dims[1] = {dim};
  if (eligible(self) && self.dim() > 0 && self.numel() > 0 &&
      reduce_into(B200_RD_ARGMIN, self, at::IntArrayRef(dims, 1), keepdim, self.scalar_type(), &v, &i))
    return {v, i};
  auto st = run_fallback(B200_OP_HANDLE("aten::min", "dim"), self, dim, keepdim);
  return {st[0].toTensor(), st[1].toTensor()};
}
std::tuple<at::Tensor&, at::Tensor&> min_dim_out(const at::Tensor& self, int64_t dim, bool keepdim, at::Tensor& v, at::Tensor& i) {
  const int64_t dims[1] = {dim};
  if (eligible(self) && self.dim() > 0 && self.numel() > 0 &&
      reduce_into(B200_RD_ARGMIN, self, at::IntArrayRef(dims, 1), keepdim, self.scalar_type(), &v, &i))
    return {v, i};
  run_fallback(B200_OP_HANDLE("aten::min", "dim_min"), self, dim, keepdim, v, i);
  return {v, i};
}
at::Tensor arg_impl(int op, const char* name, const at::Tensor& self, std::optional<int64_t> dim, bool keepdim) {
  at::Tensor i;
  if (eligible(self) && self.numel() > 0) {
    bool ok;
    if (dim.has_value() && self.dim() > 0) {
      const int64_t dims[1] = {*dim};
      ok = reduce_into(op, self, at::IntArrayRef(dims, 1), keepdim, self.scalar_type(), nullptr, &i);
    } else {
      ok = reduce_into(op, self, std::nullopt, keepdim, self.scalar_type(), nullptr, &i);
    }
    if (ok) return i;
  }
  return fallback_tensor(c10::Dispatcher::singleton().findSchemaOrThrow(name, ""), self, dim, keepdim);
}
at::Tensor argmax(const at::Tensor& self, std::optional<int64_t> dim, bool keepdim) {
  return arg_impl(B200_RD_ARGMAX, "aten::argmax", self, dim, keepdim);
}
at::Tensor argmin(const at::Tensor& self, std::optional<int64_t> dim, bool keepdim) {
  return arg_impl(B200_RD_ARGMIN, "aten::argmin", self, dim, keepdim);
}

// ------------------------------------------------------------------------------------------------ any / all
at::ScalarType bool_dtype(const at::Tensor& self) { return self.scalar_type() == at::kByte ? at::kByte : at::kBool; }
at::Tensor any_all(const at::Tensor& self) {
  at::Tensor out;
  if (eligible(self) && reduce_into(B200_RD_ANY, self, std::nullopt, false, bool_dtype(self), &out, nullptr)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::any", ""), self);
}
at::Tensor all_all(const at::Tensor& self) {
  at::Tensor out;
  if (eligible(self) && reduce_into(B200_RD_ALL, self, std::nullopt, false, bool_dtype(self), &out, nullptr)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::all", ""), self);
}
at::Tensor any_dim(const at::Tensor& self, int64_t dim, bool keepdim) {
  at::Tensor out;
  const int64_t dims[1] = {dim};
  if (eligible(self) && self.dim() > 0 &&
      reduce_into(B200_RD_ANY, self, at::IntArrayRef(dims, 1), keepdim, bool_dtype(self), &out, nullptr))
    return out;
  return fallback_tensor(B200_OP_HANDLE("aten::any", "dim"), self, dim, keepdim);
}
at::Tensor all_dim(const at::Tensor& self, int64_t dim, bool keepdim) {
  at::Tensor out;
  const int64_t dims[1] = {dim};
  if (eligible(self) && self.dim() > 0 &&
      reduce_into(B200_RD_ALL, self, at::IntArrayRef(dims, 1), keepdim, bool_dtype(self), &out, nullptr))
    return out;
  return fallback_tensor(B200_OP_HANDLE("aten::all", "dim"), self, dim, keepdim);
}
at::Tensor any_dims(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim) {
  at::Tensor out;
  if (eligible(self) && reduce_into(B200_RD_ANY, self, dim, keepdim, bool_dtype(self), &out, nullptr)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::any", "dims"), self, dim, keepdim);
}
at::Tensor all_dims(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim) {
  at::Tensor out;
  if (eligible(self) && reduce_into(B200_RD_ALL, self, dim, keepdim, bool_dtype(self), &out, nullptr)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::all", "dims"), self, dim, keepdim);
}

// ------------------------------------------------------------------------------------------------ var / std
at::Tensor var_impl(int op, const at::Tensor& self, at::OptionalIntArrayRef dim, const std::optional<at::Scalar>& correction,
                    bool keepdim, bool* ok) {
  at::Tensor out;
  *ok = eligible(self) && c10::isFloatingType(self.scalar_type()) &&
        reduce_into(op, self, dim, keepdim, self.scalar_type(), &out, nullptr, correction ? correction->toDouble() : 1.0);
  return out;
}
at::Tensor var_correction(const at::Tensor& self, at::OptionalIntArrayRef dim, const std::optional<at::Scalar>& correction, bool keepdim) {
  bool ok;
  at::Tensor out = var_impl(B200_RD_VAR, self, dim, correction, keepdim, &ok);
  if (ok) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::var", "correction"), self, dim, correction, keepdim);
}
at::Tensor std_correction(const at::Tensor& self, at::OptionalIntArrayRef dim, const std::optional<at::Scalar>& correction, bool keepdim) {
  bool ok;
  at::Tensor out = var_impl(B200_RD_STD, self, dim, correction, keepdim, &ok);
  if (ok) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::std", "correction"), self, dim, correction, keepdim);
}
std::tuple<at::Tensor, at::Tensor> var_mean_correction(const at::Tensor& self, at::OptionalIntArrayRef dim,
                                                       const std::optional<at::Scalar>& correction, bool keepdim) {
  bool ok;
  at::Tensor v = var_impl(B200_RD_VAR, self, dim, correction, keepdim, &ok);
  if (ok) return {v, mean_dim(self, dim, keepdim, std::nullopt)};
  auto st = run_fallback(B200_OP_HANDLE("aten::var_mean", "correction"), self, dim, correction, keepdim);
  return {st[0].toTensor(), st[1].toTensor()};
}
std::tuple<at::Tensor, at::Tensor> std_mean_correction(const at::Tensor& self, at::OptionalIntArrayRef dim,
                                                       const std::optional<at::Scalar>& correction, bool keepdim) {
  bool ok;
  at::Tensor v = var_impl(B200_RD_STD, self, dim, correction, keepdim, &ok);
  if (ok) return {v, mean_dim(self, dim, keepdim, std::nullopt)};
  auto st = run_fallback(B200_OP_HANDLE("aten::std_mean", "correction"), self, dim, correction, keepdim);
  return {st[0].toTensor(), st[1].toTensor()};
}

// ------------------------------------------------------------------------------------------------ vector norms
bool norm_into(const at::Tensor& self, const at::Scalar& ord, at::OptionalIntArrayRef dim, bool keepdim,
               std::optional<at::ScalarType> dtype, at::Tensor* out) {
  if (!eligible(self) || ord.isComplex()) return false;
  const auto dt = dtype.value_or(self.scalar_type());
  if (!c10::isFloatingType(dt)) return false;
  const double p = ord.toDouble();
  int op;
  if (p == 2.0) op = B200_RD_NORM2;
  else if (p == 1.0) op = B200_RD_SUMABS;
  else if (p == std::numeric_limits<double>::infinity()) op = B200_RD_ABSMAX;
  else return false;
  return reduce_into(op, cast_for(self, dt), dim, keepdim, dt, out, nullptr);
}
at::Tensor linalg_vector_norm(const at::Tensor& self, const at::Scalar& ord, at::OptionalIntArrayRef dim, bool keepdim,
                              std::optional<at::ScalarType> dtype) {
  at::Tensor out;
  if (norm_into(self, ord, dim, keepdim, dtype, &out)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::linalg_vector_norm", ""), self, ord, dim, keepdim, dtype);
}
at::Tensor& linalg_vector_norm_out(const at::Tensor& self, const at::Scalar& ord, at::OptionalIntArrayRef dim, bool keepdim,
                                   std::optional<at::ScalarType> dtype, at::Tensor& out) {
  if (norm_into(self, ord, dim, keepdim, dtype.value_or(out.scalar_type()), &out)) return out;
  run_fallback(B200_OP_HANDLE("aten::linalg_vector_norm", "out"), self, ord, dim, keepdim, dtype, out);
  return out;
}
at::Tensor norm_scalaropt_dim(const at::Tensor& self, const std::optional<at::Scalar>& p, at::IntArrayRef dim, bool keepdim) {
  at::Tensor out;
  if (norm_into(self, p.value_or(at::Scalar(2.0)), dim, keepdim, std::nullopt, &out)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::norm", "ScalarOpt_dim"), self, p, dim, keepdim);
}
at::Tensor norm_scalar(const at::Tensor& self, const at::Scalar& p) {
  at::Tensor out;
  if (norm_into(self, p, std::nullopt, false, std::nullopt, &out)) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::norm", "Scalar"), self, p);
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("sum.dim_IntList", TORCH_FN(sum_dim));
  m.impl("sum.IntList_out", TORCH_FN(sum_out));
  m.impl("mean.dim", TORCH_FN(mean_dim));
  m.impl("mean.out", TORCH_FN(mean_out));
  m.impl("prod", TORCH_FN(prod_all));
  m.impl("prod.dim_int", TORCH_FN(prod_dim));
  m.impl("amax", TORCH_FN(amax));
  m.impl("amax.out", TORCH_FN(amax_out));
  m.impl("amin", TORCH_FN(amin));
  m.impl("amin.out", TORCH_FN(amin_out));
  m.impl("max", TORCH_FN(max_all));
  m.impl("min", TORCH_FN(min_all));
  m.impl("max.dim", TORCH_FN(max_dim));
  m.impl("max.dim_max", TORCH_FN(max_dim_out));
  m.impl("min.dim", TORCH_FN(min_dim));
  m.impl("min.dim_min", TORCH_FN(min_dim_out));
  m.impl("argmax", TORCH_FN(argmax));
  m.impl("argmin", TORCH_FN(argmin));
  m.impl("any", TORCH_FN(any_all));
  m.impl("all", TORCH_FN(all_all));
  m.impl("any.dim", TORCH_FN(any_dim));
  m.impl("all.dim", TORCH_FN(all_dim));
  m.impl("any.dims", TORCH_FN(any_dims));
  m.impl("all.dims", TORCH_FN(all_dims));
  m.impl("var.correction", TORCH_FN(var_correction));
  m.impl("std.correction", TORCH_FN(std_correction));
  m.impl("var_mean.correction", TORCH_FN(var_mean_correction));
  m.impl("std_mean.correction", TORCH_FN(std_mean_correction));
  m.impl("linalg_vector_norm", TORCH_FN(linalg_vector_norm));
  m.impl("linalg_vector_norm.out", TORCH_FN(linalg_vector_norm_out));
  m.impl("norm.ScalarOpt_dim", TORCH_FN(norm_scalaropt_dim));
  m.impl("norm.Scalar", TORCH_FN(norm_scalar));
}

}  // namespace
}  // namespace ops
}  // namespace b200
