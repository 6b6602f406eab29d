// searchsorted / bucketize, histc, nonzero, unique and group norm on the backend's own kernels.
// Data-dependent output sizes (nonzero, unique) read one count back from the device, as the operators' contracts
// require.  Parity: reference torch_musa/csrc/aten/ops/{Bucketize,Unique,Nonzero,Histc,GroupNorm}.cpp.
#include "aten/Loops.h"
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <ATen/TensorOperators.h>
#include <ATen/native/Resize.h>
#include <torch/library.h>

namespace b200 {
namespace ops {
namespace {

bool ss_dtype_ok(at::ScalarType t) { return t == at::kFloat || t == at::kBFloat16 || t == at::kHalf || t == at::kLong; }

at::Tensor& searchsorted_out_impl(const at::Tensor& sorted, const at::Tensor& self, bool out_int32, bool right,
                                  const std::optional<at::Tensor>& sorter, at::Tensor& out) {
  auto dt = at::result_type(sorted, self);
  if (!ss_dtype_ok(dt)) dt = at::isIntegralType(dt, true) ? at::kLong : at::kFloat;
  const at::Tensor b = sorted.to(dt).contiguous(), v = self.to(dt).contiguous();
  TORCH_CHECK(b.dim() >= 1, "searchsorted: the sorted sequence needs at least one dimension");
  const int64_t nb = b.size(-1);
  const bool shared = b.dim() == 1;
  int64_t rows = 1, nv = v.numel();
  if (!shared) {
    TORCH_CHECK(v.dim() == b.dim() && v.sizes().slice(0, v.dim() - 1) == b.sizes().slice(0, b.dim() - 1),
                "searchsorted: leading dimensions of the sequence and the values must match");
    nv = v.size(-1);
    rows = nv ? v.numel() / nv : 0;
  }
  at::Tensor so;
  if (sorter.has_value() && sorter->defined()) so = sorter->to(at::kLong).contiguous();
  at::native::resize_output(out, v.sizes());
  at::Tensor o = out.is_contiguous() ? out : at::empty(v.sizes(), out.options());
  B200_KERNEL_CALL(b200_searchsorted(o.data_ptr(), out_int32 ? 1 : 0, b.const_data_ptr(), v.const_data_ptr(),
                                     so.defined() ? so.const_data_ptr<int64_t>() : nullptr, loops::any_dtype(dt), rows, nv, nb,
                                     shared ? 1 : 0, right ? 1 : 0, current_raw_stream(self)));
  if (!o.is_same(out)) out.copy_(o);
  return out;
}

bool side_right(bool right, std::optional<c10::string_view> side) {
  if (side.has_value()) {
    TORCH_CHECK(*side == "left" || *side == "right", "searchsorted: side must be 'left' or 'right'");
    TORCH_CHECK(!(right && *side == "left"), "searchsorted: side and right contradict each other");
    return *side == "right";
  }
  return right;
}

at::Tensor searchsorted_tensor(const at::Tensor& sorted, const at::Tensor& self, bool out_int32, bool right,
                               std::optional<c10::string_view> side, const std::optional<at::Tensor>& sorter) {
  at::Tensor out = at::empty({0}, self.options().dtype(out_int32 ? at::kInt : at::kLong));
  return searchsorted_out_impl(sorted, self, out_int32, side_right(right, side), sorter, out);
}
at::Tensor& searchsorted_tensor_out(const at::Tensor& sorted, const at::Tensor& self, bool out_int32, bool right,
                                    std::optional<c10::string_view> side, const std::optional<at::Tensor>& sorter,
                                    at::Tensor& out) {
  return searchsorted_out_impl(sorted, self, out_int32, side_right(right, side), sorter, out);
}
at::Tensor bucketize_tensor(const at::Tensor& self, const at::Tensor& boundaries, bool out_int32, bool right) {
  TORCH_CHECK(boundaries.dim() == 1, "bucketize: boundaries must be one-dimensional");
  at::Tensor out = at::empty({0}, self.options().dtype(out_int32 ? at::kInt : at::kLong));
  return searchsorted_out_impl(boundaries, self, out_int32, right, std::nullopt, out);
}
at::Tensor& bucketize_tensor_out(const at::Tensor& self, const at::Tensor& boundaries, bool out_int32, bool right,
                                 at::Tensor& out) {
  TORCH_CHECK(boundaries.dim() == 1, "bucketize: boundaries must be one-dimensional");
  return searchsorted_out_impl(boundaries, self, out_int32, right, std::nullopt, out);
}

at::Tensor histc(const at::Tensor& self, int64_t bins, const at::Scalar& min, const at::Scalar& max) {
  TORCH_CHECK(bins > 0, "histc: bins must be > 0");
  TORCH_CHECK(at::isFloatingType(self.scalar_type()), "histc: expected a floating-point tensor");
  double lo = min.toDouble(), hi = max.toDouble();
  const at::Tensor x = (self.scalar_type() == at::kDouble ? self.to(at::kFloat) : self).contiguous();
  if (lo == hi && x.numel() > 0) {
    lo = x.min().item<double>();
    hi = x.max().item<double>();
  }
  if (lo == hi) { lo -= 1; hi += 1; }
  TORCH_CHECK(lo < hi && std::isfinite(lo) && std::isfinite(hi), "histc: range of [", lo, ", ", hi, "] is not finite");
  at::Tensor counts = at::zeros({bins}, self.options().dtype(at::kFloat));
  B200_KERNEL_CALL(b200_histc(counts.data_ptr<float>(), x.const_data_ptr(), kdtype(x.scalar_type()), x.numel(), (int)bins,
                              (float)lo, (float)hi, current_raw_stream(self)));
  return counts.to(self.scalar_type());
}

at::Tensor nonzero(const at::Tensor& self) {
  at::ScalarType dt = self.scalar_type();
  at::Tensor x = self.contiguous();
  if (dt == at::kDouble) x = x.to(at::kFloat), dt = at::kFloat;
  else if (dt == at::kShort || dt == at::kChar) x = x.to(at::kInt), dt = at::kInt;
  else if (at::isComplexType(dt)) x = at::view_as_real(x).abs().sum(-1).contiguous(), dt = x.scalar_type();
  const int64_t n = x.numel();
  TORCH_CHECK(n < (1ll << 31), "nonzero: tensors with 2^31 or more elements are not supported");
  auto stream = current_raw_stream(self);
  at::Tensor linear = at::empty({n}, self.options().dtype(at::kLong));
  at::Tensor count = at::empty({1}, self.options().dtype(at::kLong));
  size_t bytes = 0;
  B200_KERNEL_CALL(b200_nonzero_linear(nullptr, &bytes, linear.data_ptr<int64_t>(), count.data_ptr<int64_t>(),
                                       x.const_data_ptr(), loops::any_dtype(dt), n, stream));
  at::Tensor temp = at::empty({(int64_t)bytes}, self.options().dtype(at::kByte));
  B200_KERNEL_CALL(b200_nonzero_linear(temp.data_ptr(), &bytes, linear.data_ptr<int64_t>(), count.data_ptr<int64_t>(),
                                       x.const_data_ptr(), loops::any_dtype(dt), n, stream));
  const int64_t nnz = count.item<int64_t>();  // the output shape depends on the data
  const int nd = (int)self.dim();
  at::Tensor coords = at::empty({nnz, nd}, self.options().dtype(at::kLong));
  if (nnz > 0 && nd > 0) {
    TORCH_CHECK(nd <= 8, "nonzero: more than 8 dimensions");
    std::vector<int64_t> sizes(self.sizes().begin(), self.sizes().end());
    B200_KERNEL_CALL(b200_unravel(coords.data_ptr<int64_t>(), linear.const_data_ptr<int64_t>(), count.const_data_ptr<int64_t>(),
                                  nnz, sizes.data(), nd, stream));
  }
  return coords;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> unique2(const at::Tensor& self, bool /*sorted*/, bool return_inverse,
                                                       bool return_counts) {
  at::ScalarType dt = self.scalar_type();
  at::Tensor flat = self.reshape({-1});
  at::ScalarType kd = dt;
  if (dt == at::kBFloat16 || dt == at::kHalf || dt == at::kDouble) kd = at::kFloat;   // exact for the 16-bit types
  else if (dt == at::kShort || dt == at::kChar || dt == at::kByte || dt == at::kBool) kd = at::kInt;
  TORCH_CHECK(kd == at::kFloat || kd == at::kInt || kd == at::kLong, "unique: unsupported dtype ", dt);
  const int64_t n = flat.numel();
  at::Tensor inverse = at::empty({0}, self.options().dtype(at::kLong)), counts = at::empty({0}, self.options().dtype(at::kLong));
  if (n == 0) return {at::empty({0}, self.options()), inverse, counts};
  auto sorted = at::sort(flat.to(kd), /*stable=*/true, 0, false);
  const at::Tensor keys = std::get<0>(sorted).contiguous(), perm = std::get<1>(sorted).contiguous();
  auto stream = current_raw_stream(self);
  at::Tensor uniq = at::empty({n}, keys.options()), cnt = at::empty({n}, self.options().dtype(at::kLong));
  at::Tensor runs = at::empty({1}, self.options().dtype(at::kLong));
  at::Tensor run_id;
  if (return_inverse) run_id = at::empty({n}, self.options().dtype(at::kLong));
  size_t bytes = 0;
  B200_KERNEL_CALL(b200_unique_sorted(nullptr, &bytes, keys.const_data_ptr(), uniq.data_ptr(), cnt.data_ptr<int64_t>(),
                                      runs.data_ptr<int64_t>(), run_id.defined() ? run_id.data_ptr<int64_t>() : nullptr,
                                      loops::any_dtype(kd), n, stream));
  at::Tensor temp = at::empty({(int64_t)bytes}, self.options().dtype(at::kByte));
  B200_KERNEL_CALL(b200_unique_sorted(temp.data_ptr(), &bytes, keys.const_data_ptr(), uniq.data_ptr(), cnt.data_ptr<int64_t>(),
                                      runs.data_ptr<int64_t>(), run_id.defined() ? run_id.data_ptr<int64_t>() : nullptr,
                                      loops::any_dtype(kd), n, stream));
  const int64_t m = runs.item<int64_t>();
  at::Tensor out = uniq.narrow(0, 0, m).to(dt);
  if (return_inverse) {
    inverse = at::empty({n}, self.options().dtype(at::kLong));
    B200_KERNEL_CALL(b200_scatter_inverse(inverse.data_ptr<int64_t>(), run_id.const_data_ptr<int64_t>(),
                                          perm.const_data_ptr<int64_t>(), n, stream));
    inverse = inverse.view(self.sizes());
  }
  if (return_counts) counts = cnt.narrow(0, 0, m).clone();
  return {out, inverse, counts};
}

// ---------------------------------------------------------------- group norm (composed from the backend's kernels)
std::tuple<at::Tensor, at::Tensor, at::Tensor> native_group_norm(const at::Tensor& X, const std::optional<at::Tensor>& w,
                                                                 const std::optional<at::Tensor>& b, int64_t N, int64_t C,
                                                                 int64_t HxW, int64_t G, double eps) {
  TORCH_CHECK(G > 0 && C % G == 0, "group_norm: channels must divide by the number of groups");
  const at::Tensor x = X.contiguous().view({N, G, (C / G) * HxW}).to(at::kFloat);
  auto vm = at::var_mean(x, at::IntArrayRef({2}), /*correction=*/at::Scalar(0), /*keepdim=*/true);
  const at::Tensor var = std::get<0>(vm), mean = std::get<1>(vm);
  const at::Tensor rstd = at::rsqrt(var + eps);
  at::Tensor y = ((x - mean) * rstd).view({N, C, HxW});
  if (w.has_value() && w->defined()) y = y * w->to(at::kFloat).view({1, C, 1});
  if (b.has_value() && b->defined()) y = y + b->to(at::kFloat).view({1, C, 1});
  return {y.view(X.sizes()).to(X.scalar_type()), mean.view({N, G}).to(X.scalar_type()), rstd.view({N, G}).to(X.scalar_type())};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> native_group_norm_backward(
    const at::Tensor& dY, const at::Tensor& X, const at::Tensor& mean, const at::Tensor& rstd,
    const std::optional<at::Tensor>& w, int64_t N, int64_t C, int64_t HxW, int64_t G, std::array<bool, 3> mask) {
  const int64_t D = (C / G) * HxW;
  const at::Tensor x = X.contiguous().view({N, G, D}).to(at::kFloat);
  const at::Tensor dy = dY.contiguous().view({N, C, HxW}).to(at::kFloat);
  const at::Tensor mu = mean.to(at::kFloat).view({N, G, 1}), rs = rstd.to(at::kFloat).view({N, G, 1});
  const at::Tensor xhat = (x - mu) * rs;
  at::Tensor dx, dw, db;
  if (mask[1]) dw = (dy * xhat.view({N, C, HxW})).sum(at::IntArrayRef({0, 2})).to(X.scalar_type());
  if (mask[2]) db = dy.sum(at::IntArrayRef({0, 2})).to(X.scalar_type());
  if (mask[0]) {
    at::Tensor dxhat = dy;
    if (w.has_value() && w->defined()) dxhat = dy * w->to(at::kFloat).view({1, C, 1});
    dxhat = dxhat.view({N, G, D});
    const at::Tensor s1 = dxhat.sum(at::IntArrayRef({2}), true), s2 = (dxhat * xhat).sum(at::IntArrayRef({2}), true);
    dx = ((dxhat * (double)D - s1 - xhat * s2) * (rs / (double)D)).view(X.sizes()).to(X.scalar_type());
  }
  return {dx, dw, db};
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("searchsorted.Tensor", TORCH_FN(searchsorted_tensor));
  m.impl("searchsorted.Tensor_out", TORCH_FN(searchsorted_tensor_out));
  m.impl("bucketize.Tensor", TORCH_FN(bucketize_tensor));
  m.impl("bucketize.Tensor_out", TORCH_FN(bucketize_tensor_out));
  m.impl("histc", TORCH_FN(histc));
  m.impl("nonzero", TORCH_FN(nonzero));
  m.impl("_unique2", TORCH_FN(unique2));
  m.impl("native_group_norm", TORCH_FN(native_group_norm));
  m.impl("native_group_norm_backward", TORCH_FN(native_group_norm_backward));
}

}  // namespace ops
}  // namespace b200
