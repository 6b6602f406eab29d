// Front-ends for quantized (per-tensor affine int8 / uint8) and sparse COO tensors on the device.
//
// Quantized tensors keep their integer payload in device memory with a quantizer attached; quantize /
// dequantize / int_repr run on the backend's element-wise kernels.  Sparse COO tensors hold device index and
// value tensors; densification, coalescing and sparse x dense products are composed from the backend's sort,
// unique, index_select and index_put kernels.  Parity: reference torch_musa/csrc/aten/quantized/* (quantizer,
// QTensor factories, int_repr / dequantize) and the sparse operator registrations of its generated op list.
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <ATen/NativeFunctions.h>
#include <ATen/SparseTensorImpl.h>
#include <ATen/TensorOperators.h>
#include <ATen/quantized/QTensorImpl.h>
#include <ATen/quantized/Quantizer.h>
#include <torch/library.h>

namespace b200 {
namespace ops {
namespace {

// ------------------------------------------------------------------ quantized
at::ScalarType underlying(at::ScalarType q) {
  switch (q) {
    case at::kQInt8: return at::kChar;
    case at::kQUInt8: return at::kByte;
    case at::kQInt32: return at::kInt;
    default: TORCH_CHECK(false, "blackwell quantized tensors support qint8, quint8 and qint32, got ", q);
  }
}
std::pair<double, double> qrange(at::ScalarType q) {
  switch (q) {
    case at::kQInt8: return {-128., 127.};
    case at::kQUInt8: return {0., 255.};
    default: return {-2147483648., 2147483647.};
  }
}

void device_copy_bytes(void* dst, const void* src, size_t n, const at::Tensor& on) {
  if (n == 0) return;
  B200_CUDA_CHECK(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToDevice, current_raw_stream(on)));
}

at::Tensor empty_affine_quantized(at::IntArrayRef size, std::optional<at::ScalarType> dtype, std::optional<at::Layout> layout,
                                  std::optional<at::Device> device, std::optional<bool> pin, double scale, int64_t zero_point,
                                  std::optional<at::MemoryFormat> mf) {
  TORCH_CHECK(dtype.has_value() && at::isQIntType(*dtype), "_empty_affine_quantized needs a quantized dtype");
  auto options = at::TensorOptions().dtype(*dtype).device(device.value_or(at::Device(kDeviceType, current_device())));
  return at::new_qtensor(size, options.memory_format(mf.value_or(at::MemoryFormat::Contiguous)),
                         at::make_per_tensor_affine_quantizer(scale, zero_point, *dtype));
}

at::Tensor quantize_per_tensor(const at::Tensor& self, double scale, int64_t zero_point, at::ScalarType dtype) {
  TORCH_CHECK(scale > 0, "quantize_per_tensor: scale must be positive");
  const at::Tensor x = self.contiguous().to(at::kFloat);
  auto [lo, hi] = qrange(dtype);
  at::Tensor ints = at::clamp(at::round(x / scale) + (double)zero_point, lo, hi).to(underlying(dtype));
  at::Tensor q = at::new_qtensor(self.sizes(), self.options().dtype(dtype),
                                 at::make_per_tensor_affine_quantizer(scale, zero_point, dtype));
  device_copy_bytes(q.data_ptr(), ints.const_data_ptr(), (size_t)ints.numel() * ints.element_size(), self);
  return q;
}

at::Tensor make_per_tensor_quantized_tensor(const at::Tensor& self, double scale, int64_t zero_point) {
  const at::ScalarType qt = self.scalar_type() == at::kChar ? at::kQInt8 : self.scalar_type() == at::kByte ? at::kQUInt8
                                                                                                            : at::kQInt32;
  TORCH_CHECK(underlying(qt) == self.scalar_type(), "_make_per_tensor_quantized_tensor expects int8, uint8 or int32");
  const at::Tensor src = self.contiguous();
  at::Tensor q = at::new_qtensor(self.sizes(), self.options().dtype(qt), at::make_per_tensor_affine_quantizer(scale, zero_point, qt));
  device_copy_bytes(q.data_ptr(), src.const_data_ptr(), (size_t)src.numel() * src.element_size(), self);
  return q;
}

const at::PerTensorAffineQuantizer& quantizer_of(const at::Tensor& q) {
  auto qz = at::get_qtensorimpl(q)->quantizer();
  TORCH_CHECK(qz->qscheme() == at::kPerTensorAffine, "only per-tensor affine quantization is supported on this device");
  return *static_cast<at::PerTensorAffineQuantizer*>(qz.get());
}

at::Tensor q_int_repr(const at::Tensor& self) {
  const at::ScalarType ut = underlying(self.scalar_type());
  at::Tensor out = at::empty(self.sizes(), at::TensorOptions().dtype(ut).device(self.device()));
  const at::Tensor src = self.is_contiguous() ? self : self.contiguous();
  device_copy_bytes(out.data_ptr(), src.data_ptr(), (size_t)out.numel() * out.element_size(), out);
  return out;
}
at::Tensor dequantize(const at::Tensor& self) {
  const auto& qz = quantizer_of(self);
  return (q_int_repr(self).to(at::kFloat) - (double)qz.zero_point()) * qz.scale();
}
double q_scale(const at::Tensor& self) { return quantizer_of(self).scale(); }
int64_t q_zero_point(const at::Tensor& self) { return quantizer_of(self).zero_point(); }
at::QScheme qscheme(const at::Tensor& self) { return at::get_qtensorimpl(self)->quantizer()->qscheme(); }
at::Tensor quantized_clone(const at::Tensor& self, std::optional<at::MemoryFormat>) {
  const auto& qz = quantizer_of(self);
  return make_per_tensor_quantized_tensor(q_int_repr(self), qz.scale(), qz.zero_point());
}

// ------------------------------------------------------------------ sparse COO
at::Tensor sparse_coo_with_dims_and_tensors(int64_t sparse_dim, int64_t dense_dim, c10::SymIntArrayRef size,
                                            const at::Tensor& indices, const at::Tensor& values,
                                            std::optional<at::ScalarType> dtype, std::optional<at::Layout> layout,
                                            std::optional<at::Device> device, std::optional<bool> pin,
                                            std::optional<bool> is_coalesced) {
  return at::native::new_with_dims_and_tensor_sparse_symint(sparse_dim, dense_dim, size, indices, values, dtype, layout, device,
                                                            pin, is_coalesced);
}

// row-major linear index of every non-zero over the sparse dimensions
at::Tensor linear_index(const at::Tensor& indices, at::IntArrayRef sizes, int64_t sparse_dim) {
  at::Tensor lin = at::zeros({indices.size(1)}, indices.options());
  int64_t mult = 1;
  for (int64_t d = sparse_dim - 1; d >= 0; --d) {
    lin = lin + indices.select(0, d) * mult;
    mult *= sizes[d];
  }
  return lin;
}

at::Tensor sparse_to_dense(const at::Tensor& self, std::optional<at::ScalarType> dtype, std::optional<bool>) {
  const int64_t sd = self.sparse_dim();
  const at::Tensor idx = self._indices(), val = self._values();
  int64_t rows = 1;
  for (int64_t d = 0; d < sd; ++d) rows *= self.size(d);
  std::vector<int64_t> flat_shape{rows};
  for (int64_t d = sd; d < self.dim(); ++d) flat_shape.push_back(self.size(d));
  at::Tensor out = at::zeros(flat_shape, val.options());
  if (val.size(0) > 0) out.index_add_(0, linear_index(idx, self.sizes(), sd), val);   // duplicates add up
  out = out.view(self.sizes());
  return dtype.has_value() ? out.to(*dtype) : out;
}

at::Tensor sparse_coalesce(const at::Tensor& self) {
  const int64_t sd = self.sparse_dim();
  const at::Tensor idx = self._indices(), val = self._values();
  if (val.size(0) < 2) {
    at::Tensor out = at::native::new_with_dims_and_tensor_sparse_symint(
        sd, self.dense_dim(), c10::fromIntArrayRefSlow(self.sizes()), idx.clone(), val.clone(), val.scalar_type(),
        at::kSparse, self.device(), std::nullopt, true);
    return out;
  }
  const at::Tensor lin = linear_index(idx, self.sizes(), sd);
  auto u = at::_unique2(lin, true, true, false);
  const at::Tensor uniq = std::get<0>(u), inverse = std::get<1>(u);
  std::vector<int64_t> vshape(val.sizes().begin(), val.sizes().end());
  vshape[0] = uniq.size(0);
  at::Tensor new_val = at::zeros(vshape, val.options());
  new_val.index_add_(0, inverse, val);
  // unravel the unique linear indices back to coordinates
  at::Tensor new_idx = at::empty({sd, uniq.size(0)}, idx.options());
  at::Tensor rem = uniq;
  for (int64_t d = sd - 1; d >= 0; --d) {
    new_idx.select(0, d).copy_(at::remainder(rem, self.size(d)));
    rem = at::floor_divide(rem, self.size(d));
  }
  return at::native::new_with_dims_and_tensor_sparse_symint(sd, self.dense_dim(), c10::fromIntArrayRefSlow(self.sizes()),
                                                            new_idx, new_val, val.scalar_type(), at::kSparse, self.device(),
                                                            std::nullopt, true);
}

// beta * self + alpha * (sparse [m, k] @ dense [k, n])
at::Tensor sparse_addmm(const at::Tensor& self, const at::Tensor& mat1, const at::Tensor& mat2, const at::Scalar& beta,
                        const at::Scalar& alpha) {
  TORCH_CHECK(mat1.is_sparse() && !mat2.is_sparse() && mat1.sparse_dim() == 2 && mat1.dense_dim() == 0 && mat2.dim() == 2,
              "addmm on this device supports sparse [m, k] x dense [k, n]");
  const at::Tensor idx = mat1._indices(), val = mat1._values();
  at::Tensor out = at::zeros({mat1.size(0), mat2.size(1)}, mat2.options());
  if (val.size(0) > 0) {
    const at::Tensor rows = at::index_select(mat2, 0, idx.select(0, 1)) * val.to(mat2.scalar_type()).unsqueeze(1);
    out.index_add_(0, idx.select(0, 0), rows);
  }
  out = out * alpha;
  if (beta.toDouble() != 0.0) out = out + self.expand_as(out) * beta;
  return out;
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("quantize_per_tensor", TORCH_FN(quantize_per_tensor));
  m.impl("_make_per_tensor_quantized_tensor", TORCH_FN(make_per_tensor_quantized_tensor));
}

TORCH_LIBRARY_IMPL(aten, QuantizedPrivateUse1, m) {
  m.impl("_empty_affine_quantized", TORCH_FN(empty_affine_quantized));
  m.impl("int_repr", TORCH_FN(q_int_repr));
  m.impl("dequantize.self", TORCH_FN(dequantize));
  m.impl("q_scale", TORCH_FN(q_scale));
  m.impl("q_zero_point", TORCH_FN(q_zero_point));
  m.impl("qscheme", TORCH_FN(qscheme));
  m.impl("clone", TORCH_FN(quantized_clone));
}

TORCH_LIBRARY_IMPL(aten, SparsePrivateUse1, m) {
  m.impl("_sparse_coo_tensor_with_dims_and_tensors", TORCH_FN(sparse_coo_with_dims_and_tensors));
  m.impl("_indices", TORCH_FN(at::native::_indices_sparse));
  m.impl("_values", TORCH_FN(at::native::_values_sparse));
  m.impl("_nnz", TORCH_FN(at::native::_nnz_sparse));
  m.impl("sparse_dim", TORCH_FN(at::native::sparse_dim_sparse));
  m.impl("dense_dim", TORCH_FN(at::native::dense_dim_sparse));
  m.impl("_dimI", TORCH_FN(at::native::sparse_dim_sparse));
  m.impl("_dimV", TORCH_FN(at::native::dense_dim_sparse));
  m.impl("is_coalesced", TORCH_FN(at::native::is_coalesced_sparse));
  m.impl("_coalesced_", TORCH_FN(at::native::_coalesced_sparse_));
  m.impl("indices", TORCH_FN(at::native::indices_sparse));
  m.impl("values", TORCH_FN(at::native::values_sparse));
  m.impl("_to_dense", TORCH_FN(sparse_to_dense));
  m.impl("_coalesce", TORCH_FN(sparse_coalesce));
  m.impl("addmm", TORCH_FN(sparse_addmm));
}

}  // namespace ops
}  // namespace b200
