// fp8 matrix products on the block-scaled tcgen05 kernel.
//
//   blackwell::scaled_mm(a, b, block_scale_a?, block_scale_b?, row_scale?, col_scale?, bias?, out_dtype)
//       a [M, K] fp8 (K contiguous), b [N, K] fp8 (K contiguous); block_scale_a [M, K/128] (1 x 128 blocks),
//       block_scale_b [N/128, K/128] (128 x 128 blocks), row_scale [M] or scalar, col_scale [N] or scalar.
//   blackwell::quantize_fp8_1x128(x, e5m2=False) -> (q, scales): per 1 x 128 block amax / 448 scaling.
//   aten::_scaled_mm: tensor-wise, row-wise and 1x128 / 128x128 block-wise scale layouts are mapped onto the
//       same kernel; anything else goes to the library through the CUDA-alias bridge.
// Parity: reference torch_musa/csrc/aten/ops/Matmul.cpp:670-681 (_scaled_mm through the vendor library).
#include "aten/FallbackCall.h"
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {

using Opt = std::optional<at::Tensor>;

bool is_fp8(at::ScalarType t) { return t == at::kFloat8_e4m3fn || t == at::kFloat8_e5m2; }
bool defined(const Opt& t) { return t.has_value() && t->defined(); }

void check_scale(const char* what, const at::Tensor& ref, const Opt& s) {
  if (!defined(s)) return;
  check_devices("scaled_mm", ref, *s);
  TORCH_CHECK(s->scalar_type() == at::kFloat, "scaled_mm: ", what, " must be float32");
}

at::Tensor scaled_mm(const at::Tensor& a, const at::Tensor& b, const Opt& bsa, const Opt& bsb, const Opt& row_scale,
                     const Opt& col_scale, const Opt& bias, at::ScalarType out_dtype) {
  TORCH_CHECK(on_device(a) && on_device(b) && a.device() == b.device(), "scaled_mm: operands must be on one blackwell device");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && is_fp8(a.scalar_type()) && is_fp8(b.scalar_type()) && a.size(1) == b.size(1),
              "scaled_mm: a [M, K] and b [N, K] must be fp8 with the same K");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1, "scaled_mm: K must be the contiguous dimension of both operands");
  const int64_t M = a.size(0), K = a.size(1), N = b.size(0);
  check_scale("block_scale_a", a, bsa);
  check_scale("block_scale_b", a, bsb);
  check_scale("row_scale", a, row_scale);
  check_scale("col_scale", a, col_scale);
  if (defined(bias)) check_devices("scaled_mm", a, *bias);
  at::Tensor out = at::empty({M, N}, a.options().dtype(out_dtype));
  if (out.numel() == 0) return out;
  b200_fp8_gemm_t g{};
  g.m = (int)M; g.n = (int)N; g.k = (int)K;
  g.lda = a.stride(0); g.ldb = b.stride(0); g.ldd = N;
  g.a_e5m2 = a.scalar_type() == at::kFloat8_e5m2;
  g.b_e5m2 = b.scalar_type() == at::kFloat8_e5m2;
  g.out_dtype = kdtype(out_dtype);
  TORCH_CHECK(g.out_dtype >= 0, "scaled_mm: output dtype must be float32, bfloat16 or float16");
  if (defined(bsa)) {
    TORCH_CHECK(bsa->dim() == 2 && bsa->size(0) == M && bsa->size(1) == (K + 127) / 128, "scaled_mm: block_scale_a must be [M, K/128]");
    g.block_scale_a = bsa->const_data_ptr<float>();
    g.bsa_stride_m = bsa->stride(0);
    g.bsa_stride_kb = bsa->stride(1);
  }
  if (defined(bsb)) {
    TORCH_CHECK(bsb->dim() == 2 && bsb->size(0) == (N + 127) / 128 && bsb->size(1) == (K + 127) / 128,
                "scaled_mm: block_scale_b must be [N/128, K/128]");
    g.block_scale_b = bsb->const_data_ptr<float>();
    g.bsb_stride_nb = bsb->stride(0);
    g.bsb_stride_kb = bsb->stride(1);
  }
  if (defined(row_scale)) {
    TORCH_CHECK(row_scale->numel() == 1 || row_scale->numel() == M, "scaled_mm: row_scale must have 1 or M elements");
    g.row_scale = row_scale->const_data_ptr<float>();
    g.row_scale_stride = row_scale->numel() == 1 ? 0 : (row_scale->dim() == 2 ? row_scale->stride(0) : row_scale->stride(-1));
  }
  if (defined(col_scale)) {
    TORCH_CHECK(col_scale->numel() == 1 || col_scale->numel() == N, "scaled_mm: col_scale must have 1 or N elements");
    g.col_scale = col_scale->const_data_ptr<float>();
    g.col_scale_stride = col_scale->numel() == 1 ? 0 : col_scale->stride(-1);
  }
  if (defined(bias)) {
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous() &&
                (bias->scalar_type() == out_dtype || bias->scalar_type() == at::kFloat), "scaled_mm: bias must be [N] in the output dtype or float32");
    g.bias = bias->const_data_ptr();
    g.bias_dtype = kdtype(bias->scalar_type());
  }
  DeviceSwitch sw(a.device().index());
  int e = b200_gemm_fp8(&g, out.mutable_data_ptr(), a.const_data_ptr(), b.const_data_ptr(), current_raw_stream(a));
  TORCH_CHECK(e != (int)cudaErrorNotSupported, "scaled_mm: layout not covered (K % 16, 16-byte aligned rows; block scales need K % 128 == 0)");
  B200_KERNEL_CALL(e);
  return out;
}

std::tuple<at::Tensor, at::Tensor> quantize_fp8_1x128(const at::Tensor& x, bool e5m2) {
  TORCH_CHECK(on_device(x) && x.dim() == 2 && kdtype(x.scalar_type()) >= 0 && x.stride(1) == 1,
              "quantize_fp8_1x128: x must be a 2-D float device tensor with contiguous rows");
  TORCH_CHECK(x.size(1) % 128 == 0, "quantize_fp8_1x128: the row length must be a multiple of 128");
  at::Tensor q = at::empty(x.sizes(), x.options().dtype(e5m2 ? at::kFloat8_e5m2 : at::kFloat8_e4m3fn));
  at::Tensor s = at::empty({x.size(0), x.size(1) / 128}, x.options().dtype(at::kFloat));
  DeviceSwitch sw(x.device().index());
  B200_KERNEL_CALL(b200_quantize_fp8_1x128(kdtype(x.scalar_type()), x.const_data_ptr(), q.mutable_data_ptr(),
                                           s.data_ptr<float>(), x.size(0), (int)x.size(1), x.stride(0), e5m2 ? 1 : 0,
                                           current_raw_stream(x)));
  return {q, s};
}

at::Tensor aten_scaled_mm(const at::Tensor& self, const at::Tensor& mat2, const at::Tensor& scale_a,
                          const at::Tensor& scale_b, const Opt& bias, const Opt& scale_result,
                          std::optional<at::ScalarType> out_dtype, bool use_fast_accum) {
  const at::ScalarType odt = out_dtype.value_or(at::kBFloat16);
  const bool layout_ok = self.dim() == 2 && mat2.dim() == 2 && is_fp8(self.scalar_type()) && is_fp8(mat2.scalar_type()) &&
                         self.stride(1) == 1 && mat2.stride(0) == 1 && !defined(scale_result) && kdtype(odt) >= 0 &&
                         on_device(scale_a) && on_device(scale_b) && scale_a.scalar_type() == at::kFloat &&
                         scale_b.scalar_type() == at::kFloat && self.size(1) % 16 == 0;
  if (layout_ok) {
    const int64_t M = self.size(0), K = self.size(1), N = mat2.size(1), KB = (K + 127) / 128;
    const at::Tensor b = mat2.t();   // [N, K], K contiguous
    if (scale_a.numel() == 1 && scale_b.numel() == 1)
      return scaled_mm(self, b, std::nullopt, std::nullopt, scale_a, scale_b, bias, odt);
    if (scale_a.numel() == M && scale_b.numel() == N && scale_a.dim() == 2 && scale_a.size(1) == 1)
      return scaled_mm(self, b, std::nullopt, std::nullopt, scale_a, scale_b.reshape({N}), bias, odt);
    if (K % 128 == 0 && scale_a.dim() == 2 && scale_a.size(0) == M && scale_a.size(1) == KB && scale_b.dim() == 2 &&
        scale_b.size(0) == KB && scale_b.size(1) == (N + 127) / 128)
      return scaled_mm(self, b, scale_a, scale_b.t(), std::nullopt, std::nullopt, bias, odt);
  }
  auto st = run_fallback(B200_OP_HANDLE("aten::_scaled_mm", ""), self, mat2, scale_a, scale_b, bias, scale_result,
                         out_dtype, use_fast_accum);
  return st.back().toTensor();
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(blackwell, m) {
  m.def("scaled_mm(Tensor a, Tensor b, Tensor? block_scale_a, Tensor? block_scale_b, Tensor? row_scale, Tensor? col_scale, "
        "Tensor? bias, ScalarType out_dtype) -> Tensor");
  m.def("quantize_fp8_1x128(Tensor x, bool e5m2=False) -> (Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(blackwell, PrivateUse1, m) {
  m.impl("scaled_mm", TORCH_FN(scaled_mm));
  m.impl("quantize_fp8_1x128", TORCH_FN(quantize_fp8_1x128));
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) { m.impl("_scaled_mm", TORCH_FN(aten_scaled_mm)); }

}  // namespace ops
}  // namespace b200
