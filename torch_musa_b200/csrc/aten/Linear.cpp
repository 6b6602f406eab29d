// mm / addmm / bmm / baddbmm / _addmm_activation on the tcgen05 GEMM kernel.
// Operand layouts are taken from the strides (a transposed view is an MN-major
// operand, not a copy), bias and activation ride in the epilogue, and anything the
// kernel does not cover (fp32/fp64/complex/int, unaligned leading dimensions) goes
// to the library GEMM through the CUDA-alias fallback.
// Parity: reference torch_musa/csrc/aten/ops/Matmul.cpp:258-344,475-497, Baddbmm.cpp.
#include "aten/FallbackCall.h"
#include "aten/Ops.h"

#include <ATen/ExpandUtils.h>
#include <ATen/Context.h>
#include <ATen/Functions.h>
#include <ATen/native/Resize.h>
#include <torch/library.h>

#include <atomic>

namespace b200 {
namespace ops {

namespace {

std::atomic<bool> g_use_tc_gemm{true};

struct Operand {
  at::Tensor t;     // keeps a contiguous copy alive if one was needed
  bool kmajor;      // reduction dim contiguous
  int64_t ld;       // leading stride in elements
  int64_t bstride;  // batch stride (3-D operands)
};

// t is [.., rows, red] for A (rows = M) or [.., red, cols] for B (viewed as [cols, red] logically).
// `red_dim` is the index of the reduction dimension among the last two.
bool describe(const at::Tensor& t, int red_dim, Operand* out) {
  const int nd = t.dim();
  const int other = (red_dim == nd - 1) ? nd - 2 : nd - 1;
  auto mk = [&](const at::Tensor& x) -> bool {
    int64_t sr = x.stride(red_dim), so = x.stride(other);
    int64_t nr = x.size(red_dim), no = x.size(other);
    if ((sr == 1 || nr == 1) && (so >= std::max<int64_t>(nr, 1)) ) {
      out->kmajor = true;
      out->ld = so;
    } else if ((so == 1 || no == 1) && sr >= std::max<int64_t>(no, 1)) {
      out->kmajor = false;
      out->ld = sr;
    } else {
      return false;
    }
    out->bstride = nd == 3 ? x.stride(0) : 0;
    out->t = x;
    return true;
  };
  if (mk(t)) return true;
  return mk(t.contiguous());
}

bool gemm_eligible(const at::Tensor& a, const at::Tensor& b) {
  if (!g_use_tc_gemm.load(std::memory_order_relaxed)) return false;
  auto dt = a.scalar_type();
  if (dt != b.scalar_type()) return false;
  // fp32 operands multiply on the tensor cores as tf32 when the caller allows that precision
  // (torch.backends.blackwell.allow_tf32 / torch.set_float32_matmul_precision); strict fp32 is a library GEMM
  if (dt == at::kFloat) {
    if (!at::globalContext().allowTF32CuBLAS()) return false;
  } else if (dt != at::kBFloat16 && dt != at::kHalf) {
    return false;
  }
  if (a.is_conj() || b.is_conj() || a.is_neg() || b.is_neg()) return false;
  if (!on_device(a) || !on_device(b) || a.device() != b.device()) return false;  // the generic route reports the mismatch
  return true;
}

// out[M,N] = alpha * a[M,K] @ b[K,N] (+ bias) ; returns false if the kernel declined
bool run_gemm(const at::Tensor& out, const at::Tensor& a, const at::Tensor& b, const at::Tensor* bias, int act,
              float alpha, bool accumulate) {
  const int nd = a.dim();
  Operand A, B;
  if (!describe(a, nd - 1, &A)) return false;
  if (!describe(b, nd - 2, &B)) return false;
  if (a.scalar_type() == at::kFloat) {
    // the tf32 kernel reads both operands with the reduction dimension contiguous: re-lay out what is not
    if (out.scalar_type() != at::kFloat || accumulate) return false;
    if (!A.kmajor && !describe(a.contiguous(), nd - 1, &A)) return false;
    if (!B.kmajor) {
      const at::Tensor bt = b.transpose(nd - 2, nd - 1).contiguous().transpose(nd - 2, nd - 1);
      if (!describe(bt, nd - 2, &B)) return false;
    }
    if (!A.kmajor || !B.kmajor) return false;
  }
  b200_gemm_desc_t g{};
  g.m = (int)a.size(nd - 2);
  g.k = (int)a.size(nd - 1);
  g.n = (int)b.size(nd - 1);
  g.a_kmajor = A.kmajor;
  g.b_kmajor = B.kmajor;
  g.lda = A.ld;
  g.ldb = B.ld;
  g.ldd = out.stride(nd - 2);
  g.in_dtype = kdtype(a.scalar_type());
  g.out_dtype = kdtype(out.scalar_type());
  g.batch = nd == 3 ? (int)a.size(0) : 1;
  g.stride_a = A.bstride;
  g.stride_b = B.bstride;
  g.stride_d = nd == 3 ? out.stride(0) : 0;
  if (bias) check_devices("addmm", out, *bias);
  check_devices("mm", out, a, b);
  g.bias = bias ? bias->const_data_ptr() : nullptr;
  g.bias_dtype = bias ? kdtype(bias->scalar_type()) : 0;
  g.act = act;
  g.accumulate = accumulate;
  g.alpha = alpha;
  if (g.out_dtype < 0 || out.stride(nd - 1) != 1) return false;
  DeviceSwitch sw(out.device().index());
  at::Tensor workspace;
  if (const size_t ws = b200_gemm_workspace_bytes(&g)) {
    workspace = at::empty({(int64_t)(ws / sizeof(float))}, out.options().dtype(at::kFloat));
    g.workspace = workspace.mutable_data_ptr();
    g.workspace_bytes = ws;
  }
  int e = b200_gemm(&g, out.mutable_data_ptr(), A.t.const_data_ptr(), B.t.const_data_ptr(), current_raw_stream(out));
  if (e == (int)cudaErrorNotSupported) return false;
  B200_KERNEL_CALL(e);
  return true;
}

at::Tensor mm(const at::Tensor& self, const at::Tensor& mat2) {
  TORCH_CHECK(self.dim() == 2 && mat2.dim() == 2, "mm: expected 2-D tensors");
  TORCH_CHECK(self.size(1) == mat2.size(0), "mat1 and mat2 shapes cannot be multiplied (", self.size(0), "x",
              self.size(1), " and ", mat2.size(0), "x", mat2.size(1), ")");
  if (gemm_eligible(self, mat2) && self.size(1) > 0) {
    at::Tensor out = at::empty({self.size(0), mat2.size(1)}, self.options());
    if (out.numel() == 0) return out;
    if (run_gemm(out, self, mat2, nullptr, 0, 1.f, false)) return out;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::mm", ""), self, mat2);
}

at::Tensor& mm_out(const at::Tensor& self, const at::Tensor& mat2, at::Tensor& out) {
  if (gemm_eligible(self, mat2) && self.dim() == 2 && mat2.dim() == 2 && self.size(1) == mat2.size(0) &&
      self.size(1) > 0 && out.scalar_type() == self.scalar_type()) {
    at::native::resize_output(out, {self.size(0), mat2.size(1)});
    if (out.numel() == 0) return out;
    if (out.stride(1) == 1 && run_gemm(out, self, mat2, nullptr, 0, 1.f, false)) return out;
  }
  run_fallback(B200_OP_HANDLE("aten::mm", "out"), self, mat2, out);
  return out;
}

at::Tensor addmm_impl(const at::Tensor& self, const at::Tensor& mat1, const at::Tensor& mat2, const at::Scalar& beta,
                      const at::Scalar& alpha, int act, bool* handled) {
  *handled = false;
  if (!(gemm_eligible(mat1, mat2) && mat1.dim() == 2 && mat2.dim() == 2 && mat1.size(1) == mat2.size(0) &&
        mat1.size(1) > 0 && self.scalar_type() == mat1.scalar_type()))
    return {};
  const int64_t M = mat1.size(0), N = mat2.size(1);
  const double b = beta.toDouble(), a = alpha.toDouble();
  // bias vector [N] (or [1,N]) with beta == 1: epilogue add
  bool row_bias = b == 1.0 && self.is_contiguous() &&
                  ((self.dim() == 1 && self.size(0) == N) || (self.dim() == 2 && self.size(0) == 1 && self.size(1) == N && M != 1));
  at::Tensor out = at::empty({M, N}, mat1.options());
  if (out.numel() == 0) { *handled = true; return out; }
  if (row_bias) {
    // alpha scales the product only; the bias is added after scaling
    if (run_gemm(out, mat1, mat2, &self, act, (float)a, false)) { *handled = true; return out; }
    return {};
  }
  if (act != 0) return {};
  if (b == 0.0) {
    if (run_gemm(out, mat1, mat2, nullptr, 0, (float)a, false)) { *handled = true; return out; }
    return {};
  }
  // general: out = beta*self (broadcast) then accumulate the product
  out.copy_(self.expand({M, N}));
  if (b != 1.0) out.mul_(beta);
  if (run_gemm(out, mat1, mat2, nullptr, 0, (float)a, true)) { *handled = true; return out; }
  return {};
}

at::Tensor addmm(const at::Tensor& self, const at::Tensor& mat1, const at::Tensor& mat2, const at::Scalar& beta,
                 const at::Scalar& alpha) {
  bool handled;
  at::Tensor out = addmm_impl(self, mat1, mat2, beta, alpha, 0, &handled);
  if (handled) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::addmm", ""), self, mat1, mat2, beta, alpha);
}

at::Tensor addmm_activation(const at::Tensor& self, const at::Tensor& mat1, const at::Tensor& mat2,
                            const at::Scalar& beta, const at::Scalar& alpha, bool use_gelu) {
  bool handled;
  at::Tensor out = addmm_impl(self, mat1, mat2, beta, alpha, use_gelu ? 2 : 1, &handled);
  if (handled) return out;
  return fallback_tensor(B200_OP_HANDLE("aten::_addmm_activation", ""), self, mat1, mat2, beta, alpha, use_gelu);
}

at::Tensor bmm(const at::Tensor& self, const at::Tensor& mat2) {
  TORCH_CHECK(self.dim() == 3 && mat2.dim() == 3, "bmm: expected 3-D tensors");
  TORCH_CHECK(self.size(0) == mat2.size(0) && self.size(2) == mat2.size(1), "bmm: incompatible shapes ", self.sizes(),
              " and ", mat2.sizes());
  if (gemm_eligible(self, mat2) && self.size(2) > 0) {
    at::Tensor out = at::empty({self.size(0), self.size(1), mat2.size(2)}, self.options());
    if (out.numel() == 0) return out;
    if (run_gemm(out, self, mat2, nullptr, 0, 1.f, false)) return out;
  }
  return fallback_tensor(B200_OP_HANDLE("aten::bmm", ""), self, mat2);
}

at::Tensor baddbmm(const at::Tensor& self, const at::Tensor& b1, const at::Tensor& b2, const at::Scalar& beta,
                   const at::Scalar& alpha) {
  if (gemm_eligible(b1, b2) && b1.dim() == 3 && b2.dim() == 3 && b1.size(2) > 0 &&
      self.scalar_type() == b1.scalar_type() && b1.size(0) == b2.size(0) && b1.size(2) == b2.size(1)) {
    at::Tensor out = at::empty({b1.size(0), b1.size(1), b2.size(2)}, b1.options());
    if (out.numel() == 0) return out;
    const double b = beta.toDouble();
    if (b == 0.0) {
      if (run_gemm(out, b1, b2, nullptr, 0, alpha.toFloat(), false)) return out;
    } else {
      out.copy_(self.expand(out.sizes()));
      if (b != 1.0) out.mul_(beta);
      if (run_gemm(out, b1, b2, nullptr, 0, alpha.toFloat(), true)) return out;
    }
  }
  return fallback_tensor(B200_OP_HANDLE("aten::baddbmm", ""), self, b1, b2, beta, alpha);
}

}  // namespace

void set_tensor_core_gemm(bool on) { g_use_tc_gemm = on; }
bool tensor_core_gemm_enabled() { return g_use_tc_gemm; }

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("mm", TORCH_FN(mm));
  m.impl("mm.out", TORCH_FN(mm_out));
  m.impl("addmm", TORCH_FN(addmm));
  m.impl("_addmm_activation", TORCH_FN(addmm_activation));
  m.impl("bmm", TORCH_FN(bmm));
  m.impl("baddbmm", TORCH_FN(baddbmm));
}

}  // namespace ops
}  // namespace b200
