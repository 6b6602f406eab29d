// Operators that stock ATen does not have, in the backend's own `blackwell::`
// namespace: rotary embedding, SwiGLU (packed / two-tensor), fused cross-entropy
// (forward keeps loss+lse, backward regenerates softmax, optionally in place),
// vocab-parallel cross-entropy pieces, residual-add RMSNorm, multi-tensor L2 norm /
// scale / LAMB, and a bounded device sleep.  Autograd formulas and fake-tensor
// rules are attached from Python (torch.library), so nothing in torch is patched.
// Parity: the reference adds these as new aten ops through torch patches
// (reference torch_patches/aten_src_ATen_native_native_functions.yaml.patch:10-83,
// torch_musa/csrc/aten/ops/RoPE.cpp, SwiGlu.cpp, Loss.cpp:547-660,
// csrc/extension/C_frontend.cpp:76-110).
#include "aten/FallbackCall.h"
#include "aten/Ops.h"

#include <ATen/Functions.h>

#include <cmath>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {

inline void check_fast(const at::Tensor& t, const char* what) {
  TORCH_CHECK(on_device(t), what, ": expected a blackwell tensor, got ", t.device());
  TORCH_CHECK(kdtype(t.scalar_type()) >= 0, what, ": unsupported dtype ", t.scalar_type(),
              " (float32, bfloat16, float16)");
}

at::Tensor rope(const at::Tensor& x, const at::Tensor& cos, const at::Tensor& sin,
                const std::optional<at::Tensor>& positions, bool interleaved, bool conj) {
  check_fast(x, "rope");
  check_devices("rope", x, cos, sin, positions);
  TORCH_CHECK(x.dim() == 4, "rope: x must be [batch, seq, heads, head_dim], got ", x.sizes());
  const int64_t B = x.size(0), S = x.size(1), H = x.size(2), D = x.size(3);
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat && cos.is_contiguous() &&
                  sin.is_contiguous() && cos.size(-1) == D / 2 && sin.size(-1) == D / 2,
              "rope: cos/sin must be contiguous float32 [positions, head_dim/2]");
  at::Tensor xin = x;
  if (x.stride(3) != 1 || x.stride(0) != x.stride(1) * S) xin = x.contiguous();
  at::Tensor out = at::empty({B, S, H, D}, x.options());
  if (out.numel() == 0) return out;
  const int64_t* pos = nullptr;
  at::Tensor p;
  if (positions.has_value() && positions->defined()) {
    p = positions->to(at::kLong).contiguous();
    TORCH_CHECK(p.numel() == B * S, "rope: positions must have batch*seq elements");
    pos = p.data_ptr<int64_t>();
  } else {
    TORCH_CHECK(cos.numel() / (D / 2) >= S, "rope: cos/sin cover ", cos.numel() / (D / 2), " positions, need ", S);
  }
  DeviceSwitch sw(x.device().index());
  B200_KERNEL_CALL(b200_rope(kdtype(x.scalar_type()), out.mutable_data_ptr(), xin.const_data_ptr(),
                             cos.data_ptr<float>(), sin.data_ptr<float>(), pos, B * S, S, (int)H, (int)D,
                             xin.stride(1), xin.stride(2), interleaved ? 1 : 0, conj ? 1 : 0, current_raw_stream(x)));
  return out;
}

const int* counts_ptr(const std::optional<at::Tensor>& counts, int* n, const char* what) {
  *n = 0;
  if (!counts.has_value() || !counts->defined()) return nullptr;
  TORCH_CHECK(counts->scalar_type() == at::kInt && counts->dim() == 1 && counts->is_contiguous() && on_device(*counts), what,
              ": row counts must be a contiguous int32 vector on the device");
  *n = (int)counts->numel();
  return counts->const_data_ptr<int>();
}

at::Tensor swiglu_rows(const at::Tensor& x, const std::optional<at::Tensor>& row_counts) {
  check_fast(x, "swiglu");
  TORCH_CHECK(x.dim() >= 1 && x.size(-1) % 2 == 0, "swiglu: last dimension must be even");
  at::Tensor xc = x.contiguous();
  const int64_t h = x.size(-1) / 2, rows = h ? x.numel() / (2 * h) : 0;
  std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end());
  shape.back() = h;
  at::Tensor out = at::empty(shape, x.options());
  int n = 0;
  const int* cp = counts_ptr(row_counts, &n, "swiglu");
  DeviceSwitch sw(x.device().index());
  B200_KERNEL_CALL(b200_swiglu_fwd_rows(kdtype(x.scalar_type()), out.mutable_data_ptr(), xc.const_data_ptr(), rows, h, cp, n,
                                        current_raw_stream(x)));
  return out;
}

at::Tensor swiglu_rows_backward(const at::Tensor& dy, const at::Tensor& x, const std::optional<at::Tensor>& row_counts) {
  check_fast(x, "swiglu_backward");
  check_devices("swiglu_backward", x, dy);
  at::Tensor xc = x.contiguous(), dyc = dy.contiguous();
  const int64_t h = x.size(-1) / 2, rows = h ? x.numel() / (2 * h) : 0;
  at::Tensor dx = at::empty_like(xc);
  int n = 0;
  const int* cp = counts_ptr(row_counts, &n, "swiglu_backward");
  DeviceSwitch sw(x.device().index());
  B200_KERNEL_CALL(b200_swiglu_bwd_rows(kdtype(x.scalar_type()), dx.mutable_data_ptr(), dyc.const_data_ptr(),
                                        xc.const_data_ptr(), rows, h, cp, n, current_raw_stream(x)));
  return dx;
}

at::Tensor swiglu(const at::Tensor& x) { return swiglu_rows(x, std::nullopt); }
at::Tensor swiglu_backward(const at::Tensor& dy, const at::Tensor& x) { return swiglu_rows_backward(dy, x, std::nullopt); }

at::Tensor silu_mul(const at::Tensor& gate, const at::Tensor& up) {
  check_fast(gate, "silu_mul");
  check_devices("silu_mul", gate, up);
  TORCH_CHECK(gate.sizes() == up.sizes() && gate.scalar_type() == up.scalar_type(), "silu_mul: shape/dtype mismatch");
  at::Tensor g = gate.contiguous(), u = up.contiguous();
  at::Tensor out = at::empty_like(g);
  DeviceSwitch sw(g.device().index());
  B200_KERNEL_CALL(b200_silu_mul_fwd(kdtype(g.scalar_type()), out.mutable_data_ptr(), g.const_data_ptr(),
                                     u.const_data_ptr(), g.numel(), current_raw_stream(g)));
  return out;
}

std::tuple<at::Tensor, at::Tensor> silu_mul_backward(const at::Tensor& dy, const at::Tensor& gate, const at::Tensor& up) {
  check_fast(gate, "silu_mul_backward");
  check_devices("silu_mul_backward", gate, dy, up);
  at::Tensor g = gate.contiguous(), u = up.contiguous(), d = dy.contiguous();
  at::Tensor dg = at::empty_like(g), du = at::empty_like(u);
  DeviceSwitch sw(g.device().index());
  B200_KERNEL_CALL(b200_silu_mul_bwd(kdtype(g.scalar_type()), dg.mutable_data_ptr(), du.mutable_data_ptr(),
                                     d.const_data_ptr(), g.const_data_ptr(), u.const_data_ptr(), g.numel(),
                                     current_raw_stream(g)));
  return {dg, du};
}

std::tuple<at::Tensor, at::Tensor> cross_entropy_fwd(const at::Tensor& logits, const at::Tensor& target,
                                                     int64_t ignore_index, double label_smoothing) {
  check_fast(logits, "cross_entropy_fwd");
  check_devices("cross_entropy_fwd", logits, target);
  TORCH_CHECK(logits.dim() == 2 && target.dim() == 1 && target.size(0) == logits.size(0) &&
                  target.scalar_type() == at::kLong && on_device(target),
              "cross_entropy_fwd: expected logits [T, V] and int64 target [T] on the device");
  at::Tensor x = logits.contiguous(), t = target.contiguous();
  const int64_t rows = x.size(0), cols = x.size(1);
  at::Tensor loss = at::empty({rows}, x.options().dtype(at::kFloat));
  at::Tensor lse = at::empty({rows}, x.options().dtype(at::kFloat));
  DeviceSwitch sw(x.device().index());
  B200_KERNEL_CALL(b200_cross_entropy_fwd(kdtype(x.scalar_type()), loss.data_ptr<float>(), lse.data_ptr<float>(),
                                          x.const_data_ptr(), t.data_ptr<int64_t>(), rows, cols, ignore_index,
                                          (float)label_smoothing, current_raw_stream(x)));
  return {loss, lse};
}

at::Tensor cross_entropy_bwd_impl(const at::Tensor& logits, const at::Tensor& lse, const at::Tensor& target,
                                  const std::optional<at::Tensor>& grad_loss, double scale, int64_t ignore_index,
                                  double label_smoothing, bool inplace) {
  check_fast(logits, "cross_entropy_bwd");
  check_devices("cross_entropy_bwd", logits, lse, target, grad_loss);
  TORCH_CHECK(!inplace || logits.is_contiguous(), "cross_entropy_bwd_: logits must be contiguous");
  at::Tensor x = logits.contiguous(), t = target.contiguous();
  const int64_t rows = x.size(0), cols = x.size(1);
  at::Tensor dx = inplace ? x : at::empty_like(x);
  const float* gp = nullptr;
  int scalar = 1;
  at::Tensor g;
  if (grad_loss.has_value() && grad_loss->defined()) {
    g = grad_loss->to(at::kFloat).contiguous();
    TORCH_CHECK(g.numel() == 1 || g.numel() == rows, "cross_entropy_bwd: grad must be scalar or per row");
    scalar = g.numel() == 1 ? 1 : 0;
    gp = g.data_ptr<float>();
  }
  DeviceSwitch sw(x.device().index());
  B200_KERNEL_CALL(b200_cross_entropy_bwd(kdtype(x.scalar_type()), dx.mutable_data_ptr(), x.const_data_ptr(),
                                          lse.data_ptr<float>(), t.data_ptr<int64_t>(), gp, scalar, (float)scale, rows,
                                          cols, ignore_index, (float)label_smoothing, current_raw_stream(x)));
  return dx;
}

at::Tensor cross_entropy_bwd(const at::Tensor& logits, const at::Tensor& lse, const at::Tensor& target,
                             const std::optional<at::Tensor>& grad_loss, double scale, int64_t ignore_index,
                             double label_smoothing) {
  return cross_entropy_bwd_impl(logits, lse, target, grad_loss, scale, ignore_index, label_smoothing, false);
}
at::Tensor& cross_entropy_bwd_(at::Tensor& logits, const at::Tensor& lse, const at::Tensor& target,
                               const std::optional<at::Tensor>& grad_loss, double scale, int64_t ignore_index,
                               double label_smoothing) {
  cross_entropy_bwd_impl(logits, lse, target, grad_loss, scale, ignore_index, label_smoothing, true);
  return logits;
}

at::Tensor online_softmax_stats(const at::Tensor& logits, const at::Tensor& target, int64_t vocab_start) {
  check_fast(logits, "online_softmax_stats");
  check_devices("online_softmax_stats", logits, target);
  at::Tensor x = logits.contiguous(), t = target.contiguous();
  at::Tensor stats = at::empty({x.size(0), 3}, x.options().dtype(at::kFloat));
  DeviceSwitch sw(x.device().index());
  B200_KERNEL_CALL(b200_online_softmax_stats(kdtype(x.scalar_type()), stats.data_ptr<float>(), x.const_data_ptr(),
                                             t.data_ptr<int64_t>(), x.size(0), x.size(1), vocab_start,
                                             current_raw_stream(x)));
  return stats;
}

at::Tensor vocab_parallel_ce_finish(at::Tensor& logits, const at::Tensor& all_stats, const at::Tensor& target,
                                    int64_t vocab_start, int64_t ignore_index) {
  check_fast(logits, "vocab_parallel_ce_finish");
  check_devices("vocab_parallel_ce_finish", logits, all_stats, target);
  TORCH_CHECK(logits.is_contiguous() && all_stats.is_contiguous() && all_stats.scalar_type() == at::kFloat &&
                  all_stats.dim() == 3 && all_stats.size(1) == logits.size(0) && all_stats.size(2) == 3,
              "vocab_parallel_ce_finish: all_stats must be contiguous float32 [world, T, 3]");
  at::Tensor t = target.contiguous();
  at::Tensor loss = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  DeviceSwitch sw(logits.device().index());
  B200_KERNEL_CALL(b200_vocab_parallel_ce_finish(kdtype(logits.scalar_type()), loss.data_ptr<float>(),
                                                 logits.mutable_data_ptr(), all_stats.data_ptr<float>(),
                                                 (int)all_stats.size(0), t.data_ptr<int64_t>(), logits.size(0),
                                                 logits.size(1), vocab_start, ignore_index, current_raw_stream(logits)));
  return loss;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> rms_norm_residual(const at::Tensor& x, const at::Tensor& residual,
                                                                 const at::Tensor& weight, double eps) {
  check_fast(x, "rms_norm_residual");
  check_devices("rms_norm_residual", x, residual, weight);
  TORCH_CHECK(x.sizes() == residual.sizes() && x.scalar_type() == residual.scalar_type() &&
                  weight.scalar_type() == x.scalar_type(),
              "rms_norm_residual: shape/dtype mismatch");
  at::Tensor xc = x.contiguous(), rc = residual.contiguous(), w = weight.contiguous();
  const int64_t cols = x.size(-1), rows = cols ? x.numel() / cols : 0;
  at::Tensor y = at::empty_like(xc), res = at::empty_like(xc);
  std::vector<int64_t> sshape(x.sizes().begin(), x.sizes().end());
  sshape.back() = 1;
  at::Tensor rstd = at::empty(sshape, x.options().dtype(at::kFloat));
  DeviceSwitch sw(x.device().index());
  B200_KERNEL_CALL(b200_rmsnorm_fwd(kdtype(x.scalar_type()), y.mutable_data_ptr(), rstd.data_ptr<float>(),
                                    xc.const_data_ptr(), w.const_data_ptr(), rc.const_data_ptr(), res.mutable_data_ptr(),
                                    rows, cols, (float)eps, current_raw_stream(x)));
  return {y, res, rstd};
}

at::Tensor decode_attention(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                            const at::Tensor& pos, std::optional<double> scale) {
  check_fast(q, "decode_attention");
  check_devices("decode_attention", q, k_cache, v_cache, pos);
  TORCH_CHECK(q.dim() == 3 && k_cache.dim() == 4 && v_cache.sizes() == k_cache.sizes() && q.size(0) == k_cache.size(0) &&
              q.size(2) == k_cache.size(3) && q.is_contiguous() && k_cache.is_contiguous() && v_cache.is_contiguous() &&
              k_cache.scalar_type() == q.scalar_type() && v_cache.scalar_type() == q.scalar_type(),
              "decode_attention: q [B, H, D] and contiguous caches [B, Hkv, max_len, D] of one dtype");
  TORCH_CHECK(pos.scalar_type() == at::kLong && pos.numel() == 1, "decode_attention: pos must be one int64 element");
  at::Tensor out = at::empty_like(q);
  DeviceSwitch sw(q.device().index());
  int e = b200_decode_attention(kdtype(q.scalar_type()), out.mutable_data_ptr(), q.const_data_ptr(), k_cache.const_data_ptr(),
                                v_cache.const_data_ptr(), reinterpret_cast<const long long*>(pos.const_data_ptr<int64_t>()),
                                (int)q.size(0), (int)q.size(1), (int)k_cache.size(1), (int)k_cache.size(2), (int)q.size(2),
                                (float)scale.value_or(1.0 / std::sqrt((double)q.size(2))), current_raw_stream(q));
  TORCH_CHECK(e != (int)cudaErrorNotSupported, "decode_attention: head_dim 128, bf16 / fp16 only");
  B200_KERNEL_CALL(e);
  return out;
}

// q / k / v: [B, 1, heads, 128] or [B, heads, 128] (views with a contiguous last dimension are fine)
at::Tensor decode_rope_cache(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& cos,
                             const at::Tensor& sin, const at::Tensor& pos, at::Tensor& k_cache, at::Tensor& v_cache) {
  check_fast(q, "decode_rope_cache");
  check_devices("decode_rope_cache", q, k, v, cos, sin, pos, k_cache, v_cache);
  auto rows = [](const at::Tensor& t, const char* name) {
    TORCH_CHECK((t.dim() == 3 || (t.dim() == 4 && t.size(1) == 1)) && t.size(-1) == 128 && t.stride(-1) == 1, "decode_rope_cache: ",
                name, " must be [B, 1, heads, 128] or [B, heads, 128] with a contiguous last dimension");
  };
  rows(q, "q"); rows(k, "k"); rows(v, "v");
  const int64_t B = q.size(0), H = q.size(-2), Hkv = k.size(-2);
  TORCH_CHECK(k.size(0) == B && v.size(0) == B && v.size(-2) == Hkv && k_cache.dim() == 4 && k_cache.size(0) == B &&
              k_cache.size(1) == Hkv && k_cache.size(3) == 128 && v_cache.sizes() == k_cache.sizes() && k_cache.is_contiguous() &&
              v_cache.is_contiguous(), "decode_rope_cache: caches must be contiguous [B, Hkv, max_len, 128]");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type() && k_cache.scalar_type() == q.scalar_type() &&
              v_cache.scalar_type() == q.scalar_type(), "decode_rope_cache: one dtype");
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat && cos.is_contiguous() && sin.is_contiguous() &&
              cos.size(-1) == 64 && sin.sizes() == cos.sizes(), "decode_rope_cache: cos / sin must be contiguous float32 [positions, 64]");
  TORCH_CHECK(pos.scalar_type() == at::kLong && pos.numel() == 1, "decode_rope_cache: pos must be one int64 element");
  at::Tensor out = at::empty({B, H, 128}, q.options());
  const int64_t strides[6] = {q.stride(0), q.stride(-2), k.stride(0), k.stride(-2), v.stride(0), v.stride(-2)};
  DeviceSwitch sw(q.device().index());
  int e = b200_decode_rope_cache(kdtype(q.scalar_type()), out.mutable_data_ptr(), q.const_data_ptr(), k.const_data_ptr(),
                                 v.const_data_ptr(), strides, cos.const_data_ptr<float>(), sin.const_data_ptr<float>(),
                                 reinterpret_cast<const long long*>(pos.const_data_ptr<int64_t>()), k_cache.mutable_data_ptr(),
                                 v_cache.mutable_data_ptr(), (int)B, (int)H, (int)Hkv, (int)k_cache.size(2), 128,
                                 (int)(cos.numel() / 64), current_raw_stream(q));
  TORCH_CHECK(e != (int)cudaErrorNotSupported, "decode_rope_cache: head_dim 128, bf16 / fp16, even strides only");
  B200_KERNEL_CALL(e);
  return out;
}

// mode 0: a [R, K] x b [G, N, K] -> [R, N];  mode 1: a [R, N] x b [G, N, K] -> [R, K];  mode 2: a [R, M], b [R, N] -> [G, M, N].
// The rows of group g are the next counts[g] packed rows; counts stays on the device.
at::Tensor grouped_mm_impl(const at::Tensor& a, const at::Tensor& b, const at::Tensor& counts, int64_t mode,
                           const std::optional<at::Tensor>& out) {
  check_fast(a, "grouped_mm");
  check_devices("grouped_mm", a, b, counts);
  TORCH_CHECK(counts.scalar_type() == at::kInt && counts.dim() == 1 && counts.is_contiguous(), "grouped_mm: counts must be int32 [groups]");
  TORCH_CHECK(a.dim() == 2 && a.scalar_type() == b.scalar_type() && (a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf),
              "grouped_mm: bf16 / fp16 operands, a two-dimensional");
  at::Tensor ac = a.contiguous(), bc = b.contiguous();
  const int64_t G = counts.size(0), R = ac.size(0);
  b200_grouped_gemm_t g{};
  g.rows = (int)R;
  g.groups = (int)G;
  g.counts = counts.const_data_ptr<int>();
  g.in_dtype = g.out_dtype = kdtype(a.scalar_type());
  std::vector<int64_t> oshape;
  if (mode == 0 || mode == 1) {
    TORCH_CHECK(bc.dim() == 3 && bc.size(0) == G && ac.size(1) == bc.size(mode == 0 ? 2 : 1), "grouped_mm: b must be [groups, N, K]");
    g.ragged_depth = 0;
    g.b_kmajor = mode == 0;
    g.k = (int)ac.size(1);
    g.n = (int)bc.size(mode == 0 ? 1 : 2);
    g.lda = ac.size(1);
    g.ldb = bc.size(2);
    g.stride_b = bc.size(1) * bc.size(2);
    oshape = {R, (int64_t)g.n};
  } else {
    TORCH_CHECK(mode == 2 && bc.dim() == 2 && bc.size(0) == R, "grouped_mm: mode 2 takes a [R, M] and b [R, N]");
    g.ragged_depth = 1;
    g.m = (int)ac.size(1);
    g.n = (int)bc.size(1);
    g.lda = ac.size(1);
    g.ldb = bc.size(1);
    g.stride_d = (int64_t)g.m * g.n;
    oshape = {G, (int64_t)g.m, (int64_t)g.n};
  }
  at::Tensor o;
  if (out.has_value() && out->defined()) {
    o = *out;
    TORCH_CHECK(o.is_contiguous() && o.scalar_type() == a.scalar_type() && o.sizes().equals(oshape), "grouped_mm: out has the wrong shape");
  } else {
    o = at::empty(oshape, a.options());
  }
  g.ldd = g.n;
  DeviceSwitch sw(a.device().index());
  int e = b200_grouped_gemm(&g, o.mutable_data_ptr(), ac.const_data_ptr(), bc.const_data_ptr(), current_raw_stream(a));
  TORCH_CHECK(e != (int)cudaErrorNotSupported, "grouped_mm: unsupported problem (at most 64 groups, widths multiples of 8)");
  B200_KERNEL_CALL(e);
  return o;
}

at::Tensor grouped_mm(const at::Tensor& a, const at::Tensor& b, const at::Tensor& counts, int64_t mode) {
  return grouped_mm_impl(a, b, counts, mode, std::nullopt);
}
at::Tensor& grouped_mm_out(const at::Tensor& a, const at::Tensor& b, const at::Tensor& counts, int64_t mode, at::Tensor& out) {
  grouped_mm_impl(a, b, counts, mode, out);
  return out;
}

void sleep_cycles(int64_t cycles) {
  B200_KERNEL_CALL(b200_sleep(cycles, get_current_stream().stream()));
}

}  // namespace

TORCH_LIBRARY(blackwell, m) {
  m.def("rope(Tensor x, Tensor cos, Tensor sin, Tensor? positions=None, bool interleaved=False, bool conj=False) -> Tensor");
  m.def("swiglu(Tensor x) -> Tensor");
  m.def("swiglu_backward(Tensor dy, Tensor x) -> Tensor");
  m.def("swiglu_rows(Tensor x, Tensor? row_counts) -> Tensor");
  m.def("swiglu_rows_backward(Tensor dy, Tensor x, Tensor? row_counts) -> Tensor");
  m.def("silu_mul(Tensor gate, Tensor up) -> Tensor");
  m.def("silu_mul_backward(Tensor dy, Tensor gate, Tensor up) -> (Tensor, Tensor)");
  m.def("cross_entropy_fwd(Tensor logits, Tensor target, int ignore_index=-100, float label_smoothing=0.0) -> (Tensor, Tensor)");
  m.def("cross_entropy_bwd(Tensor logits, Tensor lse, Tensor target, Tensor? grad_loss, float scale, int ignore_index, float label_smoothing) -> Tensor");
  m.def("cross_entropy_bwd_(Tensor(a!) logits, Tensor lse, Tensor target, Tensor? grad_loss, float scale, int ignore_index, float label_smoothing) -> Tensor(a!)");
  m.def("online_softmax_stats(Tensor logits, Tensor target, int vocab_start) -> Tensor");
  m.def("vocab_parallel_ce_finish(Tensor(a!) logits, Tensor all_stats, Tensor target, int vocab_start, int ignore_index) -> Tensor");
  m.def("rms_norm_residual(Tensor x, Tensor residual, Tensor weight, float eps) -> (Tensor, Tensor, Tensor)");
  m.def("multi_tensor_l2norm(Tensor[] tensors, bool per_tensor=False) -> (Tensor, Tensor)");
  m.def("multi_tensor_scale_(Tensor(a!)[] tensors, Tensor? inv_scale, float scale, Tensor(b!) found_inf) -> ()");
  m.def("multi_tensor_axpby_(Tensor(a!)[] out, Tensor[] x, Tensor[] y, float a, float b) -> ()");
  m.def("multi_tensor_lamb_(Tensor(a!)[] params, Tensor[] grads, Tensor(b!)[] exp_avg, Tensor(c!)[] exp_avg_sq, float lr, float beta1, float beta2, float eps, float weight_decay, int step, bool bias_correction, bool grad_averaging, bool adam_w_mode, float max_grad_norm, bool use_nvlamb, Tensor? global_grad_norm) -> ()");
  m.def("decode_attention(Tensor q, Tensor k_cache, Tensor v_cache, Tensor pos, float? scale=None) -> Tensor");
  m.def("grouped_mm(Tensor a, Tensor b, Tensor counts, int mode) -> Tensor");
  m.def("grouped_mm_out(Tensor a, Tensor b, Tensor counts, int mode, Tensor(a!) out) -> Tensor(a!)");
  m.def("decode_rope_cache(Tensor q, Tensor k, Tensor v, Tensor cos, Tensor sin, Tensor pos, Tensor(a!) k_cache, Tensor(b!) v_cache) -> Tensor");
  m.def("_sleep(int cycles) -> ()");
}

TORCH_LIBRARY_IMPL(blackwell, PrivateUse1, m) {
  m.impl("decode_attention", TORCH_FN(decode_attention));
  m.impl("decode_rope_cache", TORCH_FN(decode_rope_cache));
  m.impl("grouped_mm", TORCH_FN(grouped_mm));
  m.impl("grouped_mm_out", TORCH_FN(grouped_mm_out));
  m.impl("rope", TORCH_FN(rope));
  m.impl("swiglu", TORCH_FN(swiglu));
  m.impl("swiglu_backward", TORCH_FN(swiglu_backward));
  m.impl("swiglu_rows", TORCH_FN(swiglu_rows));
  m.impl("swiglu_rows_backward", TORCH_FN(swiglu_rows_backward));
  m.impl("silu_mul", TORCH_FN(silu_mul));
  m.impl("silu_mul_backward", TORCH_FN(silu_mul_backward));
  m.impl("cross_entropy_fwd", TORCH_FN(cross_entropy_fwd));
  m.impl("cross_entropy_bwd", TORCH_FN(cross_entropy_bwd));
  m.impl("cross_entropy_bwd_", TORCH_FN(cross_entropy_bwd_));
  m.impl("online_softmax_stats", TORCH_FN(online_softmax_stats));
  m.impl("vocab_parallel_ce_finish", TORCH_FN(vocab_parallel_ce_finish));
  m.impl("rms_norm_residual", TORCH_FN(rms_norm_residual));
}

TORCH_LIBRARY_IMPL(blackwell, CompositeExplicitAutograd, m) { m.impl("_sleep", TORCH_FN(sleep_cycles)); }

}  // namespace ops
}  // namespace b200
