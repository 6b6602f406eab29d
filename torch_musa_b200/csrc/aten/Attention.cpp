// scaled_dot_product_attention routing for the blackwell device.
//
// `_fused_sdp_choice` selects the fused path ("overrideable" in ATen's terms) for the cases the
// fused kernels cover -- fp16/bf16, head_dim <= 256, no explicit mask, 4-D [B, H, S, D] -- and the
// math decomposition otherwise, so every mask layout and dtype still works.  The fused forward
// returns (out, logsumexp, ...) and backward consumes them, exactly the contract of ATen's
// `_scaled_dot_product_fused_attention_overrideable(+_backward)`; grouped-query attention
// (fewer KV heads) is handled without expanding K/V.
// The fused implementation currently runs the library flash-attention kernels on the same memory
// through the CUDA-alias bridge.
// Parity: reference torch_musa/csrc/aten/ops/attention/mudnn/SDPBackendSelect.cpp:16-41,
// SDPUtils.h:93-213 (eligibility), SDP.cpp:470-673 (vendor flash forward/backward).
#include "aten/FallbackCall.h"
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <ATen/native/DispatchStub.h>
#include <ATen/native/transformers/attention.h>
#include <torch/library.h>

#include <atomic>
#include <cstdlib>
#include <cmath>

namespace b200 {
namespace ops {

namespace {

constexpr int64_t kMath = 0, kOverrideable = 4;
std::atomic<bool> g_fused_sdp{true};
// which kernel family serves the fused path: 0 = library flash, 1 = library cuDNN, 2 = the hand-written tcgen05
// forward and backward (head_dim 128; other head sizes fall to the library flash kernels).  Fixed between a forward
// and its backward.
std::atomic<int> g_sdp_impl{2};
std::atomic<int64_t> g_native_fwd_calls{0};
std::atomic<int64_t> g_native_bwd_calls{0};

// The hand-written forward: q [B, H, Sq, 128], k / v [B, Hkv, Sk, 128] with a contiguous last dimension.
// The cuDNN-style library kernels: head_dim <= 128; grouped-query heads only when B200_SDP_CUDNN_GQA=1 (default on).
bool cudnn_route_ok(const at::Tensor& q, const at::Tensor& k) {
  static const bool gqa = [] {
    const char* e = std::getenv("B200_SDP_CUDNN_GQA");
    return !(e && e[0] == '0');
  }();
  if (q.size(3) > 128) return false;
  return q.size(1) == k.size(1) || (gqa && q.size(1) % k.size(1) == 0);
}

bool native_fwd_eligible(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double dropout_p) {
  return q.size(3) == 128 && dropout_p == 0.0 && q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1 &&
         q.size(0) == k.size(0) && q.numel() > 0 && k.numel() > 0;
}

bool native_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, bool is_causal, std::optional<double> scale,
                at::Tensor* out, at::Tensor* lse) {
  const int64_t B = q.size(0), H = q.size(1), Sq = q.size(2), D = q.size(3), Hkv = k.size(1), Sk = k.size(2);
  // output in [B, Sq, H, D] memory viewed as [B, H, Sq, D], the layout the library kernels return
  at::Tensor o = at::empty({B, Sq, H, D}, q.options()).transpose(1, 2);
  at::Tensor l = at::empty({B, H, Sq}, q.options().dtype(at::kFloat));
  b200_attn_t a{};
  a.B = (int)B; a.H = (int)H; a.Hkv = (int)Hkv; a.Sq = (int)Sq; a.Sk = (int)Sk; a.head_dim = (int)D;
  a.dtype = kdtype(q.scalar_type());
  a.causal = is_causal ? 1 : 0;
  a.scale = (float)scale.value_or(1.0 / std::sqrt((double)D));
  a.q_sb = q.stride(0); a.q_sh = q.stride(1); a.q_ss = q.stride(2);
  a.k_sb = k.stride(0); a.k_sh = k.stride(1); a.k_ss = k.stride(2);
  a.v_sb = v.stride(0); a.v_sh = v.stride(1); a.v_ss = v.stride(2);
  a.o_sb = o.stride(0); a.o_sh = o.stride(1); a.o_ss = o.stride(2);
  DeviceSwitch sw(q.device().index());
  int e = b200_flash_attn_fwd(&a, o.mutable_data_ptr(), l.data_ptr<float>(), q.const_data_ptr(), k.const_data_ptr(),
                              v.const_data_ptr(), current_raw_stream(q));
  if (e == (int)cudaErrorNotSupported) return false;
  B200_KERNEL_CALL(e);
  g_native_fwd_calls.fetch_add(1, std::memory_order_relaxed);
  *out = o;
  *lse = l;
  return true;
}

bool stride_ok(const at::Tensor& t) {
  return t.stride(3) == 1 && t.stride(0) % 8 == 0 && t.stride(1) % 8 == 0 && t.stride(2) % 8 == 0 && t.stride(2) != 0 &&
         (t.size(0) == 1 || t.stride(0) != 0) && (t.size(1) == 1 || t.stride(1) != 0) &&
         (reinterpret_cast<uintptr_t>(t.const_data_ptr()) & 15) == 0;
}

// The hand-written backward: dq / dk / dv for the tensors of native_fwd.  Returns false when the shape is not covered.
bool native_bwd(const at::Tensor& grad_out_, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                const at::Tensor& out_, const at::Tensor& lse, bool is_causal, std::optional<double> scale,
                at::Tensor* dq, at::Tensor* dk, at::Tensor* dv) {
  const int64_t B = q.size(0), H = q.size(1), Sq = q.size(2), D = q.size(3), Hkv = k.size(1), Sk = k.size(2);
  if (D != 128 || !stride_ok(q) || !stride_ok(k) || !stride_ok(v)) return false;
  if (!lse.defined() || lse.scalar_type() != at::kFloat || lse.numel() != B * H * Sq) return false;
  at::Tensor go = stride_ok(grad_out_) ? grad_out_ : grad_out_.contiguous();
  at::Tensor o = stride_ok(out_) ? out_ : out_.contiguous();
  at::Tensor l = lse.is_contiguous() ? lse : lse.contiguous();
  at::Tensor dq32 = at::empty({B, H, Sq, D}, q.options().dtype(at::kFloat));
  at::Tensor delta = at::empty({B, H, Sq}, q.options().dtype(at::kFloat));
  at::Tensor gk = at::empty({B, Sk, Hkv, D}, k.options()).transpose(1, 2);
  at::Tensor gv = at::empty({B, Sk, Hkv, D}, v.options()).transpose(1, 2);
  b200_attn_t a{};
  a.B = (int)B; a.H = (int)H; a.Hkv = (int)Hkv; a.Sq = (int)Sq; a.Sk = (int)Sk; a.head_dim = (int)D;
  a.dtype = kdtype(q.scalar_type());
  a.causal = is_causal ? 1 : 0;
  a.scale = (float)scale.value_or(1.0 / std::sqrt((double)D));
  a.q_sb = q.stride(0); a.q_sh = q.stride(1); a.q_ss = q.stride(2);
  a.k_sb = k.stride(0); a.k_sh = k.stride(1); a.k_ss = k.stride(2);
  a.v_sb = v.stride(0); a.v_sh = v.stride(1); a.v_ss = v.stride(2);
  a.o_sb = o.stride(0); a.o_sh = o.stride(1); a.o_ss = o.stride(2);
  const int64_t extra[9] = {go.stride(0), go.stride(1), go.stride(2), gk.stride(0), gk.stride(1), gk.stride(2),
                            gv.stride(0), gv.stride(1), gv.stride(2)};
  DeviceSwitch sw(q.device().index());
  int e = b200_flash_attn_bwd(&a, dq32.data_ptr<float>(), gk.mutable_data_ptr(), gv.mutable_data_ptr(),
                              delta.data_ptr<float>(), q.const_data_ptr(), k.const_data_ptr(), v.const_data_ptr(),
                              o.const_data_ptr(), go.const_data_ptr(), l.const_data_ptr<float>(), extra,
                              current_raw_stream(q));
  if (e == (int)cudaErrorNotSupported) return false;
  B200_KERNEL_CALL(e);
  g_native_bwd_calls.fetch_add(1, std::memory_order_relaxed);
  // the fp32 accumulator becomes the gradient in [B, Sq, H, D] memory, the layout of the projections' output
  at::Tensor gq = at::empty({B, Sq, H, D}, q.options()).transpose(1, 2);
  gq.copy_(dq32);
  *dq = gq;
  *dk = gk;
  *dv = gv;
  return true;
}

bool fused_eligible(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                    const std::optional<at::Tensor>& mask, double dropout_p) {
  if (!g_fused_sdp.load(std::memory_order_relaxed)) return false;
  if (mask.has_value() && mask->defined()) return false;
  if (q.dim() != 4 || k.dim() != 4 || v.dim() != 4) return false;
  auto dt = q.scalar_type();
  if ((dt != at::kBFloat16 && dt != at::kHalf) || k.scalar_type() != dt || v.scalar_type() != dt) return false;
  const int64_t d = q.size(3);
  if (d > 256 || d % 8 != 0 || k.size(3) != d || v.size(3) != d) return false;
  if (q.size(1) % k.size(1) != 0 || k.size(1) != v.size(1)) return false;
  if (q.size(0) != k.size(0) || k.size(2) != v.size(2)) return false;
  if (q.numel() == 0 || k.numel() == 0) return false;
  (void)dropout_p;
  return true;
}

int64_t fused_sdp_choice(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                         const std::optional<at::Tensor>& mask, double dropout_p, bool is_causal,
                         std::optional<double> scale, bool enable_gqa) {
  (void)is_causal; (void)scale; (void)enable_gqa;
  return fused_eligible(q, k, v, mask, dropout_p) ? kOverrideable : kMath;
}

}  // namespace

int64_t fused_sdp_choice_stub_impl(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                   const std::optional<at::Tensor>& mask, double dropout_p, bool is_causal,
                                   std::optional<double> scale, bool enable_gqa) {
  return fused_sdp_choice(q, k, v, mask, dropout_p, is_causal, scale, enable_gqa);
}

namespace {

using FwdRet = std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, c10::SymInt, c10::SymInt, at::Tensor,
                          at::Tensor, at::Tensor>;

FwdRet sdpa_fused_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                      const std::optional<at::Tensor>& attn_bias, double dropout_p, bool is_causal,
                      bool return_debug_mask, std::optional<double> scale) {
  TORCH_CHECK(!(attn_bias.has_value() && attn_bias->defined()),
              "blackwell fused attention: explicit masks take the math path (this is a dispatch bug)");
  if (g_sdp_impl.load() == 2 && native_fwd_eligible(q, k, v, dropout_p)) {
    at::Tensor o, l;
    if (native_fwd(q, k, v, is_causal, scale, &o, &l)) {
      at::Tensor none = at::empty({0}, q.options().dtype(at::kLong));
      at::Tensor seed = at::zeros({}, q.options().dtype(at::kLong));
      return FwdRet(o, l, at::Tensor(), at::Tensor(), c10::SymInt(q.size(2)), c10::SymInt(k.size(2)), seed, seed.clone(),
                    at::empty({0}, q.options()));
    }
  }
  if (g_sdp_impl.load() == 1 && cudnn_route_ok(q, k)) {
    std::optional<at::Tensor> no_bias;
    auto st = run_fallback(B200_OP_HANDLE("aten::_scaled_dot_product_cudnn_attention", ""), q, k, v, no_bias,
                           /*compute_log_sumexp=*/true, dropout_p, is_causal, return_debug_mask, scale);
    return FwdRet(st[0].toTensor(), st[1].toTensor(), st[2].toTensor(), st[3].toTensor(), st[4].toSymInt(),
                  st[5].toSymInt(), st[6].toTensor(), st[7].toTensor(), st[8].toTensor());
  }
  auto st = run_fallback(B200_OP_HANDLE("aten::_scaled_dot_product_flash_attention", ""), q, k, v, dropout_p,
                         is_causal, return_debug_mask, scale);
  // (output, logsumexp, cum_seq_q, cum_seq_k, max_q, max_k, rng_state, unused, debug_attn_mask)
  return FwdRet(st[0].toTensor(), st[1].toTensor(), st[2].toTensor(), st[3].toTensor(), st[4].toSymInt(),
                st[5].toSymInt(), st[6].toTensor(), st[7].toTensor(), st[8].toTensor());
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> sdpa_fused_bwd(
    const at::Tensor& grad_out, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
    const at::Tensor& attn_bias, std::array<bool, 4> grad_input_mask, const at::Tensor& out,
    const at::Tensor& logsumexp, const at::Tensor& cum_seq_q, const at::Tensor& cum_seq_k, c10::SymInt max_q,
    c10::SymInt max_k, double dropout_p, bool is_causal, const at::Tensor& philox_seed,
    const at::Tensor& philox_offset, std::optional<double> scale) {
  (void)grad_input_mask;
  // a forward that ran on the hand-written kernel left no rng state and an empty cum_seq: its backward is ours too
  if (g_sdp_impl.load() == 2 && dropout_p == 0.0 && native_fwd_eligible(q, k, v, dropout_p)) {
    at::Tensor dq, dk, dv;
    if (native_bwd(grad_out, q, k, v, out, logsumexp, is_causal, scale, &dq, &dk, &dv))
      return {dq, dk, dv, at::Tensor()};
  }
  if (g_sdp_impl.load() == 1 && cudnn_route_ok(q, k)) {
    at::Tensor no_bias;
    auto st = run_fallback(B200_OP_HANDLE("aten::_scaled_dot_product_cudnn_attention_backward", ""), grad_out, q, k, v,
                           out, logsumexp, philox_seed, philox_offset, no_bias, cum_seq_q, cum_seq_k, max_q, max_k,
                           dropout_p, is_causal, scale);
    return {st[0].toTensor(), st[1].toTensor(), st[2].toTensor(), at::Tensor()};
  }
  (void)attn_bias;
  auto st = run_fallback(B200_OP_HANDLE("aten::_scaled_dot_product_flash_attention_backward", ""), grad_out, q, k, v,
                         out, logsumexp, cum_seq_q, cum_seq_k, max_q, max_k, dropout_p, is_causal, philox_seed,
                         philox_offset, scale);
  return {st[0].toTensor(), st[1].toTensor(), st[2].toTensor(), at::Tensor()};
}


// ---------------------------------------------------------------------------------------------------------------
// Packed variable-length attention: q [total_q, H, 128], k / v [total_k, Hkv, 128], cu_seqlens int32 [B + 1] on the
// device.  ONE launch of the tcgen05 forward (and of the backward) covers every sequence: a CTA reads its sequence's
// bounds from cu_seqlens and offsets its tile coordinates; nothing is read on the host.  lse is [H, total_q].
// Parity: reference torch_musa/csrc/aten/ops/attention/mudnn/SDP.cpp:678-845 (varlen entry of the vendor flash kernel).
void varlen_desc(b200_attn_t& a, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& cu_q,
                 const at::Tensor& cu_k, int64_t max_q, int64_t max_k, bool causal, std::optional<double> scale) {
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && q.size(2) == 128 && k.size(2) == 128 && v.sizes() == k.sizes(),
              "varlen_attention: q [total_q, H, 128], k / v [total_k, Hkv, 128]");
  TORCH_CHECK((q.scalar_type() == at::kBFloat16 || q.scalar_type() == at::kHalf) && k.scalar_type() == q.scalar_type() &&
              v.scalar_type() == q.scalar_type(), "varlen_attention: bf16 / fp16 only");
  TORCH_CHECK(cu_q.scalar_type() == at::kInt && cu_k.scalar_type() == at::kInt && cu_q.dim() == 1 && cu_q.sizes() == cu_k.sizes() &&
              cu_q.numel() >= 2 && cu_q.is_contiguous() && cu_k.is_contiguous(), "varlen_attention: cu_seqlens must be int32 [B + 1]");
  TORCH_CHECK(q.size(1) % k.size(1) == 0 && max_q > 0 && max_k > 0, "varlen_attention: bad head counts or lengths");
  a.B = (int)cu_q.numel() - 1;
  a.H = (int)q.size(1); a.Hkv = (int)k.size(1);
  a.Sq = (int)max_q; a.Sk = (int)max_k; a.head_dim = 128;
  a.dtype = kdtype(q.scalar_type());
  a.causal = causal ? 1 : 0;
  a.scale = (float)scale.value_or(1.0 / std::sqrt(128.0));
  a.q_ss = q.stride(0); a.q_sh = q.stride(1);
  a.k_ss = k.stride(0); a.k_sh = k.stride(1);
  a.v_ss = v.stride(0); a.v_sh = v.stride(1);
  a.cu_seqlens_q = cu_q.const_data_ptr<int>();
  a.cu_seqlens_k = cu_k.const_data_ptr<int>();
  a.total_q = (int)q.size(0);
  a.total_k = (int)k.size(0);
}

std::tuple<at::Tensor, at::Tensor> varlen_attention(const at::Tensor& q_, const at::Tensor& k_, const at::Tensor& v_,
                                                    const at::Tensor& cu_q, const at::Tensor& cu_k, int64_t max_q,
                                                    int64_t max_k, bool causal, std::optional<double> scale) {
  check_devices("varlen_attention", q_, k_, v_, cu_q, cu_k);
  at::Tensor q = q_.stride(2) == 1 ? q_ : q_.contiguous(), k = k_.stride(2) == 1 ? k_ : k_.contiguous(),
             v = v_.stride(2) == 1 ? v_ : v_.contiguous();
  b200_attn_t a{};
  varlen_desc(a, q, k, v, cu_q, cu_k, max_q, max_k, causal, scale);
  at::Tensor o = at::empty({q.size(0), q.size(1), 128}, q.options());
  at::Tensor lse = at::empty({q.size(1), q.size(0)}, q.options().dtype(at::kFloat));
  a.o_ss = o.stride(0); a.o_sh = o.stride(1);
  DeviceSwitch sw(q.device().index());
  int e = b200_flash_attn_fwd(&a, o.mutable_data_ptr(), lse.data_ptr<float>(), q.const_data_ptr(), k.const_data_ptr(),
                              v.const_data_ptr(), current_raw_stream(q));
  TORCH_CHECK(e != (int)cudaErrorNotSupported, "varlen_attention: unsupported strides or alignment");
  B200_KERNEL_CALL(e);
  g_native_fwd_calls.fetch_add(1, std::memory_order_relaxed);
  return {o, lse};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> varlen_attention_backward(
    const at::Tensor& grad_out, const at::Tensor& q_, const at::Tensor& k_, const at::Tensor& v_, const at::Tensor& out,
    const at::Tensor& lse, const at::Tensor& cu_q, const at::Tensor& cu_k, int64_t max_q, int64_t max_k, bool causal,
    std::optional<double> scale) {
  check_devices("varlen_attention_backward", grad_out, q_, k_, v_, out, lse, cu_q, cu_k);
  at::Tensor q = q_.contiguous(), k = k_.contiguous(), v = v_.contiguous(), go = grad_out.contiguous(), o = out.contiguous(),
             l = lse.contiguous();
  b200_attn_t a{};
  varlen_desc(a, q, k, v, cu_q, cu_k, max_q, max_k, causal, scale);
  TORCH_CHECK(l.scalar_type() == at::kFloat && l.numel() == q.size(0) * q.size(1), "varlen_attention_backward: lse must be [H, total_q]");
  a.o_ss = o.stride(0); a.o_sh = o.stride(1);
  at::Tensor dq32 = at::empty({q.size(1), q.size(0), 128}, q.options().dtype(at::kFloat));
  at::Tensor delta = at::empty({q.size(1), q.size(0)}, q.options().dtype(at::kFloat));
  at::Tensor gk = at::empty_like(k), gv = at::empty_like(v);
  const int64_t extra[9] = {0, go.stride(1), go.stride(0), 0, gk.stride(1), gk.stride(0), 0, gv.stride(1), gv.stride(0)};
  DeviceSwitch sw(q.device().index());
  int e = b200_flash_attn_bwd(&a, dq32.data_ptr<float>(), gk.mutable_data_ptr(), gv.mutable_data_ptr(),
                              delta.data_ptr<float>(), q.const_data_ptr(), k.const_data_ptr(), v.const_data_ptr(),
                              o.const_data_ptr(), go.const_data_ptr(), l.const_data_ptr<float>(), extra,
                              current_raw_stream(q));
  TORCH_CHECK(e != (int)cudaErrorNotSupported, "varlen_attention_backward: unsupported strides or alignment");
  B200_KERNEL_CALL(e);
  g_native_bwd_calls.fetch_add(1, std::memory_order_relaxed);
  at::Tensor gq = at::empty_like(q);
  gq.copy_(dq32.transpose(0, 1));       // fp32 [H, total, 128] accumulator -> [total, H, 128] in the input type
  return {gq, gk, gv};
}

}  // namespace

int64_t native_sdp_forward_calls() { return g_native_fwd_calls.load(); }
int64_t native_sdp_backward_calls() { return g_native_bwd_calls.load(); }
void set_fused_sdp(bool on) { g_fused_sdp = on; }
void set_sdp_impl(int impl) { g_sdp_impl = impl; }
int sdp_impl() { return g_sdp_impl; }
bool fused_sdp_enabled() { return g_fused_sdp; }

}  // namespace ops
}  // namespace b200

// F.scaled_dot_product_attention asks this per-device-type stub, not the dispatcher
namespace at::native {
REGISTER_PRIVATEUSE1_DISPATCH(_fused_sdp_choice_stub, &b200::ops::fused_sdp_choice_stub_impl)
}  // namespace at::native

namespace b200 {
namespace ops {

TORCH_LIBRARY_FRAGMENT(blackwell, m) {
  m.def("varlen_attention(Tensor q, Tensor k, Tensor v, Tensor cu_seqlens_q, Tensor cu_seqlens_k, int max_seqlen_q, int max_seqlen_k, bool causal=False, float? scale=None) -> (Tensor, Tensor)");
  m.def("varlen_attention_backward(Tensor grad_out, Tensor q, Tensor k, Tensor v, Tensor out, Tensor lse, Tensor cu_seqlens_q, Tensor cu_seqlens_k, int max_seqlen_q, int max_seqlen_k, bool causal=False, float? scale=None) -> (Tensor, Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(blackwell, PrivateUse1, m) {
  m.impl("varlen_attention", TORCH_FN(varlen_attention));
  m.impl("varlen_attention_backward", TORCH_FN(varlen_attention_backward));
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("_fused_sdp_choice", TORCH_FN(fused_sdp_choice));
  m.impl("_scaled_dot_product_fused_attention_overrideable", TORCH_FN(sdpa_fused_fwd));
  m.impl("_scaled_dot_product_fused_attention_overrideable_backward", TORCH_FN(sdpa_fused_bwd));
}

}  // namespace ops
}  // namespace b200
