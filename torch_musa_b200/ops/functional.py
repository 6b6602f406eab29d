"""Functional forms of the fused operators (autograd included)."""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F


def _on_device(t: torch.Tensor) -> bool:
    return t.device.type == "blackwell"


# ------------------------------------------------------------------------- RMSNorm
def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * weight`` over the last dimension (fp32 statistics).

    On the device this is ``aten::_fused_rms_norm`` (one kernel forward, one backward)."""
    return F.rms_norm(x, (x.shape[-1],), weight, eps)


class _RMSNormResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, eps):
        y, res, rstd = torch.ops.blackwell.rms_norm_residual(x, residual, weight, eps)
        ctx.save_for_backward(res, weight, rstd)
        return y, res

    @staticmethod
    def backward(ctx, dy, dres):
        res, weight, rstd = ctx.saved_tensors
        dx, dw = torch.ops.aten._fused_rms_norm_backward(dy.contiguous(), res, [res.shape[-1]], rstd, weight,
                                                         [True, True])
        if dres is not None:
            dx = dx + dres
        return dx, dx, dw, None


def rms_norm_residual(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """Fused ``h = x + residual; y = rms_norm(h)``; returns ``(y, h)`` (one pass over memory)."""
    if _on_device(x):
        return _RMSNormResidual.apply(x, residual, weight, eps)
    h = x + residual
    return rms_norm(h, weight, eps), h


# ------------------------------------------------------------------------- BatchNorm (+residual) (+ReLU)
class _BatchNormAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, running_var, residual, training, momentum, eps, relu):
        y, mean, invstd = torch.ops.blackwell.batch_norm_act(x, weight, bias, running_mean, running_var, residual,
                                                             training, momentum, eps, relu)
        ctx.relu, ctx.has_res, ctx.training = relu, residual is not None, training
        ctx.save_for_backward(x, y if relu else None, weight, mean, invstd)
        ctx.mark_non_differentiable(mean, invstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        if not ctx.training:
            raise RuntimeError("batch_norm_act: backward through evaluation-mode statistics is not supported; "
                               "use torch.nn.functional.batch_norm")
        x, y, weight, mean, invstd = ctx.saved_tensors
        dx, dw, db, dres = torch.ops.blackwell.batch_norm_act_backward(dy, x, y, weight, mean, invstd, ctx.relu,
                                                                       ctx.has_res)
        return (dx, dw if weight is not None else None, db if weight is not None else None, None, None,
                dres if ctx.has_res else None, None, None, None, None)


def _bn_act_fast(x, weight, bias, running_mean, running_var) -> bool:
    if not _on_device(x) or x.dtype not in (torch.bfloat16, torch.float16):
        return False
    if x.dim() == 4:
        if not x.is_contiguous(memory_format=torch.channels_last):
            return False
    elif x.dim() != 2 or not x.is_contiguous():
        return False
    if x.shape[1] % 8 != 0:
        return False
    return all(t is None or t.dtype == torch.float32 for t in (weight, bias, running_mean, running_var))


def batch_norm_act(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                   running_mean: Optional[torch.Tensor], running_var: Optional[torch.Tensor],
                   residual: Optional[torch.Tensor] = None, training: bool = True, momentum: float = 0.1,
                   eps: float = 1e-5, relu: bool = True) -> torch.Tensor:
    """``act(batch_norm(x) + residual)`` with ``act`` = ReLU or identity.

    On the device, for bf16/fp16 channels-last activations with fp32 parameters, the whole expression is one
    statistics pass plus one fused normalise/affine/add/ReLU pass (and the mirrored two passes backward);
    anywhere else it is the plain composition."""
    if _bn_act_fast(x, weight, bias, running_mean, running_var) and (residual is None or (
            residual.dtype == x.dtype and residual.shape == x.shape and residual.stride() == x.stride())):
        if training or (running_mean is not None and running_var is not None and not torch.is_grad_enabled()):
            return _BatchNormAct.apply(x, weight, bias, running_mean, running_var, residual, training, momentum, eps,
                                       relu)
    y = F.batch_norm(x, running_mean, running_var, weight, bias, training, momentum, eps)
    if residual is not None:
        y = y + residual
    return F.relu(y) if relu else y


# ------------------------------------------------------------------------- RoPE
def precompute_rope_cache(seq_len: int, head_dim: int, theta: float = 10000.0, device=None):
    """fp32 ``cos``/``sin`` tables of shape [seq_len, head_dim // 2]."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device="cpu") / head_dim))
    t = torch.arange(seq_len, dtype=torch.float32, device="cpu")
    freqs = torch.outer(t, inv)
    cos, sin = freqs.cos().contiguous(), freqs.sin().contiguous()
    if device is not None:
        cos, sin = cos.to(device), sin.to(device)
    return cos, sin


def _rope_reference(x, cos, sin, positions, interleaved, conj):
    # x [B, S, H, D]; cos/sin [P, D/2]
    B, S, H, D = x.shape
    if positions is not None:
        c = cos[positions.reshape(B, S)].unsqueeze(2)
        s = sin[positions.reshape(B, S)].unsqueeze(2)
    else:
        c = cos[:S].view(1, S, 1, D // 2)
        s = sin[:S].view(1, S, 1, D // 2)
    if conj:
        s = -s
    xf = x.float()
    if interleaved:
        x0, x1 = xf[..., 0::2], xf[..., 1::2]
        o0, o1 = x0 * c - x1 * s, x1 * c + x0 * s
        out = torch.stack((o0, o1), dim=-1).flatten(-2)
    else:
        x0, x1 = xf[..., : D // 2], xf[..., D // 2:]
        out = torch.cat((x0 * c - x1 * s, x1 * c + x0 * s), dim=-1)
    return out.to(x.dtype)


def _rope_rotate_half(x, cos, sin, positions):
    """The usual library formulation (four elementwise kernels, in the input dtype): ``x * cos + rotate_half(x) * sin``
    with full-width tables.  What a stock CUDA run of this model uses."""
    B, S, H, D = x.shape
    if positions is not None:
        c, s = cos[positions.reshape(B, S)].unsqueeze(2), sin[positions.reshape(B, S)].unsqueeze(2)
    else:
        c, s = cos[:S].view(1, S, 1, D // 2), sin[:S].view(1, S, 1, D // 2)
    c = torch.cat((c, c), dim=-1).to(x.dtype)
    s = torch.cat((s, s), dim=-1).to(x.dtype)
    x0, x1 = x[..., : D // 2], x[..., D // 2:]
    return x * c + torch.cat((-x1, x0), dim=-1) * s


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, positions, interleaved):
        ctx.save_for_backward(cos, sin, positions if positions is not None else torch.empty(0))
        ctx.has_pos = positions is not None
        ctx.interleaved = interleaved
        return torch.ops.blackwell.rope(x, cos, sin, positions, interleaved, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin, pos = ctx.saved_tensors
        dx = torch.ops.blackwell.rope(dy, cos, sin, pos if ctx.has_pos else None, ctx.interleaved, True)
        return dx, None, None, None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: Optional[torch.Tensor] = None,
         interleaved: bool = False) -> torch.Tensor:
    """Rotary position embedding of ``x`` [batch, seq, heads, head_dim].

    ``interleaved=False`` rotates the two halves of the head dimension (Llama / NeoX layout),
    ``True`` rotates adjacent pairs (GPT-J layout). Backward is the conjugate rotation."""
    if _on_device(x):
        return _Rope.apply(x, cos, sin, positions, interleaved)
    if x.is_cuda and not interleaved and x.dtype in (torch.bfloat16, torch.float16):
        return _rope_rotate_half(x, cos, sin, positions)
    return _rope_reference(x, cos, sin, positions, interleaved, False)


# ------------------------------------------------------------------------- SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return torch.ops.blackwell.swiglu(x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return torch.ops.blackwell.swiglu_backward(dy, x)


class _SwiGLURows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, counts):
        ctx.save_for_backward(x, counts)
        return torch.ops.blackwell.swiglu_rows(x, counts)

    @staticmethod
    def backward(ctx, dy):
        x, counts = ctx.saved_tensors
        return torch.ops.blackwell.swiglu_rows_backward(dy, x, counts), None


def swiglu(x: torch.Tensor, row_counts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(x[..., :h]) * x[..., h:]`` for a packed gate|up tensor.  ``row_counts`` (int32, on the device): the
    lengths of the packed row groups of a 2-D ``x``; only the first ``row_counts.sum()`` rows are computed (and get a
    gradient), the others are left as they are -- the sum is taken on the device."""
    if _on_device(x):
        if row_counts is not None:
            return _SwiGLURows.apply(x, row_counts.to(torch.int32))
        return _SwiGLU.apply(x)
    g, u = x.chunk(2, dim=-1)
    return F.silu(g) * u


gated_silu = swiglu


# ------------------------------------------------------------------------- grouped linear (expert GEMMs)
def _grouped_rows(counts: torch.Tensor, rows: int):
    out, start = [], 0
    for n in counts.tolist():
        n = max(0, min(int(n), rows - start))
        out.append((start, n))
        start += n
    return out


class _GroupedLinear(torch.autograd.Function):
    """``y[r] = x[r] @ w[g(r)].T`` over packed row groups whose lengths (``counts``, int32) stay on the device: one
    grouped tensor-core GEMM each for the product, the input gradient and the per-group weight gradients."""

    @staticmethod
    def forward(ctx, x, w, counts, out, grad_input_out):
        ctx.save_for_backward(x, w, counts)
        ctx.grad_input_out = grad_input_out
        if out is not None:
            ctx.mark_dirty(out)
            return torch.ops.blackwell.grouped_mm_out(x, w, counts, 0, out)
        return torch.ops.blackwell.grouped_mm(x, w, counts, 0)

    @staticmethod
    def backward(ctx, dy):
        x, w, counts = ctx.saved_tensors
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            if ctx.grad_input_out is not None:
                dx = torch.ops.blackwell.grouped_mm_out(dy, w, counts, 1, ctx.grad_input_out)
            else:
                dx = torch.ops.blackwell.grouped_mm(dy, w, counts, 1)
        dw = torch.ops.blackwell.grouped_mm(dy, x, counts, 2) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, out: Optional[torch.Tensor] = None,
                   grad_input_out: Optional[torch.Tensor] = None):
    """Rows of ``x`` [R, K] are packed group after group (``counts[g]`` rows for group g); ``w`` is [G, N, K].
    Returns [R, N]; rows past ``counts.sum()`` are left as they are (uninitialised without ``out``).  On the
    blackwell device nothing reads ``counts`` on the host.  ``out`` / ``grad_input_out`` name buffers the product /
    the input gradient are written into (an exchange arena, so that no copy follows)."""
    if _on_device(x) and x.dtype in (torch.bfloat16, torch.float16):
        return _GroupedLinear.apply(x, w, counts.to(torch.int32), out, grad_input_out)
    parts = [F.linear(x[s:s + n], w[g]) for g, (s, n) in enumerate(_grouped_rows(counts, x.shape[0]))]
    used = sum(p.shape[0] for p in parts)
    y = torch.cat(parts + [x.new_zeros((x.shape[0] - used, w.shape[1]))], 0)
    if out is not None:
        out.copy_(y)
        return out
    return y


class _SiluMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        ctx.save_for_backward(gate, up)
        return torch.ops.blackwell.silu_mul(gate, up)

    @staticmethod
    def backward(ctx, dy):
        gate, up = ctx.saved_tensors
        return torch.ops.blackwell.silu_mul_backward(dy, gate, up)


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` in one kernel (two-tensor SwiGLU)."""
    if _on_device(gate):
        return _SiluMul.apply(gate, up)
    return F.silu(gate) * up


# ------------------------------------------------------------------------- cross entropy
class _FusedCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, ignore_index, label_smoothing, reduction, inplace_backward):
        loss_rows, lse = torch.ops.blackwell.cross_entropy_fwd(logits, target, ignore_index, label_smoothing)
        n_valid = None
        if reduction == "mean":
            n_valid = (target != ignore_index).sum().clamp_min(1).to(torch.float32)
            out = loss_rows.sum() / n_valid
        elif reduction == "sum":
            out = loss_rows.sum()
        else:
            out = loss_rows
        ctx.save_for_backward(logits, lse, target, n_valid if n_valid is not None else torch.empty(0))
        ctx.cfg = (ignore_index, label_smoothing, reduction, inplace_backward)
        return out

    @staticmethod
    def backward(ctx, dloss):
        logits, lse, target, n_valid = ctx.saved_tensors
        ignore_index, ls, reduction, inplace = ctx.cfg
        g = dloss.to(torch.float32)
        if reduction == "mean":
            g = g / n_valid
        g = g.reshape(-1) if reduction == "none" else g.reshape(1)
        if inplace and logits.is_contiguous():
            dl = torch.ops.blackwell.cross_entropy_bwd_(logits, lse, target, g, 1.0, ignore_index, ls)
        else:
            dl = torch.ops.blackwell.cross_entropy_bwd(logits, lse, target, g, 1.0, ignore_index, ls)
        return dl, None, None, None, None, None


def fused_cross_entropy(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100,
                        label_smoothing: float = 0.0, reduction: str = "mean",
                        inplace_backward: bool = False) -> torch.Tensor:
    """Cross entropy over [T, V] logits that never materialises the probabilities.

    Forward stores only the per-row log-sum-exp; backward regenerates softmax from it.
    ``inplace_backward=True`` writes the gradient over the logits (saves T*V elements) --
    only valid when nothing else needs the logits after the loss."""
    if logits.dim() != 2:
        logits = logits.reshape(-1, logits.shape[-1])
        target = target.reshape(-1)
    if _on_device(logits):
        return _FusedCE.apply(logits, target, ignore_index, label_smoothing, reduction, inplace_backward)
    return F.cross_entropy(logits.float(), target, ignore_index=ignore_index, label_smoothing=label_smoothing,
                           reduction=reduction)


# ------------------------------------------------------------------------- misc
def multi_tensor_l2norm(tensors: List[torch.Tensor], per_tensor: bool = False):
    """Global (and optionally per-tensor) L2 norm of a list of tensors in a few launches."""
    if len(tensors) > 0 and _on_device(tensors[0]):
        total, per = torch.ops.blackwell.multi_tensor_l2norm(list(tensors), per_tensor)
        return (total, per) if per_tensor else (total, None)
    per = torch.stack([t.float().norm(2) for t in tensors]) if tensors else torch.zeros(0)
    return per.norm(2).reshape(1), (per if per_tensor else None)


def scaled_dot_product_attention(q, k, v, attn_mask=None, dropout_p: float = 0.0, is_causal: bool = False,
                                 scale: Optional[float] = None, enable_gqa: bool = False):
    """``F.scaled_dot_product_attention``; on the device it is routed to the backend's attention kernels."""
    return F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal,
                                          scale=scale, enable_gqa=enable_gqa)


# ------------------------------------------------------------------------- packed variable-length attention
class _VarlenAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, causal, scale):
        out, lse = torch.ops.blackwell.varlen_attention(q, k, v, cu_q, cu_k, max_q, max_k, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
        ctx.args = (max_q, max_k, causal, scale)
        return out

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        dq, dk, dv = torch.ops.blackwell.varlen_attention_backward(d_out, q, k, v, out, lse, cu_q, cu_k, *ctx.args)
        return dq, dk, dv, None, None, None, None, None, None


def flash_attn_varlen_func(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                           cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int,
                           softmax_scale: Optional[float] = None, causal: bool = False) -> torch.Tensor:
    """Attention over sequences of different lengths packed without padding: ``q`` [total_q, H, D], ``k`` / ``v``
    [total_k, Hkv, D]; sequence i owns rows ``cu_seqlens[i]:cu_seqlens[i + 1]`` (int32 prefix sums, on the device of
    the tensors).  Returns [total_q, H, D].  On the blackwell device with D = 128 and bf16 / fp16 the whole batch is
    one launch of the tensor-core forward (one more for the backward) and the lengths are never read on the host;
    otherwise the sequences are processed one by one with ``scaled_dot_product_attention``.  A causal mask compares
    positions inside a sequence (key index <= query index)."""
    if (_on_device(q) and q.shape[-1] == 128 and q.dtype in (torch.bfloat16, torch.float16)
            and k.dtype == q.dtype and v.dtype == q.dtype):
        return _VarlenAttention.apply(q, k, v, cu_seqlens_q.to(torch.int32), cu_seqlens_k.to(torch.int32),
                                      int(max_seqlen_q), int(max_seqlen_k), bool(causal), softmax_scale)
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    rep = q.shape[1] // k.shape[1]
    outs = []
    for i in range(len(cq) - 1):
        qi = q[cq[i]:cq[i + 1]].transpose(0, 1).unsqueeze(0)
        ki = k[ck[i]:ck[i + 1]].transpose(0, 1).unsqueeze(0)
        vi = v[ck[i]:ck[i + 1]].transpose(0, 1).unsqueeze(0)
        if rep > 1:
            ki, vi = ki.repeat_interleave(rep, 1), vi.repeat_interleave(rep, 1)
        mask = None
        if causal:
            sq, sk = qi.shape[2], ki.shape[2]
            mask = torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril()
        o = F.scaled_dot_product_attention(qi, ki, vi, attn_mask=mask, scale=softmax_scale)
        outs.append(o.squeeze(0).transpose(0, 1))
    return torch.cat(outs, 0)
