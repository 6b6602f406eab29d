"""FakeTensor (meta) rules for the ``blackwell::`` operators so they trace under torch.compile /
torch.export.  Parity: reference torch_musa/core/ops/register_fake_impl.py:10-42."""
from __future__ import annotations

import torch

_lib = torch.library


def _reg(name):
    def deco(fn):
        try:
            _lib.register_fake(f"blackwell::{name}")(fn)
        except RuntimeError:
            pass  # already registered (re-import)
        return fn
    return deco


@_reg("rope")
def _(x, cos, sin, positions=None, interleaved=False, conj=False):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


@_reg("swiglu")
def _(x):
    return x.new_empty(x.shape[:-1] + (x.shape[-1] // 2,))


@_reg("swiglu_backward")
def _(dy, x):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@_reg("silu_mul")
def _(gate, up):
    return torch.empty_like(gate, memory_format=torch.contiguous_format)


@_reg("silu_mul_backward")
def _(dy, gate, up):
    return (torch.empty_like(gate, memory_format=torch.contiguous_format),
            torch.empty_like(up, memory_format=torch.contiguous_format))


@_reg("cross_entropy_fwd")
def _(logits, target, ignore_index=-100, label_smoothing=0.0):
    r = logits.new_empty((logits.shape[0],), dtype=torch.float32)
    return r, torch.empty_like(r)


@_reg("cross_entropy_bwd")
def _(logits, lse, target, grad_loss, scale, ignore_index, label_smoothing):
    return torch.empty_like(logits, memory_format=torch.contiguous_format)


@_reg("online_softmax_stats")
def _(logits, target, vocab_start):
    return logits.new_empty((logits.shape[0], 3), dtype=torch.float32)


@_reg("vocab_parallel_ce_finish")
def _(logits, all_stats, target, vocab_start, ignore_index):
    return logits.new_empty((logits.shape[0],), dtype=torch.float32)


@_reg("rms_norm_residual")
def _(x, residual, weight, eps):
    stat = x.new_empty(x.shape[:-1] + (1,), dtype=torch.float32)
    return torch.empty_like(x), torch.empty_like(x), stat


@_reg("multi_tensor_l2norm")
def _(tensors, per_tensor=False):
    t = tensors[0]
    return t.new_empty((1,), dtype=torch.float32), t.new_empty((len(tensors) if per_tensor else 0,), dtype=torch.float32)


@_reg("batch_norm_act")
def _(input, weight, bias, running_mean, running_var, residual, training, momentum, eps, relu):
    c = input.shape[1]
    n = c if training else 0
    return (torch.empty_like(input), input.new_empty((n,), dtype=torch.float32),
            input.new_empty((n,), dtype=torch.float32))


@_reg("batch_norm_act_backward")
def _(grad_out, input, out, weight, save_mean, save_invstd, relu, has_residual):
    c = input.shape[1]
    return (torch.empty_like(input), input.new_empty((c,), dtype=torch.float32),
            input.new_empty((c,), dtype=torch.float32),
            torch.empty_like(input) if has_residual else input.new_empty((0,)))


@_reg("scaled_mm")
def _(a, b, block_scale_a, block_scale_b, row_scale, col_scale, bias, out_dtype):
    return a.new_empty((a.shape[0], b.shape[0]), dtype=out_dtype)


@_reg("quantize_fp8_1x128")
def _(x, e5m2=False):
    q = x.new_empty(x.shape, dtype=torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn)
    return q, x.new_empty((x.shape[0], x.shape[1] // 128), dtype=torch.float32)


@_reg("decode_attention")
def _(q, k_cache, v_cache, pos, scale=None):
    return torch.empty_like(q)


@_reg("grouped_mm")
def _(a, b, counts, mode):
    if mode == 2:
        return a.new_empty((counts.shape[0], a.shape[1], b.shape[1]))
    return a.new_empty((a.shape[0], b.shape[1] if mode == 0 else b.shape[2]))


@_reg("grouped_mm_out")
def _(a, b, counts, mode, out):
    return out


@_reg("varlen_attention")
def _(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=False, scale=None):
    return torch.empty_like(q, memory_format=torch.contiguous_format), q.new_empty((q.shape[1], q.shape[0]), dtype=torch.float32)


@_reg("varlen_attention_backward")
def _(grad_out, q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=False, scale=None):
    return (torch.empty_like(q, memory_format=torch.contiguous_format), torch.empty_like(k, memory_format=torch.contiguous_format),
            torch.empty_like(v, memory_format=torch.contiguous_format))


@_reg("swiglu_rows")
def _(x, row_counts):
    return x.new_empty(x.shape[:-1] + (x.shape[-1] // 2,))


@_reg("swiglu_rows_backward")
def _(dy, x, row_counts):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@_reg("decode_rope_cache")
def _(q, k, v, cos, sin, pos, k_cache, v_cache):
    return q.new_empty((q.shape[0], q.shape[-2], q.shape[-1]))
