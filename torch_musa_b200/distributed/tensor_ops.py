"""DTensor sharding rules for the backend's custom operators, so that models that keep their
activations as DTensors (sequence-parallel regions, ``use_local_output=False`` plans) can call the
fused kernels without falling back to replication.

Every rule lists the placements under which the kernel can run on the local shards unchanged:
element-wise operators accept the same ``Shard(d)`` on all operands for any ``d`` that is not the
feature dimension they split or normalise over; row-wise operators (norm + residual, cross entropy)
accept sharding over the row dimensions only; everything also runs replicated.

Parity: reference torch_musa/distributed/tensor/_ops.py:27-189 (strategies for its fused RMSNorm
forward/backward) and torch_musa/optim/__init__.py:18-29 (fused optimizer steps on DTensors).
"""
from __future__ import annotations

import torch

_registered = False


def register() -> None:
    global _registered
    if _registered:
        return
    _registered = True
    try:
        from torch.distributed.tensor import Replicate, Shard
        from torch.distributed.tensor.experimental import register_sharding
    except Exception:  # pragma: no cover  (torch built without distributed)
        return
    ops = torch.ops.blackwell

    def same_on_all(n_in: int, n_out: int, ndim: int, skip_last: int = 1):
        """Replicated, or every tensor sharded alike on one of the leading dimensions."""
        rules = [([Replicate()] * n_out, [Replicate()] * n_in)]
        for d in range(ndim - skip_last):
            rules.append(([Shard(d)] * n_out, [Shard(d)] * n_in))
        return rules

    @register_sharding(ops.silu_mul.default)
    def _silu_mul(gate, up):
        # purely element-wise: the feature dimension may be sharded as well (column-parallel gate/up projections)
        return same_on_all(2, 1, gate.ndim, skip_last=0)

    @register_sharding(ops.silu_mul_backward.default)
    def _silu_mul_bwd(dy, gate, up):
        return same_on_all(3, 2, gate.ndim, skip_last=0)

    @register_sharding(ops.swiglu.default)
    def _swiglu(x):
        # the last dimension holds [gate | up] halves: a shard of it would mix them
        return same_on_all(1, 1, x.ndim)

    @register_sharding(ops.swiglu_backward.default)
    def _swiglu_bwd(dy, x):
        return same_on_all(2, 1, x.ndim)

    @register_sharding(ops.rope.default)
    def _rope(x, cos, sin, positions=None, interleaved=False, conj=False):
        # x is [batch, seq, heads, head_dim]; batch and heads shard freely (tables replicated), the sequence does
        # not (row i of the tables belongs to position i) unless explicit positions travel with the shard
        rules = [([Replicate()], [Replicate(), Replicate(), Replicate()] + ([Replicate()] if positions is not None else []))]
        for d in (0, 2):
            if d < x.ndim - 1:
                ins = [Shard(d), Replicate(), Replicate()]
                if positions is not None:
                    ins.append(Shard(0) if d == 0 and positions.ndim == 2 else Replicate())
                rules.append(([Shard(d)], ins))
        return rules

    @register_sharding(ops.rms_norm_residual.default)
    def _rms_norm_residual(x, residual, weight, eps):
        rules = [([Replicate()] * 3, [Replicate()] * 3)]
        for d in range(x.ndim - 1):
            # outputs: normalised, new residual (shaped like x) and the per-row rstd (one dimension fewer)
            rules.append(([Shard(d), Shard(d), Shard(d)], [Shard(d), Shard(d), Replicate()]))
        return rules

    @register_sharding(ops.cross_entropy_fwd.default)
    def _ce_fwd(logits, target, ignore_index=-100, label_smoothing=0.0):
        return [([Replicate(), Replicate()], [Replicate(), Replicate()]),
                ([Shard(0), Shard(0)], [Shard(0), Shard(0)])]      # rows only: the vocabulary stays whole per rank

    @register_sharding(ops.cross_entropy_bwd.default)
    def _ce_bwd(logits, lse, target, grad_loss, scale, ignore_index, label_smoothing):
        n = 4 if grad_loss is not None else 3
        rep = [Replicate()] * n
        shard = [Shard(0), Shard(0), Shard(0)] + ([Shard(0) if getattr(grad_loss, "ndim", 0) else Replicate()] if n == 4 else [])
        return [([Replicate()], rep), ([Shard(0)], shard)]
