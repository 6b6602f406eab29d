"""Tensor parallelism with sequence-parallel activations (Megatron-style), built from two primitives:

    ag_matmul(x_shard [T/W, K], w_local [N/W, K])  ->  [T, N/W]     all-gather -> GEMM   (column-parallel layer)
    matmul_rs(x [T, K/W],      w_local [N, K/W])   ->  [T/W, N]     GEMM -> reduce-scatter (row-parallel layer)

Between layers the activations stay sharded over the flattened token dimension, so norms and residual adds
run on 1/W of the tokens.  The two primitives are each other's backward: d(ag_matmul)/dx is a matmul_rs and
d(matmul_rs)/dx is an ag_matmul, so the same two kernels serve forward and backward.

The primitives have two implementations selected per call: the fused peer-memory kernels on the blackwell
device (one kernel moves the shards over NVLink and feeds / drains the tensor-core tiles), and the plain
composition `all_gather_into_tensor` + `F.linear` / `F.linear` + `reduce_scatter_tensor` anywhere else (CPU +
gloo in the tests, CUDA + NCCL in the benchmark's stock arm).
Parity: the reference relies on stock DTensor Colwise/RowwiseParallel over its collective backend and adds
sharding rules for its custom ops (reference torch_musa/distributed/tensor/_ops.py:27-189).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

# Optional fused implementations, installed by torch_musa_b200.parallel.fused_tp when the device supports them:
#   FUSED_AG_MATMUL(x_shard, w, group) -> (y, x_full)        FUSED_MATMUL_RS(x, w, group) -> y_shard
FUSED_AG_MATMUL: Optional[Callable] = None
FUSED_MATMUL_RS: Optional[Callable] = None


class _Solo:
    """Group stand-in for a layer built with world size 1: no communication even inside a larger job."""


SOLO = _Solo()


def _world(group) -> int:
    if group is SOLO:
        return 1
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def all_gather_rows(x: torch.Tensor, group=None) -> torch.Tensor:
    w = _world(group)
    if w == 1:
        return x
    out = x.new_empty((x.shape[0] * w,) + tuple(x.shape[1:]))
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def reduce_scatter_rows(x: torch.Tensor, group=None) -> torch.Tensor:
    w = _world(group)
    if w == 1:
        return x
    out = x.new_empty((x.shape[0] // w,) + tuple(x.shape[1:]))
    dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
    return out


def _ag_matmul_impl(x_shard, w, group):
    if FUSED_AG_MATMUL is not None and x_shard.device.type == "blackwell" and _world(group) > 1:
        r = FUSED_AG_MATMUL(x_shard, w, group)
        if r is not None:
            return r
    x_full = all_gather_rows(x_shard, group)
    return F.linear(x_full, w), x_full


def _matmul_rs_impl(x, w, group):
    if FUSED_MATMUL_RS is not None and x.device.type == "blackwell" and _world(group) > 1:
        r = FUSED_MATMUL_RS(x, w, group)
        if r is not None:
            return r
    return reduce_scatter_rows(F.linear(x, w), group)


class _AGMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w, group):
        y, x_full = _ag_matmul_impl(x_shard, w, group)
        ctx.group = group
        ctx.save_for_backward(x_full, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx_shard = _matmul_rs_impl(dy, w.t(), ctx.group) if ctx.needs_input_grad[0] else None   # [T, N/W] x [N/W, K] -> RS
        dw = dy.t().matmul(x_full) if ctx.needs_input_grad[1] else None
        return dx_shard, dw, None


class _MatmulRS(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group):
        ctx.group = group
        ctx.save_for_backward(x, w)
        return _matmul_rs_impl(x, w, group)

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        dy_shard = dy_shard.contiguous()
        # dX = AG(dy) @ W ; the gathered dy is also what the weight gradient needs
        dx, dy_full = _ag_matmul_impl(dy_shard, w.t(), ctx.group)
        dw = dy_full.t().matmul(x) if ctx.needs_input_grad[1] else None
        return (dx if ctx.needs_input_grad[0] else None), dw, None


def ag_matmul(x_shard: torch.Tensor, w_local: torch.Tensor, group=None) -> torch.Tensor:
    """``all_gather(x_shard) @ w_local.T``; x_shard [T/W, K], w_local [N/W, K] -> [T, N/W]."""
    return _AGMatmul.apply(x_shard, w_local, group)


def matmul_rs(x: torch.Tensor, w_local: torch.Tensor, group=None) -> torch.Tensor:
    """``reduce_scatter(x @ w_local.T)`` over rows; x [T, K/W], w_local [N, K/W] -> [T/W, N]."""
    return _MatmulRS.apply(x, w_local, group)


class _GatherRows(torch.autograd.Function):
    """all-gather over rows whose backward is the reduce-scatter of the gradient."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_rows(g.contiguous(), ctx.group), None


def gather_rows(x: torch.Tensor, group=None) -> torch.Tensor:
    return _GatherRows.apply(x, group)


class _ShardRows(torch.autograd.Function):
    """Takes this rank's row block of a replicated tensor; backward all-gathers the gradient blocks."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = _world(group)
        if w == 1:
            return x
        r = dist.get_rank(group)
        n = x.shape[0] // w
        return x[r * n:(r + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather_rows(g.contiguous(), ctx.group), None


def shard_rows(x: torch.Tensor, group=None) -> torch.Tensor:
    return _ShardRows.apply(x, group)


class ColumnParallelLinear(nn.Module):
    """Weight [out/W, in]; input: row shard [T/W, in]; output [T, out/W]."""

    def __init__(self, in_features: int, out_features: int, world: int, group=None, device=None, dtype=None):
        super().__init__()
        assert out_features % world == 0
        self.group = SOLO if world == 1 else group
        self.weight = nn.Parameter(torch.empty(out_features // world, in_features, device=device, dtype=dtype))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        return ag_matmul(x_shard, self.weight, self.group)


class RowParallelLinear(nn.Module):
    """Weight [out, in/W]; input [T, in/W]; output: row shard [T/W, out] (summed over ranks)."""

    def __init__(self, in_features: int, out_features: int, world: int, group=None, device=None, dtype=None):
        super().__init__()
        assert in_features % world == 0
        self.group = SOLO if world == 1 else group
        self.weight = nn.Parameter(torch.empty(out_features, in_features // world, device=device, dtype=dtype))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return matmul_rs(x, self.weight, self.group)
