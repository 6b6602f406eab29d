"""Vocabulary-parallel fused cross entropy (tensor parallelism over the vocabulary dimension).

Each rank holds logits for its vocabulary shard [T, V/TP].  One kernel computes per-token
(max, sum-exp, target-logit) over the shard, the [T, 3] statistics are all-gathered (tiny), and a
second kernel combines them into the loss and overwrites the logits shard with the softmax gradient,
so backward is a scale of that buffer.
Parity: reference torch_musa/distributed/loss.py:22-136.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F


class _ParallelFusedCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, group, ignore_index, reduction):
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        T, Vs = logits.shape
        vocab_start = rank * Vs
        if logits.device.type == "blackwell":
            stats = torch.ops.blackwell.online_softmax_stats(logits, target, vocab_start)
            all_stats = torch.empty((world, T, 3), dtype=torch.float32, device=logits.device)
            dist.all_gather_into_tensor(all_stats, stats, group=group)
            grad_buf = logits.detach()  # overwritten in place with (softmax - onehot)
            loss_rows = torch.ops.blackwell.vocab_parallel_ce_finish(grad_buf, all_stats, target, vocab_start,
                                                                     ignore_index)
        else:
            lf = logits.float()
            m = lf.max(dim=-1).values
            s = (lf - m[:, None]).exp().sum(-1)
            local_t = target - vocab_start
            inside = (local_t >= 0) & (local_t < Vs)
            tl = torch.where(inside, lf.gather(1, local_t.clamp(0, Vs - 1)[:, None])[:, 0], torch.zeros_like(m))
            stats = torch.stack((m, s, tl), dim=-1).contiguous()
            gathered = [torch.empty_like(stats) for _ in range(world)]
            dist.all_gather(gathered, stats, group=group)
            all_stats = torch.stack(gathered)
            gm = all_stats[..., 0].max(dim=0).values
            gs = (all_stats[..., 1] * (all_stats[..., 0] - gm).exp()).sum(0)
            lse = gm + gs.log()
            ignored = target == ignore_index
            loss_rows = torch.where(ignored, torch.zeros_like(lse), lse - all_stats[..., 2].sum(0))
            p = (lf - lse[:, None]).exp()
            onehot = torch.zeros_like(p)
            onehot[inside, local_t[inside]] = 1.0
            grad_buf = torch.where(ignored[:, None], torch.zeros_like(p), p - onehot).to(logits.dtype)
        n_valid = (target != ignore_index).sum().clamp_min(1).to(torch.float32)
        ctx.save_for_backward(grad_buf, n_valid)
        ctx.reduction = reduction
        if reduction == "mean":
            return loss_rows.sum() / n_valid
        if reduction == "sum":
            return loss_rows.sum()
        return loss_rows

    @staticmethod
    def backward(ctx, dloss):
        grad_buf, n_valid = ctx.saved_tensors
        g = dloss.to(torch.float32)
        if ctx.reduction == "mean":
            g = g / n_valid
        if ctx.reduction == "none":
            out = grad_buf * g[:, None].to(grad_buf.dtype)
        else:
            out = grad_buf * g.to(grad_buf.dtype)
        return out, None, None, None, None


def parallel_fused_cross_entropy(logits_shard: torch.Tensor, target: torch.Tensor, group=None,
                                 ignore_index: int = -100, reduction: str = "mean") -> torch.Tensor:
    """Cross entropy over vocabulary-sharded logits [T, V/TP]; ``target`` holds global vocabulary ids.

    The logits shard is consumed (overwritten by its gradient) on the device path."""
    group = group or dist.group.WORLD
    return _ParallelFusedCE.apply(logits_shard.contiguous(), target.contiguous(), group, ignore_index, reduction)
