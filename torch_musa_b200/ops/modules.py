"""``nn.Module`` wrappers of the fused operators."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import functional as BF


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        if residual is not None:
            return BF.rms_norm_residual(x, residual, self.weight, self.eps)
        return BF.rms_norm(x, self.weight, self.eps)

    def extra_repr(self):
        return f"{self.weight.numel()}, eps={self.eps}"


class RoPE(nn.Module):
    """Rotary position embedding with a cached fp32 cos/sin table."""

    def __init__(self, head_dim: int, max_seq_len: int = 4096, theta: float = 10000.0, interleaved: bool = False):
        super().__init__()
        self.head_dim, self.max_seq_len, self.theta, self.interleaved = head_dim, max_seq_len, theta, interleaved
        cos, sin = BF.precompute_rope_cache(max_seq_len, head_dim, theta)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def forward(self, x: torch.Tensor, positions: Optional[torch.Tensor] = None):
        return BF.rope(x, self.cos, self.sin, positions, self.interleaved)


class SwishGLU(nn.Module):
    def forward(self, x: torch.Tensor):
        return BF.swiglu(x)


class FusedCrossEntropyLoss(nn.Module):
    def __init__(self, ignore_index: int = -100, label_smoothing: float = 0.0, reduction: str = "mean",
                 inplace_backward: bool = False):
        super().__init__()
        self.ignore_index, self.label_smoothing, self.reduction = ignore_index, label_smoothing, reduction
        self.inplace_backward = inplace_backward

    def forward(self, logits: torch.Tensor, target: torch.Tensor):
        return BF.fused_cross_entropy(logits, target, self.ignore_index, self.label_smoothing, self.reduction,
                                      self.inplace_backward)


class BatchNormAct2d(nn.BatchNorm2d):
    """``BatchNorm2d`` with the following ReLU (and an optional residual add before it) fused into the same
    kernel passes.  Parameters, buffers and state_dict keys are those of ``nn.BatchNorm2d``."""

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1, relu: bool = True, **kw):
        super().__init__(num_features, eps=eps, momentum=momentum, **kw)
        self.relu = relu

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        return bn_module_act(self, x, residual, self.relu)


def bn_module_act(bn: nn.BatchNorm2d, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                  relu: bool = True) -> torch.Tensor:
    """Applies an existing ``nn.BatchNorm2d`` module followed by (+ residual) (ReLU) through the fused operator."""
    training = bn.training or (bn.running_mean is None and bn.running_var is None)
    momentum = 0.0 if bn.momentum is None else bn.momentum
    if bn.training and bn.track_running_stats and bn.num_batches_tracked is not None:
        bn.num_batches_tracked.add_(1)
        if bn.momentum is None:
            momentum = 1.0 / float(bn.num_batches_tracked)
    return BF.batch_norm_act(x, bn.weight, bn.bias, bn.running_mean if (not bn.training or bn.track_running_stats) else None,
                             bn.running_var if (not bn.training or bn.track_running_stats) else None, residual, training,
                             momentum, bn.eps, relu)
