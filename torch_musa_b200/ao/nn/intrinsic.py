"""Float containers that mark a convolution block as one fusable unit: the quantization passes swap them for their
quantization-aware or quantized counterparts, and the eager path runs them as written.

Parity: reference torch_musa/core/ao/nn/intrinsic/modules/fused.py:10-48 (ConvSiLU2d, ConvBnSiLU2d, ConvAddSiLU2d).
"""
from __future__ import annotations

import torch
from torch import nn
from torch.ao.nn.intrinsic import _FusedModule


def _expect(mod, kind, where):
    if not isinstance(mod, kind):
        raise TypeError(f"{where}: expected {kind.__name__}, got {type(mod).__name__}")


class ConvSiLU2d(_FusedModule):
    """``silu(conv(x))``."""

    def __init__(self, conv: nn.Conv2d, silu: nn.SiLU):
        _expect(conv, nn.Conv2d, "ConvSiLU2d")
        _expect(silu, nn.SiLU, "ConvSiLU2d")
        super().__init__(conv, silu)


class ConvBnSiLU2d(_FusedModule):
    """``silu(bn(conv(x)))``; exists in training mode only (an eval-mode block folds the norm into the convolution)."""

    def __init__(self, conv: nn.Conv2d, bn: nn.BatchNorm2d, silu: nn.SiLU):
        _expect(conv, nn.Conv2d, "ConvBnSiLU2d")
        _expect(bn, nn.BatchNorm2d, "ConvBnSiLU2d")
        _expect(silu, nn.SiLU, "ConvBnSiLU2d")
        super().__init__(conv, bn, silu)


class ConvAddSiLU2d(_FusedModule):
    """``silu(conv(x) + other)``: the tail of a residual block."""

    def __init__(self, conv: nn.Conv2d, silu: nn.SiLU):
        _expect(conv, nn.Conv2d, "ConvAddSiLU2d")
        _expect(silu, nn.SiLU, "ConvAddSiLU2d")
        super().__init__(conv, silu)

    def forward(self, x: torch.Tensor, other: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        return self[1](self[0](x) + other)
