"""Quantization-aware training versions of the fused blocks: weights pass through a fake quantizer (after the batch
norm has been folded in, where there is one), the block's output through the activation fake quantizer that
``prepare_qat`` attaches.

Parity: reference torch_musa/core/ao/nn/intrinsic/qat/modules/conv_fused.py:19-144.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn
import torch.ao.nn.intrinsic.qat as nniqat
import torch.ao.nn.qat as nnqat
from torch.ao.nn.intrinsic import _FusedModule

from . import intrinsic


class ConvBnSiLU2d(nniqat.ConvBn2d):
    """Convolution + batch norm + SiLU with the norm folded into the fake-quantized weight (the folding arithmetic
    and the statistics handling are PyTorch's ``ConvBn2d``; only the activation differs)."""

    _FLOAT_MODULE = intrinsic.ConvBnSiLU2d
    _FLOAT_CONV_MODULE = nn.Conv2d
    _FLOAT_BN_MODULE = nn.BatchNorm2d
    _FLOAT_RELU_MODULE = nn.SiLU            # the activation that `to_float` appends
    _FUSED_FLOAT_MODULE = intrinsic.ConvSiLU2d

    def forward(self, x):
        return F.silu(self._forward(x))


class ConvSiLU2d(nnqat.Conv2d, _FusedModule):
    """Convolution + SiLU with a fake-quantized weight."""

    _FLOAT_MODULE = intrinsic.ConvSiLU2d
    _FLOAT_CONV_MODULE = nn.Conv2d
    _FLOAT_BN_MODULE = None
    _FLOAT_RELU_MODULE = nn.SiLU

    def forward(self, x):
        return F.silu(self._conv_forward(x, self.weight_fake_quant(self.weight), self.bias))


class ConvAddSiLU2d(nnqat.Conv2d, _FusedModule):
    """``silu(conv(x) + other)`` with a fake-quantized weight."""

    _FLOAT_MODULE = intrinsic.ConvAddSiLU2d
    _FLOAT_CONV_MODULE = nn.Conv2d
    _FLOAT_BN_MODULE = None
    _FLOAT_RELU_MODULE = nn.SiLU

    def forward(self, x, other):  # type: ignore[override]
        return F.silu(self._conv_forward(x, self.weight_fake_quant(self.weight), self.bias) + other)
