"""Quantized fused blocks: int8 per-channel weights and a quantized (quint8) output with the scale the observers
found.  The arithmetic is "dequantize, convolve, activate, requantize" on whatever device the block lives on: the
integer weights and their scales are plain buffers, not packed CPU parameters, so the block moves with ``.to()`` and
the convolution runs on the device's own kernels (tcgen05 implicit GEMM for bf16 on the blackwell device).

Parity: reference torch_musa/core/ao/nn/intrinsic/quantized/modules/conv_silu.py:21-98, conv_add.py:14-78 (those call
the vendor's int8 convolution; here the integer representation is kept and the product is computed in floating point).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn
from torch.nn.utils.fusion import fuse_conv_bn_weights


class _QuantizedConvAct2d(nn.Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 compute_dtype: torch.dtype = torch.float32):
        super().__init__()
        pair = lambda v: tuple(v) if isinstance(v, (tuple, list)) else (v, v)  # noqa: E731
        self.in_channels, self.out_channels, self.groups = in_channels, out_channels, groups
        self.kernel_size, self.stride, self.padding, self.dilation = pair(kernel_size), pair(stride), pair(padding), pair(dilation)
        self.compute_dtype = compute_dtype
        kh, kw = self.kernel_size
        self.register_buffer("weight_int8", torch.zeros(out_channels, in_channels // groups, kh, kw, dtype=torch.int8))
        self.register_buffer("weight_scale", torch.ones(out_channels))
        self.register_buffer("weight_zero_point", torch.zeros(out_channels, dtype=torch.int32))
        self.register_buffer("bias", torch.zeros(out_channels) if bias else None)
        self.scale, self.zero_point = 1.0, 0

    # ---- weights
    def set_weight(self, w: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor) -> None:
        """Quantizes a float weight [out, in / groups, kh, kw] per output channel (or per tensor: 0-dim qparams)."""
        scale = scale.detach().float().reshape(-1).expand(self.out_channels).clone()
        zero_point = zero_point.detach().to(torch.int32).reshape(-1).expand(self.out_channels).clone()
        q = torch.round(w.detach().float() / scale.view(-1, 1, 1, 1)) + zero_point.view(-1, 1, 1, 1)
        self.weight_int8.copy_(q.clamp(-128, 127).to(torch.int8))
        self.weight_scale.copy_(scale)
        self.weight_zero_point.copy_(zero_point)

    def weight(self) -> torch.Tensor:
        """The dequantized weight."""
        return (self.weight_int8.float() - self.weight_zero_point.view(-1, 1, 1, 1).float()) * self.weight_scale.view(-1, 1, 1, 1)

    # ---- arithmetic
    def _conv(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.dequantize() if x.is_quantized else x
        dt = self.compute_dtype
        b = None if self.bias is None else self.bias.to(dt)
        return F.conv2d(xf.to(dt), self.weight().to(dt), b, self.stride, self.padding, self.dilation, self.groups).float()

    def _requant(self, y: torch.Tensor) -> torch.Tensor:
        return torch.quantize_per_tensor(y, float(self.scale), int(self.zero_point), torch.quint8)

    # ---- conversion
    @classmethod
    def from_float(cls, mod, use_precomputed_fake_quant: bool = False):
        """From a quantization-aware block (fake quantizers carry the ranges) or from an observed float block."""
        act = getattr(mod, "activation_post_process", None)
        if act is None:
            raise ValueError(f"{type(mod).__name__} has no activation observer: run prepare / prepare_qat first")
        if hasattr(mod, "weight_fake_quant"):                       # QAT block (possibly with a batch norm to fold)
            w, b = mod.weight, mod.bias
            if getattr(mod, "bn", None) is not None:
                w, b = fuse_conv_bn_weights(w, b, mod.bn.running_mean, mod.bn.running_var, mod.bn.eps, mod.bn.weight, mod.bn.bias)
            wobs = mod.weight_fake_quant
            conv = mod
        else:                                                       # observed float block: [conv, activation]
            conv = mod[0] if isinstance(mod, nn.Sequential) else mod
            w, b = conv.weight, conv.bias
            wobs = mod.qconfig.weight()
        wobs(w.detach())
        w_scale, w_zp = wobs.calculate_qparams()
        out = cls(conv.in_channels, conv.out_channels, conv.kernel_size, conv.stride, conv.padding, conv.dilation,
                  conv.groups, b is not None)
        out.set_weight(w, w_scale, w_zp)
        if b is not None:
            out.bias.copy_(b.detach().float())
        a_scale, a_zp = act.calculate_qparams()
        out.scale, out.zero_point = float(a_scale), int(a_zp)
        return out

    def extra_repr(self) -> str:
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}, "
                f"padding={self.padding}, scale={self.scale:.6g}, zero_point={self.zero_point}")

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        super()._save_to_state_dict(destination, prefix, keep_vars)
        destination[prefix + "scale"] = torch.tensor(float(self.scale))
        destination[prefix + "zero_point"] = torch.tensor(int(self.zero_point))

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        if prefix + "scale" in state_dict:
            self.scale = float(state_dict.pop(prefix + "scale"))
            self.zero_point = int(state_dict.pop(prefix + "zero_point"))
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)


class ConvSiLU2d(_QuantizedConvAct2d):
    """Quantized ``silu(conv(x))``: quint8 in, quint8 out."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._requant(F.silu(self._conv(x)))


class ConvAddSiLU2d(_QuantizedConvAct2d):
    """Quantized ``silu(conv(x) + other)``."""

    def forward(self, x: torch.Tensor, other: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        o = other.dequantize() if other.is_quantized else other
        return self._requant(F.silu(self._conv(x) + o.float()))
