"""Fusion rules and module mappings that make the SiLU blocks first-class citizens of ``torch.ao.quantization``:
``fuse_modules`` / ``fuse_modules_qat`` accept conv + bn + SiLU patterns, ``prepare_qat`` swaps the fused float blocks
for their quantization-aware versions, ``convert`` produces the quantized blocks.

Parity: reference torch_musa/core/ao/register_helper.py:12-20 (publishes the classes into the torch.ao namespaces).
"""
from __future__ import annotations

import torch
from torch import nn
from torch.nn.utils.fusion import fuse_conv_bn_eval

from .nn import intrinsic, qat, quantized

_registered = False


def fuse_conv_silu(is_qat: bool, conv: nn.Conv2d, silu: nn.SiLU):
    return intrinsic.ConvSiLU2d(conv, silu)


def fuse_conv_bn_silu(is_qat: bool, conv: nn.Conv2d, bn: nn.BatchNorm2d, silu: nn.SiLU):
    """Training / QAT: the three stay separate inside one container (the QAT block folds the norm every step).
    Evaluation: the norm is folded into the convolution once."""
    if conv.training != bn.training:
        raise ValueError("conv and bn must be in the same mode (both training or both eval) to be fused")
    if is_qat or conv.training:
        if bn.num_features != conv.out_channels or not bn.affine or not bn.track_running_stats:
            raise ValueError("fusing needs an affine batch norm with running statistics over the conv's output channels")
        return intrinsic.ConvBnSiLU2d(conv, bn, silu)
    return intrinsic.ConvSiLU2d(fuse_conv_bn_eval(conv, bn), silu)


def register() -> None:
    """Idempotent: publishes the classes under ``torch.ao.nn.intrinsic{,.qat,.quantized}`` and adds the fusion rules
    and the float -> QAT -> quantized mappings to PyTorch's default tables."""
    global _registered
    if _registered:
        return
    import torch.ao.nn.intrinsic as nni
    import torch.ao.nn.intrinsic.qat as nniqat
    import torch.ao.nn.intrinsic.quantized as nniq
    from torch.ao.quantization import fuser_method_mappings as fm
    from torch.ao.quantization import quantization_mappings as qm

    for name in ("ConvSiLU2d", "ConvBnSiLU2d", "ConvAddSiLU2d"):
        setattr(nni, name, getattr(intrinsic, name))
        setattr(nniqat, name, getattr(qat, name))
    for name in ("ConvSiLU2d", "ConvAddSiLU2d"):
        setattr(nniq, name, getattr(quantized, name))
    fm._DEFAULT_OP_LIST_TO_FUSER_METHOD[(nn.Conv2d, nn.SiLU)] = fuse_conv_silu
    fm._DEFAULT_OP_LIST_TO_FUSER_METHOD[(nn.Conv2d, nn.BatchNorm2d, nn.SiLU)] = fuse_conv_bn_silu
    qm.DEFAULT_QAT_MODULE_MAPPINGS[intrinsic.ConvBnSiLU2d] = qat.ConvBnSiLU2d
    qm.DEFAULT_QAT_MODULE_MAPPINGS[intrinsic.ConvSiLU2d] = qat.ConvSiLU2d
    qm.DEFAULT_QAT_MODULE_MAPPINGS[intrinsic.ConvAddSiLU2d] = qat.ConvAddSiLU2d
    for src in (intrinsic.ConvSiLU2d, qat.ConvSiLU2d, qat.ConvBnSiLU2d):
        qm.DEFAULT_STATIC_QUANT_MODULE_MAPPINGS[src] = quantized.ConvSiLU2d
    for src in (intrinsic.ConvAddSiLU2d, qat.ConvAddSiLU2d):
        qm.DEFAULT_STATIC_QUANT_MODULE_MAPPINGS[src] = quantized.ConvAddSiLU2d
    _registered = True
