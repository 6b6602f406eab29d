"""Quantization support of the backend: fused conv / batch-norm / SiLU blocks in float, quantization-aware and
quantized form, their registration with ``torch.ao.quantization`` and the PT2E lowering.

    import torch_musa_b200.ao as ao
    ao.register()                                   # (done on package import)
    torch.ao.quantization.fuse_modules_qat(model, [["conv", "bn", "act"]], inplace=True)
    torch.ao.quantization.prepare_qat(model, inplace=True); ...train...; torch.ao.quantization.convert(model.eval())

Parity: reference torch_musa/core/ao/__init__.py, torch_musa/core/lowering.py.
"""
from . import nn  # noqa: F401
from .fusion import fuse_conv_bn_silu, fuse_conv_silu, register  # noqa: F401
from .lowering import lower_pt2e_quantized  # noqa: F401
from . import lowering as _lowering

register()
_lowering.install()
