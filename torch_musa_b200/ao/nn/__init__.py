"""Fused, quantization-aware and quantized convolution blocks with a SiLU activation."""
from . import intrinsic, qat, quantized  # noqa: F401
