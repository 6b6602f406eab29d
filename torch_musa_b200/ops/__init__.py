"""Functional API and ``nn.Module`` wrappers of the backend's fused operators.

Every function runs the hand-written sm_100a kernel when its inputs live on the
blackwell device and an equivalent plain-PyTorch formulation otherwise (CPU
tests, reference numerics), with identical autograd behaviour.
Parity: the reference exposes these through a patched torch (``nn.RoPE``,
``nn.SwishGLU``, ``F.rope``, ``torch.rms_norm`` routing; reference
torch_patches/torch_nn_functional.py.patch, torch_nn_modules_activation.py.patch).
"""
from .functional import (  # noqa: F401
    rms_norm,
    rms_norm_residual,
    batch_norm_act,
    rope,
    precompute_rope_cache,
    swiglu,
    grouped_linear,
    silu_mul,
    gated_silu,
    fused_cross_entropy,
    multi_tensor_l2norm,
    scaled_dot_product_attention,
    flash_attn_varlen_func,
)
from .modules import RMSNorm, RoPE, SwishGLU, FusedCrossEntropyLoss, BatchNormAct2d  # noqa: F401
from . import fake  # noqa: F401  (FakeTensor / meta rules for torch.compile)
