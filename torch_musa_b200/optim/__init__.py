"""Fused optimizers.  One multi-tensor kernel launch updates up to 128 parameter tensors;
step counters, learning-rate tensors and the GradScaler's ``found_inf`` stay on the device,
so an optimizer step never synchronises with the host.
Parity: reference torch_musa/optim/{fused_adam,fused_adamw,fused_lamb}.py, optim/__init__.py:18-29."""
from .fused import FusedAdam, FusedAdamW, FusedSGD, FusedLAMB, clip_grad_norm_  # noqa: F401
