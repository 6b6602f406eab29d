"""AMP for the blackwell device: ``torch.blackwell.amp.autocast`` / ``GradScaler`` /
``custom_fwd`` / ``custom_bwd``.  The operator policy itself is registered natively
(AutocastPrivateUse1); this module is the Python surface.
Parity: reference torch_musa/core/amp/autocast_mode.py:12-62, grad_scaler.py:10-31."""
from __future__ import annotations

import functools
from typing import Any, List

import torch


def get_amp_supported_dtype() -> List[torch.dtype]:
    return [torch.float16, torch.bfloat16]


def amp_definitely_not_available() -> bool:
    from ._lazy_init import is_available

    return not is_available()


class autocast(torch.amp.autocast_mode.autocast):
    """``with torch.blackwell.amp.autocast(dtype=torch.bfloat16):``"""

    def __init__(self, enabled: bool = True, dtype: torch.dtype = torch.bfloat16, cache_enabled: bool = True):
        super().__init__("blackwell", enabled=enabled, dtype=dtype, cache_enabled=cache_enabled)


class GradScaler(torch.amp.GradScaler):
    """Loss scaler whose unscale/inf-check and scale update run as fused device kernels."""

    def __init__(self, init_scale: float = 2.0**16, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, enabled: bool = True):
        super().__init__("blackwell", init_scale=init_scale, growth_factor=growth_factor,
                         backoff_factor=backoff_factor, growth_interval=growth_interval, enabled=enabled)


def custom_fwd(fwd=None, *, cast_inputs=None):
    return torch.amp.custom_fwd(fwd, device_type="blackwell", cast_inputs=cast_inputs)


def custom_bwd(bwd):
    return torch.amp.custom_bwd(bwd, device_type="blackwell")


def install() -> None:
    """Nothing to patch: torch.amp discovers ``get_amp_supported_dtype`` on ``torch.blackwell``."""
    return None
