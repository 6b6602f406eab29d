"""Device management API of ``torch.blackwell`` (mirror of ``torch.cuda``'s).
Parity: reference torch_musa/core/device.py:23-202."""
from __future__ import annotations

from typing import Any, List, Optional, Tuple, Union

import torch

from ._lazy_init import _lazy_init, _C

_device_t = Union[torch.device, str, int, None]


def _get_device_index(device: Any, optional: bool = False, allow_cpu: bool = False) -> int:
    """Device ordinal of ``device`` (``None`` / index-less device -> current device if ``optional``)."""
    if isinstance(device, int):
        return device
    if isinstance(device, str):
        device = torch.device(device)
    if isinstance(device, torch.device):
        if allow_cpu and device.type == "cpu":
            return -1
        if device.type != "blackwell":
            raise ValueError(f"Expected a blackwell device, but got: {device}")
        if device.index is not None:
            return device.index
        device = None
    if device is None:
        if optional:
            return current_device()
        raise ValueError(f"Expected a torch.device with a specified index or an integer, but got: {device}")
    # Stream / tensor-like objects
    idx = getattr(device, "device_index", None)
    if idx is not None:
        return int(idx)
    raise ValueError(f"Cannot infer a blackwell device index from {device!r}")


def device_count() -> int:
    return _C()._device_count()


def current_device() -> int:
    _lazy_init()
    return _C()._current_device()


def set_device(device: _device_t) -> None:
    idx = _get_device_index(device)
    if idx >= 0:
        _lazy_init()
        _C()._set_device(idx)


def _exchange_device(device: int) -> int:
    if device < 0:
        return -1
    _lazy_init()
    return _C()._exchange_device(device)


def _maybe_exchange_device(device: int) -> int:
    if device < 0:
        return -1
    _lazy_init()
    return _C()._maybe_exchange_device(device)


class _DeviceGuard:
    def __init__(self, index: int):
        self.idx = index
        self.prev_idx = -1

    def __enter__(self):
        self.prev_idx = _exchange_device(self.idx)

    def __exit__(self, *exc):
        self.idx = _maybe_exchange_device(self.prev_idx)
        return False


class device:
    """Context manager that changes the selected device (no-op for ``None`` / negative index)."""

    def __init__(self, device: Any):
        self.idx = _get_device_index(device, optional=True)
        self.prev_idx = -1

    def __enter__(self):
        self.prev_idx = _exchange_device(self.idx)

    def __exit__(self, *exc):
        self.idx = _maybe_exchange_device(self.prev_idx)
        return False


class device_of(device):
    """Context manager selecting the device of a tensor (no-op for non-blackwell tensors)."""

    def __init__(self, obj):
        idx = obj.get_device() if getattr(obj, "is_blackwell", False) or obj.device.type == "blackwell" else -1
        super().__init__(idx)


def synchronize(device: _device_t = None) -> None:
    _lazy_init()
    with globals()["device"](device):
        _C()._synchronize()


class _DeviceProperties:
    def __init__(self, d: dict):
        self.__dict__.update(d)

    def __repr__(self):
        return (
            f"_BlackwellDeviceProperties(name='{self.name}', major={self.major}, minor={self.minor}, "
            f"total_memory={self.total_memory // (1024 * 1024)}MB, "
            f"multi_processor_count={self.multi_processor_count}, uuid={self.uuid}, "
            f"L2_cache_size={self.l2_cache_size // (1024 * 1024)}MB)"
        )


def get_device_properties(device: _device_t = None) -> _DeviceProperties:
    _lazy_init()
    idx = _get_device_index(device, optional=True)
    if idx < 0 or idx >= device_count():
        raise AssertionError("Invalid device id")
    return _DeviceProperties(_C()._device_properties(idx))


def get_device_name(device: _device_t = None) -> str:
    return get_device_properties(device).name


def get_device_capability(device: _device_t = None) -> Tuple[int, int]:
    p = get_device_properties(device)
    return p.major, p.minor


def can_device_access_peer(device: _device_t, peer_device: _device_t) -> bool:
    _lazy_init()
    a, b = _get_device_index(device, optional=True), _get_device_index(peer_device)
    if a < 0 or a >= device_count():
        raise AssertionError("Invalid device id")
    if b < 0 or b >= device_count():
        raise AssertionError("Invalid peer device id")
    return _C()._can_access_peer(a, b)


def get_arch_list() -> List[str]:
    """Architectures the kernel library was compiled for."""
    return [_C()._kernels_arch()]


def is_bf16_supported(including_emulation: bool = True) -> bool:
    return True


def is_tf32_supported() -> bool:
    return True


def _sleep(cycles: int) -> None:
    """Enqueue a kernel that spins for ``cycles`` SM clocks (capped on the device side)."""
    _lazy_init()
    _C()._sleep(int(cycles))


def set_sync_debug_mode(debug_mode: Union[int, str]) -> None:
    """0/"default", 1/"warn", 2/"error": what to do on implicit host synchronisation."""
    if isinstance(debug_mode, str):
        debug_mode = {"default": 0, "warn": 1, "error": 2}[debug_mode]
    _C()._set_sync_debug_mode(int(debug_mode))


def get_sync_debug_mode() -> int:
    return _C()._get_sync_debug_mode()


def current_blas_handle():
    """cuBLAS handle (a ``cublasHandle_t`` as an integer) bound to the current device and stream.

    16-bit matrix products run on the backend's own tcgen05 kernels and never touch it; fp32 / fp64 / complex
    products are library GEMMs that run over the same memory on the current blackwell stream, and this is the
    handle they use."""
    from ._lazy_init import _lazy_init

    _lazy_init()
    import torch

    with torch.cuda.device(current_device()):
        return torch.cuda.current_blas_handle()
