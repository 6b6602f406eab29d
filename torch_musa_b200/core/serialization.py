"""Checkpoint interchange.

Storages saved from this device are tagged ``blackwell:N``.  On load, a
``blackwell:N`` tag restores onto the device, and so does a ``cuda:N`` tag when
the user maps it here (``map_location="blackwell"``): the file format is the
stock ``torch.save`` format, so checkpoints move freely between this backend and
the CUDA backend.  With the unified CPU allocator active, a storage whose host
memory is already managed memory is retagged in place (no device allocation, no
copy).  Parity: reference torch_musa/core/serialization.py:45-83,
torch_musa/__init__.py:227-262.
"""
from __future__ import annotations

import torch

_installed = False


def _tag(obj):
    if obj.device.type == "blackwell":
        return "blackwell:" + str(obj.device.index or 0)
    return None


def _validate_index(location: str) -> int:
    import torch_musa_b200 as bw

    idx = 0
    if ":" in location:
        idx = max(int(location.split(":", 1)[1]), 0)
    if not bw.is_available():
        raise RuntimeError(
            "Attempting to deserialize object on a blackwell device but torch.blackwell.is_available() is False. "
            "Use torch.load with map_location=torch.device('cpu') to map your storages to the CPU."
        )
    n = bw.device_count()
    if idx >= n:
        raise RuntimeError(
            f"Attempting to deserialize object on blackwell device {idx} but torch.blackwell.device_count() is {n}. "
            "Use torch.load with map_location to map your storages to an existing device."
        )
    return idx


def _deserialize(obj, location):
    if not isinstance(location, str) or not location.startswith("blackwell"):
        return None
    import torch_musa_b200 as bw

    idx = _validate_index(location)
    bw._lazy_init()
    if (
        bw._C._unified_cpu_allocator_enabled()
        and obj.device.type == "cpu"
        and obj.nbytes() > 0
        and bw._C._is_managed_ptr(obj.data_ptr())
    ):
        # managed host memory is device-visible: relabel the same bytes as a device storage
        return bw._C._managed_storage_to_device(obj, idx)
    with bw.device(idx):
        return obj.to(device=f"blackwell:{idx}")


def install() -> None:
    global _installed
    if _installed:
        return
    torch.serialization.register_package(11, _tag, _deserialize)
    _installed = True
