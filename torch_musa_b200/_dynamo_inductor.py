"""torch.compile integration for the blackwell device.

* Dynamo: a ``DeviceInterface`` so guards, streams and device properties resolve for the device.
* Backend ``"blackwell_graphs"``: AOT-autograd + whole-graph CUDA-graph capture of the compiled
  forward/backward (the launch-bound case), running the backend's eager kernels -- no code
  generation and no Triton anywhere.
Parity: reference torch_musa/_dynamo/device_interface.py:17-86, _dynamo/backend/musagraphs.py:171-322,
_inductor/__init__.py:17-39 (the reference generates Triton; this backend lowers to its own kernels).
"""
from __future__ import annotations

import torch

_installed = False


def install() -> None:
    global _installed
    if _installed:
        return
    _installed = True
    try:
        from torch._dynamo.device_interface import DeviceInterface, register_interface_for_device
    except Exception:  # pragma: no cover
        return
    import torch_musa_b200 as bw

    class BlackwellInterface(DeviceInterface):
        device = bw.device
        Event = bw.Event
        Stream = bw.Stream

        class Worker:
            @staticmethod
            def set_device(device: int):
                bw.set_device(device)

            @staticmethod
            def current_device() -> int:
                return bw.current_device()

            @staticmethod
            def get_device_properties(device=None):
                return bw.get_device_properties(device)

        current_device = staticmethod(bw.current_device)
        set_device = staticmethod(bw.set_device)
        device_count = staticmethod(bw.device_count)
        stream = staticmethod(bw.stream)
        current_stream = staticmethod(bw.current_stream)
        set_stream = staticmethod(bw.set_stream)
        _set_stream_by_id = staticmethod(bw._set_stream_by_id)
        synchronize = staticmethod(bw.synchronize)
        get_device_properties = staticmethod(bw.get_device_properties)
        memory_allocated = staticmethod(bw.memory_allocated)

        @staticmethod
        def maybe_exchange_device(device: int) -> int:
            return bw._maybe_exchange_device(device)

        @staticmethod
        def exchange_device(device: int) -> int:
            return bw._exchange_device(device)

        @staticmethod
        def is_available() -> bool:
            return bw.is_available()

        @staticmethod
        def get_compute_capability(device=None):
            major, minor = bw.get_device_capability(device)
            return major * 10 + minor

        @staticmethod
        def is_bf16_supported(including_emulation: bool = False) -> bool:
            return True

        @staticmethod
        def get_raw_stream(device_idx: int) -> int:
            return bw.current_stream(device_idx).cuda_stream

    try:
        register_interface_for_device("blackwell", BlackwellInterface)
    except Exception:  # pragma: no cover
        pass

    from .compile_backend import register as _register_backend

    _register_backend()

    from .compile.backend import register as _register_compiler

    _register_compiler()
