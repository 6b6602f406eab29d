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

    _install_trace_rules(bw)

    from .compile_backend import register as _register_backend

    _register_backend()

    from .compile.backend import register as _register_compiler

    _register_compiler()


# Functions of the device module that Dynamo may call while tracing and keep in the graph as calls (the same
# treatment torch.cuda's stream accessors get), and the autocast class it may enter as a context manager.
_IN_GRAPH_FUNCTIONS = ("current_stream", "default_stream", "stream")
# Queries whose answer Dynamo may bake into the graph as a constant (the second group under a guard that re-checks it),
# the treatment the same functions of torch.cuda get.
_CONSTANT_FUNCTIONS = ("is_available", "get_device_properties", "is_bf16_supported", "device_count")
_GUARDED_CONSTANT_FUNCTIONS = ("current_device", "is_initialized")


def _install_trace_rules(bw) -> None:
    """Parity: reference torch_musa/_dynamo/trace_rules.py:20-42 (in-graph functions) and
    torch_musa/_dynamo/variables/torch.py:7-13 (autocast as a supported context-manager class)."""
    try:
        from torch._dynamo import trace_rules
        from torch._dynamo.variables import TorchInGraphFunctionVariable
        from torch._dynamo.variables.torch import supported_ctx_manager_classes
    except Exception:  # pragma: no cover - Dynamo is optional in a PyTorch build
        return
    from torch._dynamo.variables import torch as torch_vars

    names = _IN_GRAPH_FUNCTIONS + _CONSTANT_FUNCTIONS + _GUARDED_CONSTANT_FUNCTIONS
    rules = {f"torch.blackwell.{name}": TorchInGraphFunctionVariable for name in names if hasattr(bw, name)}
    for name in _CONSTANT_FUNCTIONS + _GUARDED_CONSTANT_FUNCTIONS:
        torch_vars.constant_fold_functions[getattr(bw, name)] = None
    for name in _GUARDED_CONSTANT_FUNCTIONS:
        torch_vars.constant_fold_functions_need_guards[getattr(bw, name)] = None
    try:
        trace_rules.get_torch_obj_rule_map.cache_clear()          # the object -> rule map is built once and cached
        trace_rules.torch_name_rule_map[-1].update(rules)          # the table of Python (non C-binding) functions
    except Exception:  # pragma: no cover
        pass
    try:
        supported_ctx_manager_classes[bw.amp.autocast] = None
        _teach_autocast(bw)
    except Exception:  # pragma: no cover
        pass


def _teach_autocast(bw) -> None:
    """Dynamo models autocast regions with one variable class that is built from ``torch.autocast``'s arguments; the
    device module's ``autocast(enabled, dtype, cache_enabled)`` is translated into that form (device type fixed)."""
    import inspect

    from torch._dynamo.variables.ctx_manager import AutocastModeVariable
    from torch._dynamo.variables.torch import TorchCtxManagerClassVariable

    if getattr(TorchCtxManagerClassVariable.call_function, "_blackwell_autocast", False):
        return
    original = TorchCtxManagerClassVariable.call_function
    own_signature = inspect.signature(bw.amp.autocast)

    def call_function(self, tx, args, kwargs):
        if self.value is bw.amp.autocast:
            bound = own_signature.bind(*args, **kwargs)
            bound.apply_defaults()
            a = bound.arguments
            return AutocastModeVariable.create(
                torch.amp.autocast_mode.autocast, [],
                {"device_type": "blackwell", "dtype": a["dtype"], "enabled": a["enabled"], "cache_enabled": a["cache_enabled"]})
        return original(self, tx, args, kwargs)

    call_function._blackwell_autocast = True
    TorchCtxManagerClassVariable.call_function = call_function
