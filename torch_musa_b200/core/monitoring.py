"""Read-only device telemetry and the remaining small pieces of the ``torch.cuda``-shaped surface:
utilisation / temperature / power / clocks (NVML, read only: nothing here changes a setting), the process list,
compile flags of the kernel library, the BLAS-Lt handle, a ``cudart()``-style runtime namespace, and the legacy typed
storage classes.

Parity: reference torch_musa/__init__.py:60-131 (`musart`, `current_blaslt_handle`, legacy `*Storage` types) and
torch_musa/core/device.py (device telemetry helpers).
"""
from __future__ import annotations

from typing import Any, List

import torch

from ._lazy_init import _lazy_init
from .device import _get_device_index


def _C():
    from .. import _C as C

    return C


def _nvml_handle(device: Any = None):
    try:
        import pynvml
    except ImportError as e:  # pragma: no cover
        raise ModuleNotFoundError("pynvml (nvidia-ml-py) is needed for device telemetry") from e
    try:
        pynvml.nvmlInit()
    except Exception as e:
        raise RuntimeError(f"the NVML library could not be initialised: {e}") from e
    idx = _get_device_index(device, optional=True)
    return pynvml, pynvml.nvmlDeviceGetHandleByIndex(idx)


def utilization(device: Any = None) -> int:
    """Percent of the last sample period during which a kernel was running."""
    nv, h = _nvml_handle(device)
    return int(nv.nvmlDeviceGetUtilizationRates(h).gpu)


def memory_usage(device: Any = None) -> int:
    """Percent of the last sample period during which device memory was read or written."""
    nv, h = _nvml_handle(device)
    return int(nv.nvmlDeviceGetUtilizationRates(h).memory)


def temperature(device: Any = None) -> int:
    """GPU temperature in degrees Celsius."""
    nv, h = _nvml_handle(device)
    return int(nv.nvmlDeviceGetTemperature(h, nv.NVML_TEMPERATURE_GPU))


def power_draw(device: Any = None) -> int:
    """Board power in milliwatts."""
    nv, h = _nvml_handle(device)
    return int(nv.nvmlDeviceGetPowerUsage(h))


def clock_rate(device: Any = None) -> int:
    """Current SM clock in MHz."""
    nv, h = _nvml_handle(device)
    return int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))


def list_gpu_processes(device: Any = None) -> str:
    nv, h = _nvml_handle(device)
    procs = nv.nvmlDeviceGetComputeRunningProcesses(h)
    lines = [f"GPU:{_get_device_index(device, optional=True)}"]
    if not procs:
        lines.append("no processes are running")
    for p in procs:
        mem = (p.usedGpuMemory or 0) / (1 << 20)
        lines.append(f"process {p.pid:>10d} uses {mem:>12.3f} MB GPU memory")
    return "\n".join(lines)


def get_gencode_flags() -> str:
    """nvcc flags the kernel library was built with."""
    arch = _C()._kernels_arch()            # "sm_100a"
    num = arch.split("_", 1)[1]
    return f"-gencode arch=compute_{num},code={arch}"


def current_blaslt_handle() -> int:
    """cuBLASLt handle of the current device (library GEMMs only; 16-bit products use the tcgen05 kernels)."""
    _lazy_init()
    from .device import current_device

    with torch.cuda.device(current_device()):
        getter = getattr(torch._C, "_cuda_getCurrentBlasLtHandle", None)
        return int(getter()) if getter is not None else int(torch.cuda.current_blas_handle())


class _Runtime:
    """The handful of CUDA-runtime calls user code reaches for through ``torch.cuda.cudart()``."""

    @staticmethod
    def cudaHostRegister(ptr: int, size: int, flags: int = 0) -> int:
        _C()._host_register(ptr, size)
        return 0

    @staticmethod
    def cudaHostUnregister(ptr: int) -> int:
        _C()._host_unregister(ptr)
        return 0

    @staticmethod
    def cudaMemGetInfo(device: int = 0):
        from .memory import mem_get_info

        return mem_get_info(device)

    @staticmethod
    def cudaProfilerStart() -> int:
        return int(torch.cuda.cudart().cudaProfilerStart())

    @staticmethod
    def cudaProfilerStop() -> int:
        return int(torch.cuda.cudart().cudaProfilerStop())

    @staticmethod
    def cudaDeviceSynchronize() -> int:
        from .device import synchronize

        synchronize()
        return 0


def cudart() -> _Runtime:
    _lazy_init()
    return _Runtime()


# ---------------------------------------------------------------- legacy typed storages
class _classproperty:
    def __init__(self, fn):
        self.fn = fn

    def __get__(self, obj, owner):
        return self.fn(owner)


class _LegacyStorageBase(torch.storage._LegacyStorage):
    """``torch.blackwell.FloatStorage(n)``-style constructors (deprecated in torch, kept for old checkpoints and
    scripts): a typed view of an untyped device storage."""

    @classmethod
    def from_buffer(cls, *args, **kwargs):
        raise RuntimeError("from_buffer: not available for blackwell storage")

    def __new__(cls, *args, **kwargs):
        if cls is _LegacyStorageBase:
            raise RuntimeError("only the typed subclasses can be instantiated")
        if len(args) == 1 and isinstance(args[0], int) and not kwargs:
            n = args[0]
        elif not args and not kwargs:
            n = 0
        else:
            raise TypeError(f"{cls.__name__}(size) is the only supported constructor on this device")
        elem = torch.empty((), dtype=cls.dtype).element_size()
        untyped = torch.UntypedStorage(n * elem, device="blackwell")
        return torch.TypedStorage(wrap_storage=untyped, dtype=cls.dtype, _internal=True)

    @classmethod
    def _new_shared(cls, *args, **kwargs):
        raise RuntimeError("use torch.multiprocessing queues to share device tensors between processes")


def make_storage_types() -> dict:
    table = {"Float": torch.float32, "Double": torch.float64, "Half": torch.float16, "BFloat16": torch.bfloat16,
             "Long": torch.int64, "Int": torch.int32, "Short": torch.int16, "Char": torch.int8, "Byte": torch.uint8,
             "Bool": torch.bool, "ComplexFloat": torch.complex64, "ComplexDouble": torch.complex128}
    out = {}
    for name, dt in table.items():
        out[name + "Storage"] = type(name + "Storage", (_LegacyStorageBase,),
                                     {"dtype": _classproperty(lambda cls, _dt=dt: _dt),
                                      "__module__": "torch_musa_b200"})
    return out
