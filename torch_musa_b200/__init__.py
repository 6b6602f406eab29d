"""torch_musa_b200: a Blackwell-native (NVIDIA B200, sm_100a) PyTorch device backend.

Importing this package

* names PyTorch's ``PrivateUse1`` dispatch key ``"blackwell"`` (``torch.device("blackwell:0")``),
* loads the native runtime ``_C`` (device guard, stream pool, caching allocators, hooks,
  generator, hand-written sm_100a kernels registered as ATen operators, process-group backend),
* installs this package as ``torch.blackwell`` -- the mirror of ``torch.cuda`` for this device --
  and adds ``Tensor.blackwell()``, ``Tensor.is_blackwell``, ``Module.blackwell()``,
  ``UntypedStorage.blackwell()``,
* registers serialization (``blackwell:N`` tags, ``cuda:N`` checkpoints load onto the device),
  AMP autocast, the ``"bccl"`` collective backend and the torch.compile integration.

Nothing touches a GPU until the first tensor or ``torch.blackwell.init()``; the import works on a
host without any GPU (``torch.blackwell.is_available()`` is then False).

Parity: reference torch_musa/__init__.py:43-262 (backend rename, module install, patches).
"""
from __future__ import annotations

import os
import sys
import warnings

import torch

__version__ = "0.1.0"

DEVICE_TYPE = "blackwell"

# ---------------------------------------------------------------------------
# 1. backend name (must happen before anything parses a "blackwell" device string)
try:
    torch.utils.rename_privateuse1_backend(DEVICE_TYPE)
except RuntimeError as _e:  # already renamed by a previous import of this package
    if torch._C._get_privateuse1_backend_name() != DEVICE_TYPE:
        raise RuntimeError(
            f"PrivateUse1 is already named {torch._C._get_privateuse1_backend_name()!r}; "
            "torch_musa_b200 cannot share a process with another PrivateUse1 backend"
        ) from _e

# ---------------------------------------------------------------------------
# 2. native runtime
import importlib as _importlib

_native = None
_native_error = None
try:
    _native = _importlib.import_module("._C", __name__)
except ImportError as _e:  # not built yet: build in-tree once, then retry
    _native_error = _e
    if os.environ.get("B200_NO_AUTOBUILD", "0") != "1" and not os.path.exists(
        os.path.join(os.path.dirname(__file__), "_C.so")
    ):
        try:
            from . import _build

            _build.build(verbose=False)
            _native = _importlib.import_module("._C", __name__)
            _native_error = None
        except Exception as _e2:  # pragma: no cover - depends on toolchain
            _native_error = _e2
_C = _native
if _C is None:
    raise ImportError(
        "torch_musa_b200: the native runtime (_C.so / libb200_kernels.so) is missing and could not be "
        f"built: {_native_error!r}. Run `python -m torch_musa_b200._build`."
    )

_C._register_hooks()

# ---------------------------------------------------------------------------
# 3. the torch.blackwell namespace (this very package)
from .core._lazy_init import (  # noqa: E402
    _lazy_init,
    _lazy_call,
    _is_in_bad_fork,
    init,
    is_initialized,
    is_available,
)
from .core.device import (  # noqa: E402
    device,
    device_of,
    set_device,
    current_device,
    device_count,
    synchronize,
    get_device_name,
    get_device_capability,
    get_device_properties,
    can_device_access_peer,
    get_arch_list,
    is_bf16_supported,
    is_tf32_supported,
    _exchange_device,
    _maybe_exchange_device,
    _DeviceGuard,
    _get_device_index,
    _sleep,
    set_sync_debug_mode,
    get_sync_debug_mode,
    current_blas_handle,
)
from .core.stream import (  # noqa: E402
    Stream,
    ExternalStream,
    Event,
    StreamContext,
    stream,
    set_stream,
    current_stream,
    default_stream,
    _set_stream_by_id,
    is_current_stream_capturing,
)
from .core.memory import (  # noqa: E402
    empty_cache,
    memory_stats,
    memory_stats_as_nested_dict,
    memory_stats_all,
    reset_accumulated_memory_stats,
    reset_peak_memory_stats,
    reset_max_memory_allocated,
    reset_max_memory_cached,
    memory_allocated,
    max_memory_allocated,
    memory_reserved,
    max_memory_reserved,
    memory_cached,
    max_memory_cached,
    memory_snapshot,
    memory_summary,
    mem_get_info,
    set_per_process_memory_fraction,
    get_per_process_memory_fraction,
    get_allocator_backend,
    _record_memory_history,
    _snapshot,
    _dump_snapshot,
    _set_allocator_settings,
    BlackwellPluggableAllocator,
    change_current_allocator,
    MemPool,
    get_pool_checkpoint,
    set_pool_checkpoint,
    adopt_allocation,
    MemPoolContext,
    use_mem_pool,
    use_unified_cpu_allocator,
    host_memory_stats,
    OutOfMemoryError,
    caching_allocator_alloc,
    caching_allocator_delete,
)
from .core.random import (  # noqa: E402
    get_rng_state,
    get_rng_state_all,
    set_rng_state,
    set_rng_state_all,
    manual_seed,
    manual_seed_all,
    seed,
    seed_all,
    initial_seed,
    default_generators,
)
from .core import amp  # noqa: E402
from .core.amp import get_amp_supported_dtype, amp_definitely_not_available  # noqa: E402
from .graphs import (  # noqa: E402
    BlackwellGraph,
    graph,
    graph_pool_handle,
    make_graphed_callables,
    update_graph_with_profile,
)
from .core import serialization as _serialization  # noqa: E402
from .core import attrs as _attrs  # noqa: E402

CUDAGraph = BlackwellGraph  # torch.cuda-style alias used by generic code

from .core.tensor_types import make_types as _make_tensor_types  # noqa: E402

globals().update(_make_tensor_types())  # FloatTensor, HalfTensor, BFloat16Tensor, ... (legacy typed classes)

from .core.monitoring import (  # noqa: E402
    clock_rate,
    cudart,
    current_blaslt_handle,
    get_gencode_flags,
    list_gpu_processes,
    make_storage_types as _make_storage_types,
    memory_usage,
    power_draw,
    temperature,
    utilization,
)

globals().update(_make_storage_types())  # FloatStorage, HalfStorage, ... (legacy typed storages)
runtime = cudart


from .core import reductions as _reductions  # noqa: E402

_reductions.init_reductions()


def ipc_collect():
    """Drop the references this process holds on tensors it sent to other processes and that every
    receiver has released since (received mappings close with their last tensor on their own)."""
    return _reductions.ipc_collect()


def fallback_counts():
    """Operators that ran on PyTorch's CUDA kernels (same memory) instead of a hand-written kernel."""
    return dict(_C._fallback_counts())


def reset_fallback_counts():
    _C._reset_fallback_counts()


def set_fallback_logging(level: int):
    """0 = silent, 1 = count, 2 = warn once per operator."""
    _C._set_fallback_logging(int(level))


def kernel_launch_count() -> int:
    """Number of hand-written sm_100a kernels launched by this process so far."""
    return int(_C._kernel_launch_count())


def reset_kernel_launch_count():
    _C._reset_kernel_launch_count()


def _is_compiled() -> bool:
    return True


torch._register_device_module(DEVICE_TYPE, sys.modules[__name__])
_attrs.install()
_serialization.install()
amp.install()

# ---------------------------------------------------------------------------
# 4. higher layers (each is importable on a CPU-only host)
from . import ops  # noqa: E402,F401  (custom ops: autograd + fake impls)
from . import optim  # noqa: E402,F401
from . import distributed  # noqa: E402,F401  (registers the "bccl" backend)
from . import _dynamo_inductor as _compile_glue  # noqa: E402

_compile_glue.install()

if os.environ.get("PYTORCH_BLACKWELL_ALLOC_CONF", "").find("cpu:unified") >= 0:
    # the CPU allocator swap needs a live runtime; it is applied at first device use
    _lazy_call(lambda: None)


# ---------------------------------------------------------------------------
# 5. torch.cuda-style conveniences that generic code probes for
PluggableAllocator = BlackwellPluggableAllocator
fork_rng = lambda devices=None, enabled=True, **kw: torch.random.fork_rng(  # noqa: E731
    devices=devices, enabled=enabled, device_type=DEVICE_TYPE, **kw)


class BlackwellError(RuntimeError):
    """A failed runtime call, with the runtime's error name and description."""


def check_error(res: int) -> None:
    """Raises if ``res`` (a runtime status code) is not success."""
    if int(res) != 0:
        raise BlackwellError(f"runtime call failed with status {int(res)}")


class _BCCL:
    """``torch.blackwell.bccl``: version of the collective library underneath the bccl backend."""

    @staticmethod
    def version():
        v = int(_C._nccl_version()) if hasattr(_C, "_nccl_version") else 0
        return (v // 10000, (v // 100) % 100, v % 100)

    @staticmethod
    def is_available(tensors=None) -> bool:
        return hasattr(_C, "_create_process_group")


bccl = _BCCL()


class _Backends:
    """``torch.backends.blackwell``: precision switches and library version, in the shape of ``torch.backends.cudnn``."""

    @property
    def allow_tf32(self) -> bool:
        return torch.backends.cuda.matmul.allow_tf32

    @allow_tf32.setter
    def allow_tf32(self, v: bool) -> None:
        torch.backends.cuda.matmul.allow_tf32 = bool(v)
        torch.backends.cudnn.allow_tf32 = bool(v)

    @staticmethod
    def is_available() -> bool:
        return is_available()

    @staticmethod
    def version():
        return tuple(int(x) for x in (torch.version.cuda or "0.0").split("."))

    @property
    def fft_plan_cache(self):
        """FFT plan caches, one per device (``[i].size``, ``[i].max_size``, ``[i].clear()``).  Transforms run as library
        FFTs over the same memory, so the cache that matters is the library's cache of the device with the same
        ordinal.  Parity: reference torch_musa/csrc/aten/mufft (plan cache of its FFT library)."""
        return torch.backends.cuda.cufft_plan_cache

    class flags:
        """Context manager that sets ``allow_tf32`` for a block."""

        def __init__(self, allow_tf32=None):
            self.allow_tf32, self._prev = allow_tf32, None

        def __enter__(self):
            self._prev = torch.backends.blackwell.allow_tf32
            if self.allow_tf32 is not None:
                torch.backends.blackwell.allow_tf32 = self.allow_tf32
            return self

        def __exit__(self, *exc):
            torch.backends.blackwell.allow_tf32 = self._prev
            return False


torch.backends.blackwell = _Backends()
if not hasattr(torch.version, DEVICE_TYPE):
    setattr(torch.version, DEVICE_TYPE, "sm_100a / CUDA " + str(torch.version.cuda))
from . import utils, profiler, testing  # noqa: E402,F401
from . import ao  # noqa: E402,F401  (publishes the fused SiLU blocks under torch.ao.nn.intrinsic*, adds the fusion rules)


def _autoload():
    """Entry point for torch's backend autoload (``torch.backends`` entry-point group)."""
    return None
