"""Memory management API of ``torch.blackwell`` (caching allocator statistics, snapshots,
memory fraction, pluggable / unified allocators, memory pools).
Parity: reference torch_musa/core/memory.py:61-657."""
from __future__ import annotations

import collections
import contextlib
import pickle
from typing import Any, Dict, Optional, Tuple, Union

import torch

from ._lazy_init import _lazy_init, is_initialized, _C
from .device import _get_device_index

OutOfMemoryError = torch.OutOfMemoryError


def empty_cache() -> None:
    """Return every cached, unused segment to the driver (both this backend's pools and the pool that
    serves long-tail operators)."""
    if is_initialized():
        _C()._empty_cache(-1)


def memory_stats_as_nested_dict(device: Any = None) -> Dict[str, Any]:
    if not is_initialized():
        return {}
    return _C()._memory_stats(_get_device_index(device, optional=True))


def memory_stats(device: Any = None) -> Dict[str, Any]:
    """Flat ``{"allocated_bytes.all.current": ...}`` dictionary, same keys as ``torch.cuda.memory_stats``."""
    result = []

    def _recurse(prefix, obj):
        if isinstance(obj, dict):
            if len(prefix) > 0:
                prefix += "."
            for k, v in obj.items():
                _recurse(prefix + k, v)
        else:
            result.append((prefix, obj))

    _recurse("", memory_stats_as_nested_dict(device))
    result.sort()
    return collections.OrderedDict(result)


def memory_stats_all() -> Dict[int, Dict[str, Any]]:
    return {i: memory_stats(i) for i in range(_C()._device_count())}


def reset_accumulated_memory_stats(device: Any = None) -> None:
    _C()._reset_accumulated_memory_stats(_get_device_index(device, optional=True))


def reset_peak_memory_stats(device: Any = None) -> None:
    _C()._reset_peak_memory_stats(_get_device_index(device, optional=True))


reset_max_memory_allocated = reset_peak_memory_stats
reset_max_memory_cached = reset_peak_memory_stats


def memory_allocated(device: Any = None) -> int:
    return memory_stats(device).get("allocated_bytes.all.current", 0)


def max_memory_allocated(device: Any = None) -> int:
    return memory_stats(device).get("allocated_bytes.all.peak", 0)


def memory_reserved(device: Any = None) -> int:
    return memory_stats(device).get("reserved_bytes.all.current", 0)


def max_memory_reserved(device: Any = None) -> int:
    return memory_stats(device).get("reserved_bytes.all.peak", 0)


memory_cached = memory_reserved
max_memory_cached = max_memory_reserved


def mem_get_info(device: Any = None) -> Tuple[int, int]:
    """(free, total) bytes of the device as the driver sees them."""
    _lazy_init()
    return tuple(_C()._mem_get_info(_get_device_index(device, optional=True)))


def set_per_process_memory_fraction(fraction: float, device: Any = None) -> None:
    _lazy_init()
    if not isinstance(fraction, float):
        raise TypeError("Invalid type for fraction argument, must be `float`")
    if fraction < 0 or fraction > 1:
        raise ValueError(f"Invalid fraction value: {fraction}. Allowed range: 0~1")
    _C()._set_memory_fraction(fraction, _get_device_index(device, optional=True))


def get_per_process_memory_fraction(device: Any = None) -> float:
    return _C()._get_memory_fraction(_get_device_index(device, optional=True))


def get_allocator_backend() -> str:
    return _C()._allocator_backend()


def _set_allocator_settings(env: str) -> None:
    _C()._set_allocator_settings(env)


def memory_snapshot(device: Any = None):
    """List of segments with their blocks (state of the caching allocator)."""
    if not is_initialized():
        return []
    return _C()._snapshot(-1 if device is None else _get_device_index(device))


def _record_memory_history(enabled: Optional[Union[str, bool]] = "all", max_entries: int = 100000,
                           stacks: Optional[str] = None, **kwargs) -> None:
    """Start/stop recording allocator events (alloc/free/segment/oom) into a ring buffer.  ``stacks="cpp"`` (or
    ``"all"``) also stores the symbolised C++ frames of every allocation site in the trace (key ``frames``)."""
    _lazy_init()
    _C()._record_memory_history(bool(enabled) and enabled != "none", int(max_entries), stacks in ("cpp", "all"))


def _snapshot(device: Any = None) -> Dict[str, Any]:
    segs = memory_snapshot(device)
    traces = [_C()._trace(i) for i in range(_C()._device_count())] if is_initialized() else []
    return {"segments": segs, "device_traces": traces, "allocator_settings": _C()._allocator_config()}


def _dump_snapshot(filename: str = "dump_snapshot.pickle") -> None:
    with open(filename, "wb") as f:
        pickle.dump(_snapshot(), f)


def _format_size(sz: int) -> str:
    for unit in ("B  ", "KiB", "MiB", "GiB", "TiB"):
        if abs(sz) < 1024 * 10 or unit == "TiB":
            return f"{sz:6d} {unit}"
        sz //= 1024
    return str(sz)


def memory_summary(device: Any = None, abbreviated: bool = False) -> str:
    """Human-readable table of the allocator statistics."""
    idx = _get_device_index(device, optional=True)
    st = memory_stats(idx)
    rows = [
        ("Allocated memory", "allocated_bytes", True),
        ("Active memory", "active_bytes", True),
        ("Requested memory", "requested_bytes", True),
        ("Reserved memory", "reserved_bytes", True),
        ("Non-releasable memory", "inactive_split_bytes", True),
        ("Allocations", "allocation", False),
        ("Active allocs", "active", False),
        ("Reserved segments", "segment", False),
        ("Non-releasable allocs", "inactive_split", False),
    ]
    lines = ["=" * 75, f" {'blackwell memory summary, device ID ' + str(idx):^73} ", "-" * 75,
             f"  OOMs: {st.get('num_ooms', 0):<12d} |  device malloc retries: {st.get('num_alloc_retries', 0):<8d}", "=" * 75,
             f"{'Metric':<24}|{'Cur Usage':>12}|{'Peak Usage':>12}|{'Tot Alloc':>12}|{'Tot Freed':>12}", "-" * 75]
    for title, key, is_bytes in rows:
        pools = [("all", title)] if abbreviated else [("all", title), ("large_pool", "      from large pool"), ("small_pool", "      from small pool")]
        for pool, name in pools:
            vals = [st.get(f"{key}.{pool}.{f}", 0) for f in ("current", "peak", "allocated", "freed")]
            fmt = (lambda v: _format_size(v)) if is_bytes else (lambda v: f"{v:10d}")
            lines.append(f"{name:<24}|" + "|".join(f"{fmt(v):>12}" for v in vals))
        lines.append("-" * 75)
    lines.append("=" * 75)
    return "\n".join(lines) + "\n"


def caching_allocator_alloc(size: int, device: Any = None, stream=None) -> int:
    """Raw allocation from the caching allocator; returns the device address."""
    _lazy_init()
    idx = _get_device_index(device, optional=True)
    if stream is None:
        from .stream import current_stream

        stream = current_stream(idx)
    handle = stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)
    return _C()._raw_alloc(int(size), idx, handle)


def caching_allocator_delete(mem_ptr: int) -> None:
    _C()._raw_delete(int(mem_ptr))


def host_memory_stats() -> Dict[str, int]:
    """Statistics of the caching pinned-host allocator."""
    return dict(_C()._host_stats())


class BlackwellPluggableAllocator:
    """Allocator backed by ``malloc``/``free`` functions of a user shared library.

    The functions must have the C signatures
    ``void* alloc(size_t size, int device, cudaStream_t stream)`` and
    ``void free(void* ptr, size_t size, int device, cudaStream_t stream)``.
    """

    def __init__(self, path_to_so_file: str, alloc_fn_name: str, free_fn_name: str):
        self._path, self._alloc, self._free = path_to_so_file, alloc_fn_name, free_fn_name


def change_current_allocator(allocator: BlackwellPluggableAllocator) -> None:
    """Install ``allocator`` for the device. Must run before the first allocation."""
    _C()._install_pluggable_allocator(allocator._path, allocator._alloc, allocator._free)


class MemPool:
    """A private memory pool of the caching allocator; ``id`` is unique and monotonically increasing."""

    def __init__(self, allocator=None):
        self._id = tuple(_C()._new_mempool_id(True))
        self._allocator = allocator

    @property
    def id(self) -> Tuple[int, int]:
        return self._id

    @property
    def allocator(self):
        return self._allocator

    def use_count(self) -> int:
        from .device import current_device

        return _C()._pool_use_count(current_device(), self._id) if is_initialized() else 0

    def snapshot(self):
        return [s for s in memory_snapshot() if tuple(s["segment_pool_id"]) == self._id]


def get_pool_checkpoint(device: Any, pool_id: Tuple[int, int]):
    """Block layout of a private pool right now (``.live_pointers`` lists its live allocations)."""
    _lazy_init()
    return _C()._checkpoint_pool(_get_device_index(device, optional=True), tuple(pool_id))


def set_pool_checkpoint(device: Any, state, stale=()):
    """Put a private pool back into the layout of ``state``.  Everything allocated in the pool since is
    taken back (pass the tensors that still point there as ``stale`` so that they give up ownership) and
    what was live at the checkpoint is live again at the same addresses.  Returns ``(freed, created)``
    pointer lists; ``adopt_allocation`` turns a created pointer that no tensor owns into a byte tensor."""
    _lazy_init()
    return _C()._restore_pool(_get_device_index(device, optional=True), state, list(stale))


def adopt_allocation(device: Any, ptr: int, nbytes: int):
    _lazy_init()
    return _C()._adopt_allocation(_get_device_index(device, optional=True), ptr, nbytes)


class MemPoolContext:
    """Stack of active pools, thread local (introspection only)."""

    import threading as _threading

    _tls = _threading.local()

    def __init__(self, pool: MemPool):
        self.pool = pool
        self.prev = None

    def __enter__(self):
        self.prev = getattr(MemPoolContext._tls, "active", None)
        MemPoolContext._tls.active = self.pool
        return self

    def __exit__(self, *exc):
        MemPoolContext._tls.active = self.prev
        return False

    @staticmethod
    def active_pool() -> Optional[MemPool]:
        return getattr(MemPoolContext._tls, "active", None)


@contextlib.contextmanager
def use_mem_pool(pool: MemPool, device: Any = None):
    """Route allocations made on the current stream inside the block to ``pool``."""
    _lazy_init()
    idx = _get_device_index(device, optional=True)
    ctx = MemPoolContext(pool)
    ctx.__enter__()
    _C()._begin_allocate_to_pool(idx, pool.id)
    try:
        yield
    finally:
        _C()._end_allocate_to_pool(idx, pool.id)
        _C()._release_pool(idx, pool.id)
        ctx.__exit__(None, None, None)


@contextlib.contextmanager
def use_unified_cpu_allocator():
    """Inside the block CPU tensors are allocated in managed (unified) memory, so a checkpoint loaded with
    ``map_location="blackwell"`` is retagged to the device without a second allocation or a copy."""
    _lazy_init()
    prev = _C()._unified_cpu_allocator_enabled()
    _C()._set_unified_cpu_allocator(True)
    try:
        yield
    finally:
        _C()._set_unified_cpu_allocator(prev)
