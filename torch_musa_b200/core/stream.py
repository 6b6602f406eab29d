"""Streams and events of ``torch.blackwell``.

``Stream`` and ``Event`` extend the device-generic ``torch.Stream`` / ``torch.Event``
(they go through the backend's registered device guard), adding the CUDA-style
extras: ``priority``, ``cuda_stream`` (raw ``cudaStream_t``), external streams,
IPC handles and ``priority_range``.
Parity: reference torch_musa/core/stream.py:18-344.
"""
from __future__ import annotations

import ctypes
from typing import Any, Optional

import torch

from ._lazy_init import _lazy_init, _C
from .device import _get_device_index, device as _device_ctx

class Stream(torch.Stream):
    """A stream of the blackwell device: an in-order queue of kernels and copies.

    ``priority``: 0 (default) or negative for higher priority (see ``Stream.priority_range``).
    Streams come from a per-device pool (32 per priority level) and are reused round-robin.
    """

    def __new__(cls, device=None, priority: int = 0, **kwargs):
        _lazy_init()
        if "stream_id" in kwargs and "device_index" in kwargs:
            kwargs.setdefault("device_type", _device_type_enum())
            return super().__new__(cls, **kwargs)
        if "stream_ptr" in kwargs:
            idx = _get_device_index(device, optional=True)
            sid, didx, dtype = _C()._stream_from_external(int(kwargs.pop("stream_ptr")), idx)
            return super().__new__(cls, stream_id=sid, device_index=didx, device_type=dtype)
        idx = _get_device_index(device, optional=True)
        sid, didx, dtype = _C()._stream_from_pool(int(priority), idx)
        return super().__new__(cls, stream_id=sid, device_index=didx, device_type=dtype)

    @property
    def priority(self) -> int:
        return _C()._stream_priority(self.stream_id, self.device_index)

    @staticmethod
    def priority_range():
        _lazy_init()
        return _C()._stream_priority_range()

    @property
    def cuda_stream(self) -> int:
        """The raw ``cudaStream_t`` as an integer (0 for the default stream)."""
        return _C()._stream_handle(self.stream_id, self.device_index)

    @property
    def _as_parameter_(self):
        return ctypes.c_void_p(self.cuda_stream)

    def wait_event(self, event) -> None:
        event.wait(self)

    def wait_stream(self, stream) -> None:
        self.wait_event(stream.record_event())

    def record_event(self, event=None):
        if event is None:
            event = Event()
        event.record(self)
        return event

    def synchronize(self) -> None:
        _C()._stream_synchronize(self.stream_id, self.device_index)

    def is_capturing(self) -> bool:
        return _C()._stream_is_capturing(self.stream_id, self.device_index)

    def __eq__(self, o) -> bool:
        if isinstance(o, torch.Stream):
            return (self.stream_id, self.device_index, self.device_type) == (o.stream_id, o.device_index, o.device_type)
        return False

    def __hash__(self):
        return hash((self.stream_id, self.device_index, self.device_type))

    def __repr__(self):
        return f"<torch.blackwell.Stream device={self.device} cuda_stream={self.cuda_stream:#x}>"


def _device_type_enum() -> int:
    """Numeric value of c10::DeviceType::PrivateUse1."""
    return _C()._device_type_enum()


class ExternalStream(Stream):
    """Wraps a ``cudaStream_t`` created elsewhere (no ownership is taken)."""

    def __new__(cls, stream_ptr: int, device=None, **kwargs):
        return super().__new__(cls, device=device, stream_ptr=stream_ptr)


class Event(torch.Event):
    """Device event: marks a point in a stream; used for timing and cross-stream ordering."""

    def __new__(cls, enable_timing: bool = False, blocking: bool = False, interprocess: bool = False):
        ev = super().__new__(cls, device="blackwell", enable_timing=enable_timing, blocking=blocking,
                             interprocess=interprocess)
        return ev

    def record(self, stream=None) -> None:
        if stream is None:
            stream = current_stream()
        super().record(stream)

    def wait(self, stream=None) -> None:
        if stream is None:
            stream = current_stream()
        super().wait(stream)

    def elapsed_time(self, end_event) -> float:
        """Milliseconds between this event and ``end_event`` (both created with ``enable_timing=True``)."""
        return _C()._event_elapsed_time(self.event_id, end_event.event_id)

    @classmethod
    def from_ipc_handle(cls, device, handle: bytes):
        return _C()._IpcEvent.from_ipc_handle(_get_device_index(device, optional=True), handle)

    def __repr__(self):
        return f"<torch.blackwell.Event {self.event_id:#x}>" if self.event_id else "<torch.blackwell.Event uninitialized>"


def _wrap(t) -> Stream:
    sid, didx, dtype = t
    return Stream(stream_id=sid, device_index=didx, device_type=dtype)


def current_stream(device: Any = None) -> Stream:
    _lazy_init()
    return _wrap(_C()._current_stream(_get_device_index(device, optional=True)))


def default_stream(device: Any = None) -> Stream:
    _lazy_init()
    return _wrap(_C()._default_stream(_get_device_index(device, optional=True)))


def _set_stream_by_id(stream_id: int, device_index: int, device_type: int) -> None:
    _C()._set_stream(stream_id, device_index, device_type)


def set_stream(stream: Optional[torch.Stream]) -> None:
    """Make ``stream`` current (and its device the selected device)."""
    if stream is None:
        return
    _lazy_init()
    _set_stream_by_id(stream.stream_id, stream.device_index, stream.device_type)


class StreamContext:
    """``with torch.blackwell.stream(s):`` -- run the body with ``s`` current on its device."""

    def __init__(self, stream: Optional[torch.Stream]):
        self.stream = stream
        self.idx = _get_device_index(None, optional=True) if stream is not None else -1
        self.src_prev_stream = None
        self.dst_prev_stream = None

    def __enter__(self):
        cur = self.stream
        if cur is None or self.idx == -1:
            return
        self.src_prev_stream = current_stream(None)
        if self.src_prev_stream.device_index != cur.device_index:
            with _device_ctx(cur.device_index):
                self.dst_prev_stream = current_stream(cur.device_index)
        set_stream(cur)

    def __exit__(self, *exc):
        cur = self.stream
        if cur is None or self.idx == -1:
            return False
        if self.src_prev_stream.device_index != cur.device_index:
            set_stream(self.dst_prev_stream)
        set_stream(self.src_prev_stream)
        return False


def stream(stream: Optional[torch.Stream]) -> StreamContext:
    return StreamContext(stream)


def is_current_stream_capturing() -> bool:
    """True while a graph capture is under way on the current stream."""
    from ._lazy_init import is_initialized

    if not is_initialized():
        return False
    return current_stream().is_capturing()
