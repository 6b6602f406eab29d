"""Lazy initialisation of the blackwell runtime.

Nothing touches the GPU at import.  The first device use (torch's own
``device_lazy_init`` looks up ``torch.blackwell._lazy_init``) initialises the
runtime, then drains calls queued before init (seeds, for example).  A process
forked after init must not touch the device again: the child is "poisoned" and
raises a clear error (use the spawn start method).
Parity: reference torch_musa/core/_lazy_init.py:26-137.
"""
from __future__ import annotations

import threading
import traceback
from typing import Callable, List, Tuple

import torch

_initialized = False
_tls = threading.local()
_init_lock = threading.Lock()
_queued_calls: List[Tuple[Callable[[], None], List[str]]] = []


def _C():
    import torch_musa_b200

    return torch_musa_b200._C


def is_available() -> bool:
    """True when at least one B200-class CUDA device is visible."""
    return _C()._device_count() > 0


def is_initialized() -> bool:
    return _initialized and not _is_in_bad_fork()


def _is_in_bad_fork() -> bool:
    return _C()._is_in_bad_fork()


def _lazy_call(fn: Callable[[], None], **kwargs) -> None:
    """Run ``fn`` now if the runtime is up, else right after it comes up."""
    if is_initialized():
        fn()
        return
    _queued_calls.append((fn, traceback.format_stack()))


def init() -> None:
    """Initialise the runtime eagerly (normally implicit)."""
    _lazy_init()


def _lazy_init() -> None:
    global _initialized
    if is_initialized() or getattr(_tls, "is_initializing", False):
        return
    with _init_lock:
        if is_initialized():
            return
        if _is_in_bad_fork():
            raise RuntimeError(
                "Cannot re-initialize blackwell in forked subprocess. To use blackwell with multiprocessing, "
                "you must use the 'spawn' start method"
            )
        if not is_available():
            raise RuntimeError(
                "torch.blackwell: no device found (is a CUDA driver installed and a B200 visible? "
                "torch.blackwell.is_available() is False)"
            )
        _C()._init()
        _tls.is_initializing = True
        try:
            for fn, stack in _queued_calls:
                try:
                    fn()
                except Exception as e:  # pragma: no cover
                    raise RuntimeError(
                        f"blackwell call failed lazily at initialization with error: {e}\n\n"
                        f"call was originally invoked at:\n\n{''.join(stack)}"
                    ) from e
            _queued_calls.clear()
        finally:
            _tls.is_initializing = False
        _initialized = True
