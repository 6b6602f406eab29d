"""Pickling of device tensors and events for ``torch.multiprocessing`` queues and pipes.

A tensor is sent as a description of where its storage lives (the cudaIpc handle of its
segment, or the file descriptors of its memory chunks when expandable segments are on) and is
rebuilt in the receiving process as a view of the same device memory.  The sender keeps the
tensor alive until the receiver lets go of it: every shared storage has a reference counter in
a small file under ``/dev/shm`` that the receiver's storage decrements when it is freed, and
``ipc_collect()`` (also run on every send) drops the sender-side references whose counter is
back to zero.

Parity: reference torch_musa/core/reductions.py:1-17 (event pickling) and
torch_musa/csrc/core/StorageSharing.cpp:63-323, MusaIPCTypes.cpp:25-57 (storage sharing, limbo).
"""
from __future__ import annotations

import atexit
import itertools
import os
import threading
from multiprocessing.reduction import DupFd, ForkingPickler

import torch

_lock = threading.Lock()
_sent = {}          # counter path -> tensor kept alive for the receiver
_seq = itertools.count()
_installed = False


def _C():
    from .. import _C as C

    return C


def _counter_path() -> str:
    return f"/dev/shm/b200_ipc_{os.getpid()}_{next(_seq)}"


def ipc_collect() -> int:
    """Drop the sender-side references of shared tensors that every receiver has released.
    Returns how many are still held."""
    with _lock:
        for path in list(_sent):
            try:
                n = _C()._ipc_counter_add(path, 0)
            except RuntimeError:
                n = 0
            if n <= 0:
                del _sent[path]
                _C()._ipc_counter_unlink(path)
        return len(_sent)


def _cleanup():
    for path in list(_sent):
        try:
            os.unlink(path)
        except OSError:
            pass
    _sent.clear()


def rebuild_tensor(cls, size, stride, offset, dtype, requires_grad, info):
    C = _C()
    if info["pid"] == os.getpid():
        # sent to ourselves (a queue read by the sending process): the memory is already mapped here
        with _lock:
            base = _sent.get(info["counter"])
        if base is None:
            raise RuntimeError("the shared tensor was already released by its sender")
        u8 = base
        C._ipc_counter_add(info["counter"], -1)
        storage = u8.untyped_storage()
    else:
        if info["kind"] == "ipc":
            u8 = C._open_shared_ipc(info["device"], info["handle"], info["offset"], info["nbytes"], info["counter"])
        else:
            fds = [f.detach() for f in info["fds"]]
            u8 = C._open_shared_fds(info["device"], fds, info["chunk_bytes"], info["offset"], info["nbytes"],
                                    info["counter"])
        storage = u8.untyped_storage()
    t = torch.empty((0,), dtype=dtype, device=u8.device).set_(storage, offset, size, stride)
    if cls is torch.nn.Parameter:
        t = torch.nn.Parameter(t, requires_grad=requires_grad)
    else:
        t.requires_grad_(requires_grad)
    return t


def reduce_tensor(t: torch.Tensor):
    if t.requires_grad and not t.is_leaf:
        raise RuntimeError("Cowardly refusing to serialize non-leaf tensor which requires_grad: detach() it first")
    ipc_collect()
    C = _C()
    info = dict(C._share_storage(t))
    if info["kind"] == "fd":
        raw = info["fds"]
        info["fds"] = [DupFd(fd) for fd in raw]   # duplicates; ours can go
        for fd in raw:
            os.close(fd)
    path = _counter_path()
    C._ipc_counter_create(path, 1)
    info["counter"] = path
    with _lock:
        _sent[path] = t.detach()
    cls = torch.nn.Parameter if isinstance(t, torch.nn.Parameter) else torch.Tensor
    return rebuild_tensor, (cls, tuple(t.size()), tuple(t.stride()), t.storage_offset(), t.dtype, t.requires_grad,
                            info)


def rebuild_event(device, handle):
    from .stream import Event

    return Event.from_ipc_handle(device, handle)


def reduce_event(event):
    return rebuild_event, (event.device_index, event.ipc_handle())


def init_reductions() -> None:
    """Route blackwell tensors through this module; every other tensor keeps torch's own reducer."""
    global _installed
    if _installed:
        return
    _installed = True
    import torch.multiprocessing.reductions as tr

    stock = tr.reduce_tensor

    def reduce(t):
        if t.device.type == "blackwell":
            return reduce_tensor(t)
        return stock(t)

    for cls in (torch.Tensor, torch.nn.Parameter):
        ForkingPickler.register(cls, reduce)
    try:
        ForkingPickler.register(_C()._IpcEvent, reduce_event)
    except Exception:  # pragma: no cover
        pass
    atexit.register(_cleanup)
