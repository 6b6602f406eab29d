"""Registration of the ``"bccl"`` collective backend with ``torch.distributed``.

``dist.init_process_group("bccl")`` (or ``backend="cpu:gloo,blackwell:bccl"``) creates the native
process group: NCCL communicators (bootstrap, broadcast, barrier, gather/scatter, point-to-point,
and every collective by default) plus hand-written P2P kernels over peer-mapped symmetric memory
for the hot paths.  Parity: reference torch_musa/csrc/distributed/Register.cpp:75-209.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_registered = False


def is_bccl_available() -> bool:
    import torch_musa_b200 as bw

    return hasattr(bw._C, "_create_process_group")


def _create(dist_backend_opts, pg_options):
    import torch_musa_b200 as bw

    if not is_bccl_available():
        raise RuntimeError("the bccl backend was not compiled into torch_musa_b200._C")
    store = dist_backend_opts.store
    rank = dist_backend_opts.group_rank
    size = dist_backend_opts.group_size
    timeout = dist_backend_opts.timeout
    bw._lazy_init()
    return bw._C._create_process_group(store, rank, size, timeout, pg_options)


def register_backend() -> None:
    global _registered
    if _registered or not dist.is_available():
        return
    try:
        dist.Backend.register_backend("bccl", _create, extended_api=True, devices=["blackwell"])
    except Exception:  # already registered by an earlier import in this interpreter
        pass
    dist.is_bccl_available = is_bccl_available
    _registered = True
