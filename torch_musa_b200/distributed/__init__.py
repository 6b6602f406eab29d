"""Distributed layer: the ``"bccl"`` process-group backend for the blackwell device, symmetric
(peer-mapped) memory, fused collective kernels and the parallelism helpers built on them."""
from __future__ import annotations

from .backend import register_backend, is_bccl_available  # noqa: F401

register_backend()
