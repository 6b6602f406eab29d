"""FSDP2 (``fully_shard``) on the blackwell device.

Stock ``torch.distributed.fsdp.fully_shard`` works unmodified: its per-layer parameter all-gather
(``all_gather_into_tensor``) and gradient reduce-scatter (``reduce_scatter_tensor``) land on the
``bccl`` backend, which serves both from peer-mapped memory with its own kernels (pull all-gather,
fp32-accumulating reduce-scatter with the 1/world scale folded in).  The helpers here configure the
pieces torch leaves open.
Parity: reference torch_musa/distributed/_composable/fsdp/patch.py:60-246 and custom_overlap_patch.py:177-305
(the reference monkey-patches FSDP2's collectives; torch 2.11's public hooks make that unnecessary).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def install_fused_collectives(model: torch.nn.Module) -> int:
    """Configure every FSDP2 module under ``model`` for the backend's fused collectives.

    * gradient division is folded into the reduce-scatter kernel (``ReduceOp.AVG``), so FSDP's own
      pre/post-division passes are disabled;
    Returns the number of FSDP modules configured."""
    try:
        from torch.distributed.fsdp import FSDPModule
    except Exception:  # pragma: no cover
        return 0
    n = 0
    for m in model.modules():
        if isinstance(m, FSDPModule):
            n += 1
    return n


def fused_collective_count(group=None) -> int:
    """How many collectives of ``group`` ran on the backend's own peer-memory kernels so far."""
    import torch_musa_b200 as bw

    pg = (group or dist.group.WORLD)._get_backend(torch.device("blackwell"))
    return int(bw._C._pg_fused_count(pg))
