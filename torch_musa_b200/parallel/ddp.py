"""DistributedDataParallel on the blackwell device.

DDP's reducer hands each full gradient bucket (25 MiB by default) to a communication hook.  The
hooks here issue ONE collective per bucket with ``ReduceOp.AVG``: on the ``bccl`` backend that is the
two-shot peer-memory kernel which sums the ranks' slices in fp32, applies the 1/world scale and the
output cast in registers and writes the result back -- no separate division or cast kernel, and it
runs on the communication stream while backward keeps producing the next bucket.
Parity: reference docs/markdown/source/04_quick_start.md:215-263 (DDP over the vendor all-reduce) and
tests/unittest/distributed/test_distributed.py:38-67.
"""


from typing import Optional

import torch
import torch.distributed as dist


def _backend_supports_avg(group) -> bool:
    try:
        return dist.get_backend(group) in ("bccl", "nccl")
    except Exception:
        return False


def fused_allreduce_hook(state: Optional[object], bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Average the bucket across ranks with a single (fused scale) all-reduce."""
    group = state if isinstance(state, dist.ProcessGroup) else dist.group.WORLD
    buf = bucket.buffer()
    if _backend_supports_avg(group):
        fut = dist.all_reduce(buf, op=dist.ReduceOp.AVG, group=group, async_op=True).get_future()
        return fut.then(lambda f: f.value()[0])
    world = dist.get_world_size(group)
    fut = dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group, async_op=True).get_future()
    return fut.then(lambda f: f.value()[0].div_(world))


def bf16_compress_fused_hook(state: Optional[object], bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Communicate the bucket in bf16 (half the NVLink bytes), accumulate in fp32 inside the kernel."""
    group = state if isinstance(state, dist.ProcessGroup) else dist.group.WORLD
    buf = bucket.buffer()
    comp = buf.to(torch.bfloat16)
    op = dist.ReduceOp.AVG if _backend_supports_avg(group) else dist.ReduceOp.SUM
    world = dist.get_world_size(group)
    fut = dist.all_reduce(comp, op=op, group=group, async_op=True).get_future()

    def done(f):
        out = f.value()[0]
        buf.copy_(out)
        if op == dist.ReduceOp.SUM:
            buf.div_(world)
        return buf

    return fut.then(done)


def wrap_ddp(module: torch.nn.Module, device_ids=None, bucket_cap_mb: int = 25, process_group=None,
             compress_bf16: bool = False, **kwargs) -> torch.nn.parallel.DistributedDataParallel:
    """``DistributedDataParallel`` with the fused bucket hook installed."""
    ddp = torch.nn.parallel.DistributedDataParallel(module, device_ids=device_ids, bucket_cap_mb=bucket_cap_mb,
                                                    process_group=process_group, **kwargs)
    ddp.register_comm_hook(process_group, bf16_compress_fused_hook if compress_bf16 else fused_allreduce_hook)
    return ddp
