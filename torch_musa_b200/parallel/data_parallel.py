"""Single-process multi-device helpers in the shape of ``torch.nn.parallel.comm``: ``broadcast_coalesced``, ``scatter``,
``gather`` and ``reduce_add`` over device-to-device copies, plus a small ``DataParallel`` that replicates a module over
the visible blackwell devices, splits the batch, runs the replicas on their own streams and gathers the outputs.
Meant for quick experiments; multi-process DDP (``parallel/ddp.py``) is the performance path.
Parity: reference torch_musa/csrc/core/PythonComm.cpp:14-67 and its patches of torch/nn/parallel/{comm,_functions}.py.
"""
from __future__ import annotations

import copy
from typing import List, Optional, Sequence

import torch


def _dev(d) -> torch.device:
    if isinstance(d, int):
        return torch.device("blackwell", d)
    return torch.device(d)


def broadcast(tensor: torch.Tensor, devices: Sequence) -> List[torch.Tensor]:
    return [tensor if tensor.device == _dev(d) else tensor.to(_dev(d), non_blocking=True) for d in devices]


def broadcast_coalesced(tensors: Sequence[torch.Tensor], devices: Sequence, buffer_size: int = 10 << 20) -> List[List[torch.Tensor]]:
    """Copies ``tensors`` to every device, packing small tensors of one dtype into buffers of ``buffer_size`` bytes so
    that each device receives a few large copies instead of many small ones."""
    out: List[List[Optional[torch.Tensor]]] = [[None] * len(tensors) for _ in devices]
    groups = {}
    for i, t in enumerate(tensors):
        groups.setdefault(t.dtype, []).append(i)
    for dtype, idxs in groups.items():
        chunk, size = [], 0
        batches = []
        for i in idxs:
            n = tensors[i].numel() * tensors[i].element_size()
            if chunk and size + n > buffer_size:
                batches.append(chunk)
                chunk, size = [], 0
            chunk.append(i)
            size += n
        if chunk:
            batches.append(chunk)
        for batch in batches:
            flat = torch.cat([tensors[i].reshape(-1) for i in batch])
            for di, d in enumerate(devices):
                f = flat if flat.device == _dev(d) else flat.to(_dev(d), non_blocking=True)
                off = 0
                for i in batch:
                    n = tensors[i].numel()
                    out[di][i] = f[off:off + n].view_as(tensors[i])
                    off += n
    return out  # type: ignore[return-value]


def scatter(tensor: torch.Tensor, devices: Sequence, chunk_sizes: Optional[Sequence[int]] = None, dim: int = 0) -> List[torch.Tensor]:
    chunks = tensor.split(list(chunk_sizes), dim) if chunk_sizes is not None else tensor.chunk(len(devices), dim)
    return [c.to(_dev(d), non_blocking=True) for c, d in zip(chunks, devices)]


def gather(tensors: Sequence[torch.Tensor], dim: int = 0, destination=None) -> torch.Tensor:
    dst = _dev(destination) if destination is not None else tensors[0].device
    return torch.cat([t.to(dst, non_blocking=True) for t in tensors], dim)


def reduce_add(tensors: Sequence[torch.Tensor], destination=None) -> torch.Tensor:
    dst = _dev(destination) if destination is not None else tensors[0].device
    acc = tensors[0].to(dst).clone()
    for t in tensors[1:]:
        acc += t.to(dst, non_blocking=True)
    return acc


class DataParallel(torch.nn.Module):
    def __init__(self, module: torch.nn.Module, device_ids: Optional[Sequence[int]] = None, output_device=None, dim: int = 0):
        super().__init__()
        import torch_musa_b200 as bw

        self.module, self.dim = module, dim
        self.device_ids = list(device_ids) if device_ids is not None else list(range(max(bw.device_count(), 1)))
        self.output_device = output_device if output_device is not None else self.device_ids[0]

    def forward(self, *inputs):
        import torch_musa_b200 as bw

        if len(self.device_ids) == 1:
            return self.module(*inputs)
        replicas = [self.module] + [copy.deepcopy(self.module).to(_dev(d)) for d in self.device_ids[1:]]
        shards = [scatter(x, self.device_ids, dim=self.dim) if isinstance(x, torch.Tensor) else [x] * len(self.device_ids)
                  for x in inputs]
        outs = []
        for i, (rep, d) in enumerate(zip(replicas, self.device_ids)):
            with bw.device(d):
                outs.append(rep(*[s[i] for s in shards]))
        return gather(outs, self.dim, self.output_device)
