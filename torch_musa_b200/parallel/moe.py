"""Expert parallelism: token dispatch / combine for mixture-of-experts layers.

Two interchangeable implementations of the same contract

    recv, rows_per_local_expert, ctx = dispatch(x [T, d], idx [T, K])
    out [T, d]                      = combine(y [R, d], gates [T, K], ctx)

``recv`` holds the rows this rank's experts must process, grouped by local expert (all rows of local
expert 0, then expert 1, ...); ``y`` is what the experts computed for those rows, in the same order.
``rows_per_local_expert`` is a list, or -- fused exchange, the default -- an int32 device tensor: ``recv`` is then
the whole capacity-sized receive buffer and the grouped expert GEMMs (``ops.grouped_linear``) read the counts on
the device, so that no host synchronisation sits in the layer.

* ``FusedExpertExchange`` (blackwell device): the kernels of ``csrc/kernels/moe.cu``.  Dispatch is ONE
  kernel that exchanges the per-expert counts through peer memory, derives every row's destination and
  writes token rows straight into the destination GPU's receive buffer over NVLink; combine is ONE kernel
  that pulls the expert outputs back and applies the gate weights in registers.  No send buffer, no sort,
  no split-size all-to-all, and the backward passes are the mirrored kernels.
* ``ReferenceExpertExchange`` (any device / backend): sort by expert, ``all_to_all_single`` of split sizes
  and of the rows, re-sort by local expert -- what stock PyTorch code does.  It is the numerics oracle of
  the tests and the baseline arm of the benchmark.

Parity: the reference has no expert parallelism; its all_to_all is a loop of send/recv pairs
(reference torch_musa/csrc/distributed/ProcessGroupMCCL.cpp:4022-4117).
"""
from __future__ import annotations

import os

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist



def _group_info(group) -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


# ------------------------------------------------------------------------------------------------ reference
class ReferenceExpertExchange:
    """Sort + all_to_all_single implementation (differentiable through torch.distributed.nn)."""

    def __init__(self, num_experts: int, group=None):
        self.E = num_experts
        self.group = group
        self.rank, self.world = _group_info(group)
        assert num_experts % self.world == 0
        self.E_local = num_experts // self.world

    def _a2a(self, t, out_splits, in_splits):
        if self.world == 1:
            return t
        from torch.distributed.nn.functional import all_to_all_single

        out = t.new_empty((sum(out_splits),) + tuple(t.shape[1:]))
        return all_to_all_single(out, t, out_splits, in_splits, group=self.group)

    def dispatch(self, x: torch.Tensor, idx: torch.Tensor, slot: int = 0):
        T, K = idx.shape
        flat = idx.reshape(-1).long()
        order = torch.argsort(flat, stable=True)                       # pairs sorted by global expert
        counts = torch.bincount(flat, minlength=self.E)
        send = x[order // K]
        if self.world > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.group)   # [W, E_local]: rows from source s for my expert j
        else:
            recv_counts = counts
        in_splits = counts.view(self.world, self.E_local).sum(1).tolist()
        rc = recv_counts.view(self.world, self.E_local)
        out_splits = rc.sum(1).tolist()
        recv = self._a2a(send, out_splits, in_splits)                   # grouped by source rank, then local expert
        # regroup by local expert, sources in rank order inside an expert
        rc_l = rc.tolist()
        seg_expert = torch.tensor([j for s in range(self.world) for j in range(self.E_local)], device=recv.device)
        seg_len = torch.tensor([rc_l[s][j] for s in range(self.world) for j in range(self.E_local)], device=recv.device)
        row_expert = torch.repeat_interleave(seg_expert, seg_len)
        regroup = torch.argsort(row_expert, stable=True)
        rows_per_expert = rc.sum(0).tolist()
        ctx = (order, regroup, in_splits, out_splits, T, K)
        return recv[regroup], rows_per_expert, ctx

    def expert_buffers(self, slot: int = 0):
        """(output buffer, input-gradient buffer) the expert GEMMs may write into directly: none here."""
        return None, None

    def combine(self, y: torch.Tensor, gates: torch.Tensor, ctx, slot: int = 0) -> torch.Tensor:
        order, regroup, in_splits, out_splits, T, K = ctx
        back = torch.empty_like(y)
        back = back.index_copy(0, regroup, y)                           # undo the regrouping
        ret = self._a2a(back, in_splits, out_splits)                    # rows return to their source, expert-sorted
        pair = torch.empty_like(ret).index_copy(0, order, ret)          # undo the expert sort: pair order (t, k)
        pair = pair.view(T, K, -1)
        return (pair.float() * gates.unsqueeze(-1).float()).sum(1).to(y.dtype)


# ------------------------------------------------------------------------------------------------ fused
class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx, ex, slot):
        sm = ex.sm
        slots, counts = sm.moe_count(idx, ex.E)
        pos, recv_counts = sm.moe_dispatch(x, idx, slots, counts, ex.E, ex.cap_rows, ex.recv_off(slot), 0)
        ctx.ex, ctx.T, ctx.d = ex, x.shape[0], x.shape[1]
        ctx.save_for_backward(idx, pos)
        ctx.mark_non_differentiable(pos, recv_counts)
        return pos, recv_counts

    @staticmethod
    def backward(ctx, _dpos, _dcounts):
        return None, None, None, None


class _Receive(torch.autograd.Function):
    """The received rows as an autograd node: its backward returns the gradient rows to their source tokens."""

    @staticmethod
    def forward(ctx, x, idx, pos, ex, slot, rows):
        ctx.ex, ctx.rows = ex, rows
        ctx.save_for_backward(idx, pos)
        return ex.recv_view(slot)[:rows]

    @staticmethod
    def backward(ctx, d_recv):
        ex = ctx.ex
        idx, pos = ctx.saved_tensors
        if d_recv.data_ptr() != ex.drecv_view().data_ptr():       # the grouped input-gradient GEMM wrote it in place
            ex.drecv_view()[: ctx.rows].copy_(d_recv)
        dx = ex.sm.moe_gather(idx, pos, None, ex.d, ex.E, ex.drecv_off())
        return dx, None, None, None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, gates, idx, pos, ex, slot):
        rows = y.shape[0]
        if y.data_ptr() != ex.y_view(slot).data_ptr():             # the grouped down projection wrote it in place
            ex.y_view(slot)[:rows].copy_(y)
        out = ex.sm.moe_gather(idx, pos, gates, ex.d, ex.E, ex.y_off(slot))
        ctx.ex, ctx.slot, ctx.rows = ex, slot, rows
        ctx.save_for_backward(gates, idx, pos)
        return out

    @staticmethod
    def backward(ctx, d_out):
        ex = ctx.ex
        gates, idx, pos = ctx.saved_tensors
        d_out = d_out.contiguous()
        d_gates = ex.sm.moe_gather_dot(d_out, idx, pos, ex.E, ex.y_off(ctx.slot))
        ex.sm.moe_scatter(d_out, idx, pos, gates, ex.E, ex.dy_off())
        # with device-side counts the rows go to the expert GEMMs where they are (their consumers run before the
        # next layer's backward scatters into this buffer again: its input depends on them)
        d_y = ex.dy_view() if ctx.rows == ex.cap_rows else ex.dy_view()[: ctx.rows].clone()
        return d_y, d_gates, None, None, None, None


class FusedExpertExchange:
    """Peer-memory implementation; ``slots`` independent (receive, output) buffer pairs, one per MoE layer, so
    the rows a layer saved for its backward stay valid while later layers run."""

    def __init__(self, num_experts: int, d_model: int, cap_rows: int, slots: int = 1, group=None, device=None):
        import torch_musa_b200 as bw

        self.E, self.d, self.cap_rows, self.slots = num_experts, d_model, int(cap_rows), slots
        self.group = group
        self.host_counts = os.environ.get("B200_MOE_HOST_COUNTS", "0") == "1"
        self.rank, self.world = _group_info(group)
        assert num_experts % self.world == 0 and d_model % 8 == 0
        self.E_local = num_experts // self.world
        self.device = torch.device(device if device is not None else f"blackwell:{bw.current_device()}")
        self._region = (self.cap_rows * d_model * 2 + 255) // 256 * 256
        self._table = (self.world * num_experts * 4 + 255) // 256 * 256
        total = self._table + (2 * slots + 2) * self._region
        from torch_musa_b200.parallel._symm import group_store_and_key  # this file also loads stand-alone (no package)

        store, key = group_store_and_key(group, "moe_arena")
        self.sm = bw._C._create_symmetric_memory(store, key, self.rank, self.world, self.device.index or 0, total)
        if not self.sm.ok:
            raise RuntimeError(f"expert-parallel arena unavailable: {self.sm.why_not}")

    # ---- arena layout: [count table][recv slot 0][y slot 0][recv slot 1][y slot 1]...[dy][drecv]
    def recv_off(self, slot): return self._table + (2 * slot) * self._region
    def y_off(self, slot): return self._table + (2 * slot + 1) * self._region
    def dy_off(self): return self._table + (2 * self.slots) * self._region
    def drecv_off(self): return self._table + (2 * self.slots + 1) * self._region
    def _view(self, off): return self.sm.local_tensor(off, [self.cap_rows, self.d], torch.bfloat16)
    def recv_view(self, slot): return self._view(self.recv_off(slot))
    def y_view(self, slot): return self._view(self.y_off(slot))
    def dy_view(self): return self._view(self.dy_off())
    def drecv_view(self): return self._view(self.drecv_off())

    def dispatch(self, x: torch.Tensor, idx: torch.Tensor, slot: int = 0):
        """Returns (received rows, rows per local expert, context for `combine`).  By default the counts stay on
        the device (an int32 tensor; the received rows are the whole capacity-sized buffer and the grouped expert
        GEMMs read the counts themselves); ``host_counts`` brings them to the host as a list, which costs a
        synchronisation per layer."""
        idx32 = idx.to(torch.int32).contiguous()
        pos, recv_counts = _Dispatch.apply(x.contiguous(), idx32, self, slot)
        if not self.host_counts:
            recv = _Receive.apply(x, idx32, pos, self, slot, self.cap_rows)
            return recv, recv_counts, (idx32, pos)
        rows_per_expert = recv_counts.tolist()
        rows = min(sum(rows_per_expert), self.cap_rows)
        recv = _Receive.apply(x, idx32, pos, self, slot, rows)
        return recv, rows_per_expert, (idx32, pos)

    def expert_buffers(self, slot: int = 0):
        """(output buffer, input-gradient buffer) for the grouped expert GEMMs: this slot's combine source and the
        buffer the dispatch backward gathers from."""
        if self.host_counts:
            return None, None
        return self.y_view(slot), self.drecv_view()

    def combine(self, y: torch.Tensor, gates: torch.Tensor, ctx, slot: int = 0) -> torch.Tensor:
        idx32, pos = ctx
        return _Combine.apply(y, gates.float().contiguous(), idx32, pos, self, slot)

    def check(self) -> None:
        st = self.sm.take_status()
        if st:
            raise RuntimeError(f"an expert-exchange kernel gave up on a bounded wait (status {st})")


def make_expert_exchange(num_experts: int, d_model: int, tokens_per_rank: int, top_k: int, slots: int = 1, group=None,
                         device=None, capacity_factor: float = 2.0):
    """The fused exchange on the blackwell device, the reference one elsewhere."""
    dev = torch.device(device) if device is not None else None
    if dev is not None and dev.type == "blackwell":
        _, world = _group_info(group)
        cap = int(capacity_factor * tokens_per_rank * top_k)
        return FusedExpertExchange(num_experts, d_model, cap, slots, group, dev)
    return ReferenceExpertExchange(num_experts, group)
