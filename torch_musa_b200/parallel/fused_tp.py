"""Fused tensor-parallel primitives on the blackwell device.

``FusedTensorParallel`` owns a peer-mapped arena for the activation shards and installs
``tensor_parallel.FUSED_AG_MATMUL``: all-gather -> GEMM as ONE kernel launch -- a few CTAs stream the peers'
row shards over NVLink (bulk copies peer HBM -> shared memory -> local HBM, no multicast) into the local
[M, K] operand while the remaining SM pairs already run tcgen05 tiles on the 256-row panels that have
arrived, own shard first.  Shapes the kernel does not cover (M % (256 * world), K % 64) fall back to
all_gather + GEMM; the choice depends on shapes only, so every rank takes the same branch.
Parity: the reference has no fused collective path; its FSDP/TP all-gathers are separate vendor-library
calls (reference torch_musa/csrc/distributed/ProcessGroupMCCL.cpp:4678-4735).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import tensor_parallel as TP
from ._symm import group_store_and_key


class FusedTensorParallel:
    FLAG_BYTES = 1 << 20

    def __init__(self, max_shard_bytes: int, max_rows: int, group=None, device=None, copier_pairs: int = 16,
                 max_partial_bytes: int = 0, reducer_pairs: int = 16):
        import torch_musa_b200 as bw

        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = torch.device(device if device is not None else f"blackwell:{bw.current_device()}")
        self.max_shard_bytes = (int(max_shard_bytes) + 255) // 256 * 256
        self.copier_pairs, self.reducer_pairs = copier_pairs, reducer_pairs
        self.max_partial_bytes = (int(max_partial_bytes) + 1023) // 1024 * 1024
        self.partial_off = (self.max_shard_bytes + 1023) // 1024 * 1024
        self.flag_off = self.partial_off + self.max_partial_bytes
        total = self.flag_off + self.FLAG_BYTES
        store, key = group_store_and_key(group, "tp_arena")
        self.sm = bw._C._create_symmetric_memory(store, key, self.rank, self.world,
                                                 self.device.index or 0, total)
        if not self.sm.ok:
            raise RuntimeError(f"tensor-parallel arena unavailable: {self.sm.why_not}")
        self.flags = torch.zeros(max(1, max_rows // 256), dtype=torch.int32, device=self.device)
        self.sm.local_tensor(self.flag_off, [self.FLAG_BYTES // 4], torch.int32).zero_()
        bw.synchronize()
        dist.barrier(group)          # every rank's flag table is zero before anyone's kernel can raise a flag in it
        self.calls = self.rs_calls = 0

    def _helper_pairs(self, pull_bytes: float, flops: float, limit: int) -> int:
        """SM pairs that move data instead of multiplying: the count that minimises max(transfer, GEMM) under a
        measured model -- p pairs pull about 35 * p^0.75 GB/s from the peers (99 / 166 / 280 GB/s at 4 / 8 / 16
        pairs) and the GEMM runs on the remaining 74 - p pairs at about 1.3 PFLOP/s in total."""
        best, best_t = 1, float("inf")
        for p in range(1, limit + 1):
            t = max(pull_bytes / (35e9 * p ** 0.75), flops / 1.3e15 * 74.0 / (74 - p))
            if t < best_t:
                best, best_t = p, t
        return best

    def ag_matmul(self, x_shard: torch.Tensor, w: torch.Tensor, group):
        rows, K = x_shard.shape
        M = rows * self.world
        if (x_shard.dtype not in (torch.bfloat16, torch.float16) or w.dtype != x_shard.dtype or M % (256 * self.world)
                or K % 64 or rows * K * x_shard.element_size() > self.max_shard_bytes or M // 256 > self.flags.numel()):
            return None
        N = w.shape[0]
        pairs = self._helper_pairs((self.world - 1) * rows * K * 2.0, 2.0 * M * N * K, self.copier_pairs)
        y, x_full = self.sm.gemm_allgather(x_shard.contiguous(), w, 0, self.flags, pairs)
        self.calls += 1
        return y, x_full

    def matmul_rs(self, x: torch.Tensor, w: torch.Tensor, group):
        M, K = x.shape
        N = w.shape[0]
        flag_words = self.world * (M // 256 // self.world + 1) * (N // 256 + 1) * 2
        if (x.dtype not in (torch.bfloat16, torch.float16) or w.dtype != x.dtype or M % (256 * self.world) or N % 256
                or K % 8 or self.world > 8 or M * N * 2 > self.max_partial_bytes or flag_words * 4 > self.FLAG_BYTES):
            return None
        pairs = self._helper_pairs((self.world - 1) * (M // self.world) * N * 2.0, 2.0 * M * N * K, self.reducer_pairs)
        y = self.sm.gemm_reduce_scatter(x.contiguous(), w, self.partial_off, self.flag_off, pairs)
        self.rs_calls += 1
        return y

    def install(self) -> "FusedTensorParallel":
        TP.FUSED_AG_MATMUL = self.ag_matmul
        if self.max_partial_bytes:
            TP.FUSED_MATMUL_RS = self.matmul_rs
        return self

    def uninstall(self) -> None:
        if TP.FUSED_AG_MATMUL == self.ag_matmul:
            TP.FUSED_AG_MATMUL = None
        if TP.FUSED_MATMUL_RS == self.matmul_rs:
            TP.FUSED_MATMUL_RS = None

    def check(self) -> None:
        import torch_musa_b200 as bw

        st = self.sm.take_status() or bw._C._gemm_status(True)
        if st:
            raise RuntimeError(f"a fused tensor-parallel kernel gave up on a bounded wait (status {st})")
