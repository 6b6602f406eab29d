#!/usr/bin/env python
"""Collective micro-benchmark on the bccl backend: the hand-written peer-memory kernels against NCCL for the
same call, same process, same buffers.

  python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmark/comm_bench.py [--max-mb 64]

For every operation and size one JSON line on rank 0:
  {"op", "bytes", "world", "fused_us", "nccl_us", "fused_busbw_gbs", "nccl_busbw_gbs", "frac_of_link"}
Times are CUDA-event times on the launching stream, max over ranks.  Bus bandwidth follows the usual
conventions (all-reduce 2(n-1)/n, all-gather / reduce-scatter / all-to-all (n-1)/n of the full buffer);
`frac_of_link` divides the per-GPU bytes that must cross NVLink by the time and by the measured 770 GB/s
peer-copy bandwidth per direction.
Parity: the reference has no collective benchmark; its distributed tests only check values
(reference tests/unittest/distributed/test_distributed.py).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import torch_musa_b200 as bw  # noqa: E402

LINK_GBS = 770.0


def timed(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    bw.synchronize()
    dist.barrier()
    s, e = bw.Event(enable_timing=True), bw.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    bw.synchronize()
    t = torch.tensor([s.elapsed_time(e) * 1e3 / iters], dtype=torch.float32).to(f"blackwell:{bw.current_device()}")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.cpu())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    bw.set_device(local)
    dev = torch.device("blackwell", local)
    dist.init_process_group("bccl", rank=rank, world_size=world)
    pg = dist.distributed_c10d._get_default_group()._get_backend(dev)
    sizes = [s << 20 for s in (1, 4, 16, 64, 256) if s <= a.max_mb]

    def both(fn):
        bw._C._pg_set_fused(pg, True)
        before = bw._C._pg_fused_count(pg)
        f = timed(fn, a.iters)
        used = bw._C._pg_fused_count(pg) > before
        bw._C._pg_set_fused(pg, False)
        n = timed(fn, a.iters)
        bw._C._pg_set_fused(pg, True)
        return f, n, used

    for nbytes in sizes:
        cases = []
        x32 = torch.randn(nbytes // 4, device=dev)
        cases.append(("all_reduce_fp32_avg", nbytes, 2.0 * (world - 1) / world,
                      lambda: dist.all_reduce(x32, op=dist.ReduceOp.AVG)))
        x16 = torch.randn(nbytes // 2, device=dev, dtype=torch.bfloat16)
        cases.append(("all_reduce_bf16_sum", nbytes, 2.0 * (world - 1) / world, lambda: dist.all_reduce(x16)))
        shard = torch.randn(nbytes // 2 // world, device=dev, dtype=torch.bfloat16)
        full = torch.empty(nbytes // 2 // world * world, device=dev, dtype=torch.bfloat16)
        cases.append(("all_gather_bf16", full.numel() * 2, (world - 1) / world,
                      lambda: dist.all_gather_into_tensor(full, shard)))
        g32 = torch.randn(nbytes // 4 // world * world, device=dev)
        o32 = torch.empty(nbytes // 4 // world, device=dev)
        cases.append(("reduce_scatter_fp32_avg", g32.numel() * 4, (world - 1) / world,
                      lambda: dist.reduce_scatter_tensor(o32, g32, op=dist.ReduceOp.AVG)))
        a_in = torch.randn(nbytes // 2 // world * world, device=dev, dtype=torch.bfloat16)
        a_out = torch.empty_like(a_in)
        cases.append(("all_to_all_bf16", a_in.numel() * 2, (world - 1) / world,
                      lambda: dist.all_to_all_single(a_out, a_in)))
        for name, total, factor, fn in cases:
            f_us, n_us, used = both(fn)
            if rank == 0:
                cross = total * factor / (2.0 if name.startswith("all_reduce") else 1.0)  # bytes in per GPU per phase
                print(json.dumps({
                    "op": name, "bytes": total, "world": world, "fused_kernel_used": used,
                    "fused_us": round(f_us, 1), "nccl_us": round(n_us, 1),
                    "fused_busbw_gbs": round(total * factor / f_us / 1e3, 1),
                    "nccl_busbw_gbs": round(total * factor / n_us / 1e3, 1),
                    "frac_of_link": round((total * factor / f_us / 1e3) / (LINK_GBS * (2.0 if name.startswith("all_reduce") else 1.0)), 3),
                }), flush=True)
    st = bw._C._pg_symmetric_memory(pg, local).take_status() if hasattr(bw._C, "_pg_symmetric_memory") else 0
    if rank == 0 and st:
        print(json.dumps({"warning": "a peer-memory kernel gave up on a bounded wait", "status": st}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
