#!/usr/bin/env python
"""Gradient reduce-scatter + fp32 cast + sharded AdamW: the one-kernel-per-bucket path against reduce_scatter_tensor
followed by the fused multi-tensor AdamW and the bf16 cast (three passes over the shard plus the collective).

  python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmark/zero_bench.py [--mparams 256]

One JSON line on rank 0 with both times (CUDA events, max over ranks), the bytes that cross NVLink and the roofline
fraction: max(bytes in per GPU / 770 GB/s, local HBM traffic of the update / measured copy bandwidth) / fused time.
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
from torch_musa_b200.parallel.zero import ShardedFusedAdamW  # noqa: E402


def timed(fn, dev, iters=5, warmup=2):
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
    t = torch.tensor([s.elapsed_time(e) * 1e3 / iters], dtype=torch.float32).to(dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.cpu())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mparams", type=int, default=256, help="millions of bf16 parameters")
    ap.add_argument("--bucket-mb", type=int, default=32)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    bw.set_device(local)
    dev = torch.device("blackwell", local)
    dist.init_process_group("bccl", rank=rank, world_size=world)
    n = a.mparams << 20
    params = [torch.nn.Parameter((torch.randn(n // 8, device=dev) * 0.02).to(torch.bfloat16)) for _ in range(8)]
    opt = ShardedFusedAdamW(params, lr=1e-3, bucket_mb=a.bucket_mb)
    assert opt.fused, "the fused path needs the blackwell device and more than one rank"
    opt.flat_g.normal_(0, 0.01)
    fused = timed(opt.step, dev)

    # unfused composition on the same buffers
    chunk = opt.bs * world
    shard32 = torch.zeros(opt.n_buckets * opt.bs, device=dev)
    ref_p = torch.nn.Parameter(opt.p32.clone())
    ref_opt = torch.optim.AdamW([ref_p], lr=1e-3, fused=True)

    def unfused():
        for b in range(opt.n_buckets):
            g = opt.flat_g[b * chunk:(b + 1) * chunk]
            dist.reduce_scatter_tensor(shard32[b * opt.bs:(b + 1) * opt.bs], g.float(), op=dist.ReduceOp.AVG)
        ref_p.grad = shard32
        ref_opt.step()
        p16 = ref_p.detach().to(torch.bfloat16)
        for b in range(opt.n_buckets):
            dist.all_gather_into_tensor(opt.flat_p[b * chunk:(b + 1) * chunk], p16[b * opt.bs:(b + 1) * opt.bs])

    unf = timed(unfused, dev)
    total = opt.n_buckets * chunk
    cross_in = (world - 1) / world * total * 2.0 * 2           # gradient slices in + parameter slices in, bf16
    hbm = (total / world) * (4 * 3 * 2 + 2) + total * 2 * 2     # master + moments read/write, bf16 shard, grad + param buffers
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {"hbm_gbs": 6650.0}
    roof_us = max(cross_in / 770e9, hbm / (peaks["hbm_gbs"] * 1e9)) * 1e6
    if rank == 0:
        print(json.dumps({"op": "reduce_scatter_adamw_allgather", "world": world, "params_m": a.mparams, "bucket_mb": a.bucket_mb,
                          "fused_us": round(fused, 1), "unfused_us": round(unf, 1), "speedup": round(unf / fused, 2),
                          "nvlink_bytes_in_per_gpu": int(cross_in), "roofline_us": round(roof_us, 1),
                          "roofline_frac": round(roof_us / fused, 3)}))
    bw.synchronize()
    opt.check()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
