#!/usr/bin/env python
"""Fused tensor-parallel primitives against their unfused compositions, same process and buffers.

  python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmark/tp_bench.py [--tokens 16384]

Per case one JSON line on rank 0: op, shape, helper SM pairs, fused_us, unfused_us (all_gather/reduce_scatter through
the process group + the plain GEMM), gemm_only_us, and the roofline figures: time of the FLOPs at the measured GEMM
peak, time of the bytes that must cross NVLink at 770 GB/s, and achieved = max(of the two) / fused time.
CUDA-event times on the launching stream, max over ranks.
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
import torch.nn.functional as F  # noqa: E402

import torch_musa_b200 as bw  # noqa: E402
from torch_musa_b200.parallel import tensor_parallel as TP  # noqa: E402
from torch_musa_b200.parallel.fused_tp import FusedTensorParallel  # noqa: E402

LINK_GBS = 770.0


def peak_tflops():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["bf16_tflops"], "measured"
    return 1590.0, "fallback"


def timed(fn, dev, iters=10, warmup=3):
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
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--pairs", type=int, nargs="*", default=[4, 8, 12, 16])
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    bw.set_device(local)
    dev = torch.device("blackwell", local)
    dist.init_process_group("bccl", rank=rank, world_size=world)
    T, D = a.tokens, a.dim
    ctx = FusedTensorParallel(max_shard_bytes=T // world * max(D, 11008) * 2, max_rows=T, device=dev,
                              max_partial_bytes=T * D * 2, copier_pairs=16, reducer_pairs=16)
    peak, src = peak_tflops()
    cases = [("qkv", 12288), ("gate_up", 22016), ("copy_only", 256)]
    for name, n_full in cases:
        N = max(256, n_full // world // 8 * 8)
        x_shard = (torch.randn(T // world, D, device=dev) * 0.1).to(torch.bfloat16)
        w = (torch.randn(N, D, device=dev) * 0.02).to(torch.bfloat16)
        x_full = TP.all_gather_rows(x_shard)
        unfused = timed(lambda: F.linear(TP.all_gather_rows(x_shard), w), dev, a.iters)
        gemm = timed(lambda: F.linear(x_full, w), dev, a.iters)
        flops, cross = 2.0 * T * N * D, (world - 1) * (T // world) * D * 2.0
        for pairs in a.pairs:
            fused = timed(lambda: ctx.sm.gemm_allgather(x_shard, w, 0, ctx.flags, pairs), dev, a.iters)
            t_f, t_l = flops / (peak * 1e12) * 1e6, cross / (LINK_GBS * 1e9) * 1e6
            if rank == 0:
                print(json.dumps({"op": "allgather_gemm", "case": name, "shape": [T, N, D], "world": world, "pairs": pairs,
                                  "fused_us": round(fused, 1), "unfused_us": round(unfused, 1), "gemm_only_us": round(gemm, 1),
                                  "flops_us_at_" + src + "_peak": round(t_f, 1), "nvlink_us_at_770": round(t_l, 1),
                                  "roofline_frac": round(max(t_f, t_l) / fused, 3),
                                  "pull_gbs": round(cross / fused / 1e3, 1)}), flush=True)
    for name, k_full in [("o_proj", 4096), ("down", 11008), ("reduce_only", 64 * world)]:
        K = max(64, k_full // world // 8 * 8)
        x = (torch.randn(T, K, device=dev) * 0.1).to(torch.bfloat16)
        w = (torch.randn(D, K, device=dev) * 0.02).to(torch.bfloat16)
        unfused = timed(lambda: TP.reduce_scatter_rows(F.linear(x, w)), dev, a.iters)
        gemm = timed(lambda: F.linear(x, w), dev, a.iters)
        flops, cross = 2.0 * T * D * K, (world - 1) * (T // world) * D * 2.0
        for pairs in a.pairs:
            fused = timed(lambda: ctx.sm.gemm_reduce_scatter(x, w, ctx.partial_off, ctx.flag_off, pairs), dev, a.iters)
            t_f, t_l = flops / (peak * 1e12) * 1e6, cross / (LINK_GBS * 1e9) * 1e6
            if rank == 0:
                print(json.dumps({"op": "gemm_reduce_scatter", "case": name, "shape": [T, D, K], "world": world, "pairs": pairs,
                                  "fused_us": round(fused, 1), "unfused_us": round(unfused, 1), "gemm_only_us": round(gemm, 1),
                                  "flops_us_at_" + src + "_peak": round(t_f, 1), "nvlink_us_at_770": round(t_l, 1),
                                  "roofline_frac": round(max(t_f, t_l) / fused, 3),
                                  "pull_gbs": round(cross / fused / 1e3, 1)}), flush=True)
    bw.synchronize()
    ctx.check()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
