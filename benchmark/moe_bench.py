#!/usr/bin/env python
"""Expert-parallel token exchange: the fused dispatch / combine kernels against sort + all_to_all_single.

  python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmark/moe_bench.py [--tokens 8192]

One JSON line per phase on rank 0 (CUDA events, max over ranks): time of the fused kernel(s), time of the reference
exchange, bytes that must cross NVLink per GPU and the fraction of the 770 GB/s link figure the fused path reaches.
Router logits are N(0,1) per token (balanced loads), top-2, d_model 4096, bf16.
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
from torch_musa_b200.parallel.moe import FusedExpertExchange, ReferenceExpertExchange  # noqa: E402


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
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=8)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    bw.set_device(local)
    dev = torch.device("blackwell", local)
    dist.init_process_group("bccl", rank=rank, world_size=world)
    T, D, E, K = a.tokens, a.dim, a.experts, 2
    torch.manual_seed(rank)
    x = (torch.randn(T, D, device=dev) * 0.1).to(torch.bfloat16)
    _, idx = torch.topk(torch.randn(T, E, device=dev), K, dim=-1)
    gates = torch.full((T, K), 0.5, device=dev)
    fused = FusedExpertExchange(E, D, cap_rows=2 * T * K, slots=1, device=dev)
    ref = ReferenceExpertExchange(E)
    state = {}

    def f_dispatch():
        with torch.no_grad():
            state["f"] = fused.dispatch(x, idx, 0)

    def f_combine():
        with torch.no_grad():
            recv, rows, ctx = state["f"]
            state["fo"] = fused.combine(recv, gates, ctx, 0)

    def r_dispatch():
        with torch.no_grad():
            state["r"] = ref.dispatch(x, idx, 0)

    def r_combine():
        with torch.no_grad():
            recv, rows, ctx = state["r"]
            state["ro"] = ref.combine(recv, gates, ctx, 0)

    td, rd = timed(f_dispatch, dev), timed(r_dispatch, dev)
    tc, rc = timed(f_combine, dev), timed(r_combine, dev)
    cross = (world - 1) / world * T * K * D * 2.0
    if rank == 0:
        for name, f, r in (("dispatch", td, rd), ("combine", tc, rc)):
            print(json.dumps({"op": "moe_" + name, "world": world, "tokens_per_gpu": T, "top_k": K, "d_model": D,
                              "fused_us": round(f, 1), "all_to_all_us": round(r, 1), "speedup": round(r / f, 2),
                              "nvlink_bytes_per_gpu": int(cross), "roofline_us_at_770": round(cross / 770e3, 1),
                              "frac_of_link": round(cross / 770e3 / f, 3),
                              "note": "fused time includes the row-count read on the host (dispatch) and the copy of the "
                                      "expert output into the arena (combine)"}), flush=True)
    bw.synchronize()
    fused.check()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
