#!/usr/bin/env python
"""Decode throughput of the Llama-7B architecture with a static KV cache: eager step loop against the same step
replayed from a device graph.

  python benchmark/decode_bench.py [--batch 32] [--kv 2048] [--layers 32] [--tokens 32]
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmark/decode_bench.py   (tensor parallel:
      every rank holds 1/W of the heads and of the KV cache, two all-reduces per layer inside the captured step)

One JSON line: {"op": "decode", "batch", "kv_len", "eager_ms_per_token", "graph_ms_per_token", "graph_tokens_per_s", ...}.
Random-init bf16 weights, random prompt; CUDA-event times after warm-up.
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

import torch_musa_b200 as bw  # noqa: E402
from torch_musa_b200.models import Llama, LlamaConfig  # noqa: E402
from torch_musa_b200.models.decode import LlamaDecoder, shard_for_tensor_parallel  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--kv", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--tokens", type=int, default=32)
    a = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("blackwell", local)
    group = None
    if world > 1:
        import torch.distributed as dist

        bw.set_device(local)
        dist.init_process_group("bccl", rank=rank, world_size=world)
        group = dist.group.WORLD
    cfg = LlamaConfig(n_layers=a.layers, max_seq_len=a.kv + a.tokens * 3 + 8, fused_qkv=world == 1,
                      fused_gate_up=world == 1)
    torch.manual_seed(0)
    with torch.device(dev):
        model = Llama(cfg).to(torch.bfloat16).eval()
    model.init_rope_cache(dev)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
    if world > 1:
        shard_for_tensor_parallel(model, rank, world)
    torch.manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (a.batch, a.kv)).to(dev)
    dec = LlamaDecoder(model, a.batch, cfg.max_seq_len, device=dev, tp_group=group)
    dec.prefill(prompt)

    def timed(n):
        bw.synchronize()
        s, e = bw.Event(enable_timing=True), bw.Event(enable_timing=True)
        s.record()
        dec.decode(n)
        e.record()
        bw.synchronize()
        return s.elapsed_time(e) / n

    dec.decode(4)
    eager = timed(a.tokens)
    dec.capture()
    dec.decode(4)
    graph = timed(a.tokens)
    if world > 1:
        t = torch.tensor([eager, graph], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)          # max over ranks
        eager, graph = float(t[0]), float(t[1])
        if rank != 0:
            del dec          # the captured graph references the communicator: release it before the group goes
            dist.destroy_process_group()
            return
    print(json.dumps({"op": "decode", "tp": world, "model": f"llama-7b dims, {a.layers} layers", "batch": a.batch, "kv_len": a.kv,
                      "eager_ms_per_token": round(eager, 3), "graph_ms_per_token": round(graph, 3),
                      "graph_tokens_per_s": round(a.batch / graph * 1e3, 1), "speedup": round(eager / graph, 2)}))
    if world > 1:
        del dec
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
