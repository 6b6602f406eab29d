#!/usr/bin/env python
"""Trains a tiny Llama for a few steps on the blackwell device (or on the CPU when no B200 is visible) with the
fused optimizer and bf16 autocast.

    python examples/python/train_tiny_llama.py [--steps 20] [--device blackwell|cpu]
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402

import torch_musa_b200 as bw  # noqa: E402  (registers the device, the bccl backend and the fused operators)
from torch_musa_b200.models import Llama, llama_tiny_config  # noqa: E402


def main(argv=None) -> float:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--device", default="blackwell" if bw.is_available() else "cpu")
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    torch.manual_seed(0)
    cfg = llama_tiny_config()
    model = Llama(cfg).to(dev)
    fused = dev.type == "blackwell"
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, fused=fused)
    tokens = torch.randint(0, cfg.vocab_size, (4, 33), device=dev)          # one batch, memorised: the loss must fall

    def step():
        with torch.autocast(dev.type, dtype=torch.bfloat16):
            loss = model(tokens[:, :-1], tokens[:, 1:])
        opt.zero_grad(set_to_none=False)
        loss.backward()
        opt.step()
        return loss

    first = last = None
    for _ in range(a.steps):
        last = float(step().detach())
        first = last if first is None else first
    print(f"device {dev}: loss {first:.3f} -> {last:.3f} over {a.steps} steps")
    return last


if __name__ == "__main__":
    main()
