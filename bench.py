#!/usr/bin/env python
"""Headline benchmark: Llama-7B training throughput (tokens/s) with FSDP2 per-layer sharding.

  python bench.py --gpus N --steps K --warmup W            (N > 1: launched under torch.distributed.run)
  python bench.py --impl reference ...                     (the unmodified reference: unavailable, see below)
  python bench.py --impl stock ...                         (same model on stock PyTorch CUDA + NCCL)

Config (BASELINE.json): 32 layers, d_model 4096, 32 heads, SwiGLU FFN 11008, RMSNorm eps 1e-5, RoPE theta 1e4,
vocab 32000, seq 4096, micro-batch 1 per GPU, bf16 compute with fp32 master weights / fp32 gradient reduce,
fused AdamW lr 3e-4, synthetic token ids uniform in [0, 32000) from a seed, random-init weights.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

REFERENCE_UNAVAILABLE = (
    "the reference (MooreThreads/torch_musa) needs the MUSA SDK (mcc, muDNN, MCCL) and a patched torch 2.7.1; "
    "its offline pip install stops in setup.py (ModuleNotFoundError: ahocorasick) and no MUSA device exists here"
)


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference", "stock"])
    p.add_argument("--layers", type=int, default=32, help="debug only: fewer layers makes the number invalid")
    p.add_argument("--seq", type=int, default=4096)
    p.add_argument("--micro-batch", type=int, default=1)
    p.add_argument("--parallelism", default="auto", choices=["auto", "fsdp", "single"])
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--config", default="llama_fsdp", choices=["llama_fsdp", "resnet50_ddp", "moe_ep", "llama_tp"],
                   help="llama_fsdp: the headline Llama-7B FSDP2 step; resnet50_ddp: ResNet-50 DDP images/s")
    p.add_argument("--batch", type=int, default=256, help="resnet50_ddp: images per GPU")
    p.add_argument("--trace", default=None, help="debug: also run two extra steps under torch.profiler and write "
                   "a chrome trace per rank to this path prefix (never inside the timed region)")
    return p.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()  # our own child, by handle
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def _load_by_path(name, rel):
    """Loads one file of the package as a stand-alone module (the stock arm must not import the backend)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "torch_musa_b200", rel))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def main_resnet(args):
    """ResNet-50 DDP training throughput: bf16 autocast over fp32 master weights, channels-last, per-GPU batch
    256 of 3x224x224 N(0,1) images, SGD momentum 0.9 (fused multi-tensor optimizer), 25 MB gradient buckets."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    ours = args.impl == "ours"
    if ours:
        import torch_musa_b200 as bw
        from torch_musa_b200.models import resnet50

        devmod, devtype, backend = bw, "blackwell", "bccl"
    else:
        devmod, devtype, backend = torch.cuda, "cuda", "nccl"
        resnet50 = _load_by_path("_stock_resnet", "models/resnet.py").resnet50
    device = torch.device(devtype, local_rank)
    devmod.set_device(local_rank)
    use_ddp = world > 1
    if use_ddp:
        dist.init_process_group(backend=backend, rank=rank, world_size=world, device_id=device if not ours else None)

    torch.manual_seed(1234)
    model = resnet50(1000).to(device).to(memory_format=torch.channels_last)
    if use_ddp:
        if ours:
            from torch_musa_b200.parallel.ddp import wrap_ddp

            net = wrap_ddp(model, device_ids=[local_rank], bucket_cap_mb=25, gradient_as_bucket_view=True)
        else:
            net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], bucket_cap_mb=25,
                                                            gradient_as_bucket_view=True)
    else:
        net = model
    if ours:
        from torch_musa_b200.optim import FusedSGD

        opt = FusedSGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    else:
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4, fused=True)

    B = args.batch
    gen = torch.Generator().manual_seed(1000 + rank)
    n_batches = 2
    host_x = [torch.randn(B, 3, 224, 224, generator=gen).pin_memory() for _ in range(n_batches)]
    host_t = [torch.randint(0, 1000, (B,), generator=gen).pin_memory() for _ in range(n_batches)]
    dev_x = [x.to(device).contiguous(memory_format=torch.channels_last) for x in host_x]
    dev_t = [t.to(device) for t in host_t]

    def step(x, t):
        with torch.autocast(devtype, dtype=torch.bfloat16):
            loss = F.cross_entropy(net(x), t)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def barrier():
        if use_ddp:
            dist.barrier()
        devmod.synchronize()

    for i in range(args.warmup):
        step(dev_x[i % n_batches], dev_t[i % n_batches])
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if ours:
        bw.reset_kernel_launch_count()
    ev0, ev1 = devmod.Event(enable_timing=True), devmod.Event(enable_timing=True)
    barrier()
    ev0.record()
    for i in range(args.steps):
        loss = step(dev_x[i % n_batches], dev_t[i % n_batches])
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    launches = bw.kernel_launch_count() if ours else 0
    final_loss = float(loss.detach().float().cpu())

    e2e_ms, h2d, d2h = 0.0, 0, 0
    if not args.no_e2e:
        barrier()
        ev2, ev3 = devmod.Event(enable_timing=True), devmod.Event(enable_timing=True)
        ev2.record()
        for i in range(args.steps):
            x = host_x[i % n_batches].to(device, non_blocking=True).contiguous(memory_format=torch.channels_last)
            t = host_t[i % n_batches].to(device, non_blocking=True)
            h2d += x.numel() * x.element_size() + t.numel() * t.element_size()
            lv = step(x, t).detach().float().cpu()
            d2h += lv.numel() * lv.element_size()
        ev3.record()
        barrier()
        e2e_ms = ev2.elapsed_time(ev3)
    clocks = sampler.stop() if rank == 0 else None
    if args.trace:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            for i in range(2):
                step(dev_x[i % n_batches], dev_t[i % n_batches])
            barrier()
        prof.export_chrome_trace(f"{args.trace}.rank{rank}.json")
    if use_ddp:
        t = torch.tensor([ms_total, e2e_ms], dtype=torch.float64).to(device).float()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = float(t[0].cpu()), float(t[1].cpu())
    ms_per_step = ms_total / args.steps
    imgs = B * world
    if rank == 0:
        out = {
            "metric": "resnet50_ddp_train_images_per_s", "value": imgs / (ms_per_step / 1e3), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (images N(0,1), labels uniform in [0,1000) from a seed; random-init weights)",
            "impl": args.impl,
            "config": {"model": "resnet-50 (torchvision layout, 1000 classes)", "global_batch": imgs,
                       "image": "3x224x224", "parallelism": f"ddp{world}, 25 MB buckets" if use_ddp else "single device",
                       "precision": "bf16 autocast, fp32 master weights, channels-last",
                       "optimizer": "fused multi-tensor SGD momentum 0.9",
                       "cache": "activations per step (several GB) are far larger than the 126 MB L2"},
            "final_loss": final_loss, "gpu_launches": launches, "clocks": clocks,
        }
        if not args.no_e2e:
            out["e2e"] = {"value": imgs / (e2e_ms / args.steps / 1e3), "unit": "images/s",
                          "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": d2h // args.steps}
        if ours:
            out["fallback_ops"] = len(bw.fallback_counts())
            if os.environ.get("B200_BENCH_VERBOSE"):
                sys.stderr.write("fallbacks: " + json.dumps(sorted(bw.fallback_counts().items(), key=lambda kv: -kv[1])) + "\n")
        print(json.dumps(out))
    if use_ddp:
        dist.destroy_process_group()
    return 0


def _stock_package():
    """Loads the model files under a throw-away package name so that the stock arm never imports the backend."""
    import types

    for name in ("_stock_pkg", "_stock_pkg.ops", "_stock_pkg.models", "_stock_pkg.parallel"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__path__ = []
            sys.modules[name] = m
    sys.modules["_stock_pkg.ops"].functional = _load_by_path("_stock_pkg.ops.functional", "ops/functional.py")
    llama = _load_by_path("_stock_pkg.models.llama", "models/llama.py")
    moe = _load_by_path("_stock_pkg.models.moe", "models/moe.py")
    pmoe = _load_by_path("_stock_pkg.parallel.moe", "parallel/moe.py")
    sys.modules["_stock_pkg.parallel"].tensor_parallel = _load_by_path("_stock_pkg.parallel.tensor_parallel",
                                                                       "parallel/tensor_parallel.py")
    _load_by_path("_stock_pkg.parallel.loss", "parallel/loss.py")
    sys.modules["_stock_pkg"].ops = sys.modules["_stock_pkg.ops"]
    sys.modules["_stock_pkg"].parallel = sys.modules["_stock_pkg.parallel"]
    return llama, moe, pmoe


def main_tp(args):
    """Llama-7B architecture, tensor parallel over all ranks (column-parallel q/k/v/gate/up, row-parallel o/down,
    sequence-parallel norms, vocabulary-parallel loss), bf16, one sequence of 2048 tokens per GPU in the batch
    (batch 8 x 2048 at TP=8); forward + backward + fused AdamW step."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    ours = args.impl == "ours"
    if ours:
        import torch_musa_b200 as bw
        from torch_musa_b200.models.llama import LlamaConfig
        from torch_musa_b200.models.llama_tp import TPLlama

        devmod, devtype, backend = bw, "blackwell", "bccl"
    else:
        devmod, devtype, backend = torch.cuda, "cuda", "nccl"
        llama_mod, _, _ = _stock_package()
        LlamaConfig = llama_mod.LlamaConfig
        TPLlama = _load_by_path("_stock_pkg.models.llama_tp", "models/llama_tp.py").TPLlama
    device = torch.device(devtype, local_rank)
    devmod.set_device(local_rank)
    if world > 1:
        dist.init_process_group(backend=backend, rank=rank, world_size=world, device_id=device if not ours else None)

    B, S = world, 2048
    cfg = LlamaConfig(n_layers=args.layers, max_seq_len=S)
    torch.manual_seed(1234)
    with torch.device(device):
        model = TPLlama(cfg, world).to(torch.bfloat16)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
    fused = None
    if ours and world > 1:
        from torch_musa_b200.parallel.fused_tp import FusedTensorParallel

        T = B * S
        # all-gather -> GEMM runs as one launch; GEMM -> reduce-scatter stays GEMM + the backend's reduce-scatter kernel
        # unless B200_TP_FUSED_RS=1 (the one-launch version is slower with few ranks, see profiles/)
        fused_rs = os.environ.get("B200_TP_FUSED_RS", "0") == "1"
        fused = FusedTensorParallel(max_shard_bytes=T // world * cfg.dim * 2, max_rows=T, device=device,
                                    max_partial_bytes=T * cfg.dim * 2 if fused_rs else 0).install()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    gen = torch.Generator().manual_seed(1000)          # every rank sees the same batch: tensor parallelism
    n_batches = 4
    host_tokens = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen).pin_memory() for _ in range(n_batches)]
    dev_tokens = [t.to(device) for t in host_tokens]
    partial_grad = model.replicated_parameters()

    def step(tok):
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        if world > 1:
            flat = torch.cat([p.grad.reshape(-1) for p in partial_grad])
            dist.all_reduce(flat)
            off = 0
            for p in partial_grad:
                p.grad.copy_(flat[off:off + p.numel()].view_as(p.grad))
                off += p.numel()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        devmod.synchronize()

    for i in range(args.warmup):
        step(dev_tokens[i % n_batches])
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if ours:
        bw.reset_kernel_launch_count()
    ev0, ev1 = devmod.Event(enable_timing=True), devmod.Event(enable_timing=True)
    barrier()
    ev0.record()
    for i in range(args.steps):
        loss = step(dev_tokens[i % n_batches])
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    launches = bw.kernel_launch_count() if ours else 0
    final_loss = float(loss.detach().float().cpu())
    e2e_ms, h2d, d2h = 0.0, 0, 0
    if not args.no_e2e:
        barrier()
        ev2, ev3 = devmod.Event(enable_timing=True), devmod.Event(enable_timing=True)
        ev2.record()
        for i in range(args.steps):
            tok = host_tokens[i % n_batches].to(device, non_blocking=True)
            h2d += tok.numel() * tok.element_size()
            lv = step(tok).detach().float().cpu()
            d2h += lv.numel() * lv.element_size()
        ev3.record()
        barrier()
        e2e_ms = ev2.elapsed_time(ev3)
    clocks = sampler.stop() if rank == 0 else None
    if args.trace:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            for i in range(2):
                step(dev_tokens[i % n_batches])
            barrier()
        prof.export_chrome_trace(f"{args.trace}.rank{rank}.json")
    fused_calls = None
    if fused is not None:
        fused.check()
        fused_calls = {"allgather_gemm": fused.calls, "gemm_reduce_scatter": fused.rs_calls}
    if world > 1:
        t = torch.tensor([ms_total, e2e_ms], dtype=torch.float64).to(device).float()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = float(t[0].cpu()), float(t[1].cpu())
    ms_per_step = ms_total / args.steps
    toks = B * S
    if rank == 0:
        out = {
            "metric": "llama7b_tp_train_tokens_per_s", "value": toks / (ms_per_step / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (token ids uniform in [0,32000) from a seed; random-init weights)", "impl": args.impl,
            "config": {"model": "llama-7b (32L d4096 h32 ffn11008 vocab32000)" if args.layers == 32 else f"llama-7b-dims-{args.layers}L (INVALID: reduced layers)",
                       "global_batch": B, "seq_len": S,
                       "parallelism": f"tp{world}: colwise q/k/v/gate/up, rowwise o/down, sequence-parallel norms, vocab-parallel loss",
                       "optimizer": "fused AdamW lr 3e-4 on bf16 parameters", "fused_collective_calls": fused_calls,
                       "cache": "weights and activations per step are far larger than the 126 MB L2"},
            "final_loss": final_loss, "gpu_launches": launches, "clocks": clocks,
        }
        if not args.no_e2e:
            out["e2e"] = {"value": toks / (e2e_ms / args.steps / 1e3), "unit": "tokens/s",
                          "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": d2h // args.steps}
        if ours:
            out["fallback_ops"] = len(bw.fallback_counts())
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main_moe(args):
    """Mixtral-style MoE decoder, expert parallel over all ranks: 8 layers, d 4096, 8 SwiGLU experts of 14336,
    top-2 router, 8192 tokens per GPU, bf16 parameters and activations, fused AdamW; forward + backward + step."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    ours = args.impl == "ours"
    if ours:
        import torch_musa_b200 as bw
        from torch_musa_b200.models import MoEConfig, MoETransformer
        from torch_musa_b200.parallel import moe as pmoe

        devmod, devtype, backend = bw, "blackwell", "bccl"
    else:
        devmod, devtype, backend = torch.cuda, "cuda", "nccl"
        _, moe_mod, pmoe = _stock_package()
        MoEConfig, MoETransformer = moe_mod.MoEConfig, moe_mod.MoETransformer
    device = torch.device(devtype, local_rank)
    devmod.set_device(local_rank)
    if world > 1:
        dist.init_process_group(backend=backend, rank=rank, world_size=world, device_id=device if not ours else None)

    B, S = 2, 4096
    cfg = MoEConfig(n_layers=args.layers if args.layers != 32 else 8, max_seq_len=S, synthetic_router_logits=True)
    torch.manual_seed(1234)
    with torch.device(device):
        model = MoETransformer(cfg, ep_world=world).to(torch.bfloat16)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
    if ours:
        exchange = pmoe.make_expert_exchange(cfg.n_experts, cfg.dim, B * S, cfg.top_k, slots=cfg.n_layers, device=device,
                                             capacity_factor=cfg.capacity_factor)
    else:
        exchange = pmoe.ReferenceExpertExchange(cfg.n_experts)
    model.set_exchange(exchange)
    replicated = model.replicated_parameters()
    experts = model.expert_parameters()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

    gen = torch.Generator().manual_seed(1000 + rank)
    n_batches = 4
    host_tokens = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen).pin_memory() for _ in range(n_batches)]
    dev_tokens = [t.to(device) for t in host_tokens]

    def sync_grads():
        if world == 1:
            return
        grads = [p.grad for p in replicated if p.grad is not None]
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, op=dist.ReduceOp.AVG)
        off = 0
        for g in grads:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()
        torch._foreach_mul_([p.grad for p in experts if p.grad is not None], 1.0 / world)

    def step(tok):
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        sync_grads()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        devmod.synchronize()

    for i in range(args.warmup):
        step(dev_tokens[i % n_batches])
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if ours:
        bw.reset_kernel_launch_count()
    ev0, ev1 = devmod.Event(enable_timing=True), devmod.Event(enable_timing=True)
    barrier()
    ev0.record()
    for i in range(args.steps):
        loss = step(dev_tokens[i % n_batches])
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    launches = bw.kernel_launch_count() if ours else 0
    final_loss = float(loss.detach().float().cpu())
    e2e_ms, h2d, d2h = 0.0, 0, 0
    if not args.no_e2e:
        barrier()
        ev2, ev3 = devmod.Event(enable_timing=True), devmod.Event(enable_timing=True)
        ev2.record()
        for i in range(args.steps):
            tok = host_tokens[i % n_batches].to(device, non_blocking=True)
            h2d += tok.numel() * tok.element_size()
            lv = step(tok).detach().float().cpu()
            d2h += lv.numel() * lv.element_size()
        ev3.record()
        barrier()
        e2e_ms = ev2.elapsed_time(ev3)
    clocks = sampler.stop() if rank == 0 else None
    if args.trace:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            for i in range(2):
                step(dev_tokens[i % n_batches])
            barrier()
        prof.export_chrome_trace(f"{args.trace}.rank{rank}.json")
    if ours:
        exchange.check()
    if world > 1:
        t = torch.tensor([ms_total, e2e_ms], dtype=torch.float64).to(device).float()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = float(t[0].cpu()), float(t[1].cpu())
    ms_per_step = ms_total / args.steps
    toks = B * S * world
    if rank == 0:
        out = {
            "metric": "moe_ep_train_tokens_per_s", "value": toks / (ms_per_step / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (token ids uniform in [0,32000) from a seed; random-init weights)", "impl": args.impl,
            "config": {"model": f"mixtral-style moe ({cfg.n_layers}L d4096 h32/kv8, 8 experts x ffn14336, top-2)",
                       "global_batch": B * world, "seq_len": S, "tokens_per_gpu": B * S,
                       "parallelism": f"ep{world} ({cfg.n_experts // world} expert(s) per GPU), replicated attention/router",
                       "expert_gemm": "bf16", "router": "top-2 softmax over logits drawn N(0,1) per token", "optimizer": "fused AdamW lr 3e-4 on bf16 parameters",
                       "cache": "weights and activations per step are far larger than the 126 MB L2"},
            "final_loss": final_loss, "gpu_launches": launches, "clocks": clocks,
        }
        if not args.no_e2e:
            out["e2e"] = {"value": toks / (e2e_ms / args.steps / 1e3), "unit": "tokens/s",
                          "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": d2h // args.steps}
        if ours:
            out["fallback_ops"] = len(bw.fallback_counts())
            if os.environ.get("B200_BENCH_VERBOSE"):
                sys.stderr.write("fallbacks: " + json.dumps(sorted(bw.fallback_counts().items(), key=lambda kv: -kv[1])) + "\n")
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    args = parse()
    deadline = int(os.environ.get("B200_BENCH_DUMP_AFTER_S", "900"))
    if deadline > 0:
        # a run normally ends within two minutes; one that is still alive after the deadline prints every thread's
        # Python stack and exits instead of occupying the GPUs until somebody kills it (0 disables)
        import faulthandler

        faulthandler.dump_traceback_later(deadline, exit=True)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.config == "resnet50_ddp":
        return main_resnet(args)
    if args.config == "moe_ep":
        return main_moe(args)
    if args.config == "llama_tp":
        return main_tp(args)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")

    ours = args.impl == "ours"
    if ours:
        import torch_musa_b200 as bw

        devmod, devtype, backend = bw, "blackwell", "bccl"
        have_backend = bw.distributed.is_bccl_available()
    else:
        devmod, devtype, backend = torch.cuda, "cuda", "nccl"
        have_backend = True
    device = torch.device(devtype, local_rank)
    devmod.set_device(local_rank)

    par = args.parallelism
    if par == "auto":
        par = "fsdp" if (have_backend or world > 1) else "single"
    if world > 1 and par != "fsdp":
        raise SystemExit("multi-GPU runs use FSDP2")
    if par == "fsdp":
        dist.init_process_group(backend=backend, rank=rank, world_size=world, device_id=device if not ours else None)

    if ours:
        from torch_musa_b200.models import Llama, LlamaConfig
    else:
        # The stock arm must not load the blackwell backend (it would become the process's accelerator):
        # load the model definition and its plain-PyTorch functional fallbacks straight from their files.
        import importlib.util
        import types

        pkg = types.ModuleType("_stock_pkg"); pkg.__path__ = []
        opsp = types.ModuleType("_stock_pkg.ops"); opsp.__path__ = []
        sys.modules["_stock_pkg"], sys.modules["_stock_pkg.ops"] = pkg, opsp
        modelsp = types.ModuleType("_stock_pkg.models"); modelsp.__path__ = []
        sys.modules["_stock_pkg.models"] = modelsp

        def _load(name, path):
            spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "torch_musa_b200", path))
            mod = importlib.util.module_from_spec(spec)
            sys.modules[name] = mod
            spec.loader.exec_module(mod)
            return mod

        opsp.functional = _load("_stock_pkg.ops.functional", "ops/functional.py")
        _llama = _load("_stock_pkg.models.llama", "models/llama.py")
        Llama, LlamaConfig = _llama.Llama, _llama.LlamaConfig

    cfg = LlamaConfig(n_layers=args.layers, max_seq_len=args.seq)
    torch.manual_seed(1234)
    with torch.device("meta"):
        model = Llama(cfg)

    if par == "fsdp":
        from torch.distributed.fsdp import fully_shard, MixedPrecisionPolicy
        from torch.distributed.device_mesh import init_device_mesh

        mesh = init_device_mesh(devtype, (world,))
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
        for layer in model.layers:
            fully_shard(layer, mesh=mesh, mp_policy=mp)
        fully_shard(model, mesh=mesh, mp_policy=mp)
        model.to_empty(device=device)
        if ours:
            from torch_musa_b200.parallel import fsdp as bw_fsdp

            bw_fsdp.install_fused_collectives(model)
    else:
        model.to_empty(device=device)
        model = model.to(torch.bfloat16)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
            else:
                p.fill_(1.0)
        model.init_rope_cache(device)

    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

    B, S = args.micro_batch, args.seq
    gen = torch.Generator().manual_seed(1000 + rank)
    n_batches = 4
    host_tokens = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen).pin_memory() for _ in range(n_batches)]
    dev_tokens = [t.to(device) for t in host_tokens]

    def step(tok):
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def barrier():
        if par == "fsdp":
            dist.barrier()
        devmod.synchronize()

    for i in range(args.warmup):
        step(dev_tokens[i % n_batches])
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # ---- device-timed region: inputs already on the device
    if ours:
        bw.reset_kernel_launch_count()
    ev0, ev1 = devmod.Event(enable_timing=True), devmod.Event(enable_timing=True)
    barrier()
    ev0.record()
    for i in range(args.steps):
        loss = step(dev_tokens[i % n_batches])
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    launches = bw.kernel_launch_count() if ours else 0
    final_loss = float(loss.detach().float().cpu())

    # ---- end-to-end region: pinned host tokens -> device each step, loss read back each step
    e2e = None
    if not args.no_e2e:
        barrier()
        t0 = time.perf_counter()
        ev2, ev3 = devmod.Event(enable_timing=True), devmod.Event(enable_timing=True)
        ev2.record()
        h2d = d2h = 0
        for i in range(args.steps):
            tok = host_tokens[i % n_batches].to(device, non_blocking=True)
            h2d += tok.numel() * tok.element_size()
            l = step(tok)
            lv = l.detach().float().cpu()  # device -> host read of the step's result
            d2h += lv.numel() * lv.element_size()
        ev3.record()
        barrier()
        e2e_ms = max(ev2.elapsed_time(ev3), (time.perf_counter() - t0) * 1e3 * 0.0)
        e2e = {"ms_total": e2e_ms, "h2d": h2d // args.steps, "d2h": d2h // args.steps}

    clocks = sampler.stop() if rank == 0 else None

    if args.trace:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            for i in range(2):
                step(dev_tokens[i % n_batches])
            barrier()
        prof.export_chrome_trace(f"{args.trace}.rank{rank}.json")

    # max over ranks
    if par == "fsdp" and world > 1:
        t = torch.tensor([ms_total, e2e["ms_total"] if e2e else 0.0], dtype=torch.float64).to(device).float()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t[0].cpu())
        if e2e:
            e2e["ms_total"] = float(t[1].cpu())

    tokens_per_step = B * S * world
    ms_per_step = ms_total / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)
    if rank == 0:
        out = {
            "metric": "llama7b_fsdp2_train_tokens_per_s",
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic (token ids uniform in [0,32000) from a seed; random-init weights)",
            "impl": args.impl,
            "config": {
                "model": "llama-7b (32L d4096 h32 ffn11008 vocab32000)" if args.layers == 32 else f"llama-7b-dims-{args.layers}L (INVALID: reduced layers)",
                "global_batch": B * world,
                "seq_len": S,
                "parallelism": (f"fsdp2x{world} per-layer, bf16 params / fp32 master+reduce" if par == "fsdp" else "single-device bf16"),
                "optimizer": "fused AdamW lr 3e-4",
                "cache": "working set per step (13.5 GB bf16 weights + activations) is far larger than the 126 MB L2",
            },
            "final_loss": final_loss,
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if e2e:
            out["e2e"] = {"value": tokens_per_step / (e2e["ms_total"] / args.steps / 1e3), "unit": "tokens/s",
                          "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]}
        if ours:
            out["fallback_ops"] = len(bw.fallback_counts())
            if os.environ.get("B200_BENCH_VERBOSE"):
                sys.stderr.write("fallbacks: " + json.dumps(sorted(bw.fallback_counts().items(), key=lambda kv: -kv[1])) + "\n")
        print(json.dumps(out))
    if par == "fsdp":
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
