#!/usr/bin/env python
"""Headline benchmark: Llama-7B training throughput (tokens/s) with FSDP2 per-layer sharding.

  python bench.py --gpus N --steps K --warmup W            (N > 1: launched under torch.distributed.run)
  python bench.py --impl reference ...                     (the unmodified reference: unavailable, see below)
  python bench.py --impl stock ...                         (same model on stock PyTorch CUDA + NCCL)
  python bench.py --config resnet50_ddp|llama_tp|moe_ep    (the other configurations of the baseline table)

Config (headline): 32 layers, d_model 4096, 32 heads, SwiGLU FFN 11008, RMSNorm eps 1e-5, RoPE theta 1e4,
vocab 32000, seq 4096, micro-batch 1 per GPU, bf16 compute with fp32 master weights / fp32 gradient reduce,
fused AdamW lr 3e-4, synthetic token ids uniform in [0, 32000) from a seed, random-init weights.
Prints ONE JSON line on rank 0.  After its own measurement the "ours" arm runs the stock arm as a child process on
the same GPUs (same N, steps and warm-up; never overlapping a timed region) and reports ``vs_baseline`` = own value /
stock value; ``--no-baseline`` skips that.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading

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
    p.add_argument("--no-baseline", action="store_true", help="do not run the stock arm after the measurement")
    p.add_argument("--fsdp-mode", default="fused_adamw", choices=["fused_adamw", "fused", "stock_collectives"],
                   help="ours, llama_fsdp: AdamW inside the gradient reduce kernel / fused gather+reduce with the "
                        "ordinary fused AdamW / torch's FSDP2 collectives on the process group")
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


class Env:
    """Process-level facts every workload needs: rank, device module, backend names."""

    def __init__(self, args):
        import torch

        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        self.ours = args.impl == "ours"
        if self.ours:
            import torch_musa_b200 as bw

            self.bw, self.devmod, self.devtype, self.backend = bw, bw, "blackwell", "bccl"
        else:
            self.bw, self.devmod, self.devtype, self.backend = None, torch.cuda, "cuda", "nccl"
        self.device = torch.device(self.devtype, self.local_rank)
        self.devmod.set_device(self.local_rank)
        self.pg = False

    def init_pg(self):
        import torch.distributed as dist

        dist.init_process_group(backend=self.backend, rank=self.rank, world_size=self.world,
                                device_id=self.device if not self.ours else None)
        self.pg = True

    def barrier(self):
        if self.pg:
            import torch.distributed as dist

            dist.barrier()
        self.devmod.synchronize()


class Workload:
    """What one configuration provides to the timing scaffold."""

    metric = unit = ""
    data = "synthetic"
    units_per_step = 0            # tokens or images per step over all ranks
    config: dict = {}
    host_batches: list = []       # per batch: tuple of pinned host tensors

    def to_device(self, host, non_blocking=False):
        raise NotImplementedError

    def step(self, batch):        # one full training step; returns the loss tensor
        raise NotImplementedError

    def extra(self) -> dict:      # keys added to the JSON line
        return {}


# ------------------------------------------------------------------------------------------------ workloads
class LlamaFSDP(Workload):
    """Llama-7B, FSDP2 per layer, bf16 parameters for compute over fp32 masters, fp32 gradient reduce, AdamW."""

    metric, unit = "llama7b_fsdp2_train_tokens_per_s", "tokens/s"
    data = "synthetic (token ids uniform in [0,32000) from a seed; random-init weights)"

    def __init__(self, args, env: Env):
        import torch

        ours = env.ours
        have_backend = env.bw.distributed.is_bccl_available() if ours else True
        par = args.parallelism
        if par == "auto":
            par = "fsdp" if (have_backend or env.world > 1) else "single"
        if env.world > 1 and par != "fsdp":
            raise SystemExit("multi-GPU runs use FSDP2")
        if par == "fsdp":
            env.init_pg()
        if ours:
            from torch_musa_b200.models import Llama, LlamaConfig
        else:
            llama_mod, _, _ = _stock_package()
            Llama, LlamaConfig = llama_mod.Llama, llama_mod.LlamaConfig
        cfg = LlamaConfig(n_layers=args.layers, max_seq_len=args.seq)
        torch.manual_seed(1234)
        with torch.device("meta"):
            model = Llama(cfg)
        self.engine = None
        mode = args.fsdp_mode if (ours and par == "fsdp") else "stock_collectives"
        if par == "fsdp":
            from torch.distributed.device_mesh import init_device_mesh
            from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

            mesh = init_device_mesh(env.devtype, (env.world,))
            mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
            for layer in model.layers:
                fully_shard(layer, mesh=mesh, mp_policy=mp)
            fully_shard(model, mesh=mesh, mp_policy=mp)
            model.to_empty(device=env.device)
        else:
            model.to_empty(device=env.device)
            model = model.to(torch.bfloat16)
        with torch.no_grad():
            for p in model.parameters():
                if p.dim() >= 2:
                    p.normal_(0.0, 0.02)
                else:
                    p.fill_(1.0)
            model.init_rope_cache(env.device)
        hp = dict(lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
        if mode != "stock_collectives":
            from torch_musa_b200.parallel import fsdp as bw_fsdp

            try:
                self.engine = bw_fsdp.install_fused_collectives(model, fused_adamw=dict(hp, eps=1e-8) if mode == "fused_adamw" else None)
            except (RuntimeError, ValueError) as e:
                # the peer-mapped arena could not be set up (the same on every rank: its creation is collective); the
                # step then runs on the process group's all_gather / reduce_scatter and says so in its record
                self.install_error = f"{type(e).__name__}: {e}"[:300]
                mode = "stock_collectives"
        if self.engine is not None and self.engine.optimizer is not None:
            opt = self.engine.optimizer
        else:
            opt = torch.optim.AdamW(model.parameters(), fused=True, **hp)
        self.model, self.opt, self.env, self.par, self.mode = model, opt, env, par, mode
        B, S = args.micro_batch, args.seq
        gen = torch.Generator().manual_seed(1000 + env.rank)
        self.host_batches = [(torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen).pin_memory(),) for _ in range(4)]
        self.units_per_step = B * S * env.world
        self.config = {
            "model": "llama-7b (32L d4096 h32 ffn11008 vocab32000)" if args.layers == 32 else f"llama-7b-dims-{args.layers}L (INVALID: reduced layers)",
            "global_batch": B * env.world, "seq_len": S,
            "parallelism": (f"fsdp2x{env.world} per-layer, bf16 params / fp32 master+reduce" if par == "fsdp" else "single-device bf16"),
            "optimizer": "fused AdamW lr 3e-4" + (" (inside the gradient reduce kernel)" if mode == "fused_adamw" else ""),
            "collectives": {"fused_adamw": "own kernels: gather into final layout, reduce + AdamW epilogue",
                            "fused": "own kernels: gather into final layout, reduce to fp32 shard",
                            "stock_collectives": "process group all_gather / reduce_scatter"}[mode] if par == "fsdp" else "none",
            "cache": "working set per step (13.5 GB bf16 weights + activations) is far larger than the 126 MB L2",
        }

    def to_device(self, host, non_blocking=False):
        return (host[0].to(self.env.device, non_blocking=non_blocking),)

    def step(self, batch):
        tok = batch[0]
        loss = self.model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        return loss

    def extra(self):
        out = {}
        if getattr(self, "install_error", None):
            out["fused_install_error"] = self.install_error
        if self.engine is not None:
            self.engine.check()
            out["fused_collective_count"] = self.engine.fused_collective_count
            out["fused_kernel_calls"] = dict(self.engine.calls)
            if self.engine.skipped:
                out["fused_skipped_groups"] = self.engine.skipped
        return out


class ResNetDDP(Workload):
    """ResNet-50 DDP: bf16 autocast over fp32 master weights, channels-last, per-GPU batch 256 of 3x224x224 N(0,1)
    images, SGD momentum 0.9 (fused multi-tensor optimizer), 25 MB gradient buckets."""

    metric, unit = "resnet50_ddp_train_images_per_s", "images/s"
    data = "synthetic (images N(0,1), labels uniform in [0,1000) from a seed; random-init weights)"

    def __init__(self, args, env: Env):
        import torch

        ours = env.ours
        if ours:
            from torch_musa_b200.models import resnet50
        else:
            resnet50 = _load_by_path("_stock_resnet", "models/resnet.py").resnet50
        use_ddp = env.world > 1
        if use_ddp:
            env.init_pg()
        torch.manual_seed(1234)
        model = resnet50(1000).to(env.device).to(memory_format=torch.channels_last)
        if use_ddp:
            if ours:
                from torch_musa_b200.parallel.ddp import wrap_ddp

                net = wrap_ddp(model, device_ids=[env.local_rank], bucket_cap_mb=25, gradient_as_bucket_view=True)
            else:
                net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[env.local_rank], bucket_cap_mb=25,
                                                                gradient_as_bucket_view=True)
        else:
            net = model
        if ours:
            from torch_musa_b200.optim import FusedSGD

            opt = FusedSGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
        else:
            opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4, fused=True)
        self.net, self.opt, self.env = net, opt, env
        B = args.batch
        gen = torch.Generator().manual_seed(1000 + env.rank)
        self.host_batches = [(torch.randn(B, 3, 224, 224, generator=gen).pin_memory(),
                              torch.randint(0, 1000, (B,), generator=gen).pin_memory()) for _ in range(2)]
        self.units_per_step = B * env.world
        self.config = {"model": "resnet-50 (torchvision layout, 1000 classes)", "global_batch": B * env.world,
                       "image": "3x224x224", "parallelism": f"ddp{env.world}, 25 MB buckets" if use_ddp else "single device",
                       "precision": "bf16 autocast, fp32 master weights, channels-last",
                       "optimizer": "fused multi-tensor SGD momentum 0.9",
                       "cache": "activations per step (several GB) are far larger than the 126 MB L2"}

    def to_device(self, host, non_blocking=False):
        import torch

        x = host[0].to(self.env.device, non_blocking=non_blocking).contiguous(memory_format=torch.channels_last)
        return (x, host[1].to(self.env.device, non_blocking=non_blocking))

    def step(self, batch):
        import torch
        import torch.nn.functional as F

        with torch.autocast(self.env.devtype, dtype=torch.bfloat16):
            loss = F.cross_entropy(self.net(batch[0]), batch[1])
        loss.backward()
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        return loss


class LlamaTP(Workload):
    """Llama-7B architecture, tensor parallel over all ranks (column-parallel q/k/v/gate/up, row-parallel o/down,
    sequence-parallel norms, vocabulary-parallel loss), bf16, one sequence of 2048 tokens per GPU in the batch
    (batch 8 x 2048 at TP=8); forward + backward + fused AdamW step."""

    metric, unit = "llama7b_tp_train_tokens_per_s", "tokens/s"
    data = "synthetic (token ids uniform in [0,32000) from a seed; random-init weights)"

    def __init__(self, args, env: Env):
        import torch

        ours, world = env.ours, env.world
        if ours:
            from torch_musa_b200.models.llama import LlamaConfig
            from torch_musa_b200.models.llama_tp import TPLlama
        else:
            llama_mod, _, _ = _stock_package()
            LlamaConfig = llama_mod.LlamaConfig
            TPLlama = _load_by_path("_stock_pkg.models.llama_tp", "models/llama_tp.py").TPLlama
        if world > 1:
            env.init_pg()
        B, S = world, 2048
        cfg = LlamaConfig(n_layers=args.layers, max_seq_len=S)
        torch.manual_seed(1234)
        with torch.device(env.device):
            model = TPLlama(cfg, world).to(torch.bfloat16)
        with torch.no_grad():
            for p in model.parameters():
                if p.dim() >= 2:
                    p.normal_(0.0, 0.02)
        self.fused = None
        if ours and world > 1:
            from torch_musa_b200.parallel.fused_tp import FusedTensorParallel

            T = B * S
            # all-gather -> GEMM runs as one launch; GEMM -> reduce-scatter stays GEMM + the backend's reduce-scatter
            # kernel unless B200_TP_FUSED_RS=1 (the one-launch version is slower with few ranks, see profiles/)
            fused_rs = os.environ.get("B200_TP_FUSED_RS", "0") == "1"
            self.fused = FusedTensorParallel(max_shard_bytes=T // world * cfg.dim * 2, max_rows=T, device=env.device,
                                             max_partial_bytes=T * cfg.dim * 2 if fused_rs else 0).install()
        self.opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
        gen = torch.Generator().manual_seed(1000)          # every rank sees the same batch: tensor parallelism
        self.host_batches = [(torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen).pin_memory(),) for _ in range(4)]
        self.partial_grad = model.replicated_parameters()
        self.model, self.env = model, env
        self.units_per_step = B * S
        self.config = {"model": "llama-7b (32L d4096 h32 ffn11008 vocab32000)" if args.layers == 32 else f"llama-7b-dims-{args.layers}L (INVALID: reduced layers)",
                       "global_batch": B, "seq_len": S,
                       "parallelism": f"tp{world}: colwise q/k/v/gate/up, rowwise o/down, sequence-parallel norms, vocab-parallel loss",
                       "optimizer": "fused AdamW lr 3e-4 on bf16 parameters",
                       "cache": "weights and activations per step are far larger than the 126 MB L2"}

    def to_device(self, host, non_blocking=False):
        return (host[0].to(self.env.device, non_blocking=non_blocking),)

    def step(self, batch):
        import torch
        import torch.distributed as dist

        tok = batch[0]
        loss = self.model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        if self.env.world > 1:
            flat = torch.cat([p.grad.reshape(-1) for p in self.partial_grad])
            dist.all_reduce(flat)
            off = 0
            for p in self.partial_grad:
                p.grad.copy_(flat[off:off + p.numel()].view_as(p.grad))
                off += p.numel()
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        return loss

    def extra(self):
        if self.fused is None:
            return {}
        self.fused.check()
        return {"fused_collective_calls": {"allgather_gemm": self.fused.calls, "gemm_reduce_scatter": self.fused.rs_calls}}


class MoEEP(Workload):
    """Mixtral-style MoE decoder, expert parallel over all ranks: 8 layers, d 4096, 8 SwiGLU experts of 14336,
    top-2 router, 8192 tokens per GPU, bf16 parameters and activations, fused AdamW; forward + backward + step."""

    metric, unit = "moe_ep_train_tokens_per_s", "tokens/s"
    data = "synthetic (token ids uniform in [0,32000) from a seed; random-init weights)"

    def __init__(self, args, env: Env):
        import torch

        ours, world = env.ours, env.world
        if ours:
            from torch_musa_b200.models import MoEConfig, MoETransformer
            from torch_musa_b200.parallel import moe as pmoe
        else:
            _, moe_mod, pmoe = _stock_package()
            MoEConfig, MoETransformer = moe_mod.MoEConfig, moe_mod.MoETransformer
        if world > 1:
            env.init_pg()
        B, S = 2, 4096
        cfg = MoEConfig(n_layers=args.layers if args.layers != 32 else 8, max_seq_len=S, synthetic_router_logits=True)
        torch.manual_seed(1234)
        with torch.device(env.device):
            model = MoETransformer(cfg, ep_world=world).to(torch.bfloat16)
        with torch.no_grad():
            for p in model.parameters():
                if p.dim() >= 2:
                    p.normal_(0.0, 0.02)
        if ours:
            self.exchange = pmoe.make_expert_exchange(cfg.n_experts, cfg.dim, B * S, cfg.top_k, slots=cfg.n_layers,
                                                      device=env.device, capacity_factor=cfg.capacity_factor)
        else:
            self.exchange = pmoe.ReferenceExpertExchange(cfg.n_experts)
        model.set_exchange(self.exchange)
        self.replicated = model.replicated_parameters()
        self.experts = model.expert_parameters()
        self.opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
        gen = torch.Generator().manual_seed(1000 + env.rank)
        self.host_batches = [(torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen).pin_memory(),) for _ in range(4)]
        self.model, self.env = model, env
        self.units_per_step = B * S * world
        self.config = {"model": f"mixtral-style moe ({cfg.n_layers}L d4096 h32/kv8, 8 experts x ffn14336, top-2)",
                       "global_batch": B * world, "seq_len": S, "tokens_per_gpu": B * S,
                       "parallelism": f"ep{world} ({cfg.n_experts // world} expert(s) per GPU), replicated attention/router",
                       "expert_gemm": getattr(cfg, "expert_gemm", "bf16"),
                       "router": "top-2 softmax over logits drawn N(0,1) per token",
                       "optimizer": "fused AdamW lr 3e-4 on bf16 parameters",
                       "cache": "weights and activations per step are far larger than the 126 MB L2"}

    def to_device(self, host, non_blocking=False):
        return (host[0].to(self.env.device, non_blocking=non_blocking),)

    def step(self, batch):
        import torch
        import torch.distributed as dist

        tok = batch[0]
        loss = self.model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        if self.env.world > 1:
            grads = [p.grad for p in self.replicated if p.grad is not None]
            flat = torch.cat([g.reshape(-1) for g in grads])
            dist.all_reduce(flat, op=dist.ReduceOp.AVG)
            off = 0
            for g in grads:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()
            torch._foreach_mul_([p.grad for p in self.experts if p.grad is not None], 1.0 / self.env.world)
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        return loss

    def extra(self):
        if self.env.ours:
            self.exchange.check()
        return {}


WORKLOADS = {"llama_fsdp": LlamaFSDP, "resnet50_ddp": ResNetDDP, "llama_tp": LlamaTP, "moe_ep": MoEEP}


# ------------------------------------------------------------------------------------------------ scaffold
def measure(args, env: Env, wl: Workload) -> dict:
    """Warm-up, the device-timed region (inputs resident), the end-to-end region (pinned host inputs copied in and
    the loss read back every step), clocks sampled during both; times are CUDA events, max over ranks."""
    import torch
    import torch.distributed as dist

    devmod, rank = env.devmod, env.rank
    nb = len(wl.host_batches)
    dev_batches = [wl.to_device(h) for h in wl.host_batches]
    for i in range(args.warmup):
        wl.step(dev_batches[i % nb])
    env.barrier()
    sampler = ClockSampler(env.local_rank)
    if rank == 0:
        sampler.start()
    if env.ours:
        env.bw.reset_kernel_launch_count()
    ev0, ev1 = devmod.Event(enable_timing=True), devmod.Event(enable_timing=True)
    env.barrier()
    ev0.record()
    for i in range(args.steps):
        loss = wl.step(dev_batches[i % nb])
    ev1.record()
    env.barrier()
    ms_total = ev0.elapsed_time(ev1)
    launches = env.bw.kernel_launch_count() if env.ours else 0
    final_loss = float(loss.detach().float().cpu())

    e2e_ms, h2d, d2h = 0.0, 0, 0
    if not args.no_e2e:
        env.barrier()
        ev2, ev3 = devmod.Event(enable_timing=True), devmod.Event(enable_timing=True)
        ev2.record()
        for i in range(args.steps):
            batch = wl.to_device(wl.host_batches[i % nb], non_blocking=True)
            h2d += sum(t.numel() * t.element_size() for t in wl.host_batches[i % nb])
            lv = wl.step(batch).detach().float().cpu()      # device -> host read of the step's result
            d2h += lv.numel() * lv.element_size()
        ev3.record()
        env.barrier()
        e2e_ms = ev2.elapsed_time(ev3)
    clocks = sampler.stop() if rank == 0 else None
    if args.trace:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            for i in range(2):
                wl.step(dev_batches[i % nb])
            env.barrier()
        prof.export_chrome_trace(f"{args.trace}.rank{rank}.json")
    extra = wl.extra()
    if env.pg and env.world > 1:
        t = torch.tensor([ms_total, e2e_ms], dtype=torch.float64).to(env.device).float()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = float(t[0].cpu()), float(t[1].cpu())
    ms_per_step = ms_total / args.steps
    out = {
        "metric": wl.metric, "value": wl.units_per_step / (ms_per_step / 1e3), "unit": wl.unit, "n_gpus": env.world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": wl.data, "impl": args.impl,
        "config": wl.config, "final_loss": final_loss, "gpu_launches": launches, "clocks": clocks,
    }
    if not args.no_e2e:
        out["e2e"] = {"value": wl.units_per_step / (e2e_ms / args.steps / 1e3), "unit": wl.unit,
                      "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": d2h // args.steps}
    out.update(extra)
    if env.ours:
        out["fallback_ops"] = len(env.bw.fallback_counts())
        if out["fallback_ops"]:
            # which operators ran on a library kernel instead of one of this repository's (name: calls)
            out["fallback_op_names"] = dict(sorted(env.bw.fallback_counts().items(), key=lambda kv: -kv[1])[:12])
        if os.environ.get("B200_BENCH_VERBOSE") and rank == 0:
            sys.stderr.write("fallbacks: " + json.dumps(sorted(env.bw.fallback_counts().items(), key=lambda kv: -kv[1])) + "\n")
    else:
        out["sdpa_backend"] = os.environ.get("_B200_STOCK_SDPA", "default")
    return out


def run_stock_child(args, world: int) -> dict:
    """Runs the stock arm (same configuration, N, steps, warm-up) as a child process and returns its JSON line."""
    cmd = [sys.executable]
    port = int(os.environ.get("MASTER_PORT", "29511")) + 17     # this process's store still owns the original port
    if world > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                "--master-port", str(port)]
    cmd += [os.path.abspath(__file__), "--impl", "stock", "--gpus", str(world), "--steps", str(args.steps), "--warmup",
            str(args.warmup), "--config", args.config, "--layers", str(args.layers), "--seq", str(args.seq),
            "--micro-batch", str(args.micro_batch), "--batch", str(args.batch)]
    if args.no_e2e:
        cmd.append("--no-e2e")
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_PORT",
                                                           "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK",
                                                           "TORCHELASTIC_RUN_ID", "GROUP_WORLD_SIZE", "ROLE_WORLD_SIZE",
                                                           "TORCHELASTIC_RESTART_COUNT", "TORCHELASTIC_MAX_RESTARTS",
                                                           "TORCHELASTIC_USE_AGENT_STORE", "TORCH_NCCL_ASYNC_ERROR_HANDLING",
                                                           "TORCHELASTIC_ERROR_FILE")}
    env["MASTER_PORT"] = str(port)
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=840, env=env)
    except subprocess.TimeoutExpired:
        return {"error": "stock arm did not finish in 840 s"}
    for line in reversed(r.stdout.strip().splitlines()):
        line = line.strip()
        if line.startswith("{") and '"metric"' in line:
            try:
                return json.loads(line)
            except ValueError:
                continue
    return {"error": f"stock arm exited {r.returncode}: {(r.stderr or r.stdout)[-400:]}"}


def main():
    args = parse()
    deadline = int(os.environ.get("B200_BENCH_DUMP_AFTER_S", "1500"))
    if deadline > 0:
        # a run normally ends within a few minutes; one that is still alive after the deadline prints every thread's
        # Python stack and exits instead of occupying the GPUs until somebody kills it (0 disables)
        import faulthandler

        faulthandler.dump_traceback_later(deadline, exit=True)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.impl == "stock":
        import torch
        from torch.nn.attention import SDPBackend, sdpa_kernel

        # the best stock attention on this GPU first (cuDNN fused attention), the others as fall-backs
        ctx = sdpa_kernel([SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION,
                           SDPBackend.MATH], set_priority=True)
        ctx.__enter__()
        os.environ["_B200_STOCK_SDPA"] = "priority: cudnn, flash, efficient, math"
    env = Env(args)
    wl = WORKLOADS[args.config](args, env)
    out = measure(args, env, wl)
    world, rank = env.world, env.rank
    if env.pg:
        import torch.distributed as dist

        dist.destroy_process_group()
    if rank != 0:
        return 0
    if env.ours and not args.no_baseline:
        # free this process's device memory before the stock arm needs it (the other ranks have exited by now or
        # are about to: nothing of this run is timed any more)
        import gc

        import torch

        del wl
        gc.collect()
        env.bw.synchronize()
        env.bw.empty_cache()
        base = run_stock_child(args, world)
        if "value" in base:
            out["vs_baseline"] = out["value"] / base["value"]
            out["baseline"] = {"impl": "stock PyTorch CUDA + NCCL, same box, same run", "value": base["value"],
                               "ms_per_step": base["ms_per_step"], "e2e": (base.get("e2e") or {}).get("value"),
                               "sdpa_backend": base.get("sdpa_backend"), "steps": base["steps"], "warmup": base["warmup"]}
            if out.get("e2e") and base.get("e2e"):
                out["baseline"]["e2e_ratio"] = out["e2e"]["value"] / base["e2e"]["value"]
        else:
            out["baseline"] = base
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
