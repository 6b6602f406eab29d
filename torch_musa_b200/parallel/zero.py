"""Data-parallel training with a sharded optimizer whose gradient reduce-scatter, fp32 cast and AdamW update are
ONE kernel per bucket.

``ShardedFusedAdamW`` flattens bf16 parameters (and their gradients) into one buffer cut into buckets of
``world * bucket`` elements; rank r owns slice r of every bucket: an fp32 master copy and both Adam moments of that
slice only (optimizer state / world per GPU).  ``step()`` runs, per bucket,

  1. ``reduce_scatter_adamw``: every rank reads its slice of the bucket's gradients from all peers over NVLink,
     sums them in fp32 registers, applies the 1/world scale and the AdamW update to its master slice and moments and
     writes the updated bf16 slice -- the reduced gradient never exists in memory;
  2. an all-gather of the updated bf16 slices back into the flat parameter buffer (the backend's pull kernel).

Parity: the reference reduces gradients with a library reduce-scatter and then launches its fused optimizer
(reference torch_musa/distributed/fsdp/_runtime_utils.py:71-130, torch_musa/optim/fused_adamw.py); there is no
fused path.
"""
from __future__ import annotations

from typing import Iterable, List

import torch
import torch.distributed as dist

from ._symm import group_store_and_key


class ShardedFusedAdamW:
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, group=None, bucket_mb: int = 32, fused: bool = True):
        import torch_musa_b200 as bw

        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        assert self.params and all(p.dtype == torch.bfloat16 for p in self.params), "bf16 parameters expected"
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        dev = self.params[0].device
        self.device = dev
        total = sum(p.numel() for p in self.params)
        self.bs = max(8, (bucket_mb << 20) // 2 // self.world // 8 * 8)          # elements per rank per bucket
        chunk = self.bs * self.world
        self.n_buckets = (total + chunk - 1) // chunk
        padded = self.n_buckets * chunk
        self.flat_p = torch.zeros(padded, dtype=torch.bfloat16, device=dev)
        self.flat_g = torch.zeros(padded, dtype=torch.bfloat16, device=dev)
        off = 0
        with torch.no_grad():
            for p in self.params:
                n = p.numel()
                self.flat_p[off:off + n].copy_(p.reshape(-1))
                p.data = self.flat_p[off:off + n].view_as(p)
                p.grad = self.flat_g[off:off + n].view_as(p)
                off += n
        shard = self.n_buckets * self.bs
        self.p32 = torch.empty(shard, dtype=torch.float32, device=dev)
        for b in range(self.n_buckets):
            src = self.flat_p[b * chunk + self.rank * self.bs: b * chunk + (self.rank + 1) * self.bs]
            self.p32[b * self.bs:(b + 1) * self.bs].copy_(src)
        self.m = torch.zeros_like(self.p32)
        self.v = torch.zeros_like(self.p32)
        self.p16 = torch.empty(self.bs, dtype=torch.bfloat16, device=dev)
        self.step_t = torch.zeros((), dtype=torch.float32, device=dev)
        self.fused = fused and dev.type == "blackwell" and self.world > 1
        self.sm = None
        if self.fused:
            store, key = group_store_and_key(group, "zero_arena")
            self.sm = bw._C._create_symmetric_memory(store, key, self.rank, self.world,
                                                     dev.index or 0, 2 * chunk * 2)
            if not self.sm.ok:
                self.fused, self.sm = False, None

    def zero_grad(self) -> None:
        """Gradients live in the flat buffer (views): zero it in one pass."""
        self.flat_g.zero_()
        for p, g in zip(self.params, self._grad_views()):
            p.grad = g

    def _grad_views(self):
        off = 0
        for p in self.params:
            n = p.numel()
            yield self.flat_g[off:off + n].view_as(p)
            off += n

    def _grads_finite(self) -> bool:
        """True when no gradient element on any rank is inf / nan (one small all-reduce and one host read)."""
        ok = torch.isfinite(self.flat_g).all().to(torch.float32).reshape(1)
        if self.world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        return bool(ok.item() > 0)

    def step_with_scaler(self, scaler) -> bool:
        """One step under dynamic loss scaling (``torch.amp.GradScaler`` used as the holder of the scale and of its
        growth / backoff policy): gradients are divided by the scale inside the update kernel; a step whose gradients
        are not finite on some rank is skipped on every rank and the scale backs off; after ``growth_interval`` good
        steps in a row the scale grows.  Returns whether the update was applied."""
        scale = float(scaler.get_scale())
        applied = self.step(grad_scale=scale, check_finite=True)
        self._good_steps = getattr(self, "_good_steps", 0) + 1 if applied else 0
        def set_scale(value: float) -> None:
            try:
                scaler.update(value)
            except AssertionError:      # the scaler creates its state on the first `scale()` call: make that call
                scaler.scale(torch.zeros((), device=self.device))
                scaler.update(value)

        if not applied:
            set_scale(scale * scaler.get_backoff_factor())
        elif self._good_steps >= scaler.get_growth_interval():
            set_scale(scale * scaler.get_growth_factor())
            self._good_steps = 0
        return applied

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, check_finite: bool = False) -> bool:
        """``grad_scale``: the factor the loss was multiplied by (the gradients are divided by it on the fly);
        ``check_finite``: leave parameters and state untouched and return False when a gradient is inf / nan."""
        if check_finite and not self._grads_finite():
            return False
        self.step_t += 1
        chunk = self.bs * self.world
        b1, b2 = self.betas
        inv = 1.0 / float(grad_scale)
        for b in range(self.n_buckets):
            g = self.flat_g[b * chunk:(b + 1) * chunk]
            sl = slice(b * self.bs, (b + 1) * self.bs)
            if self.fused:
                self.sm.reduce_scatter_adamw(g, self.p32[sl], self.m[sl], self.v[sl], self.p16, self.step_t, self.lr, b1,
                                             b2, self.eps, self.wd, inv / self.world)
            else:
                if self.world > 1:
                    gs = torch.empty(self.bs, dtype=torch.float32, device=self.device)
                    dist.reduce_scatter_tensor(gs, g.float(), op=dist.ReduceOp.SUM, group=self.group)
                    gs *= inv / self.world
                else:
                    gs = g.float() * inv if inv != 1.0 else g.float()
                p, m, v = self.p32[sl], self.m[sl], self.v[sl]
                step = float(self.step_t)
                p.mul_(1 - self.lr * self.wd)
                m.mul_(b1).add_(gs, alpha=1 - b1)
                v.mul_(b2).addcmul_(gs, gs, value=1 - b2)
                denom = (v.sqrt() / (1 - b2 ** step) ** 0.5).add_(self.eps)
                p.addcdiv_(m, denom, value=-self.lr / (1 - b1 ** step))
                self.p16.copy_(p)
            out = self.flat_p[b * chunk:(b + 1) * chunk]
            if self.world > 1:
                dist.all_gather_into_tensor(out, self.p16, group=self.group)
            else:
                out.copy_(self.p16)
        return True

    def check(self) -> None:
        if self.sm is not None:
            st = self.sm.take_status()
            if st:
                raise RuntimeError(f"a sharded-optimizer kernel gave up on a bounded wait (status {st})")

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self) -> dict:
        """This rank's shard of the optimizer state (fp32 master weights and both moments, bucket-major as the step
        uses them) plus the hyper-parameters; save one per rank, or gather with ``full_state_dict``."""
        return {"step": float(self.step_t), "lr": self.lr, "betas": tuple(self.betas), "eps": self.eps,
                "weight_decay": self.wd, "world": self.world, "rank": self.rank, "bucket_elems": self.bs,
                "master": self.p32.detach().cpu(), "exp_avg": self.m.detach().cpu(), "exp_avg_sq": self.v.detach().cpu()}

    def load_state_dict(self, sd: dict) -> None:
        if sd["world"] != self.world or sd["rank"] != self.rank or sd["bucket_elems"] != self.bs:
            raise ValueError("optimizer shard was saved for a different world size, rank or bucket size")
        self.lr, self.betas, self.eps, self.wd = sd["lr"], tuple(sd["betas"]), sd["eps"], sd["weight_decay"]
        self.step_t.fill_(sd["step"])
        with torch.no_grad():
            self.p32.copy_(sd["master"])
            self.m.copy_(sd["exp_avg"])
            self.v.copy_(sd["exp_avg_sq"])
            # parameters follow the restored master weights
            chunk = self.bs * self.world
            for b in range(self.n_buckets):
                self.p16.copy_(self.p32[b * self.bs:(b + 1) * self.bs])
                out = self.flat_p[b * chunk:(b + 1) * chunk]
                if self.world > 1:
                    dist.all_gather_into_tensor(out, self.p16, group=self.group)
                else:
                    out.copy_(self.p16)

    def full_state_dict(self) -> dict:
        """Per-parameter ``exp_avg`` / ``exp_avg_sq`` / fp32 master tensors in the parameters' shapes, assembled from
        every rank's shard (a collective call).  The layout torch's AdamW uses, for tools that expect it."""
        def gather(shard: torch.Tensor) -> torch.Tensor:
            chunk = self.bs * self.world
            full = torch.empty(self.n_buckets * chunk, dtype=shard.dtype, device=shard.device)
            for b in range(self.n_buckets):
                out = full[b * chunk:(b + 1) * chunk]
                piece = shard[b * self.bs:(b + 1) * self.bs].contiguous()
                if self.world > 1:
                    dist.all_gather_into_tensor(out, piece, group=self.group)
                else:
                    out.copy_(piece)
            return full
        flats = {"master": gather(self.p32), "exp_avg": gather(self.m), "exp_avg_sq": gather(self.v)}
        state, off = {}, 0
        for i, p in enumerate(self.params):
            n = p.numel()
            state[i] = {k: v[off:off + n].view_as(p).cpu() for k, v in flats.items()}
            state[i]["step"] = float(self.step_t)
            off += n
        return {"state": state, "param_groups": [{"lr": self.lr, "betas": tuple(self.betas), "eps": self.eps,
                                                  "weight_decay": self.wd, "params": list(range(len(self.params)))}]}
