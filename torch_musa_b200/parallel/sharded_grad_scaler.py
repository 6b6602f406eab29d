"""Loss scaling for sharded (FSDP / ZeRO) training.

A rank only sees its shard of every gradient, so "did any gradient overflow?" has to be agreed on by the whole
process group before anybody steps: otherwise some ranks skip the step and the shards of one parameter diverge.
``ShardedGradScaler`` unscales the local shards (one fused multi-tensor kernel per device and dtype on the blackwell
device, plain tensor math for CPU-offloaded shards), reduces ONE found-inf flag with ``MAX`` over the group, and only
then decides.  It accepts DTensor parameters (FSDP2) as well as flat-parameter shards (FSDP1) and keeps
``torch.amp.GradScaler``'s interface and ``state_dict`` format.

Parity: reference torch_musa/distributed/fsdp/sharded_grad_scaler.py:34-374 (a port of torch's scaler to the MUSA
device); this one is written against the public tensor API and has no per-device replicator machinery, because a
rank drives exactly one device.
"""
from __future__ import annotations

from collections import defaultdict
from enum import Enum
from typing import Dict, Iterable, List, Optional

import torch
import torch.distributed as dist


class _Stage(Enum):
    READY = 0
    UNSCALED = 1
    STEPPED = 2


def _local(t: torch.Tensor) -> torch.Tensor:
    return t._local_tensor if hasattr(t, "_local_tensor") else t


class ShardedGradScaler:
    def __init__(self, device: str = "blackwell", init_scale: float = 2.0 ** 16, growth_factor: float = 2.0,
                 backoff_factor: float = 0.5, growth_interval: int = 2000, enabled: bool = True,
                 process_group=None):
        if growth_factor <= 1.0 or not 0.0 < backoff_factor < 1.0:
            raise ValueError("growth_factor must be > 1 and backoff_factor in (0, 1)")
        self._device = device
        self._enabled = enabled
        self._init_scale, self._growth_factor, self._backoff_factor = init_scale, growth_factor, backoff_factor
        self._growth_interval = growth_interval
        self.process_group = process_group
        self._scale: Optional[torch.Tensor] = None        # fp32 scalar on the first loss's device
        self._growth_tracker: Optional[torch.Tensor] = None
        self._per_optimizer: Dict[int, dict] = defaultdict(lambda: {"stage": _Stage.READY, "found_inf": None})

    # ---------------------------------------------------------------- state
    def is_enabled(self) -> bool:
        return self._enabled

    def _lazy_init(self, device: torch.device) -> None:
        if self._scale is None:
            self._scale = torch.full((), self._init_scale, dtype=torch.float32, device=device)
            self._growth_tracker = torch.zeros((), dtype=torch.int32, device=device)

    def get_scale(self) -> float:
        if not self._enabled:
            return 1.0
        return self._init_scale if self._scale is None else float(self._scale)

    def get_growth_factor(self) -> float:
        return self._growth_factor

    def get_backoff_factor(self) -> float:
        return self._backoff_factor

    def get_growth_interval(self) -> int:
        return self._growth_interval

    def state_dict(self) -> dict:
        if not self._enabled:
            return {}
        return {"scale": self.get_scale(), "growth_factor": self._growth_factor,
                "backoff_factor": self._backoff_factor, "growth_interval": self._growth_interval,
                "_growth_tracker": 0 if self._growth_tracker is None else int(self._growth_tracker)}

    def load_state_dict(self, sd: dict) -> None:
        if not self._enabled:
            return
        if not sd:
            raise RuntimeError("the state dict comes from a disabled scaler")
        self._init_scale = sd["scale"]
        self._growth_factor, self._backoff_factor = sd["growth_factor"], sd["backoff_factor"]
        self._growth_interval = sd["growth_interval"]
        if self._scale is not None:
            self._scale.fill_(sd["scale"])
            self._growth_tracker.fill_(sd["_growth_tracker"])
        else:
            self._pending_tracker = sd["_growth_tracker"]

    # ---------------------------------------------------------------- scale
    def scale(self, outputs):
        """Multiplies a loss (or a nested list / tuple of losses) by the current scale."""
        if not self._enabled:
            return outputs
        if isinstance(outputs, torch.Tensor):
            self._lazy_init(outputs.device)
            if hasattr(self, "_pending_tracker"):
                self._growth_tracker.fill_(self._pending_tracker)
                del self._pending_tracker
            # the product keeps the loss's dtype: FSDP's mixed precision returns 16-bit losses
            return outputs * self._scale.to(device=outputs.device, dtype=outputs.dtype, non_blocking=True)
        if isinstance(outputs, (list, tuple)):
            return type(outputs)(self.scale(o) for o in outputs)
        raise ValueError("outputs must be a tensor or a list / tuple of tensors")

    # ---------------------------------------------------------------- unscale
    def _unscale_shards(self, grads: List[torch.Tensor], inv_scale: torch.Tensor) -> torch.Tensor:
        """Divides the local gradient shards by the scale in place; returns a 0/1 fp32 flag on the scale's device."""
        found = torch.zeros((), dtype=torch.float32, device=inv_scale.device)
        buckets: Dict[tuple, List[torch.Tensor]] = defaultdict(list)
        for g in grads:
            buckets[(g.device, g.dtype)].append(g)
        for (dev, _dt), items in buckets.items():
            if dev.type == "cpu":
                # offloaded shards: no fused kernel on the host
                bad = False
                for g in items:
                    g.mul_(inv_scale.to("cpu", g.dtype) if g.dtype != torch.float16 else float(inv_scale))
                    bad = bad or not bool(torch.isfinite(g).all())
                if bad:
                    found.fill_(1.0)
            else:
                flag = torch.zeros(1, dtype=torch.float32, device=dev)
                torch._amp_foreach_non_finite_check_and_unscale_(items, flag, inv_scale.to(dev).reshape(()))
                found = torch.maximum(found, flag.reshape(()).to(found.device))
        return found

    def unscale_(self, optimizer) -> None:
        if not self._enabled:
            return
        st = self._per_optimizer[id(optimizer)]
        if st["stage"] is _Stage.UNSCALED:
            raise RuntimeError("unscale_() has already been called on this optimizer since the last update().")
        if st["stage"] is _Stage.STEPPED:
            raise RuntimeError("unscale_() is being called after step().")
        if self._scale is None:
            raise RuntimeError("Attempted unscale_ but _scale is None; call scale(loss) first")
        grads = []
        for group in optimizer.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = _local(p.grad)
                if g.is_sparse:
                    g = g.coalesce()._values()
                if g.numel():
                    grads.append(g)
        inv_scale = self._scale.double().reciprocal().float()
        found = self._unscale_shards(grads, inv_scale)
        # one flag for the whole group: every rank takes the same decision
        if dist.is_available() and dist.is_initialized():
            pg = self.process_group
            if dist.get_world_size(pg) > 1:
                backend = dist.get_backend(pg)
                if found.device.type == "cpu" and backend not in ("gloo",):
                    carrier = found.to(self._device)
                    dist.all_reduce(carrier, op=dist.ReduceOp.MAX, group=pg)
                    found = carrier.to("cpu")
                else:
                    dist.all_reduce(found, op=dist.ReduceOp.MAX, group=pg)
        st["found_inf"] = found
        st["stage"] = _Stage.UNSCALED

    # ---------------------------------------------------------------- step / update
    def step(self, optimizer, *args, **kwargs):
        if not self._enabled:
            return optimizer.step(*args, **kwargs)
        st = self._per_optimizer[id(optimizer)]
        if st["stage"] is _Stage.STEPPED:
            raise RuntimeError("step() has already been called since the last update().")
        if st["stage"] is _Stage.READY:
            self.unscale_(optimizer)
        ret = None
        if float(st["found_inf"]) == 0.0:
            ret = optimizer.step(*args, **kwargs)
        st["stage"] = _Stage.STEPPED
        return ret

    def update(self, new_scale=None) -> None:
        if not self._enabled or self._scale is None:
            return
        if new_scale is not None:
            self._scale.fill_(float(new_scale))
        else:
            flags = [s["found_inf"] for s in self._per_optimizer.values() if s["found_inf"] is not None]
            if not flags:
                raise RuntimeError("No inf checks were recorded prior to update.")
            found = flags[0].to(self._scale.device)
            for f in flags[1:]:
                found = torch.maximum(found, f.to(self._scale.device))
            if self._scale.device.type == "cpu":
                if float(found) > 0:
                    self._scale.mul_(self._backoff_factor)
                    self._growth_tracker.zero_()
                else:
                    self._growth_tracker.add_(1)
                    if int(self._growth_tracker) >= self._growth_interval:
                        self._scale.mul_(self._growth_factor)
                        self._growth_tracker.zero_()
            else:
                torch._amp_update_scale_(self._scale, self._growth_tracker, found.reshape(1), self._growth_factor,
                                         self._backoff_factor, self._growth_interval)
        self._per_optimizer.clear()
