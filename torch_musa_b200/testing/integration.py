"""End-to-end training / evaluation runs with quality gates: the harness behind "train this model for a few epochs on
this device under these execution strategies and require top-1 accuracy above X".

    run = IntegrationRun(model=resnet18(), optimizer=lambda p: torch.optim.Adam(p, 1e-3), loss_fn=nn.CrossEntropyLoss(),
                         train_batches=train_loader, test_batches=test_loader, epochs=2, device="blackwell",
                         strategies=[TF32(True), AMP(torch.bfloat16), ChannelsLast()],
                         evaluators={"top": TopKAccuracy((1, 5))},
                         gates={"top.top1": GreaterThan(0.80), "top.top5": GreaterThan(0.98)})
    report = run.run()          # raises AssertionError naming every gate that failed; report holds metrics and timings

Strategies come in three kinds, distinguished by the hooks they override: a *global* context around the whole run
(TF32), a *model transform* applied once before training (channels-last), a *step* context around every forward pass
(autocast).  Evaluators accumulate (prediction, target) pairs and produce a dict of numbers; gates address them as
"<evaluator>.<key>" (or "train_loss" / "seconds_per_epoch").  No dataset or checkpoint is downloaded here: callers hand
in iterables of (input, target) batches.

Parity: reference torch_musa/testing/integration/{config,strategy,evalautor,assertion,metrics}.py and the recipes in
tests/integration/vision/resnet/test_resnet_train.py:21-76 (ResNet-50 on CIFAR-10 with top-1 / top-5 gates).
"""
from __future__ import annotations

import contextlib
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch


# ------------------------------------------------------------------------------------------------ strategies
class Strategy:
    """Base: every hook is a no-op."""

    name = "strategy"

    def global_context(self):
        return contextlib.nullcontext()

    def transform(self, model: torch.nn.Module, device: torch.device) -> torch.nn.Module:
        return model

    def transform_input(self, x):
        return x

    def step_context(self, device: torch.device):
        return contextlib.nullcontext()


class TF32(Strategy):
    """fp32 matrix products on the tensor cores at tf32 precision (or strictly fp32 when disabled) for the run."""

    name = "tf32"

    def __init__(self, enabled: bool = True):
        self.enabled = enabled

    @contextlib.contextmanager
    def global_context(self):
        prev = (torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32)
        torch.backends.cuda.matmul.allow_tf32 = torch.backends.cudnn.allow_tf32 = self.enabled
        try:
            yield
        finally:
            torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = prev


class AMP(Strategy):
    """Autocast around every forward pass (loss included)."""

    name = "amp"

    def __init__(self, dtype: torch.dtype = torch.bfloat16, enabled: bool = True):
        self.dtype, self.enabled = dtype, enabled

    def step_context(self, device: torch.device):
        return torch.autocast(device.type, dtype=self.dtype, enabled=self.enabled)


class ChannelsLast(Strategy):
    """NHWC memory format for the model's 4-D parameters and for 4-D inputs."""

    name = "channels_last"

    def transform(self, model, device):
        return model.to(memory_format=torch.channels_last)

    def transform_input(self, x):
        return x.contiguous(memory_format=torch.channels_last) if isinstance(x, torch.Tensor) and x.dim() == 4 else x


# ------------------------------------------------------------------------------------------------ evaluators
class Evaluator:
    def append(self, prediction: torch.Tensor, target: torch.Tensor) -> None:
        raise NotImplementedError

    def evaluate(self) -> Dict[str, float]:
        raise NotImplementedError

    def zero_state(self) -> None:
        raise NotImplementedError


class TopKAccuracy(Evaluator):
    """Fraction of samples whose target is among the k highest scores: keys ``top<k>``."""

    def __init__(self, ks: Sequence[int] = (1,)):
        self.ks = tuple(sorted(ks))
        self.zero_state()

    def zero_state(self):
        self.hits, self.n = {k: 0 for k in self.ks}, 0

    def append(self, prediction, target):
        top = prediction.detach().float().topk(min(self.ks[-1], prediction.shape[-1]), dim=-1).indices.cpu()
        t = target.detach().cpu().view(-1, 1)
        for k in self.ks:
            self.hits[k] += int((top[:, :k] == t).any(-1).sum())
        self.n += t.shape[0]

    def evaluate(self):
        return {f"top{k}": self.hits[k] / max(self.n, 1) for k in self.ks}


class F1Score(Evaluator):
    """Binary F1 over thresholded scores (or boolean predictions): keys ``precision``, ``recall``, ``f1``."""

    def __init__(self, threshold: float = 0.5):
        self.threshold = threshold
        self.zero_state()

    def zero_state(self):
        self.tp = self.fp = self.fn = 0

    def append(self, prediction, target):
        p = prediction.detach().cpu()
        p = p if p.dtype == torch.bool else p.float() > self.threshold
        t = target.detach().cpu().bool()
        self.tp += int((p & t).sum())
        self.fp += int((p & ~t).sum())
        self.fn += int((~p & t).sum())

    def evaluate(self):
        prec = self.tp / max(self.tp + self.fp, 1)
        rec = self.tp / max(self.tp + self.fn, 1)
        return {"precision": prec, "recall": rec, "f1": 2 * prec * rec / max(prec + rec, 1e-12)}


class JaccardIndex(Evaluator):
    """Intersection over union of boolean masks, accumulated over the batches: key ``iou``."""

    def __init__(self, threshold: float = 0.5):
        self.threshold = threshold
        self.zero_state()

    def zero_state(self):
        self.inter = self.union = 0

    def append(self, prediction, target):
        p = prediction.detach().cpu()
        p = p if p.dtype == torch.bool else p.float() > self.threshold
        t = target.detach().cpu().bool()
        self.inter += int((p & t).sum())
        self.union += int((p | t).sum())

    def evaluate(self):
        return {"iou": self.inter / max(self.union, 1)}


# ------------------------------------------------------------------------------------------------ gates
class Gate:
    def check(self, value) -> Optional[str]:
        """None when the value passes, else a message."""
        raise NotImplementedError


class GreaterThan(Gate):
    def __init__(self, bound: float):
        self.bound = bound

    def check(self, value):
        return None if value > self.bound else f"{value:.6g} is not greater than {self.bound:.6g}"


class LessThan(Gate):
    def __init__(self, bound: float):
        self.bound = bound

    def check(self, value):
        return None if value < self.bound else f"{value:.6g} is not less than {self.bound:.6g}"


# ------------------------------------------------------------------------------------------------ the run
Batch = Tuple[Any, torch.Tensor]


@dataclass
class IntegrationRun:
    model: torch.nn.Module
    loss_fn: Callable
    train_batches: Optional[Iterable[Batch]] = None          # None: evaluation only
    test_batches: Optional[Iterable[Batch]] = None
    optimizer: Optional[Callable[[Iterable[torch.nn.Parameter]], torch.optim.Optimizer]] = None
    epochs: int = 1
    device: Any = "cpu"
    strategies: List[Strategy] = field(default_factory=list)
    evaluators: Dict[str, Evaluator] = field(default_factory=dict)
    gates: Dict[str, Gate] = field(default_factory=dict)
    grad_scaler: Optional[Any] = None                        # e.g. torch.amp.GradScaler for fp16 autocast
    log: Optional[Callable[[str], None]] = None

    def summary(self) -> str:
        mode = "train+eval" if self.train_batches is not None else "eval"
        names = ", ".join(s.name for s in self.strategies) or "none"
        return f"{type(self.model).__name__} [{mode}] on {self.device}, strategies: {names}, epochs: {self.epochs}"

    # -- helpers
    def _to(self, x, dev):
        if isinstance(x, torch.Tensor):
            x = x.to(dev)
            for s in self.strategies:
                x = s.transform_input(x)
            return x
        if isinstance(x, (list, tuple)):
            return type(x)(self._to(v, dev) for v in x)
        if isinstance(x, dict):
            return {k: self._to(v, dev) for k, v in x.items()}
        return x

    def _forward(self, model, x):
        if isinstance(x, dict):
            return model(**x)
        if isinstance(x, (list, tuple)):
            return model(*x)
        return model(x)

    @contextlib.contextmanager
    def _step(self, dev):
        with contextlib.ExitStack() as stack:
            for s in self.strategies:
                stack.enter_context(s.step_context(dev))
            yield

    def _sync(self, dev):
        if dev.type != "cpu":
            mod = getattr(torch, dev.type, None)
            if mod is not None and hasattr(mod, "synchronize"):
                mod.synchronize()

    # -- the run
    def run(self) -> Dict[str, Any]:
        dev = torch.device(self.device)
        say = self.log or (lambda _m: None)
        say(self.summary())
        report: Dict[str, Any] = {"summary": self.summary()}
        with contextlib.ExitStack() as stack:
            for s in self.strategies:
                stack.enter_context(s.global_context())
            model = self.model.to(dev)
            for s in self.strategies:
                model = s.transform(model, dev)
            if self.train_batches is not None:
                if self.optimizer is None:
                    raise ValueError("training needs an optimizer factory")
                opt = self.optimizer(model.parameters())
                model.train()
                per_epoch = []
                for epoch in range(self.epochs):
                    self._sync(dev)
                    t0, total, n = time.perf_counter(), 0.0, 0
                    for x, y in self.train_batches:
                        x, y = self._to(x, dev), self._to(y, dev)
                        with self._step(dev):
                            loss = self.loss_fn(self._forward(model, x), y)
                        opt.zero_grad(set_to_none=True)
                        if self.grad_scaler is not None:
                            self.grad_scaler.scale(loss).backward()
                            self.grad_scaler.step(opt)
                            self.grad_scaler.update()
                        else:
                            loss.backward()
                            opt.step()
                        total += float(loss.detach())
                        n += 1
                    self._sync(dev)
                    per_epoch.append(time.perf_counter() - t0)
                    report["train_loss"] = total / max(n, 1)
                    say(f"epoch {epoch}: loss {report['train_loss']:.4f} in {per_epoch[-1]:.2f} s")
                report["seconds_per_epoch"] = sum(per_epoch) / max(len(per_epoch), 1)
            if self.test_batches is not None and self.evaluators:
                model.eval()
                for ev in self.evaluators.values():
                    ev.zero_state()
                with torch.no_grad():
                    for x, y in self.test_batches:
                        x, y = self._to(x, dev), self._to(y, dev)
                        with self._step(dev):
                            out = self._forward(model, x)
                        for ev in self.evaluators.values():
                            ev.append(out, y)
                for name, ev in self.evaluators.items():
                    for key, value in ev.evaluate().items():
                        report[f"{name}.{key}"] = value
        failures = []
        for key, gate in self.gates.items():
            if key not in report:
                failures.append(f"{key}: no such metric (have {sorted(k for k in report if k != 'summary')})")
                continue
            msg = gate.check(report[key])
            if msg:
                failures.append(f"{key}: {msg}")
        report["gates_passed"] = not failures
        if failures:
            raise AssertionError("integration gates failed: " + "; ".join(failures) + f" [{self.summary()}]")
        return report


def default_strategy_sets() -> List[List[Strategy]]:
    """The combinations a recipe is normally run under: plain fp32, tf32, bf16 autocast, fp16 autocast."""
    return [[TF32(False)], [TF32(True)], [AMP(torch.bfloat16)], [AMP(torch.float16)]]
