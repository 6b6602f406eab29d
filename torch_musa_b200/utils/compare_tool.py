"""Debugging modes: run every operator on the CPU as well and compare (``CompareWithCPU``), or scan every
operator's outputs for NaN / Inf (``NanInfTracker``), with the module path that issued the operator.

Both are ``TorchDispatchMode``s, so they see the ATen operators after autograd and autocast, exactly what the
device executes.  Usage::

    with CompareWithCPU(atol=1e-3, rtol=1e-3, verbose=False) as cmp, ModuleTracker(model):
        model(x).sum().backward()
    print(cmp.summary())

Parity: reference torch_musa/utils/compare_tool.py:718-1031 (CompareWithCPU, NanInfTracker, module tracker).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
from torch.utils._python_dispatch import TorchDispatchMode
from torch.utils._pytree import tree_flatten, tree_map

_module_stack: List[str] = []


class ModuleTracker:
    """Records which ``nn.Module`` (by qualified name) is executing, for the reports of the modes below."""

    def __init__(self, root: torch.nn.Module):
        self.root = root
        self._handles = []

    def __enter__(self):
        for name, mod in self.root.named_modules():
            label = name or type(self.root).__name__
            def _enter(m, a, label=label):
                _module_stack.append(label)

            def _leave(m, a, o):
                if _module_stack:
                    _module_stack.pop()

            self._handles.append(mod.register_forward_pre_hook(_enter))
            self._handles.append(mod.register_forward_hook(_leave))
        return self

    def __exit__(self, *exc):
        for h in self._handles:
            h.remove()
        self._handles.clear()
        _module_stack.clear()


def current_module() -> str:
    return _module_stack[-1] if _module_stack else "<no module>"


def _to_cpu(x):
    if isinstance(x, torch.Tensor) and x.device.type != "cpu":
        y = x.detach().cpu()
        return y.float() if y.dtype in (torch.bfloat16, torch.float16) else y
    if isinstance(x, torch.Tensor):
        return x.detach()
    return x


_SKIP = ("aten::empty", "aten::_to_copy", "aten::copy_", "aten::detach", "aten::view", "aten::_unsafe_view",
         "aten::as_strided", "aten::native_dropout", "aten::uniform_", "aten::normal_", "aten::randn", "aten::rand",
         "aten::bernoulli_", "aten::lift_fresh", "aten::alias", "aten::empty_like", "aten::empty_strided",
         "aten::new_empty")


class CompareWithCPU(TorchDispatchMode):
    """Re-executes every device operator on CPU copies of its inputs (fp32 for half types) and compares."""

    def __init__(self, atol: float = 1e-3, rtol: float = 1e-3, verbose: bool = False, device_type: str = "blackwell",
                 raise_on_mismatch: bool = False):
        super().__init__()
        self.atol, self.rtol, self.verbose = atol, rtol, verbose
        self.device_type = device_type
        self.raise_on_mismatch = raise_on_mismatch
        self.records: List[Dict[str, Any]] = []

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        out = func(*args, **kwargs)
        name = func._schema.name
        flat_in, _ = tree_flatten((args, kwargs))
        on_dev = any(isinstance(t, torch.Tensor) and t.device.type == self.device_type for t in flat_in)
        if not on_dev or name.startswith(_SKIP):
            return out
        try:
            ref = func(*tree_map(_to_cpu, args), **tree_map(_to_cpu, kwargs))
        except Exception as e:  # operators without a CPU kernel (custom fused ops) cannot be cross-checked
            self.records.append({"op": name, "module": current_module(), "status": "no-cpu", "detail": str(e)[:80]})
            return out
        flat_o, _ = tree_flatten(out)
        flat_r, _ = tree_flatten(ref)
        worst, ok = 0.0, True
        for o, r in zip(flat_o, flat_r):
            if not (isinstance(o, torch.Tensor) and isinstance(r, torch.Tensor)) or not o.is_floating_point():
                continue
            a, b = o.detach().cpu().float(), r.float()
            if a.shape != b.shape:
                ok = False
                continue
            if a.numel():
                diff = (a - b).abs()
                worst = max(worst, float(diff.max()))
                tol = self.atol + self.rtol * b.abs()
                if o.dtype in (torch.bfloat16, torch.float16):
                    tol = tol + 1e-2 * b.abs().max().clamp_min(1.0)
                ok = ok and bool((diff <= tol).all())
        rec = {"op": name, "module": current_module(), "status": "ok" if ok else "MISMATCH", "max_abs_diff": worst}
        self.records.append(rec)
        if self.verbose or not ok:
            print(f"[compare] {rec['status']:8s} {name} in {rec['module']} max|diff|={worst:.3e}")
        if not ok and self.raise_on_mismatch:
            raise RuntimeError(f"{name} disagrees with the CPU reference (max abs diff {worst:.3e}) in {rec['module']}")
        return out

    def mismatches(self) -> List[Dict[str, Any]]:
        return [r for r in self.records if r["status"] == "MISMATCH"]

    def summary(self) -> str:
        n = len(self.records)
        bad = self.mismatches()
        lines = [f"{n} operators compared, {len(bad)} mismatches, "
                 f"{sum(r['status'] == 'no-cpu' for r in self.records)} without a CPU reference"]
        lines += [f"  {r['op']} in {r['module']}: max|diff|={r['max_abs_diff']:.3e}" for r in bad[:20]]
        return "\n".join(lines)


class NanInfTracker(TorchDispatchMode):
    """Reports (or raises at) the first operator whose output contains NaN or Inf."""

    def __init__(self, raise_error: bool = True):
        super().__init__()
        self.raise_error = raise_error
        self.hits: List[Dict[str, Any]] = []

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        out = func(*args, **(kwargs or {}))
        flat, _ = tree_flatten(out)
        for i, t in enumerate(flat):
            if isinstance(t, torch.Tensor) and t.is_floating_point() and t.numel():
                finite = torch.isfinite(t.detach())
                if not bool(finite.all()):
                    td = t.detach()
                    rec = {"op": func._schema.name, "module": current_module(), "output": i,
                           "nan": int(torch.isnan(td).sum()), "inf": int(torch.isinf(td).sum())}
                    self.hits.append(rec)
                    msg = (f"{rec['op']} produced {rec['nan']} NaN / {rec['inf']} Inf in output {i} "
                           f"(module {rec['module']})")
                    if self.raise_error:
                        raise FloatingPointError(msg)
                    print("[nan-inf] " + msg)
        return out
