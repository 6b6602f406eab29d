"""Operator-level debugging modes.

* ``OpDumper``: records every dispatched operator that touches the device (or all, if asked): name, argument
  shapes / dtypes / strides, simple statistics of inputs and outputs, and optionally the tensors themselves as
  ``.pt`` files, so a failing step can be replayed operator by operator on another machine.
* ``DoubleToFloat``: runs fp64 operators in fp32 and casts the results back.  fp64 arithmetic runs at a small
  fraction of the fp32 rate on this GPU; the mode trades the precision for that speed in code that only uses
  doubles out of habit (index arithmetic, schedules), and reports which operators it touched.

Both are ``TorchDispatchMode`` context managers and work on any device (the CPU tests run them on CPU tensors).
Parity: reference torch_musa/csrc/utils/register_wrapper.cpp:29-131 (per-operator wrapper that dumps inputs and
outputs and casts double arguments to float for kernels without fp64 support).
"""
from __future__ import annotations

import json
import os
import re
from collections import Counter
from typing import Any, Dict, List, Optional

import torch
from torch.utils._python_dispatch import TorchDispatchMode
from torch.utils._pytree import tree_flatten, tree_map


def _describe(t: Any, stats: bool) -> Any:
    if not isinstance(t, torch.Tensor):
        return repr(t) if not isinstance(t, (int, float, bool, str, type(None))) else t
    d: Dict[str, Any] = {"shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", ""), "device": str(t.device),
                         "stride": list(t.stride())}
    if stats and t.numel() and (t.is_floating_point() or t.dtype in (torch.int32, torch.int64, torch.bool)):
        f = t.detach().float()
        d.update(min=float(f.min()), max=float(f.max()), mean=float(f.mean()),
                 nan=int(torch.isnan(f).sum()), inf=int(torch.isinf(f).sum()))
    return d


class OpDumper(TorchDispatchMode):
    def __init__(self, directory: Optional[str] = None, ops: str = ".*", device_type: Optional[str] = "blackwell",
                 save_tensors: bool = False, stats: bool = True, max_records: int = 10000):
        super().__init__()
        self.directory = directory
        self.pattern = re.compile(ops)
        self.device_type = device_type
        self.save_tensors = save_tensors
        self.stats = stats
        self.max_records = max_records
        self.records: List[Dict[str, Any]] = []
        if directory:
            os.makedirs(directory, exist_ok=True)

    def _wanted(self, name: str, flat: List[Any]) -> bool:
        if not self.pattern.search(name):
            return False
        if self.device_type is None:
            return True
        return any(isinstance(a, torch.Tensor) and a.device.type == self.device_type for a in flat)

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        out = func(*args, **kwargs)
        name = func._schema.name + ("." + func._schema.overload_name if func._schema.overload_name else "")
        flat_in, _ = tree_flatten((args, kwargs))
        if len(self.records) < self.max_records and self._wanted(name, flat_in):
            idx = len(self.records)
            flat_out, _ = tree_flatten(out)
            rec = {"index": idx, "op": name,
                   "inputs": [_describe(a, self.stats) for a in flat_in],
                   "outputs": [_describe(a, self.stats) for a in flat_out]}
            self.records.append(rec)
            if self.directory and self.save_tensors:
                cpu = lambda t: t.detach().cpu() if isinstance(t, torch.Tensor) else t  # noqa: E731
                torch.save({"op": name, "args": tree_map(cpu, args), "kwargs": tree_map(cpu, kwargs),
                            "out": tree_map(cpu, out)},
                           os.path.join(self.directory, f"{idx:06d}_{name.replace('::', '.')}.pt"))
        return out

    def __exit__(self, *exc):
        r = super().__exit__(*exc)
        if self.directory:
            with open(os.path.join(self.directory, "ops.json"), "w") as f:
                json.dump(self.records, f, indent=1)
        return r

    def summary(self) -> Counter:
        return Counter(r["op"] for r in self.records)

    def first_non_finite(self) -> Optional[Dict[str, Any]]:
        """The first recorded operator whose output holds a NaN or Inf while its inputs did not."""
        for r in self.records:
            bad_out = any(isinstance(o, dict) and (o.get("nan") or o.get("inf")) for o in r["outputs"])
            bad_in = any(isinstance(i, dict) and (i.get("nan") or i.get("inf")) for i in r["inputs"])
            if bad_out and not bad_in:
                return r
        return None


class DoubleToFloat(TorchDispatchMode):
    # operators whose meaning depends on the dtype argument itself
    _SKIP = re.compile(r"aten::(_to_copy|to|empty|empty_like|empty_strided|zeros|ones|full|arange|scalar_tensor|"
                       r"_local_scalar_dense|item|copy_|clone|detach|view|_unsafe_view|as_strided|lift_fresh)")

    def __init__(self, device_type: Optional[str] = "blackwell"):
        super().__init__()
        self.device_type = device_type
        self.touched: Counter = Counter()

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        name = func._schema.name
        flat, _ = tree_flatten((args, kwargs))
        has64 = any(isinstance(a, torch.Tensor) and a.dtype == torch.float64 and
                    (self.device_type is None or a.device.type == self.device_type) for a in flat)
        if not has64 or self._SKIP.match(name) or func._schema.is_mutable:
            return func(*args, **kwargs)
        down = lambda a: a.to(torch.float32) if isinstance(a, torch.Tensor) and a.dtype == torch.float64 else a  # noqa: E731
        out = func(*tree_map(down, args), **tree_map(down, kwargs))
        self.touched[name] += 1
        up = lambda a: a.to(torch.float64) if isinstance(a, torch.Tensor) and a.dtype == torch.float32 else a  # noqa: E731
        return tree_map(up, out)
