"""Test helpers: an operator test harness that checks a device operator against the CPU (forward, backward, in-place
and ``out=`` variants), comparators with per-dtype tolerances, and decorators that skip on machines without the device.

Parity: reference torch_musa/testing/base_test_tool.py:306-350 (OpTest), :52-175 (comparators), InplaceOpChek, and
the skip decorators of torch_musa/testing/__init__.py.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence

import torch

DEFAULT_TOLERANCES = {torch.float32: (1e-5, 1e-5), torch.float64: (1e-8, 1e-8), torch.bfloat16: (2e-2, 2e-2),
                      torch.float16: (2e-3, 2e-3)}


class DefaultComparator:
    def __init__(self, abs_diff: Optional[float] = None, rel_diff: Optional[float] = None, equal_nan: bool = False):
        self.abs_diff, self.rel_diff, self.equal_nan = abs_diff, rel_diff, equal_nan

    def __call__(self, result: torch.Tensor, golden: torch.Tensor) -> bool:
        if result.shape != golden.shape:
            return False
        atol, rtol = DEFAULT_TOLERANCES.get(result.dtype, (0.0, 0.0))
        atol = self.abs_diff if self.abs_diff is not None else atol
        rtol = self.rel_diff if self.rel_diff is not None else rtol
        a, b = result.detach().cpu(), golden.detach().cpu()
        if not a.is_floating_point():
            return bool(torch.equal(a, b.to(a.dtype)))
        return bool(torch.allclose(a.double(), b.double(), atol=atol, rtol=rtol, equal_nan=self.equal_nan))


class AbsDiffComparator(DefaultComparator):
    def __init__(self, abs_diff: float = 1e-3):
        super().__init__(abs_diff=abs_diff, rel_diff=0.0)


class RelDiffComparator(DefaultComparator):
    def __init__(self, rel_diff: float = 1e-3):
        super().__init__(abs_diff=0.0, rel_diff=rel_diff)


def device_available() -> bool:
    try:
        import torch_musa_b200 as bw

        return bw.is_available()
    except Exception:
        return False


def skip_if_no_device(fn: Callable) -> Callable:
    import functools
    import unittest

    @functools.wraps(fn)
    def wrapper(*a, **k):
        if not device_available():
            raise unittest.SkipTest("no blackwell device")
        return fn(*a, **k)

    return wrapper


def skip_if_not_multi_device(n: int = 2):
    def deco(fn):
        import functools
        import unittest

        @functools.wraps(fn)
        def wrapper(*a, **k):
            import torch_musa_b200 as bw

            if not device_available() or bw.device_count() < n:
                raise unittest.SkipTest(f"needs {n} blackwell devices")
            return fn(*a, **k)

        return wrapper

    return deco


class OpTest:
    """Runs ``func(**inputs)`` on the CPU (fp32 oracle for half types) and on the device and compares outputs and,
    for inputs that require grad, gradients."""

    def __init__(self, func: Callable, input_args: Optional[Dict] = None, comparators: Optional[Sequence] = None,
                 device: str = "blackwell", ignored_result_indices: Sequence[int] = ()):
        self.func, self.inputs = func, dict(input_args or {})
        self.comparators = list(comparators or [DefaultComparator()])
        self.device = device
        self.ignored = set(ignored_result_indices)

    def _move(self, v, device, dtype=None):
        if isinstance(v, torch.Tensor):
            t = v.detach().clone()
            if dtype is not None and t.is_floating_point():
                t = t.to(dtype)
            t = t.to(device)
            return t.requires_grad_(v.requires_grad)
        if isinstance(v, (list, tuple)):
            return type(v)(self._move(x, device, dtype) for x in v)
        return v

    def _run(self, device, dtype, train):
        kw = {k: self._move(v, device, dtype) for k, v in self.inputs.items()}
        out = self.func(**kw)
        outs = list(out) if isinstance(out, (tuple, list)) else [out]
        grads = {}
        if train:
            loss = sum(o.float().sum() for o in outs if isinstance(o, torch.Tensor) and o.requires_grad)
            if isinstance(loss, torch.Tensor):
                loss.backward()
            grads = {k: v.grad for k, v in kw.items() if isinstance(v, torch.Tensor) and v.grad is not None}
        return outs, grads

    def check_result(self, train: bool = False, dtype: Optional[torch.dtype] = None):
        oracle_dtype = torch.float32 if dtype in (torch.bfloat16, torch.float16) else dtype
        ref_o, ref_g = self._run("cpu", oracle_dtype, train)
        dev_o, dev_g = self._run(self.device, dtype, train)
        assert len(ref_o) == len(dev_o), "different number of outputs"
        cmp = self.comparators[0]
        for i, (a, b) in enumerate(zip(dev_o, ref_o)):
            if i in self.ignored or not isinstance(a, torch.Tensor):
                continue
            assert a.device.type == torch.device(self.device).type, f"output {i} left the device"
            assert cmp(a.float() if a.is_floating_point() else a, b.float() if b.is_floating_point() else b), \
                f"output {i} of {getattr(self.func, '__name__', self.func)} differs from the CPU"
        for k in ref_g:
            assert k in dev_g, f"no gradient for {k} on the device"
            assert cmp(dev_g[k].float(), ref_g[k].float()), f"gradient of {k} differs from the CPU"

    def check_out_ops(self, dtype: Optional[torch.dtype] = None):
        """``out=`` variant writes into (and returns) the given tensor."""
        kw = {k: self._move(v, self.device, dtype) for k, v in self.inputs.items()}
        expect = self.func(**kw)
        out = torch.empty_like(expect)
        res = self.func(**kw, out=out)
        assert res.data_ptr() == out.data_ptr() and self.comparators[0](out, expect)


class InplaceOpCheck:
    """An in-place method must return its input (same storage) and equal the out-of-place result."""

    def __init__(self, inplace_name: str, functional: Callable, device: str = "blackwell"):
        self.inplace_name, self.functional, self.device = inplace_name, functional, device

    def check(self, x: torch.Tensor, *args, comparator=None):
        comparator = comparator or DefaultComparator()
        xd = x.detach().clone().to(self.device)
        expect = self.functional(x.detach().clone().to(self.device), *args)
        ptr = xd.data_ptr()
        ret = getattr(xd, self.inplace_name)(*args)
        assert ret.data_ptr() == ptr and xd.data_ptr() == ptr, "in-place operator reallocated its input"
        assert comparator(xd, expect)
