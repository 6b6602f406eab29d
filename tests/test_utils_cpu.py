"""Developer utilities that need no GPU: debugging dispatch modes, profiler analyses, test harness."""
import pytest
import torch

from torch_musa_b200.utils import CompareWithCPU, ModuleTracker, NanInfTracker
from torch_musa_b200 import profiler as bprof
from torch_musa_b200.testing import DefaultComparator, InplaceOpCheck, OpTest


def test_compare_and_nan_modes():
    m = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.ReLU())
    with CompareWithCPU(device_type="cpu") as c, ModuleTracker(m):
        m(torch.randn(2, 4)).sum().backward()
    assert c.records and not c.mismatches() and any(r["module"] == "0" for r in c.records)
    with pytest.raises(FloatingPointError, match="NaN"):
        with NanInfTracker():
            torch.log(torch.tensor([-1.0]))
    with NanInfTracker(raise_error=False) as t:
        torch.log(torch.tensor([-1.0]))
    assert t.hits and t.hits[0]["nan"] == 1


def test_profiler_analyses():
    from torch.profiler import ProfilerActivity, profile

    a, b = torch.randn(33, 17), torch.randn(17, 9)
    with profile(activities=[ProfilerActivity.CPU], record_shapes=True) as prof:
        for _ in range(3):
            (a @ b).relu()
        torch.zeros(4).to(torch.float64)
    ev = bprof.BasicEvaluation(prof)
    assert "aten::mm" in ev.ops and ev.ops["aten::mm"].calls == 3
    finds = bprof.find_antipatterns(prof)
    assert any(f.pattern == "matmul dimension alignment" for f in finds)
    assert "anti-pattern" in bprof.report(prof)


def test_op_harness_on_cpu():
    x = torch.randn(3, 5, requires_grad=True)
    OpTest(lambda input: torch.tanh(input) * 2, {"input": x}, device="cpu").check_result(train=True)
    OpTest(torch.add, {"input": torch.randn(4), "other": torch.randn(4)}, device="cpu").check_out_ops()
    InplaceOpCheck("mul_", torch.mul, device="cpu").check(torch.randn(6), 3.0)
    assert not DefaultComparator()(torch.zeros(2), torch.ones(2))
