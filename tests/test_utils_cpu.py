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


def test_sharded_adamw_single_process_matches_torch():
    from torch_musa_b200.parallel.zero import ShardedFusedAdamW

    torch.manual_seed(0)
    base = [torch.randn(64, 32) * 0.1, torch.randn(32) * 0.1]
    ps = [torch.nn.Parameter(b.to(torch.bfloat16)) for b in base]
    ref = [torch.nn.Parameter(b.to(torch.bfloat16).float()) for b in base]
    o = ShardedFusedAdamW(ps, lr=1e-2, weight_decay=0.1, bucket_mb=1)
    r = torch.optim.AdamW(ref, lr=1e-2, weight_decay=0.1)
    for _ in range(3):
        o.zero_grad()
        for p, q in zip(ps, ref):
            g = (torch.randn(p.shape) * 0.05).to(torch.bfloat16)
            p.grad.copy_(g)
            q.grad = g.float()
        o.step()
        r.step()
    assert max(float((p.float() - q).abs().max()) for p, q in zip(ps, ref)) < 4e-3
    # checkpoint round trip: a fresh optimizer over fresh parameters continues exactly where this one stands
    sd = o.state_dict()
    ps2 = [torch.nn.Parameter(torch.zeros_like(p)) for p in ps]
    o2 = ShardedFusedAdamW(ps2, lr=1.0, weight_decay=0.0, bucket_mb=1)
    o2.load_state_dict(sd)
    assert all(torch.equal(a, b) for a, b in zip(ps, ps2))
    for opt, params in ((o, ps), (o2, ps2)):
        opt.zero_grad()
        for p in params:
            p.grad.copy_(torch.ones_like(p) * 0.25)
        opt.step()
    assert all(torch.equal(a, b) for a, b in zip(ps, ps2))
    full = o.full_state_dict()
    assert full["state"][0]["exp_avg"].shape == ps[0].shape and full["param_groups"][0]["lr"] == 1e-2


def test_comm_helpers_on_cpu_tensors():
    from torch_musa_b200.parallel import data_parallel as dp

    ts = [torch.randn(3, 4), torch.arange(5), torch.randn(7)]
    out = dp.broadcast_coalesced(ts, ["cpu", "cpu"], buffer_size=64)
    assert all(torch.equal(a, b) for copy_ in out for a, b in zip(copy_, ts))
    x = torch.arange(12.0).view(6, 2)
    parts = dp.scatter(x, ["cpu", "cpu", "cpu"])
    assert torch.equal(dp.gather(parts), x) and torch.equal(dp.reduce_add(parts), parts[0] + parts[1] + parts[2])


def test_kv_cache_decoder_matches_full_recompute_on_cpu():
    from torch_musa_b200.models import Llama, llama_tiny_config
    from torch_musa_b200.models.decode import LlamaDecoder

    cfg = llama_tiny_config(n_kv_heads=2)
    torch.manual_seed(0)
    m = Llama(cfg).eval()
    prompt = torch.randint(0, cfg.vocab_size, (3, 5))
    d = LlamaDecoder(m, 3, 32)
    d.prefill(prompt)
    got = d.decode(6)
    seq, want = prompt.clone(), []
    with torch.no_grad():
        for _ in range(6):
            nxt = m(seq)[:, -1].argmax(-1, keepdim=True)
            want.append(nxt)
            seq = torch.cat([seq, nxt], 1)
    assert torch.equal(got, torch.cat(want, 1))


def test_cpp_example_builds():
    """The stand-alone C++ example compiles and links against the in-tree kernel library (running it needs a GPU)."""
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.exists(os.path.join(root, "torch_musa_b200", "libb200_kernels.so")):
        import pytest

        pytest.skip("kernel library not built")
    r = subprocess.run(["make", "-C", os.path.join(root, "examples", "cpp"), "-B"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


def test_op_dumper_and_double_to_float(tmp_path):
    import json
    import torch
    from torch_musa_b200.utils.op_debug import DoubleToFloat, OpDumper

    x = torch.randn(4, 5)
    with OpDumper(str(tmp_path), ops="aten::(mm|log)", device_type=None, save_tensors=True) as d:
        y = x @ x.t()
        z = torch.log(y - 100.0)          # NaNs appear here
        _ = z + 1
    assert d.summary() == {"aten::mm": 1, "aten::log": 1}
    bad = d.first_non_finite()
    assert bad is not None and bad["op"] == "aten::log" and bad["outputs"][0]["nan"] > 0
    listed = json.load(open(tmp_path / "ops.json"))
    assert [r["op"] for r in listed] == ["aten::mm", "aten::log"]
    saved = torch.load(tmp_path / "000000_aten.mm.pt")
    assert torch.equal(saved["out"], y)

    a = torch.randn(8, 8, dtype=torch.float64)
    with DoubleToFloat(device_type=None) as m:
        b = a @ a
        c = torch.sin(b)
    assert b.dtype == torch.float64 and c.dtype == torch.float64
    assert m.touched["aten::mm"] == 1 and m.touched["aten::sin"] == 1
    assert not torch.equal(b, a @ a) and torch.allclose(b, a @ a, rtol=1e-4, atol=1e-4)   # computed in fp32


def _isolated_probe(x):
    import os

    return {"pid": os.getpid(), "twice": 2 * x}


def _rank_sum_body(rank, world, offset):
    import torch
    import torch.distributed as dist

    t = torch.tensor([float(rank + offset)])
    dist.all_reduce(t)
    assert float(t) == sum(r + offset for r in range(world))


def test_multi_process_harness():
    import os
    from torch_musa_b200.testing.distributed import MultiProcessTestCase, spawn_isolated_test

    out = spawn_isolated_test(_isolated_probe, 21)
    assert out["twice"] == 42 and out["pid"] != os.getpid()

    class Suite(MultiProcessTestCase):
        world_size = 3

    Suite().run_on_ranks(_rank_sum_body, 10)


def test_op_coverage_report_reads_the_dispatcher():
    from torch_musa_b200.utils import op_coverage

    r = op_coverage.report()
    assert r["native_base_operators"] > 150 and "mm" in r["native_by_base"] and "convolution_overrideable" in r["native_by_base"]
    assert any(n.startswith("blackwell::") for n in r["custom_operators"])
    assert r["covered_of_cuda"] <= r["cuda_base_operators"] and "mm" not in r["fallback_base_operators"]
    assert op_coverage.main(["--missing", "3"]) == 0


def test_integration_run_with_strategies_and_gates():
    """The end-to-end harness: a small classifier trained under autocast + channels-last must pass its accuracy gates;
    an unreachable gate is reported by name; evaluators compute what they say."""
    from torch import nn
    from torch_musa_b200.testing import integration as it

    torch.manual_seed(0)
    centres = torch.randn(4, 3, 4, 4) * 2.0

    def batches(n, seed):
        g = torch.Generator().manual_seed(seed)
        out = []
        for _ in range(n):
            y = torch.randint(0, 4, (32,), generator=g)
            out.append((centres[y] + 0.3 * torch.randn(32, 3, 4, 4, generator=g), y))
        return out

    def make():
        return nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.ReLU(), nn.Flatten(), nn.Linear(8 * 16, 4))

    lines = []
    run = it.IntegrationRun(model=make(), loss_fn=nn.CrossEntropyLoss(), train_batches=batches(30, 1), test_batches=batches(5, 2),
                            optimizer=lambda p: torch.optim.Adam(p, lr=1e-2), epochs=2, device="cpu",
                            strategies=[it.TF32(False), it.AMP(torch.bfloat16), it.ChannelsLast()],
                            evaluators={"top": it.TopKAccuracy((1, 2))},
                            gates={"top.top1": it.GreaterThan(0.9), "top.top2": it.GreaterThan(0.95), "train_loss": it.LessThan(0.5)},
                            log=lines.append)
    report = run.run()
    assert report["gates_passed"] and report["top.top1"] > 0.9 and report["seconds_per_epoch"] > 0
    assert "amp" in lines[0] and "channels_last" in lines[0] and len(lines) == 3
    bad = it.IntegrationRun(model=make(), loss_fn=nn.CrossEntropyLoss(), test_batches=batches(2, 3),
                            evaluators={"top": it.TopKAccuracy((1,))}, gates={"top.top1": it.GreaterThan(0.99), "nope": it.LessThan(1)})
    with pytest.raises(AssertionError, match="top.top1.*not greater than.*nope: no such metric"):
        bad.run()
    f1 = it.F1Score()
    f1.append(torch.tensor([0.9, 0.8, 0.1, 0.7]), torch.tensor([1, 0, 0, 1]))
    assert abs(f1.evaluate()["f1"] - 0.8) < 1e-9                      # tp 2, fp 1, fn 0
    j = it.JaccardIndex()
    j.append(torch.tensor([True, True, False, False]), torch.tensor([True, False, True, False]))
    assert abs(j.evaluate()["iou"] - 1 / 3) < 1e-9
    assert len(it.default_strategy_sets()) == 4


def test_cmake_description_configures(tmp_path):
    """The CMake build of the kernel library (an alternative to the package's own build script) configures: the
    compiler is found, the options parse, every kernel source is picked up.  (Compiling all kernels takes minutes and is
    what the package build already does.)"""
    import os
    import shutil
    import subprocess

    if not shutil.which("cmake") or not os.path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("cmake or nvcc not available")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run(["cmake", "-S", root, "-B", str(tmp_path), "-DCMAKE_CUDA_COMPILER=/usr/local/cuda/bin/nvcc",
                        "-DB200_USE_ASAN=ON", "-DB200_WERROR=ON"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    made = open(os.path.join(str(tmp_path), "CMakeFiles", "b200_kernels.dir", "build.make")).read()
    for name in ("gemm_tcgen05.cu", "gemm_grouped.cu", "attention_bwd.cu", "conv_tcgen05.cu", "decode_attn.cu"):
        assert name in made, name


def test_host_paths_of_grouped_linear_and_varlen_attention():
    """The device-independent compositions behind `grouped_linear`, `swiglu(row_counts=...)` and `flash_attn_varlen_func`
    (what runs on any other device, and the oracle of the GPU tests) against explicit per-group / per-sequence loops."""
    import torch.nn.functional as F
    from torch_musa_b200.ops import flash_attn_varlen_func, grouped_linear, swiglu

    torch.manual_seed(0)
    x, w = torch.randn(20, 6, requires_grad=True), torch.randn(3, 4, 6, requires_grad=True)
    counts = torch.tensor([5, 0, 9], dtype=torch.int32)
    y = grouped_linear(x, w, counts)
    assert y.shape == (20, 4) and torch.allclose(y[:5], x[:5] @ w[0].t()) and torch.allclose(y[5:14], x[5:14] @ w[2].t())
    assert bool((y[14:] == 0).all())
    y.sum().backward()
    assert torch.allclose(w.grad[1], torch.zeros(4, 6)) and bool((x.grad[14:] == 0).all())
    out = torch.full((20, 4), 7.0)
    assert grouped_linear(x.detach(), w.detach(), counts, out) is out and bool((out[14:] == 0).all())
    g = torch.randn(4, 8)
    assert torch.allclose(swiglu(g, counts), F.silu(g[:, :4]) * g[:, 4:])          # the host path computes every row
    lens = [3, 7, 1]
    cu = torch.tensor([0, 3, 10, 11], dtype=torch.int32)
    q, k, v = torch.randn(11, 4, 8), torch.randn(11, 2, 8), torch.randn(11, 2, 8)
    got = flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True)
    s = 0
    for n in lens:
        qi, ki, vi = (t[s:s + n].transpose(0, 1) for t in (q, k, v))
        ki, vi = ki.repeat_interleave(2, 0), vi.repeat_interleave(2, 0)
        att = (qi @ ki.transpose(-1, -2)) / 8 ** 0.5
        att = att.masked_fill(~torch.ones(n, n, dtype=torch.bool).tril(), float("-inf")).softmax(-1)
        assert torch.allclose(got[s:s + n].transpose(0, 1), att @ vi, atol=1e-5)
        s += n


def test_sharded_adamw_dynamic_loss_scaling():
    """Scaled gradients give the same update as unscaled ones; a non-finite gradient skips the step and backs the
    scale off; good steps grow it again."""
    from torch_musa_b200.parallel.zero import ShardedFusedAdamW

    torch.manual_seed(0)
    base = [torch.randn(40, 16) * 0.1, torch.randn(16) * 0.1]
    a = [torch.nn.Parameter(b.to(torch.bfloat16)) for b in base]
    b = [torch.nn.Parameter(b.to(torch.bfloat16)) for b in base]
    oa = ShardedFusedAdamW(a, lr=1e-2, bucket_mb=1)
    ob = ShardedFusedAdamW(b, lr=1e-2, bucket_mb=1)
    scaler = torch.amp.GradScaler("cpu", init_scale=256.0, growth_interval=2)
    grads = [(torch.randn(p.shape) * 0.05).to(torch.bfloat16) for p in a]
    for p, q, g in zip(a, b, grads):
        p.grad.copy_(g)
        q.grad.copy_((g.float() * 256.0).to(torch.bfloat16))      # what backward of a scaled loss produces
    oa.step()
    assert ob.step_with_scaler(scaler) is True
    assert all(torch.allclose(p.float(), q.float(), atol=1e-2) for p, q in zip(a, b))
    before = [q.detach().clone() for q in b]
    b[0].grad[0, 0] = float("inf")
    assert ob.step_with_scaler(scaler) is False and scaler.get_scale() == 128.0
    assert all(torch.equal(x, q) for x, q in zip(before, b)) and float(ob.step_t) == 1.0
    ob.zero_grad()
    assert ob.step_with_scaler(scaler) and ob.step_with_scaler(scaler) and scaler.get_scale() == 256.0


def test_python_examples_run_on_cpu():
    import importlib.util
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def load(name):
        spec = importlib.util.spec_from_file_location(name, os.path.join(root, "examples", "python", name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    assert load("train_tiny_llama").main(["--steps", "8", "--device", "cpu"]) < 3.0      # starts near ln(512) = 6.2
    assert load("quantize_conv_block").main() < 0.2


def test_experts_accept_device_side_counts():
    """The expert block gives the same rows whether the per-expert counts arrive as a list (host) or as an int32 tensor
    (the form the fused exchange hands over, with a capacity-sized row buffer)."""
    from torch_musa_b200.models.moe import Experts

    torch.manual_seed(0)
    ex = Experts(3, 16, 24)
    rows = torch.randn(20, 16)
    counts = [6, 0, 9]
    want = ex(rows[:15], counts)
    got = ex(rows, torch.tensor(counts, dtype=torch.int32))          # 5 rows of slack past the last expert
    assert got.shape == (20, 16) and torch.allclose(got[:15], want, atol=1e-6)
