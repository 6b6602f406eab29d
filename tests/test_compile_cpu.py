"""Compile stack without a GPU: code generation and run-time compilation of fused groups (fake tensors
on the device), the partitioner's validity rules, the native graph runner and ahead-of-time packages on
CPU tensors.  Mirrors what reference tests/unittest/inductor/*.py and export tests check per layer."""
import os

import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode
from torch.fx.experimental.proxy_tensor import make_fx


def _trace_fake(fn, *shapes_dtypes):
    with FakeTensorMode(allow_non_fake_inputs=True):
        args = [torch.empty(s, dtype=d, device="blackwell") for s, d in shapes_dtypes]
        return make_fx(fn)(*args)


def test_pointwise_group_becomes_one_kernel(bw):
    from torch_musa_b200.compile import lower

    def f(x, y, w):
        h = torch.nn.functional.silu(x) * y + w
        z = torch.tanh(h) * 0.5 + (h > 0).to(h.dtype)
        return z, z.sum(-1)

    gm = _trace_fake(f, ((64, 256), torch.bfloat16), ((64, 256), torch.bfloat16), ((256,), torch.float32))
    kernels = lower.partition_pointwise(gm)
    assert len(kernels) == 1
    info = next(iter(kernels.values()))
    assert info["shape"] == (64, 256) and info["n_ops"] == 8 and info["vec"] == 8
    assert "sigmoidf(x0)" in info["source"] and "tanhf" in info["source"]
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert targets == [torch.ops.aten.sum.dim_IntList]          # everything element-wise left the outer graph
    ok, why = bw._C._jit_available()
    if not ok:
        pytest.skip(why)
    k = lower.get_kernel(info)                                  # compiled for sm_100a right here, without a GPU
    assert len(k.cubin) > 1000 and k.entry == info["entry"]
    desc = lower.describe_program(gm, kernels)
    assert [i["kind"] for i in desc["instrs"]] == ["fused", "op"]
    assert len(lower.instantiate(desc)) == 2


def test_partitioner_rejects_groups_with_outputs_of_different_shapes(bw):
    from torch_musa_b200.compile import lower

    def f(x, s):
        a = torch.exp(s) * 2.0           # [64, 1]
        b = x * a + 1.0                  # [64, 256]
        return a, b

    gm = _trace_fake(f, ((64, 256), torch.float32), ((64, 1), torch.float32))
    kernels = lower.partition_pointwise(gm)
    for info in kernels.values():        # whatever was grouped has one output shape
        assert len({tuple(info["shape"])}) == 1
    out = [n for n in gm.graph.nodes if n.op == "output"][0]
    assert len(out.args[0]) == 2


def test_addmm_activation_pass(bw):
    from torch_musa_b200.compile import lower

    def f(b, x, w):
        return torch.relu(torch.addmm(b, x, w))

    gm = _trace_fake(f, ((32,), torch.bfloat16), ((8, 16), torch.bfloat16), ((16, 32), torch.bfloat16))
    assert lower.fuse_addmm_activation(gm) == 1
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert targets == [torch.ops.aten._addmm_activation.default]


def test_native_runner_executes_cpu_graph(bw):
    from torch_musa_b200.compile import lower

    def f(x, w, b):
        h = torch.addmm(b, x, w)
        a, i = torch.topk(h, 3, dim=-1)
        parts = torch.split(h, [2, 6], dim=1)
        return torch.cat([parts[1], parts[0]], dim=1).relu(), a, i

    x, w, b = torch.randn(4, 5), torch.randn(5, 8), torch.randn(8)
    gm = make_fx(f)(x, w, b)
    runner, desc = lower.lower(gm, fuse=False)
    out = runner.run([x, w, b])
    ref = f(x, w, b)
    assert len(out) == 3
    for o, r in zip(out, ref):
        assert torch.equal(o, r)
    assert runner.runs == 1 and runner.op_calls >= 5
    # slots are released as soon as their last reader has run
    assert any(i["free"] for i in desc["instrs"])


def test_aot_package_roundtrip_on_cpu(bw, tmp_path):
    from torch_musa_b200 import export

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.l1 = torch.nn.Linear(16, 32)
            self.l2 = torch.nn.Linear(32, 4)
            self.register_buffer("calls", torch.zeros((), dtype=torch.long))

        def forward(self, x, scale):
            self.calls.add_(1)
            return {"y": self.l2(torch.tanh(self.l1(x))) * scale, "n": self.calls + 0}

    m = M().eval()
    x = torch.randn(3, 16)
    path = export.aot_compile(m, (x, 2.0), os.path.join(tmp_path, "m.b200pkg"))
    ref = M().eval()
    ref.load_state_dict(m.state_dict())
    loaded = export.aot_load(path)
    out = loaded(x, 2.0)
    exp = ref(x, 2.0)
    assert torch.allclose(out["y"], exp["y"], atol=1e-6) and int(out["n"]) == int(exp["n"])
    out = loaded(x, 2.0)                 # the buffer update persisted inside the loaded model
    assert int(out["n"]) == int(exp["n"]) + 1
    with pytest.raises(TypeError):
        loaded(x)


def test_dynamo_traces_device_module_calls_without_graph_breaks(bw):
    """Device queries fold into the graph as constants, the device module's autocast class is a context manager Dynamo
    knows, the stream accessors are in-graph functions: a function that uses them compiles as ONE graph."""
    from torch._dynamo import trace_rules
    from torch._dynamo.variables import TorchInGraphFunctionVariable

    rule_map = trace_rules.get_torch_obj_rule_map()
    for fn in (bw.current_stream, bw.default_stream, bw.stream, bw.is_available, bw.current_device):
        assert rule_map.get(fn) is TorchInGraphFunctionVariable, fn

    def f(x):
        with bw.amp.autocast(dtype=torch.bfloat16):
            y = x @ x
        return y + (1 if bw.is_available() else 2) + bw.device_count()

    x = torch.randn(4, 4)
    compiled = torch.compile(f, backend="eager", fullgraph=True)      # fullgraph: any graph break raises
    assert torch.allclose(compiled(x), f(x))


def test_aot_c_shim_is_exported_and_reports_errors(bw):
    """The C ABI for ahead-of-time compiled code: device-type code, and a failure that comes back as a status plus a
    message instead of a C++ exception (no device here, so every index is out of range)."""
    import ctypes

    lib = ctypes.CDLL(bw._C.__file__)
    assert lib.aoti_torch_device_type_blackwell() == torch._C._autograd.DeviceType.PrivateUse1.value
    lib.b200_shim_last_error.restype = ctypes.c_char_p
    handle = ctypes.c_void_p()
    if not bw.is_available():
        assert lib.aoti_torch_create_blackwell_guard(0, ctypes.byref(handle)) == 1
        assert b"out of range" in lib.b200_shim_last_error()
    assert lib.aoti_torch_create_blackwell_guard(0, None) == 1 and b"null" in lib.b200_shim_last_error()
    assert lib.aoti_torch_delete_blackwell_guard(None) == 0          # deleting nothing is fine


def test_every_generated_operator_compiles_without_a_gpu(bw):
    """One fused group per family that together use every operator the code generator knows; each generated source
    is compiled for sm_100a right here (NVRTC needs no device), so a typo in any expression template fails on the CPU."""
    from torch_musa_b200.compile import codegen, lower

    ok, why = bw._C._jit_available()
    if not ok:
        pytest.skip(why)
    F = torch.nn.functional
    aten = torch.ops.aten

    def unary(x):
        a = torch.exp(x) + torch.exp2(x) + torch.expm1(x) + torch.log(x.abs() + 1) + torch.log2(x.abs() + 1) + torch.log1p(x.abs())
        b = torch.sqrt(x.abs()) + torch.rsqrt(x.abs() + 1) + torch.reciprocal(x + 3) + torch.tanh(x) + torch.sigmoid(x) + torch.relu(x)
        c = F.silu(x) + torch.erf(x) + torch.sin(x) + torch.cos(x) + (-x) + F.gelu(x) + F.gelu(x, approximate="tanh") + F.leaky_relu(x, 0.2)
        d = torch.tan(x) + torch.asin(x.clamp(-0.9, 0.9)) + torch.acos(x.clamp(-0.9, 0.9)) + torch.atan(x) + torch.sinh(x) + torch.cosh(x)
        e = torch.asinh(x) + torch.acosh(x.abs() + 1.5) + torch.atanh(x.clamp(-0.9, 0.9)) + torch.erfc(x) + torch.log10(x.abs() + 1)
        f = torch.floor(x) + torch.ceil(x) + torch.trunc(x) + torch.round(x) + torch.sign(x) + torch.isnan(x).to(x.dtype)
        return a + b + c + d + e + f

    def binary(x, y):
        a = torch.maximum(x, y) + torch.minimum(x, y) + x.pow(2) + x.abs().pow(y) + torch.where(x > y, x, y) - torch.sub(x, y, alpha=2)
        b = (x < y).to(x.dtype) + (x >= 0.5).to(x.dtype) + (x <= y).to(x.dtype) + (x == y).to(x.dtype) + (x != 1.0).to(x.dtype)
        c = torch.logical_and(x > 0, y > 0).to(x.dtype) + torch.logical_or(x > 0, y > 0).to(x.dtype) + torch.logical_not(x > 0).to(x.dtype)
        d = torch.clamp(x, -1.0, 1.0) + torch.clamp_min(x, 0.1) + torch.clamp_max(y, 0.9) + (2.0 - x) + x / (y.abs() + 1) * 3.0
        e = torch.atan2(x, y) + torch.fmod(x, y.abs() + 1)
        return a + b + c + d + e

    def backward_forms(g, y):
        return (aten.sigmoid_backward(g, y) + aten.tanh_backward(g, y) + aten.threshold_backward(g, y, 0.0) + aten.silu_backward(g, y)
                + aten.gelu_backward(g, y) + aten.gelu_backward(g, y, approximate="tanh")).to(torch.float16)

    seen, n_kernels = set(), 0
    for fn, n_in, dt in ((unary, 1, torch.float32), (binary, 2, torch.bfloat16), (backward_forms, 2, torch.float32)):
        gm = _trace_fake(fn, *[((32, 128), dt)] * n_in)
        before = {n.target for n in gm.graph.nodes if n.op == "call_function"}
        kernels = lower.partition_pointwise(gm)
        assert kernels, fn.__name__
        for info in kernels.values():
            k = lower.get_kernel(info)                     # NVRTC, sm_100a
            assert len(k.cubin) > 1000
            n_kernels += 1
        after = {n.target for n in gm.graph.nodes if n.op == "call_function"}
        seen |= before - after                             # what moved into generated code
    missing = [t for t in codegen.OPS if t not in seen and "Scalar" not in str(t) and "prims" not in str(t)]
    assert len(missing) <= 6, missing                      # a few overload aliases (rsub.Tensor, pow.Tensor_Tensor ...) at most
    assert n_kernels >= 3
