"""torch.compile on the device: numerics of generated fused kernels against eager (dense, broadcast,
strided, mixed dtypes), training through the compiled forward+backward, graph trees, the default
``torch.compile(model)`` route, and ahead-of-time packages.
Mirrors reference tests/unittest/inductor/test_basic.py / test_musagraph_trees.py / export tests."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "blackwell"


class MLP(torch.nn.Module):
    def __init__(self, d=256, h=512):
        super().__init__()
        self.a = torch.nn.Linear(d, h)
        self.b = torch.nn.Linear(h, d)
        self.n = torch.nn.LayerNorm(d)

    def forward(self, x):
        h = torch.nn.functional.gelu(self.a(x), approximate="tanh")
        h = self.b(h)
        h = torch.tanh(h) * 0.5 + torch.sigmoid(h) * x
        return self.n(h + x)


def _pair(dtype=torch.bfloat16):
    torch.manual_seed(0)
    m = MLP().to(DEV).to(dtype)
    ref = MLP().to(dtype)
    ref.load_state_dict({k: v.cpu() for k, v in m.state_dict().items()})
    return m, ref


@pytest.mark.parametrize("graphs", [False, True])
def test_compiled_training_step_matches_cpu(bw, graphs):
    from torch_musa_b200 import compile as bc

    bc.graph_trees.reset()
    before = dict(bc.stats)
    m, ref = _pair()
    cm = torch.compile(m, backend="blackwell", options={"graphs": graphs})
    x = torch.randn(64, 256, dtype=torch.bfloat16)
    xd = x.to(DEV).requires_grad_(True)
    for _ in range(4):                       # warm-up, record, replay, replay
        m.zero_grad()
        xd.grad = None
        out = cm(xd)
        out.float().pow(2).mean().backward()
    xr = x.clone().requires_grad_(True)
    r = ref(xr)
    r.float().pow(2).mean().backward()
    assert (out.cpu().float() - r.float()).abs().max() < 0.06
    assert (xd.grad.cpu().float() - xr.grad.float()).abs().max() < 2e-3
    assert (m.a.weight.grad.cpu().float() - ref.a.weight.grad.float()).abs().max() < 2e-3
    assert bc.stats["fused_kernels"] > before["fused_kernels"]
    assert bc.stats["graphs_fallback"] == before["graphs_fallback"]
    if graphs:
        st = bc.graph_trees.get_manager(bw.current_device()).stats
        assert st["recorded"] == 2 and st["replayed"] >= 2      # forward node and its backward child
        assert bc.graph_trees.get_manager(bw.current_device()).node_count() == 2


def test_fused_kernel_addressing_modes(bw):
    """One generated kernel, every operand layout: dense, trailing / leading broadcast, scalar, strided."""
    def f(x, row, col, s, strided):
        return (torch.exp(x * 0.1) * row + col) * s - torch.relu(strided), (x > 0) & (row > 0)

    cf = torch.compile(f, backend="blackwell")
    torch.manual_seed(1)
    x = torch.randn(48, 256)
    cases = [
        (x, torch.randn(256), torch.randn(48, 1), torch.randn(()), torch.randn(48, 256)),
        (x, torch.randn(256), torch.randn(48, 1), torch.randn(()), torch.randn(256, 48).t()),   # generic path
    ]
    for args in cases:
        for dt in (torch.float32, torch.bfloat16):
            a = [t.to(dt) for t in args]
            ref = f(*[t.float() for t in a])
            out = cf(*[t.to(DEV) for t in a])
            tol = 1e-5 if dt == torch.float32 else 0.05
            assert (out[0].cpu().float() - ref[0]).abs().max() <= tol * max(1.0, float(ref[0].abs().max()))
            assert torch.equal(out[1].cpu(), ref[1])


def test_default_compile_route_and_reduce_overhead(bw):
    from torch_musa_b200 import compile as bc

    bc.graph_trees.reset()
    m, ref = _pair()
    x = torch.randn(32, 256, dtype=torch.bfloat16)
    lowered, epilogues = bc.stats["graphs_lowered"], bc.stats["addmm_epilogues"]
    with torch.no_grad():
        out = torch.compile(m)(x.to(DEV))                   # no backend named: still lands on this compiler
        assert bc.stats["graphs_lowered"] > lowered
        assert bc.stats["addmm_epilogues"] > epilogues      # gelu(linear(x)) runs in the GEMM's epilogue
        assert (out.cpu().float() - ref(x).float()).abs().max() < 0.06
        cm = torch.compile(m, mode="reduce-overhead")
        for _ in range(3):
            out = cm(x.to(DEV))
        assert (out.cpu().float() - ref(x).float()).abs().max() < 0.06
    assert bc.graph_trees.get_manager(bw.current_device()).stats["replayed"] >= 1


def test_graph_tree_paths(bw):
    """Two compiled functions called in sequence form a path; the second one reads the first one's output in place."""
    from torch_musa_b200 import compile as bc

    bc.graph_trees.reset()
    f = torch.compile(lambda x: torch.tanh(x) * 2.0 + 1.0, backend="blackwell", options={"graphs": True})
    g = torch.compile(lambda y, z: torch.sigmoid(y) * z - 0.5, backend="blackwell", options={"graphs": True})
    mgr = bc.graph_trees.get_manager(bw.current_device())
    z = bc.mark_static(torch.randn(1024, device=DEV))
    for i in range(4):
        x = torch.full((1024,), 0.1 * i, device=DEV)
        y = f(x)
        out = g(y, z)
        ref = torch.sigmoid(torch.tanh(x.cpu()) * 2.0 + 1.0) * z.cpu() - 0.5
        assert torch.allclose(out.cpu(), ref, atol=1e-5), i
        del y, out
    assert mgr.node_count() == 2 and mgr.stats["recorded"] == 2, mgr.stats
    root = next(iter(mgr.roots.values()))
    child = next(iter(root.children.values()))
    assert not child.copy_inputs                 # both inputs fixed: parent's output and the marked tensor
    assert len(root.copy_inputs) == 1            # a fresh `x` every call is copied in


def test_aot_package_on_device(bw, tmp_path):
    from torch_musa_b200 import export

    m, ref = _pair()
    m.eval()
    x = torch.randn(16, 256, dtype=torch.bfloat16)
    path = export.aot_compile(m, (x.to(DEV),), os.path.join(tmp_path, "mlp.b200pkg"))
    import zipfile
    names = zipfile.ZipFile(path).namelist()
    assert any(n.endswith(".cubin") for n in names) and "program.pkl" in names
    loaded = export.aot_load(path)
    out = loaded(x.to(DEV))
    assert (out.cpu().float() - ref(x).float()).abs().max() < 0.06
    assert loaded.runner.fused_launches >= 1


def test_aot_c_shim_guards_and_streams(bw):
    """The C ABI for ahead-of-time compiled code on a device: a stream guard makes a raw stream current and restores
    the previous one, the device guard restores its device, the current-stream query returns the raw handle."""
    import ctypes

    lib = ctypes.CDLL(bw._C.__file__)
    dev = bw.current_device()
    cur = ctypes.c_void_p()
    assert lib.aoti_torch_get_current_blackwell_stream(dev, ctypes.byref(cur)) == 0
    assert (cur.value or 0) == bw.current_stream(dev).cuda_stream
    side = bw.Stream(dev)
    guard = ctypes.c_void_p()
    assert lib.aoti_torch_create_blackwell_stream_guard(ctypes.c_void_p(side.cuda_stream), dev, ctypes.byref(guard)) == 0
    assert bw.current_stream(dev).cuda_stream == side.cuda_stream
    x = torch.ones(1024, device=DEV) * 3                       # work issued under the guard runs on `side`
    assert lib.aoti_torch_delete_blackwell_stream_guard(guard) == 0
    assert bw.current_stream(dev).cuda_stream == (cur.value or 0)
    side.synchronize()
    assert float(x.sum()) == 3072.0
    dguard = ctypes.c_void_p()
    assert lib.aoti_torch_create_blackwell_guard(dev, ctypes.byref(dguard)) == 0
    assert lib.aoti_torch_blackwell_guard_set_index(dguard, dev) == 0
    assert lib.aoti_torch_blackwell_guard_set_index(dguard, 1 << 20) == 1       # refused, status instead of a throw
    assert lib.aoti_torch_delete_blackwell_guard(dguard) == 0 and bw.current_device() == dev
