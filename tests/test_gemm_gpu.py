"""tcgen05 GEMM against a plain fp32 matmul on the CPU, over tile-edge shapes, every operand
layout (K-major / MN-major, i.e. the forward, dgrad and wgrad forms), epilogues and batching."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def ref_close(out, ref, k, dt):
    out, ref = out.float().cpu(), ref.float()
    # bf16 inputs are exact in the reference; error comes from output rounding + fp32 accumulation order
    eps = 2 ** -8 if dt == torch.bfloat16 else 2 ** -11
    tol = eps * ref.abs().max().item() + 1e-3 * (k ** 0.5) * 0.05
    err = (out - ref).abs().max().item()
    if err > tol:
        bad = ((out - ref).abs() > tol).nonzero()
        print(f"max err {err} tol {tol}; first bad idx {bad[:5].tolist()} of {bad.shape[0]}")
    return err <= tol


@pytest.fixture(autouse=True)
def _check_status(bw):
    bw._C._gemm_status(True) if hasattr(bw._C, "_gemm_status") else None
    yield
    if hasattr(bw._C, "_gemm_status"):
        bw.synchronize()
        assert bw._C._gemm_status(False) == 0, "a tcgen05 GEMM launch gave up on a bounded wait"


SHAPES = [(128, 256, 64), (128, 256, 128), (256, 512, 256), (1, 8, 8), (5, 24, 40), (127, 255, 72), (129, 257, 136),
          (300, 1000, 520), (1024, 1024, 1024), (4096, 4096, 512), (64, 11008, 256), (2048, 512, 4096)]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_mm_nt(bw, dev, m, n, k, dt):
    """y = x @ W^T : both operands K-major (the nn.Linear forward)."""
    assert bw._C._gemm_available()
    x, w = torch.randn(m, k).to(dt), torch.randn(n, k).to(dt)
    bw.reset_kernel_launch_count()
    y = x.to(dev) @ w.to(dev).t()
    assert bw.kernel_launch_count() in (1, 2), "mm did not run on the hand-written GEMM (1 launch, or 2 with split-K)"
    assert ref_close(y, x.float() @ w.float().t(), k, dt)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (136, 264, 136), (512, 1024, 320), (4096, 4096, 256)])
def test_mm_all_layouts(bw, dev, m, n, k):
    dt = torch.bfloat16
    a, b = torch.randn(m, k).to(dt), torch.randn(k, n).to(dt)
    ref = a.float() @ b.float()
    ad, bd = a.to(dev), b.to(dev)
    at_d = a.t().contiguous().to(dev).t()      # [m,k] view, M contiguous  (MN-major A)
    bt_d = b.t().contiguous().to(dev).t()      # [k,n] view, K contiguous  (K-major B)
    for A, B, name in [(ad, bd, "A:K B:MN"), (ad, bt_d, "A:K B:K"), (at_d, bd, "A:MN B:MN"), (at_d, bt_d, "A:MN B:K")]:
        bw.reset_kernel_launch_count()
        y = A @ B
        assert bw.kernel_launch_count() == 1, name
        assert ref_close(y, ref, k, dt), name


@pytest.mark.parametrize("config", [1, 2, 3])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (136, 264, 136), (384, 392, 520), (1000, 3000, 264),
                                   (4096, 4096, 512), (2048, 11008, 4096)])
def test_mm_every_tile_config(bw, dev, m, n, k, config):
    """Single-CTA 128x256 and SM-pair 256x256 tiles give the same product in all four layouts."""
    dt = torch.bfloat16
    a, b = torch.randn(m, k).to(dt), torch.randn(k, n).to(dt)
    ref = a.float() @ b.float()
    ad, bd = a.to(dev), b.to(dev)
    at_d = a.t().contiguous().to(dev).t()
    bt_d = b.t().contiguous().to(dev).t()
    bias = torch.randn(n).to(dt)
    prev = bw._C._gemm_force_config(config)
    try:
        for A, B, name in [(ad, bd, "A:K B:MN"), (ad, bt_d, "A:K B:K"), (at_d, bd, "A:MN B:MN"), (at_d, bt_d, "A:MN B:K")]:
            bw.reset_kernel_launch_count()
            y = A @ B
            assert bw.kernel_launch_count() in (1, 2), name
            assert ref_close(y, ref, k, dt), f"{name} config {config}"
        y = torch.addmm(bias.to(dev), ad, bd)
        assert ref_close(y, ref + bias.float(), k, dt), f"addmm config {config}"
    finally:
        bw._C._gemm_force_config(prev)
    bw.synchronize()
    assert bw._C._gemm_status(False) == 0


@pytest.mark.parametrize("m,n,k", [(64, 256, 50176), (128, 256, 16384), (2048, 512, 12544), (264, 136, 8200)])
def test_split_k(bw, dev, m, n, k):
    """Few output tiles and a long K (weight gradients): K is split across SMs, partial products are summed in fp32."""
    dt = torch.bfloat16
    a, b = (torch.randn(m, k) * 0.5).to(dt), (torch.randn(k, n) * 0.5).to(dt)
    ref = a.float() @ b.float()
    ad, bd = a.to(dev), b.to(dev)
    at_d = a.t().contiguous().to(dev).t()
    bias = torch.randn(n).to(dt)
    for A, B, name in [(ad, bd, "A:K B:MN"), (at_d, bd, "A:MN B:MN"), (ad, b.t().contiguous().to(dev).t(), "A:K B:K")]:
        bw.reset_kernel_launch_count()
        y = A @ B
        assert bw.kernel_launch_count() == 2, f"{name}: expected the split GEMM plus its reduction"
        assert ref_close(y, ref, k, dt), name
    y = torch.addmm(bias.to(dev), ad, bd)
    assert ref_close(y, ref + bias.float(), k, dt)
    bw.synchronize()
    assert bw._C._gemm_status(False) == 0


def test_linear_autograd(bw, dev):
    dt = torch.bfloat16
    x, w, b = torch.randn(384, 512).to(dt), torch.randn(768, 512).to(dt), torch.randn(768).to(dt)
    g = torch.randn(384, 768).to(dt)
    xd, wd, bd = (t.to(dev).detach().clone().requires_grad_() for t in (x, w, b))
    xr, wr, br = (t.float().detach().clone().requires_grad_() for t in (x, w, b))
    y = torch.nn.functional.linear(xd, wd, bd)
    y.backward(g.to(dev))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert ref_close(y, yr.detach(), 512, dt)
    assert ref_close(xd.grad, xr.grad, 768, dt)
    assert ref_close(wd.grad, wr.grad, 384, dt)
    assert torch.allclose(bd.grad.float().cpu(), br.grad, atol=0.5, rtol=2e-2)


def test_addmm_and_activation(bw, dev):
    dt = torch.bfloat16
    x, w, b = torch.randn(200, 256).to(dt), torch.randn(256, 520).to(dt), torch.randn(520).to(dt)
    y = torch.addmm(b.to(dev), x.to(dev), w.to(dev))
    assert ref_close(y, b.float() + x.float() @ w.float(), 256, dt)
    y2 = torch.addmm(b.to(dev), x.to(dev), w.to(dev), beta=0.5, alpha=2.0)
    assert ref_close(y2, 0.5 * b.float() + 2.0 * (x.float() @ w.float()), 256, dt)
    c = torch.randn(200, 520).to(dt)
    y3 = torch.addmm(c.to(dev), x.to(dev), w.to(dev))
    assert ref_close(y3, c.float() + x.float() @ w.float(), 256, dt)
    y4 = torch._addmm_activation(b.to(dev), x.to(dev), w.to(dev), use_gelu=True)
    assert ref_close(y4, torch.nn.functional.gelu(b.float() + x.float() @ w.float()), 256, dt)


def test_bmm(bw, dev):
    dt = torch.bfloat16
    a, b = torch.randn(6, 130, 72).to(dt), torch.randn(6, 72, 264).to(dt)
    bw.reset_kernel_launch_count()
    y = torch.bmm(a.to(dev), b.to(dev))
    assert bw.kernel_launch_count() == 1
    assert ref_close(y, torch.bmm(a.float(), b.float()), 72, dt)
    y2 = torch.bmm(a.to(dev), b.to(dev).transpose(1, 2).contiguous().transpose(1, 2))
    assert ref_close(y2, torch.bmm(a.float(), b.float()), 72, dt)


def test_unsupported_shapes_fall_back(bw, dev):
    # K not a multiple of 8 (unaligned leading stride) and fp32 inputs take the library route and stay correct
    a, b = torch.randn(33, 30).bfloat16(), torch.randn(30, 17).bfloat16()
    assert ref_close(a.to(dev) @ b.to(dev), a.float() @ b.float(), 30, torch.bfloat16)
    c, d = torch.randn(64, 64), torch.randn(64, 64)
    assert torch.allclose((c.to(dev) @ d.to(dev)).cpu(), c @ d, atol=1e-2, rtol=1e-2)


def test_gemm_switch(bw, dev):
    a, b = torch.randn(256, 256).bfloat16().to(dev), torch.randn(256, 256).bfloat16().to(dev)
    y1 = a @ b
    bw._C._set_tensor_core_gemm(False)
    try:
        bw.reset_kernel_launch_count()
        y2 = a @ b
        assert bw.kernel_launch_count() == 0
    finally:
        bw._C._set_tensor_core_gemm(True)
    assert torch.allclose(y1.float().cpu(), y2.float().cpu(), atol=0.25, rtol=2e-2)


def test_fp32_matmul_as_tf32_on_tensor_cores(bw, dev):
    """fp32 operands run on the tcgen05 kernel as tf32 when that precision is allowed, on the library GEMM otherwise."""
    torch.manual_seed(0)
    a, b = torch.randn(300, 520), torch.randn(520, 264)
    bias = torch.randn(264)
    ref = (a.double() @ b.double()).float()
    ad, bd = a.to(dev), b.to(dev)
    prev = torch.backends.blackwell.allow_tf32
    try:
        torch.backends.blackwell.allow_tf32 = False
        bw.reset_fallback_counts()
        strict = ad @ bd
        assert any("mm" in k for k in bw.fallback_counts())
        assert (strict.cpu() - ref).abs().max() < 1e-3
        torch.backends.blackwell.allow_tf32 = True
        bw.reset_fallback_counts()
        fast = ad @ bd                                     # b is [K, N] row-major: re-laid out K-major first
        lin = torch.nn.functional.linear(ad, bd.t().contiguous(), bias.to(dev))    # both operands K-major as stored
        assert not any("mm" in k for k in bw.fallback_counts()), bw.fallback_counts()
        scale = float(ref.abs().max())
        assert (fast.cpu() - ref).abs().max() < 4e-3 * scale        # 10-bit mantissa
        assert (fast.cpu() - ref).abs().max() > 1e-6 * scale        # ... so really not fp32 arithmetic
        assert (lin.cpu() - (ref + bias)).abs().max() < 4e-3 * scale
        assert bw._C._gemm_status() == 0
    finally:
        torch.backends.blackwell.allow_tf32 = prev


@pytest.mark.parametrize("counts,R", [([130, 0, 77, 256], 520), ([64, 64], 128), ([5], 64), ([200, 300, 1, 63, 129], 1024)])
def test_grouped_gemm_device_side_counts(bw, dev, counts, R):
    """The three grouped products (forward, input gradient, per-group weight gradient) against fp32 loops; the
    group lengths are only ever read on the device, rows past their sum stay untouched."""
    from torch_musa_b200.ops import grouped_linear

    torch.manual_seed(0)
    G, K, N = len(counts), 192, 328
    x = (torch.randn(R, K) * 0.5).to(torch.bfloat16)
    w = (torch.randn(G, N, K) * 0.1).to(torch.bfloat16)
    dy = (torch.randn(R, N) * 0.5).to(torch.bfloat16)
    cnt = torch.tensor(counts, dtype=torch.int32)
    used = sum(counts)
    # fp32 oracle
    y_ref, dx_ref, dw_ref, s = torch.zeros(R, N), torch.zeros(R, K), torch.zeros(G, N, K), 0
    for g, n in enumerate(counts):
        y_ref[s:s + n] = x[s:s + n].float() @ w[g].float().t()
        dx_ref[s:s + n] = dy[s:s + n].float() @ w[g].float()
        dw_ref[g] = dy[s:s + n].float().t() @ x[s:s + n].float()
        s += n
    xd, wd = x.to(dev).requires_grad_(), w.to(dev).requires_grad_()
    out = torch.full((R, N), 7.0, dtype=torch.bfloat16, device=dev)
    bw.reset_fallback_counts()
    y = grouped_linear(xd, wd, cnt.to(dev), out)
    y.backward(dy.to(dev))
    assert bw._C._gemm_status() == 0
    assert (y[:used].float().cpu() - y_ref[:used]).abs().max() < 3e-2 * max(1.0, float(y_ref.abs().max()))
    assert bool((y[used:] == 7.0).all())                       # rows of no group are not written
    assert (xd.grad[:used].float().cpu() - dx_ref[:used]).abs().max() < 3e-2 * max(1.0, float(dx_ref.abs().max()))
    assert (wd.grad.float().cpu() - dw_ref).abs().max() < 3e-2 * max(1.0, float(dw_ref.abs().max()))
    # the host implementation of the same contract (any device) agrees
    y_cpu = grouped_linear(x.float(), w.float(), cnt)
    assert torch.allclose(y_cpu[:used], y_ref[:used], atol=1e-4)
