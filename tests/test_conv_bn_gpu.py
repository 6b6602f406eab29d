"""Convolution (1x1 on the tcgen05 GEMM, other filters on the implicit-GEMM tcgen05 kernels, the rest on library
kernels) and the hand-written channels-last batch-norm / pooling kernels, against fp32 CPU references."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))


@pytest.mark.parametrize("cin,cout,hw", [(64, 256, 14), (256, 64, 7), (128, 128, 9)])
def test_pointwise_conv_runs_on_gemm(bw, dev, cin, cout, hw):
    dt = torch.bfloat16
    x = torch.randn(4, cin, hw, hw).to(dt)
    w = (torch.randn(cout, cin, 1, 1) * 0.05).to(dt)
    g = torch.randn(4, cout, hw, hw).to(dt)
    xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
    yr = F.conv2d(xr, wr)
    yr.backward(g.float())
    xd = x.to(dev).contiguous(memory_format=torch.channels_last).requires_grad_()
    wd = w.to(dev).requires_grad_()
    hits = bw._C._pointwise_conv_hits()
    bw.reset_kernel_launch_count()
    y = F.conv2d(xd, wd)
    assert bw._C._pointwise_conv_hits() == hits + 1 and bw.kernel_launch_count() == 1
    assert y.is_contiguous(memory_format=torch.channels_last) and y.shape == yr.shape
    y.backward(g.to(dev).contiguous(memory_format=torch.channels_last))
    assert rel_err(y, yr) < 2e-2
    assert rel_err(xd.grad, xr.grad) < 2e-2
    assert rel_err(wd.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("k,stride,pad,groups", [(3, 1, 1, 1), (3, 2, 1, 1), (1, 2, 0, 1), (7, 2, 3, 1), (3, 1, 1, 4)])
def test_general_conv(bw, dev, k, stride, pad, groups):
    dt = torch.bfloat16
    cin = 16 if k != 7 else 3 * groups
    x = torch.randn(2, cin, 20, 20).to(dt)
    w = (torch.randn(32, cin // groups, k, k) * 0.1).to(dt)
    b = torch.randn(32).to(dt)
    xr, wr, br = x.float().requires_grad_(), w.float().requires_grad_(), b.float().requires_grad_()
    yr = F.conv2d(xr, wr, br, stride, pad, 1, groups)
    yr.sum().backward()
    xd, wd, bd = x.to(dev).requires_grad_(), w.to(dev).requires_grad_(), b.to(dev).requires_grad_()
    y = F.conv2d(xd, wd, bd, stride, pad, 1, groups)
    y.sum().backward()
    assert rel_err(y, yr) < 3e-2 and rel_err(xd.grad, xr.grad) < 3e-2
    assert rel_err(wd.grad, wr.grad) < 3e-2 and rel_err(bd.grad, br.grad) < 3e-2


# (N, Cin, H, W, Cout, R, S, stride, pad): ResNet-50's filter shapes on small images, plus ragged edge cases
IMPLICIT_CASES = [
    (4, 64, 14, 14, 64, 3, 3, 1, 1),
    (2, 128, 28, 28, 128, 3, 3, 2, 1),
    (3, 256, 14, 14, 512, 1, 1, 2, 0),
    (2, 3, 32, 32, 64, 7, 7, 2, 3),       # RGB stem: channels padded to 8
    (5, 72, 9, 11, 40, 3, 3, 1, 1),       # nothing a multiple of the tile sizes
    (2, 64, 13, 13, 136, 3, 3, 2, 1),     # odd extent with stride 2, ragged output channels
    (1, 16, 8, 8, 16, 5, 3, 1, 2),        # asymmetric filter, padding wider than the filter needs
    (2, 192, 7, 7, 192, 3, 3, 1, 1),
]


@pytest.mark.parametrize("case", IMPLICIT_CASES)
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_implicit_gemm_conv(bw, dev, case, dt):
    N, C, H, W, K, R, S, stride, pad = case
    torch.manual_seed(0)
    x = torch.randn(N, C, H, W).to(dt)
    w = (torch.randn(K, C, R, S) * (1.0 / (C * R * S) ** 0.5)).to(dt)
    b = torch.randn(K).to(dt)
    xr, wr, br = x.float().requires_grad_(), w.float().requires_grad_(), b.float().requires_grad_()
    yr = F.conv2d(xr, wr, br, stride, pad)
    g = torch.randn_like(yr).to(dt)
    yr.backward(g.float())
    xd = x.to(dev).contiguous(memory_format=torch.channels_last).requires_grad_()
    wd = w.to(dev).contiguous(memory_format=torch.channels_last).requires_grad_()
    bd = b.to(dev).requires_grad_()
    hits = bw._C._implicit_conv_hits()
    bw.reset_fallback_counts()
    y = F.conv2d(xd, wd, bd, stride, pad)
    y.backward(g.to(dev).contiguous(memory_format=torch.channels_last))
    bw.synchronize()
    assert bw._C._implicit_conv_hits() == hits + 2 and bw._C._conv_status(True) == 0
    assert not any("conv" in k for k in bw.fallback_counts()), bw.fallback_counts()
    assert y.shape == yr.shape and y.is_contiguous(memory_format=torch.channels_last)
    tol = 2e-2 if dt == torch.bfloat16 else 4e-3
    assert rel_err(y, yr) < tol
    assert rel_err(xd.grad, xr.grad) < tol
    assert rel_err(wd.grad, wr.grad) < tol
    assert rel_err(bd.grad, br.grad) < tol


def test_implicit_gemm_conv_standard_layout_inputs(bw, dev):
    """NCHW-contiguous activations and filters are converted on the way in; gradients come back in the callers' layouts."""
    x = torch.randn(2, 32, 10, 10).to(torch.bfloat16)
    w = (torch.randn(48, 32, 3, 3) * 0.06).to(torch.bfloat16)
    xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
    yr = F.conv2d(xr, wr, None, 1, 1)
    yr.square().sum().backward()
    xd, wd = x.to(dev).requires_grad_(), w.to(dev).requires_grad_()
    y = F.conv2d(xd, wd, None, 1, 1)
    y.float().square().sum().backward()
    assert wd.grad.is_contiguous() and wd.grad.shape == w.shape
    assert rel_err(y, yr) < 2e-2 and rel_err(xd.grad, xr.grad) < 3e-2 and rel_err(wd.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("shape", [(8, 64, 14, 14), (4, 256, 7, 7), (3, 8, 5, 5), (64, 128)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_batch_norm_training(bw, dev, shape, dt):
    C = shape[1]
    x = (torch.randn(*shape) * 2 + 0.5).to(dt)
    w, b = torch.rand(C) + 0.5, torch.randn(C)
    g = torch.randn(*shape).to(dt)
    rm, rv = torch.zeros(C), torch.ones(C)
    xr, wr, br = x.float().requires_grad_(), w.clone().requires_grad_(), b.clone().requires_grad_()
    rm_r, rv_r = rm.clone(), rv.clone()
    yr = F.batch_norm(xr, rm_r, rv_r, wr, br, True, 0.1, 1e-5)
    yr.backward(g.float())
    fmt = torch.channels_last if len(shape) == 4 else torch.contiguous_format
    xd = x.to(dev).contiguous(memory_format=fmt).requires_grad_()
    wd, bd = w.to(dev).requires_grad_(), b.to(dev).requires_grad_()
    rm_d, rv_d = rm.to(dev), rv.to(dev)
    bw.reset_kernel_launch_count()
    y = F.batch_norm(xd, rm_d, rv_d, wd, bd, True, 0.1, 1e-5)
    assert bw.kernel_launch_count() == 2, "batch norm forward did not run on the two hand-written passes"
    y.backward(g.to(dev).contiguous(memory_format=fmt))
    tol = 2e-2 if dt == torch.bfloat16 else 4e-3
    assert rel_err(y, yr) < tol
    assert rel_err(xd.grad, xr.grad) < tol * 2
    assert rel_err(wd.grad, wr.grad) < tol and rel_err(bd.grad, br.grad) < tol
    assert rel_err(rm_d, rm_r) < 1e-3 and rel_err(rv_d, rv_r) < 1e-3
    # evaluation mode uses the running statistics
    ye = F.batch_norm(xd.detach(), rm_d, rv_d, wd.detach(), bd.detach(), False, 0.1, 1e-5)
    yer = F.batch_norm(x.float(), rm_r, rv_r, w, b, False, 0.1, 1e-5)
    assert rel_err(ye, yer) < tol


@pytest.mark.parametrize("relu,residual", [(True, False), (True, True), (False, True)])
def test_fused_batch_norm_act(bw, dev, relu, residual):
    from torch_musa_b200.ops import batch_norm_act

    dt, shape, C = torch.bfloat16, (8, 64, 10, 10), 64
    x = torch.randn(*shape).to(dt)
    r = torch.randn(*shape).to(dt) if residual else None
    w, b, g = torch.rand(C) + 0.5, torch.randn(C) * 0.3, torch.randn(*shape).to(dt)
    xr, wr, br = x.float().requires_grad_(), w.clone().requires_grad_(), b.clone().requires_grad_()
    rr = r.float().requires_grad_() if residual else None
    yr = F.batch_norm(xr, None, None, wr, br, True, 0.1, 1e-5)
    if residual:
        yr = yr + rr
    if relu:
        yr = F.relu(yr)
    yr.backward(g.float())
    cl = torch.channels_last
    xd = x.to(dev).contiguous(memory_format=cl).requires_grad_()
    rd = r.to(dev).contiguous(memory_format=cl).requires_grad_() if residual else None
    wd, bd = w.to(dev).requires_grad_(), b.to(dev).requires_grad_()
    bw.reset_kernel_launch_count()
    y = batch_norm_act(xd, wd, bd, None, None, rd, True, 0.1, 1e-5, relu)
    assert bw.kernel_launch_count() == 2
    y.backward(g.to(dev).contiguous(memory_format=cl))
    assert rel_err(y, yr) < 2e-2 and rel_err(xd.grad, xr.grad) < 4e-2
    assert rel_err(wd.grad, wr.grad) < 2e-2 and rel_err(bd.grad, br.grad) < 2e-2
    if residual:
        assert rel_err(rd.grad, rr.grad) < 2e-2


def test_resnet18_step_matches_cpu(bw, dev):
    """One autocast training step of a small ResNet: loss and a first-layer gradient agree with fp32 CPU."""
    from torch_musa_b200.models import resnet, resnet18

    torch.manual_seed(0)
    ref = resnet18(num_classes=10)
    x, t = torch.randn(8, 3, 64, 64), torch.randint(0, 10, (8,))
    fused = resnet.FUSED_BN_ACT
    try:
        resnet.FUSED_BN_ACT = None
        loss_ref = F.cross_entropy(ref(x), t)
        loss_ref.backward()
    finally:
        resnet.FUSED_BN_ACT = fused
    import copy

    m = copy.deepcopy(ref)
    m.zero_grad()
    m = m.to(dev).to(memory_format=torch.channels_last)
    xd = x.to(dev).contiguous(memory_format=torch.channels_last)
    with torch.autocast("blackwell", dtype=torch.bfloat16):
        loss = F.cross_entropy(m(xd), t.to(dev))
    loss.backward()
    assert abs(float(loss) - float(loss_ref)) < 0.08, (float(loss), float(loss_ref))
    g, gr = m.fc.weight.grad, ref.fc.weight.grad
    assert rel_err(g, gr) < 0.15


@pytest.mark.parametrize("cl", [True, False])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_pooling_forward_backward(bw, dev, cl, dt):
    """max / average pooling on the pooling kernels against CPU autograd (ResNet's 3x3 stride-2 max pool included)."""
    import torch.nn.functional as F

    bw.reset_fallback_counts()
    torch.manual_seed(0)
    x = torch.randn(3, 16, 23, 19).to(dt)
    if cl:
        x = x.contiguous(memory_format=torch.channels_last)
    tol = 1e-5 if dt == torch.float32 else 2e-2
    cases = [
        lambda t: F.max_pool2d(t, 3, 2, 1),
        lambda t: F.max_pool2d(t, 2, 2),
        lambda t: F.max_pool2d(t, (3, 2), (1, 2), (1, 0), dilation=(2, 1)),
        lambda t: F.avg_pool2d(t, 3, 2, 1),
        lambda t: F.avg_pool2d(t, 2, 2, count_include_pad=False),
        lambda t: F.avg_pool2d(t, 3, 1, 1, count_include_pad=False),
        lambda t: F.adaptive_avg_pool2d(t, 1),
    ]
    for fn in cases:
        xr = x.float().clone().requires_grad_()
        xd = x.to(dev).requires_grad_()
        r, o = fn(xr), fn(xd)
        assert o.shape == r.shape
        assert torch.allclose(o.float().cpu(), r, atol=tol, rtol=tol)
        g = torch.randn_like(r)
        r.backward(g)
        o.backward(g.to(dt).to(dev))
        assert torch.allclose(xd.grad.float().cpu(), xr.grad, atol=tol * 4, rtol=tol * 4)
    assert not any("pool" in k for k in bw.fallback_counts()), bw.fallback_counts()


def test_deterministic_mode(bw, dev):
    """With deterministic algorithms on, the weight gradient is bit-identical from run to run (no split over pixels),
    and index_put_ with accumulate leaves its atomic kernel for the sort-based route."""
    torch.manual_seed(0)
    x = torch.randn(8, 64, 28, 28, dtype=torch.bfloat16, device=dev).contiguous(memory_format=torch.channels_last)
    w = (torch.randn(64, 64, 3, 3, dtype=torch.bfloat16, device=dev) * 0.05).contiguous(memory_format=torch.channels_last)
    g = torch.randn(8, 64, 28, 28, dtype=torch.bfloat16, device=dev).contiguous(memory_format=torch.channels_last)

    def wgrad():
        wd = w.detach().requires_grad_()
        F.conv2d(x, wd, None, 1, 1).backward(g)
        return wd.grad.float()

    base = wgrad()
    torch.use_deterministic_algorithms(True)
    try:
        a, b = wgrad(), wgrad()
        assert torch.equal(a, b)
        assert rel_err(a, base) < 1e-2
        t = torch.zeros(16, device=dev)
        bw.reset_fallback_counts()
        t.index_put_((torch.tensor([1, 1, 3], device=dev),), torch.ones(3, device=dev), accumulate=True)
        assert t.cpu().tolist()[:4] == [0.0, 2.0, 0.0, 1.0]
        assert any("index_put" in k for k in bw.fallback_counts())
    finally:
        torch.use_deterministic_algorithms(False)
