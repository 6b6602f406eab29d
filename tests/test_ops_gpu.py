"""Numerics of the hand-written operator kernels against plain PyTorch fp32 on the CPU
(the reference's OpTest discipline: CPU is the oracle; reference
torch_musa/testing/base_test_tool.py:306-350)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16, torch.float16]


def tol(dt):
    return {torch.float32: (1e-5, 1e-5), torch.bfloat16: (2e-2, 2e-2), torch.float16: (2e-3, 2e-3)}[dt]


def leaf(t, dev=None, dtype=None):
    """A fresh leaf tensor (never an alias of `t`, even when no conversion is needed)."""
    t = t.detach().clone()
    if dtype is not None:
        t = t.to(dtype)
    if dev is not None:
        t = t.to(dev)
    return t.requires_grad_()


def close(a, b, dt, scale=1.0):
    atol, rtol = tol(dt)
    a, b = a.float().cpu(), b.float().cpu()
    # absolute tolerance relative to the magnitude of the reference (values are O(1) in most tests)
    mag = max(1.0, float(b.abs().max())) if b.numel() else 1.0
    ok = torch.allclose(a, b, atol=atol * scale * mag, rtol=rtol)
    if not ok:
        print("max abs diff", (a - b).abs().max().item(), "ref max", b.abs().max().item())
    return ok


@pytest.mark.parametrize("dt", DTYPES)
def test_elementwise(bw, dev, dt):
    bw.reset_kernel_launch_count()
    a, b = torch.randn(333, 77).to(dt), torch.randn(333, 77).to(dt)
    da, db = a.to(dev), b.to(dev)
    ra, rb = a.float(), b.float()
    assert close(da + db, ra + rb, dt)
    assert close(torch.add(da, db, alpha=0.5), ra + 0.5 * rb, dt)
    assert close(da - db, ra - rb, dt)
    assert close(da * db, ra * rb, dt, 4)
    assert close(da / (db.abs() + 1), ra / (rb.abs() + 1), dt)
    assert close(da * 3.0, ra * 3.0, dt, 4)
    assert close(F.relu(da), F.relu(ra), dt)
    assert close(F.gelu(da), F.gelu(ra), dt)
    assert close(F.gelu(da, approximate="tanh"), F.gelu(ra, approximate="tanh"), dt)
    assert close(F.silu(da), F.silu(ra), dt)
    assert close(torch.sigmoid(da), torch.sigmoid(ra), dt)
    assert close(torch.tanh(da), torch.tanh(ra), dt)
    assert close(torch.exp(da * 0.1), torch.exp((a * 0.1).float()), dt, 2)
    assert close(da.abs().sqrt(), ra.abs().sqrt(), dt)
    assert close(-da, -ra, dt)
    c = da.clone()
    c.add_(db)
    c.mul_(db)
    assert close(c, (a + b).to(dt).float() * rb, dt, 8)
    z = torch.zeros(1000, dtype=dt, device=dev)
    z.fill_(2.5)
    assert float(z.float().sum()) == 2500.0
    z.zero_()
    assert float(z.float().sum()) == 0.0
    assert bw.kernel_launch_count() > 10


@pytest.mark.parametrize("dt", DTYPES)
def test_activation_backward(bw, dev, dt):
    for fn in (F.relu, F.gelu, F.silu, torch.sigmoid, torch.tanh):
        x = torch.randn(129, 65).to(dt)
        xd = x.to(dev).detach().clone().requires_grad_()
        xr = x.float().detach().clone().requires_grad_()
        g = torch.randn(129, 65).to(dt)
        fn(xd).backward(g.to(dev))
        fn(xr).backward(g.float())
        assert close(xd.grad, xr.grad, dt, 2), fn


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("shape", [(4, 33, 1024), (300, 4096), (17, 8192), (5, 24576)])
def test_rms_norm(bw, dev, dt, shape):
    x = torch.randn(*shape).to(dt)
    w = (torch.randn(shape[-1]) * 0.1 + 1).to(dt)
    g = torch.randn(*shape).to(dt)
    xd, wd = x.to(dev).detach().clone().requires_grad_(), w.to(dev).detach().clone().requires_grad_()
    xr, wr = x.float().detach().clone().requires_grad_(), w.float().detach().clone().requires_grad_()
    bw.reset_kernel_launch_count()
    y = F.rms_norm(xd, (shape[-1],), wd, 1e-5)
    y.backward(g.to(dev))
    if shape[-1] * x.element_size() <= 65536:  # rows up to 64 KB stay in registers; longer rows use the generic route
        assert bw.kernel_launch_count() >= 2
    yr = F.rms_norm(xr, (shape[-1],), wr, 1e-5)
    yr.backward(g.float())
    assert close(y, yr, dt)
    assert close(xd.grad, xr.grad, dt, 2)
    rows = x.numel() // shape[-1]
    assert close(wd.grad, wr.grad, dt, max(2.0, rows ** 0.5))


def test_rms_norm_residual(bw, dev):
    from torch_musa_b200.ops import rms_norm_residual

    dt = torch.bfloat16
    x, r = torch.randn(64, 4096).to(dt), torch.randn(64, 4096).to(dt)
    w = torch.ones(4096).to(dt)
    y, h = rms_norm_residual(x.to(dev), r.to(dev), w.to(dev), 1e-5)
    href = (x.float() + r.float()).to(dt)
    assert torch.equal(h.cpu(), href)
    assert close(y, F.rms_norm(href.float(), (4096,), w.float(), 1e-5), dt)


@pytest.mark.parametrize("dt", DTYPES)
def test_layer_norm(bw, dev, dt):
    x = torch.randn(6, 50, 768).to(dt)
    w, b = (torch.randn(768) * 0.1 + 1).to(dt), (torch.randn(768) * 0.1).to(dt)
    g = torch.randn(6, 50, 768).to(dt)
    xd, wd, bd = x.to(dev).detach().clone().requires_grad_(), w.to(dev).detach().clone().requires_grad_(), b.to(dev).detach().clone().requires_grad_()
    xr, wr, br = x.float().detach().clone().requires_grad_(), w.float().detach().clone().requires_grad_(), b.float().detach().clone().requires_grad_()
    F.layer_norm(xd, (768,), wd, bd).backward(g.to(dev))
    F.layer_norm(xr, (768,), wr, br).backward(g.float())
    assert close(F.layer_norm(xd, (768,), wd, bd), F.layer_norm(xr, (768,), wr, br), dt)
    assert close(xd.grad, xr.grad, dt, 2)
    assert close(wd.grad, wr.grad, dt, 20)
    assert close(bd.grad, br.grad, dt, 20)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cols", [8, 1000, 32000, 50257])
def test_softmax(bw, dev, dt, cols):
    x = (torch.randn(33, cols) * 3).to(dt)
    g = torch.randn(33, cols).to(dt)
    for fn in (F.softmax, F.log_softmax):
        xd = x.to(dev).detach().clone().requires_grad_()
        xr = x.float().detach().clone().requires_grad_()
        y = fn(xd, dim=-1)
        y.backward(g.to(dev))
        yr = fn(xr, dim=-1)
        yr.backward(g.float())
        assert close(y, yr, dt), fn
        assert close(xd.grad, xr.grad, dt, 4), fn


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cols", [1000, 32000])
def test_fused_cross_entropy(bw, dev, dt, cols):
    from torch_musa_b200.ops import fused_cross_entropy

    T = 257
    x = (torch.randn(T, cols) * 2).to(dt)
    t = torch.randint(0, cols, (T,))
    t[::7] = -100
    for ls in (0.0, 0.1):
        xd = x.to(dev).detach().clone().requires_grad_()
        xr = x.float().detach().clone().requires_grad_()
        loss = fused_cross_entropy(xd, t.to(dev), label_smoothing=ls)
        loss.backward()
        ref = F.cross_entropy(xr, t, label_smoothing=ls)
        ref.backward()
        assert abs(float(loss) - float(ref)) < (1e-4 if dt == torch.float32 else 2e-2)
        atol = {torch.float32: 1e-7, torch.bfloat16: 1e-4, torch.float16: 1e-5}[dt]
        assert torch.allclose(xd.grad.float().cpu(), xr.grad, atol=atol, rtol=2e-2)
    # in-place backward overwrites the logits with the gradient
    xd = x.to(dev).detach().clone().requires_grad_()
    xc = xd.clone()
    loss = fused_cross_entropy(xc, t.to(dev), inplace_backward=True)
    loss.backward()
    xr = x.float().detach().clone().requires_grad_()
    F.cross_entropy(xr, t).backward()
    atol = {torch.float32: 1e-7, torch.bfloat16: 1e-4, torch.float16: 1e-5}[dt]
    assert torch.allclose(xd.grad.float().cpu(), xr.grad, atol=atol, rtol=2e-2)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("interleaved", [False, True])
def test_rope(bw, dev, dt, interleaved):
    from torch_musa_b200.ops import rope, precompute_rope_cache
    from torch_musa_b200.ops.functional import _rope_reference

    B, S, H, D = 2, 77, 4, 128
    cos, sin = precompute_rope_cache(128, D)
    x = torch.randn(B, S, H, D).to(dt)
    g = torch.randn(B, S, H, D).to(dt)
    xd = x.to(dev).detach().clone().requires_grad_()
    y = rope(xd, cos.to(dev), sin.to(dev), None, interleaved)
    y.backward(g.to(dev))
    xr = x.float().detach().clone().requires_grad_()
    yr = _rope_reference(xr, cos, sin, None, interleaved, False)
    yr.backward(g.float())
    assert close(y, yr, dt)
    assert close(xd.grad, xr.grad, dt)
    # strided input (slice of a fused qkv projection) and explicit positions
    qkv = torch.randn(B, S, 3 * H, D).to(dt)
    pos = torch.randint(0, 128, (B, S))
    yq = rope(qkv.to(dev)[:, :, H:2 * H], cos.to(dev), sin.to(dev), pos.to(dev), interleaved)
    assert close(yq, _rope_reference(qkv[:, :, H:2 * H].float(), cos, sin, pos, interleaved, False), dt)


@pytest.mark.parametrize("dt", DTYPES)
def test_swiglu_and_silu_mul(bw, dev, dt):
    from torch_musa_b200.ops import swiglu, silu_mul

    x = torch.randn(37, 2 * 1376).to(dt)
    g = torch.randn(37, 1376).to(dt)
    xd = x.to(dev).detach().clone().requires_grad_()
    xr = x.float().detach().clone().requires_grad_()
    y = swiglu(xd)
    y.backward(g.to(dev))
    a, b = xr.chunk(2, -1)
    yr = F.silu(a) * b
    yr.backward(g.float())
    assert close(y, yr, dt, 2) and close(xd.grad, xr.grad, dt, 4)
    p, q = torch.randn(1000, 33).to(dt), torch.randn(1000, 33).to(dt)
    pd, qd = p.to(dev).detach().clone().requires_grad_(), q.to(dev).detach().clone().requires_grad_()
    pr, qr = p.float().detach().clone().requires_grad_(), q.float().detach().clone().requires_grad_()
    go = torch.randn(1000, 33).to(dt)
    silu_mul(pd, qd).backward(go.to(dev))
    (F.silu(pr) * qr).backward(go.float())
    assert close(pd.grad, pr.grad, dt, 4) and close(qd.grad, qr.grad, dt, 4)


@pytest.mark.parametrize("dt", DTYPES)
def test_embedding(bw, dev, dt):
    w = torch.randn(1000, 256).to(dt)
    idx = torch.randint(0, 1000, (4, 333))
    wd = w.to(dev).detach().clone().requires_grad_()
    wr = w.float().detach().clone().requires_grad_()
    g = torch.randn(4, 333, 256).to(dt)
    y = F.embedding(idx.to(dev), wd)
    y.backward(g.to(dev))
    F.embedding(idx, wr).backward(g.float())
    assert torch.equal(y.cpu(), F.embedding(idx, w))
    assert close(wd.grad, wr.grad, dt, 4)
    torch.use_deterministic_algorithms(True)
    try:
        wd2 = w.to(dev).detach().clone().requires_grad_()
        F.embedding(idx.to(dev), wd2).backward(g.to(dev))
        assert close(wd2.grad, wr.grad, dt, 4)
    finally:
        torch.use_deterministic_algorithms(False)


def test_dropout(bw, dev):
    x = torch.ones(1 << 20, device=dev, dtype=torch.bfloat16).requires_grad_()
    y = F.dropout(x, 0.25, training=True)
    keep = float((y != 0).float().mean())
    assert 0.74 < keep < 0.76
    assert float(y.float().max()) == pytest.approx(1 / 0.75, rel=1e-2)
    y.sum().backward()
    assert torch.equal((x.grad != 0).cpu(), (y != 0).cpu())


def test_reductions_via_kernel_library(bw, dev):
    # exercised through clip_grad_norm_ / multi_tensor_l2norm
    from torch_musa_b200.ops import multi_tensor_l2norm

    ts = [torch.randn(n) for n in (1, 1000, 70000, 300000)]
    total, per = multi_tensor_l2norm([t.to(dev) for t in ts], per_tensor=True)
    ref = torch.stack([t.norm() for t in ts])
    assert torch.allclose(per.cpu(), ref, rtol=1e-4)
    assert float(total) == pytest.approx(float(ref.norm()), rel=1e-4)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hq,hkv,causal", [(4, 4, True), (8, 2, True), (4, 4, False)])
def test_sdpa_fused_routing(bw, dev, dt, hq, hkv, causal):
    """F.scaled_dot_product_attention takes the fused path (no materialised score matrix) and matches math."""
    B, S, D = 2, 256, 64
    q, k, v = torch.randn(B, hq, S, D).to(dt), torch.randn(B, hkv, S, D).to(dt), torch.randn(B, hkv, S, D).to(dt)
    g = torch.randn(B, hq, S, D).to(dt)
    qd, kd, vd = (leaf(t, dev) for t in (q, k, v))
    qr, kr, vr = (leaf(t, None, torch.float32) for t in (q, k, v))
    bw.reset_fallback_counts()
    o = F.scaled_dot_product_attention(qd, kd, vd, is_causal=causal, enable_gqa=(hq != hkv))
    o.backward(g.to(dev))
    names = bw.fallback_counts()
    assert not any("bmm" in n for n in names), "attention fell to the math decomposition"
    orf = F.scaled_dot_product_attention(qr, kr, vr, is_causal=causal, enable_gqa=(hq != hkv))
    orf.backward(g.float())
    assert close(o, orf, dt, 2)
    assert close(qd.grad, qr.grad, dt, 4) and close(kd.grad, kr.grad, dt, 4) and close(vd.grad, vr.grad, dt, 4)
    # an explicit mask still works (math path)
    mask = torch.rand(S, S) > 0.5
    om = F.scaled_dot_product_attention(qd.detach()[:, :hkv], kd.detach(), vd.detach(), attn_mask=mask.to(dev))
    omr = F.scaled_dot_product_attention(qr.detach()[:, :hkv], kr.detach(), vr.detach(), attn_mask=mask)
    assert close(om, omr, dt, 4)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_cat_and_strided_copy(bw, dev, dt):
    """cat along every dim, the backward of split (one cat), and strided / converting copies on the row kernel."""
    xs = [torch.randn(4, n, 64).to(dt) for n in (8, 24, 16)]
    for d in (0, 1, 2, -1):
        shapes = [x if d in (1,) else x[:, :8] for x in xs]
        ref = torch.cat(shapes, dim=d)
        bw.reset_kernel_launch_count()
        out = torch.cat([s.to(dev) for s in shapes], dim=d)
        assert bw.kernel_launch_count() >= (1 if d == 0 else len(shapes))   # outermost dim: one launch for all pieces
        assert torch.equal(out.cpu(), ref)
    # many small pieces of an integer type (what data-parallel wrappers flatten every step), odd byte counts,
    # more pieces than one launch takes
    pieces = [torch.arange(n, dtype=torch.int64) + 1000 * i for i, n in enumerate([1] * 140 + [3, 0, 5, 17])]
    bw.reset_fallback_counts()
    got = torch.cat([p.to(dev) for p in pieces])
    assert torch.equal(got.cpu(), torch.cat(pieces)) and not bw.fallback_counts()
    odd = [torch.randint(0, 255, (n,), dtype=torch.uint8) for n in (1, 15, 16, 33, 70001)]
    assert torch.equal(torch.cat([o.to(dev) for o in odd]).cpu(), torch.cat(odd))
    # legacy: 1-D empty tensors are skipped
    out = torch.cat([torch.empty(0, device=dev, dtype=dt), xs[0].to(dev)], dim=1)
    assert torch.equal(out.cpu(), xs[0])
    # split backward
    w = leaf(torch.randn(16, 96), dev, dt)
    a, b, c = w.view(16, 3, 32).split([1, 1, 1], dim=1)
    (a.float().sum() + 2 * b.float().sum() + 3 * c.float().sum()).backward()
    assert torch.equal(w.grad.float().cpu().view(16, 3, 32)[:, 2], torch.full((16, 32), 3.0))
    # converting copy into a column block of a wider fp32 matrix (rows of 128 elements)
    src = torch.randn(2, 128).to(dt)
    dst = torch.zeros(2, 512, device=dev)
    dst[:, 256:384].copy_(src.to(dev))
    ref = torch.zeros(2, 512)
    ref[:, 256:384] = src.float()
    assert torch.equal(dst.cpu(), ref)


@pytest.mark.parametrize("world", [1, 2, 8])
def test_chunk_cat(bw, dev, world):
    """The reduce-scatter copy-in: chunk r of every gradient goes to row r, bf16 -> fp32, with zero padding."""
    grads = [torch.randn(64, 32), torch.randn(16, 8, 4), torch.randn(24), torch.randn(13, 16)]
    grads16 = [g.to(torch.bfloat16) for g in grads]
    ref = torch._chunk_cat(grads16, dim=0, num_chunks=world).float()
    dg = [g.to(dev) for g in grads16]
    out = torch._chunk_cat(dg, dim=0, num_chunks=world)
    assert out.dtype == torch.bfloat16 and torch.equal(out.float().cpu(), ref)
    out32 = torch.full(ref.shape, 7.0, device=dev)
    torch._chunk_cat(dg, dim=0, num_chunks=world, out=out32)
    assert torch.equal(out32.cpu(), ref)


def test_mixed_device_arguments_raise(bw, dev):
    """A host tensor among the arguments of a hand-written operator is rejected on the host, before any launch."""
    from torch_musa_b200 import ops as BO

    x = torch.randn(1, 4, 2, 8, device=dev, dtype=torch.bfloat16)
    cos, sin = BO.precompute_rope_cache(4, 8)          # host tables
    with pytest.raises(RuntimeError, match="same device"):
        torch.ops.blackwell.rope(x, cos, sin)
    h = torch.randn(4, 16, device=dev, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="same device"):
        F.rms_norm(h, (16,), torch.ones(16, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="same device"):
        torch.ops.blackwell.cross_entropy_fwd(h.float(), torch.zeros(4, dtype=torch.long))
    bw.synchronize()


def test_swiglu_limited_to_live_rows(bw, dev):
    """Packed row groups with device-side lengths: only the first sum(counts) rows are computed / get a gradient."""
    from torch_musa_b200.ops import swiglu

    torch.manual_seed(0)
    x = torch.randn(40, 256).to(torch.bfloat16)
    counts = torch.tensor([7, 0, 12], dtype=torch.int32)
    live = int(counts.sum())
    xd = x.to(dev).requires_grad_()
    y = swiglu(xd, counts.to(dev))
    g, u = x.float().chunk(2, -1)
    ref = torch.nn.functional.silu(g) * u
    assert (y[:live].float().cpu() - ref[:live]).abs().max() < 2e-2
    dy = torch.randn(40, 128).to(torch.bfloat16)
    y.backward(dy.to(dev))
    xr = x.float().requires_grad_()
    gr, ur = xr.chunk(2, -1)
    (torch.nn.functional.silu(gr) * ur)[:live].backward(dy.float()[:live])
    assert (xd.grad[:live].float().cpu() - xr.grad[:live]).abs().max() < 3e-2
