"""The general reduce kernels against the CPU results of the same reductions: every operator, rows / columns /
middle dimensions / several dimensions / full reductions, short and very long rows (split reductions), every input
type, NaN propagation, and a check that none of them took the library fallback.
Parity: reference tests/unittest/operator/test_reduce.py, test_max_min.py, test_var_std.py (CPU-oracle comparisons)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(fn, x, dev, tol=None, **kw):
    ref = fn(x, **kw)
    out = fn(x.to(dev), **kw)
    refs = ref if isinstance(ref, tuple) else (ref,)
    outs = out if isinstance(out, tuple) else (out,)
    for o, r in zip(outs, refs):
        assert o.dtype == r.dtype, (o.dtype, r.dtype)
        assert o.shape == r.shape, (o.shape, r.shape)
        if r.dtype.is_floating_point:
            t = tol or {torch.float32: 2e-5, torch.float64: 1e-10, torch.bfloat16: 3e-2, torch.float16: 5e-3}[r.dtype]
            assert torch.allclose(o.cpu().double(), r.double(), atol=t, rtol=t, equal_nan=True), \
                (o.cpu().double() - r.double()).abs().max()
        else:
            assert torch.equal(o.cpu(), r)


SHAPES_DIMS = [((37, 53), -1), ((37, 53), 0), ((6, 17, 33), 1), ((6, 17, 33), (0, 2)), ((6, 17, 33), (1, 2)),
               ((6, 17, 33), None), ((5, 1, 7), 1), ((4096, 64), 1), ((3, 200000), 1), ((200000, 3), 0), ((1 << 20,), 0)]


@pytest.mark.parametrize("shape,dim", SHAPES_DIMS)
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_sum_mean_amax_amin(bw, dev, shape, dim, dt):
    bw.reset_fallback_counts()
    x = (torch.randn(shape) * 0.5).to(dt)
    kw = {} if dim is None else {"dim": dim}
    big = max(shape) > 10000
    tol = (5e-1 if dt == torch.bfloat16 else 2e-3) if big else None
    _check(torch.sum, x, dev, tol=tol, **kw)
    _check(torch.mean, x, dev, **kw)
    _check(torch.sum, x, dev, tol=tol, keepdim=True, **({"dim": dim} if dim is not None else {"dim": list(range(len(shape)))}))
    if dim is not None:
        _check(torch.amax, x, dev, **kw)
        _check(torch.amin, x, dev, **kw)
    else:
        _check(torch.max, x, dev)
        _check(torch.min, x, dev)
    assert not bw.fallback_counts(), bw.fallback_counts()


@pytest.mark.parametrize("dt", [torch.float32, torch.float64, torch.float16, torch.int64, torch.int32, torch.uint8, torch.bool])
def test_every_dtype(bw, dev, dt):
    bw.reset_fallback_counts()
    g = torch.Generator().manual_seed(0)
    x = torch.randint(0, 5, (9, 31), generator=g).to(dt) if not dt.is_floating_point else torch.randn(9, 31, generator=g).to(dt)
    _check(torch.sum, x, dev, dim=1)
    _check(torch.sum, x, dev)
    _check(torch.any, x, dev, dim=0)
    _check(torch.all, x, dev, dim=1)
    _check(torch.any, x, dev)
    _check(torch.all, x, dev)
    if dt != torch.bool:
        _check(torch.prod, x[:, :6], dev, dim=1)
        _check(torch.amax, x, dev, dim=0)
        _check(torch.argmax, x, dev, dim=1)
        _check(torch.argmin, x, dev)
        _check(lambda t: torch.max(t, dim=0), x, dev)
        _check(lambda t: torch.min(t, dim=1, keepdim=True), x, dev)
    assert not bw.fallback_counts(), bw.fallback_counts()


def test_sum_dtype_argument_and_out(bw, dev):
    bw.reset_fallback_counts()
    x = torch.randn(8, 300).to(torch.bfloat16)
    _check(lambda t: torch.sum(t, dim=1, dtype=torch.float32), x, dev)
    _check(lambda t: torch.sum(t.float(), dim=1, dtype=torch.float64), x, dev)
    _check(lambda t: torch.mean(t, dim=0, dtype=torch.float32), x, dev)
    out = torch.empty(0, device=dev)
    torch.sum(x.float().to(dev), dim=0, out=out)
    assert torch.allclose(out.cpu(), x.float().sum(0), atol=1e-4)
    # a non-contiguous input (transposed view) and a non-adjacent pair of dimensions
    y = torch.randn(5, 7, 9)
    _check(lambda t: t.transpose(0, 2).sum(dim=1), y, dev)
    _check(lambda t: t.permute(2, 0, 1).amax(dim=(0, 2)), y, dev)
    assert not bw.fallback_counts(), bw.fallback_counts()


def test_var_std_norm(bw, dev):
    bw.reset_fallback_counts()
    x = torch.randn(33, 129) * 3 + 5
    for kw in ({"dim": 1}, {"dim": 0, "unbiased": False}, {"dim": (0, 1), "correction": 2}, {}):
        _check(torch.var, x, dev, tol=1e-4, **kw)
        _check(torch.std, x, dev, tol=1e-4, **kw)
    _check(lambda t: torch.var_mean(t, dim=1), x, dev, tol=1e-4)
    _check(lambda t: torch.std_mean(t, dim=0), x, dev, tol=1e-4)
    _check(lambda t: torch.var(t.bfloat16(), dim=1), x, dev)
    for p in (1, 2, float("inf")):
        _check(lambda t, p=p: torch.linalg.vector_norm(t, ord=p, dim=1), x, dev, tol=1e-4)
        _check(lambda t, p=p: torch.linalg.vector_norm(t, ord=p), x, dev, tol=1e-4)
        _check(lambda t, p=p: t.norm(p, dim=0), x, dev, tol=1e-4)
    _check(lambda t: t.norm(), x, dev, tol=1e-4)
    _check(lambda t: torch.logsumexp(t, dim=1), x, dev, tol=1e-4)
    assert not any(k.split("::")[1].split(".")[0] in ("var", "std", "var_mean", "std_mean", "linalg_vector_norm", "norm",
                                                      "sum", "amax", "exp", "log") for k in bw.fallback_counts()), bw.fallback_counts()


def test_nan_and_ties(bw, dev):
    x = torch.tensor([[1.0, float("nan"), 3.0, 3.0], [2.0, 2.0, -1.0, 0.0]])
    _check(torch.amax, x, dev, dim=1)
    _check(torch.argmax, x, dev, dim=1)          # NaN wins; ties -> first index
    _check(torch.argmin, x, dev, dim=1)
    _check(lambda t: torch.max(t, dim=1), x, dev)
    _check(torch.sum, x, dev, dim=1)
    e = torch.zeros(0, 4)
    _check(torch.sum, e, dev, dim=0)
    _check(torch.sum, e, dev)
    _check(torch.all, e, dev)
