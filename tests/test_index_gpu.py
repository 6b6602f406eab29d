"""Indexing, scan and selection kernels against the CPU results: index_select, gather, scatter / scatter_add,
advanced indexing (reads and writes, with accumulation), tril / triu, arange, cumsum, sort, topk,
split_with_sizes_copy, one_hot; none may take the library fallback; an out-of-range index is reported, not a fault.
Parity: reference tests/unittest/operator/test_{index,index_select,gather,scatter,tril,arange,cumsum,sort,topk}.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _same(out, ref, tol=0.0):
    assert out.dtype == ref.dtype, (out.dtype, ref.dtype)
    assert out.shape == ref.shape, (out.shape, ref.shape)
    if ref.dtype.is_floating_point and tol:
        assert torch.allclose(out.cpu().float(), ref.float(), atol=tol, rtol=tol)
    else:
        assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.int64, torch.bool, torch.float64])
def test_index_select_gather(bw, dev, dt):
    bw.reset_fallback_counts()
    x = (torch.randn(7, 9, 12) * 10).to(dt)
    for dim, n in ((0, 5), (1, 20), (2, 3), (-1, 1)):
        idx = torch.randint(0, x.size(dim), (n,))
        _same(torch.index_select(x.to(dev), dim, idx.to(dev)), torch.index_select(x, dim, idx))
        _same(torch.index_select(x.to(dev), dim, idx.int().to(dev)), torch.index_select(x, dim, idx.int()))
    for dim in (0, 1, 2):
        shape = [4, 5, 6]
        idx = torch.randint(0, x.size(dim), shape)
        _same(torch.gather(x.to(dev), dim, idx.to(dev)), torch.gather(x, dim, idx))
    _same(torch.index_select(x.transpose(0, 2).to(dev), 1, torch.tensor([8, 0]).to(dev)),
          torch.index_select(x.transpose(0, 2), 1, torch.tensor([8, 0])))
    assert not bw.fallback_counts(), bw.fallback_counts()


def test_scatter_family_and_one_hot(bw, dev):
    bw.reset_fallback_counts()
    x = torch.zeros(6, 8)
    idx = torch.stack([torch.randperm(8)[:5] for _ in range(6)])          # unique per row: deterministic assign
    src = torch.randn(6, 5)
    _same(x.to(dev).scatter(1, idx.to(dev), src.to(dev)), x.scatter(1, idx, src))
    _same(x.to(dev).scatter(1, idx.to(dev), 3.5), x.scatter(1, idx, 3.5))
    dup = torch.randint(0, 8, (6, 40))
    big = torch.randn(6, 40)
    _same(x.to(dev).scatter_add(1, dup.to(dev), big.to(dev)), x.scatter_add(1, dup, big), tol=1e-5)
    xi = torch.zeros(5, 7, dtype=torch.int64)
    di = torch.randint(0, 5, (30, 7))
    _same(xi.to(dev).scatter_add(0, di.to(dev), torch.ones(30, 7, dtype=torch.int64).to(dev)),
          xi.scatter_add(0, di, torch.ones(30, 7, dtype=torch.int64)))
    d = x.to(dev)
    d.scatter_add_(1, dup.to(dev), big.to(dev))
    _same(d, x.clone().scatter_add_(1, dup, big), tol=1e-5)
    lab = torch.randint(0, 10, (33,))
    _same(torch.nn.functional.one_hot(lab.to(dev), 10), torch.nn.functional.one_hot(lab, 10))
    assert not any("scatter" in k for k in bw.fallback_counts()), bw.fallback_counts()


def test_advanced_indexing(bw, dev):
    bw.reset_fallback_counts()
    x = torch.randn(6, 7, 8)
    i = torch.tensor([5, 0, 0, 3, -1])
    j = torch.tensor([1, 2, 6, -2, 0])
    d = x.to(dev)
    _same(d[i.to(dev)], x[i])
    _same(d[i.to(dev), j.to(dev)], x[i, j])
    _same(d[:, j.to(dev)], x[:, j])
    _same(d[:, i.to(dev).view(5, 1) % 7, j.to(dev).view(1, 5)], x[:, i.view(5, 1) % 7, j.view(1, 5)])
    _same(d[i.to(dev).view(1, 5).expand(2, 5)], x[i.view(1, 5).expand(2, 5)])
    # writes
    y, yd = x.clone(), x.to(dev)
    rows = torch.tensor([4, 1])
    y[rows] = 0.5
    yd[rows.to(dev)] = 0.5
    _same(yd, y)
    vals = torch.randn(2, 8)
    y[rows, 3] = vals
    yd[rows.to(dev), 3] = vals.to(dev)
    _same(yd, y)
    acc_i = torch.tensor([0, 0, 2, 0])
    upd = torch.randn(4, 7, 8)
    y.index_put_((acc_i,), upd, accumulate=True)
    yd.index_put_((acc_i.to(dev),), upd.to(dev), accumulate=True)
    _same(yd, y, tol=1e-5)
    emb = torch.nn.Embedding(50, 16)
    tok = torch.randint(0, 50, (4, 9))
    _same(emb.weight.detach().to(dev)[tok.to(dev)], emb.weight.detach()[tok])
    assert not any(k.startswith("aten::index") or "_index_put" in k for k in bw.fallback_counts()), bw.fallback_counts()


def test_out_of_range_index_is_reported_not_a_fault(bw, dev):
    x = torch.arange(10.0).to(dev)
    bad = torch.tensor([3, 12]).to(dev)
    out = torch.index_select(x, 0, bad)                  # clamped access
    with pytest.raises(IndexError, match="index out of range"):
        bw.synchronize()
    assert out.cpu()[0] == 3.0
    assert float((x + 1).sum().cpu()) == 55.0            # the context is alive
    bw.synchronize()


def test_tril_triu_arange_cumsum(bw, dev):
    bw.reset_fallback_counts()
    x = torch.randn(3, 9, 11)
    for k in (-2, 0, 3):
        _same(torch.tril(x.to(dev), k), torch.tril(x, k))
        _same(torch.triu(x.to(dev), k), torch.triu(x, k))
    m = torch.ones(6, 6, dtype=torch.bool)
    _same(torch.tril(m.to(dev)), torch.tril(m))
    _same(torch.arange(17, device=dev), torch.arange(17))
    _same(torch.arange(3, 40, 4, device=dev), torch.arange(3, 40, 4))
    _same(torch.arange(0.0, 1.0, 0.125, device=dev), torch.arange(0.0, 1.0, 0.125))
    _same(torch.arange(10, 0, -3, device=dev, dtype=torch.int32), torch.arange(10, 0, -3, dtype=torch.int32))
    y = torch.randn(5, 3000)
    _same(torch.cumsum(y.to(dev), 1), torch.cumsum(y, 1), tol=1e-3)
    _same(torch.cumsum(y.to(dev), 0), torch.cumsum(y, 0), tol=1e-4)
    yi = torch.randint(0, 9, (4, 77))
    _same(torch.cumsum(yi.to(dev), -1), torch.cumsum(yi, -1))
    _same(torch.cumsum(yi.int().to(dev), 0), torch.cumsum(yi.int(), 0))
    assert not bw.fallback_counts(), bw.fallback_counts()


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.int64, torch.int32])
def test_sort_topk(bw, dev, dt):
    bw.reset_fallback_counts()
    g = torch.Generator().manual_seed(3)
    x = torch.randperm(40 * 300, generator=g).reshape(40, 300)            # distinct values: a unique order
    x = (x.float() / 7 - 500).to(dt) if dt.is_floating_point and dt != torch.bfloat16 else x.to(dt) if dt != torch.bfloat16 else (x % 251 * 4).to(dt)
    for dim, desc in ((1, False), (1, True), (0, False)):
        v, i = torch.sort(x.to(dev), dim=dim, descending=desc, stable=True)
        rv, ri = torch.sort(x, dim=dim, descending=desc, stable=True)
        _same(v, rv)
        _same(i, ri)
    _same(torch.argsort(x.to(dev), dim=1, stable=True), torch.argsort(x, dim=1, stable=True))
    if dt.is_floating_point:
        small = torch.randn(1000, 8, generator=g).to(dt)
        v, i = torch.topk(small.to(dev), 2, dim=-1)
        rv, ri = torch.topk(small, 2, dim=-1)
        _same(v, rv)
        assert torch.equal(torch.gather(small, 1, i.cpu()), rv)
        v, i = torch.topk(small.to(dev), 3, dim=-1, largest=False)
        _same(v, torch.topk(small, 3, dim=-1, largest=False)[0])
    wide = x[:, :200]
    v, i = torch.topk(wide.to(dev), 20, dim=1)                             # beyond the small kernel: sort + slice
    _same(v, torch.topk(wide, 20, dim=1)[0])
    assert not bw.fallback_counts(), bw.fallback_counts()


def test_split_with_sizes_copy(bw, dev):
    bw.reset_fallback_counts()
    x = torch.randn(4, 30)
    outs = [torch.empty(4, n, device=dev) for n in (5, 10, 15)]
    torch.split_with_sizes_copy(x.to(dev), [5, 10, 15], dim=1, out=outs)
    for o, r in zip(outs, x.split([5, 10, 15], dim=1)):
        _same(o, r.contiguous())
    assert not bw.fallback_counts(), bw.fallback_counts()


# ---------------------------------------------------------------- searchsorted / histc / nonzero / unique / group norm
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.int64])
@pytest.mark.parametrize("right", [False, True])
def test_searchsorted_and_bucketize(bw, dev, dt, right):
    torch.manual_seed(0)
    if dt == torch.int64:
        b = torch.sort(torch.randint(-50, 50, (37,)))[0]
        v = torch.randint(-60, 60, (5, 19))
    else:
        b = torch.sort(torch.randn(37))[0].to(dt)
        v = torch.randn(5, 19).to(dt)
        v[0, :5] = b[3:8]                                    # exact hits: left / right differ
    bw.reset_fallback_counts()
    assert torch.equal(torch.bucketize(v.to(dev), b.to(dev), right=right).cpu(), torch.bucketize(v, b, right=right))
    out32 = torch.searchsorted(b.to(dev), v.to(dev), out_int32=True, right=right)
    assert out32.dtype == torch.int32 and torch.equal(out32.cpu().long(), torch.searchsorted(b, v, right=right))
    rows = torch.sort(torch.randn(5, 23), dim=-1)[0]         # one sorted row per row of values
    vv = torch.randn(5, 7)
    assert torch.equal(torch.searchsorted(rows.to(dev), vv.to(dev), right=right).cpu(),
                       torch.searchsorted(rows, vv, right=right))
    unsorted = torch.randn(31)
    so = torch.argsort(unsorted)
    assert torch.equal(torch.searchsorted(unsorted.to(dev), vv[0].to(dev), sorter=so.to(dev)).cpu(),
                       torch.searchsorted(unsorted, vv[0], sorter=so))
    assert not bw.fallback_counts(), bw.fallback_counts()


def test_histc_nonzero_unique(bw, dev):
    torch.manual_seed(1)
    x = torch.randn(10007)
    bw.reset_fallback_counts()
    assert torch.equal(torch.histc(x.to(dev), bins=64, min=-3, max=3).cpu(), torch.histc(x, bins=64, min=-3, max=3))
    assert torch.equal(torch.histc(x.to(dev), bins=10000).cpu(), torch.histc(x, bins=10000))   # range from the data
    m = torch.randn(7, 11, 5) > 0.3
    assert torch.equal(torch.nonzero(m.to(dev)).cpu(), torch.nonzero(m))
    f = torch.randn(300).to(torch.bfloat16) * (torch.rand(300) > 0.5)
    assert torch.equal(torch.nonzero(f.to(dev)).cpu(), torch.nonzero(f))
    assert torch.nonzero(torch.zeros(5, 3, device=dev)).shape == (0, 2)
    for t in (torch.randint(0, 40, (13, 29)), torch.randn(500).round(decimals=1), torch.randn(257).to(torch.bfloat16)):
        u, inv, cnt = torch.unique(t.to(dev), return_inverse=True, return_counts=True)
        ur, invr, cntr = torch.unique(t, return_inverse=True, return_counts=True)
        assert torch.equal(u.cpu(), ur) and torch.equal(inv.cpu(), invr) and torch.equal(cnt.cpu(), cntr)
    assert torch.equal(torch.unique(torch.tensor([3, 1, 3], device=dev)).cpu(), torch.tensor([1, 3]))
    assert not bw.fallback_counts(), bw.fallback_counts()


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_group_norm(bw, dev, dt):
    torch.manual_seed(2)
    x = torch.randn(3, 32, 7, 5).to(dt)
    w, b = torch.rand(32) + 0.5, torch.randn(32)
    g = torch.randn(3, 32, 7, 5).to(dt)
    xr, wr, br = x.clone().float().requires_grad_(), w.clone().requires_grad_(), b.clone().requires_grad_()
    yr = torch.nn.functional.group_norm(xr, 8, wr, br, 1e-5)
    yr.backward(g.float())
    xd = x.to(dev).requires_grad_()
    wd, bd = w.to(dt).to(dev).requires_grad_(), b.to(dt).to(dev).requires_grad_()
    bw.reset_fallback_counts()
    y = torch.nn.functional.group_norm(xd, 8, wd, bd, 1e-5)
    y.backward(g.to(dev))
    assert not bw.fallback_counts(), bw.fallback_counts()
    tol = 1e-4 if dt == torch.float32 else 3e-2
    for a, r in ((y, yr), (xd.grad, xr.grad), (wd.grad, wr.grad), (bd.grad, br.grad)):
        assert (a.float().cpu() - r).abs().max() <= tol * max(1.0, float(r.abs().max()))
