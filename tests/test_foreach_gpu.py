"""The _foreach_* pointwise family on the multi-tensor kernel against per-tensor CPU results, including lists the fused
kernel does not cover (mixed dtypes, views), which run tensor by tensor on the general loops.
Parity: reference tests/unittest/operator/test_foreach_*.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lists(dev, dt, n=7):
    g = torch.Generator().manual_seed(11)
    shapes = [(5,), (33, 17), (1,), (4096,), (3, 5, 7), (1025,), (64, 64)][:n]
    cpu = [torch.randn(s, generator=g).to(dt) for s in shapes]
    return cpu, [t.to(dev) for t in cpu]


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_foreach_ops(bw, dev, dt):
    bw.reset_fallback_counts()
    tol = 1e-6 if dt == torch.float32 else 2e-2
    a, ad = _lists(dev, dt)
    b, bd = _lists(dev, dt)
    b = [t.abs() + 0.5 for t in b]
    bd = [t.abs() + 0.5 for t in bd]

    def same(xs, ys):
        for x, y in zip(xs, ys):
            assert x.dtype == y.dtype and torch.allclose(x.cpu().float(), y.float(), atol=tol, rtol=tol)

    before = bw.kernel_launch_count()
    same(torch._foreach_add(ad, bd, alpha=0.5), torch._foreach_add(a, b, alpha=0.5))
    assert bw.kernel_launch_count() - before <= 2, "the list should run as one or two launches"
    same(torch._foreach_mul(ad, 1.5), torch._foreach_mul(a, 1.5))
    same(torch._foreach_mul(ad, bd), torch._foreach_mul(a, b))
    same(torch._foreach_div(ad, bd), torch._foreach_div(a, b))
    same(torch._foreach_sqrt(bd), torch._foreach_sqrt(b))
    same(torch._foreach_neg(ad), torch._foreach_neg(a))
    same(torch._foreach_maximum(ad, bd), torch._foreach_maximum(a, b))
    for inplace, args, kw in (("_foreach_add_", (bd,), {"alpha": 2.0}), ("_foreach_mul_", (0.9,), {}), ("_foreach_addcmul_", (bd, bd), {"value": 0.1}),
                              ("_foreach_addcdiv_", (bd, bd), {"value": -0.3}), ("_foreach_lerp_", (bd, 0.25), {}), ("_foreach_sub_", (bd,), {}),
                              ("_foreach_div_", (2.0,), {})):
        cpu_args = tuple([t.cpu() for t in x] if isinstance(x, list) else x for x in args)
        ad = [t.to(dev) for t in a]          # same starting values: the device rounds once per fused op, the host per step
        getattr(torch, inplace)(ad, *args, **kw)
        getattr(torch, inplace)(a, *cpu_args, **kw)
        same(ad, a)
    torch._foreach_zero_(ad)
    assert all(float(t.abs().sum().cpu()) == 0 for t in ad)
    torch._foreach_copy_(ad, bd)
    same(ad, b)
    assert not bw.fallback_counts(), bw.fallback_counts()


def test_foreach_uncovered_lists_run_per_tensor(bw, dev):
    bw.reset_fallback_counts()
    a = [torch.randn(4, 6), torch.randn(8).double(), torch.arange(6).reshape(2, 3)]
    ad = [t.to(dev) for t in a]
    ad[0] = ad[0].t()                     # a view: not dense in the list's sense
    a[0] = a[0].t()
    for x, y in zip(torch._foreach_mul(ad, 2), torch._foreach_mul(a, 2)):
        assert x.dtype == y.dtype and torch.equal(x.cpu(), y)
    torch._foreach_add_(ad, 1)
    torch._foreach_add_(a, 1)
    for x, y in zip(ad, a):
        assert torch.equal(x.cpu(), y)
    assert not bw.fallback_counts(), bw.fallback_counts()
