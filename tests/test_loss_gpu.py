"""Loss functions (MSE, NLL with weights / ignore_index, BCE, and the composite KL / L1 / BCE-with-logits) forward and
backward against CPU autograd, with no library fallback.
Parity: reference tests/unittest/operator/test_loss.py, test_nll_loss.py, test_bce.py."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _fwd_bwd(fn, dev, *inputs, tol=1e-5):
    cpu = [t.clone().requires_grad_(t.is_floating_point() and i == 0) for i, t in enumerate(inputs)]
    d = [t.to(dev).requires_grad_(t.is_floating_point() and i == 0) for i, t in enumerate(inputs)]
    r, o = fn(*cpu), fn(*d)
    assert torch.allclose(o.cpu(), r, atol=tol, rtol=tol), (o.cpu() - r).abs().max()
    g = torch.randn_like(r)
    r.backward(g)
    o.backward(g.to(dev))
    assert torch.allclose(d[0].grad.cpu(), cpu[0].grad, atol=tol, rtol=tol), (d[0].grad.cpu() - cpu[0].grad).abs().max()


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_losses(bw, dev, reduction):
    bw.reset_fallback_counts()
    x, t = torch.randn(12, 7), torch.randn(12, 7)
    _fwd_bwd(lambda a, b: F.mse_loss(a, b, reduction=reduction), dev, x, t)
    _fwd_bwd(lambda a, b: F.l1_loss(a, b, reduction=reduction), dev, x, t)
    logp = torch.log_softmax(torch.randn(20, 9), -1)
    tgt = torch.randint(0, 9, (20,))
    tgt[3] = -100
    w = torch.rand(9) + 0.5
    _fwd_bwd(lambda a, b: F.nll_loss(a, b, reduction=reduction), dev, logp, tgt)
    _fwd_bwd(lambda a, b, c: F.nll_loss(a, b, weight=c, reduction=reduction), dev, logp, tgt, w)
    p, y = torch.rand(10, 5) * 0.9 + 0.05, torch.rand(10, 5)
    _fwd_bwd(lambda a, b: F.binary_cross_entropy(a, b, reduction=reduction), dev, p, y, tol=1e-4)
    _fwd_bwd(lambda a, b: F.binary_cross_entropy_with_logits(a, b, reduction=reduction), dev, x[:10, :5], y, tol=1e-4)
    _fwd_bwd(lambda a, b: F.kl_div(a, b, reduction="sum" if reduction == "mean" else reduction), dev, logp, torch.softmax(torch.randn(20, 9), -1))
    _fwd_bwd(lambda a, b: F.cross_entropy(a, b, reduction=reduction), dev, torch.randn(20, 9), tgt.clamp_min(0))
    assert not bw.fallback_counts(), bw.fallback_counts()
