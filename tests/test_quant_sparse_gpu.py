"""Quantized (per-tensor affine) and sparse COO tensors on the device against the CPU implementations.
Mirrors reference tests/unittest/operator/test_quantized*.py and the sparse cases of test_tensor.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("qdt", [torch.qint8, torch.quint8])
def test_quantize_dequantize_roundtrip(bw, dev, qdt):
    torch.manual_seed(0)
    x = torch.randn(5, 33) * 3
    zp = 3 if qdt == torch.qint8 else 120
    qr = torch.quantize_per_tensor(x, 0.05, zp, qdt)
    q = torch.quantize_per_tensor(x.to(dev), 0.05, zp, qdt)
    assert q.is_quantized and q.device.type == "blackwell" and q.q_scale() == 0.05 and q.q_zero_point() == zp
    assert q.qscheme() == torch.per_tensor_affine
    assert torch.equal(q.int_repr().cpu(), qr.int_repr())
    assert torch.allclose(q.dequantize().cpu(), qr.dequantize())
    q2 = torch._make_per_tensor_quantized_tensor(q.int_repr(), 0.1, zp)
    assert torch.allclose(q2.dequantize().cpu(), (qr.int_repr().float() - zp) * 0.1)
    e = torch._empty_affine_quantized((4, 4), scale=0.5, zero_point=1, dtype=qdt, device=dev)
    assert e.is_quantized and e.q_scale() == 0.5 and tuple(e.shape) == (4, 4)


def test_sparse_coo_tensor(bw, dev):
    torch.manual_seed(1)
    i = torch.tensor([[0, 1, 1, 3, 0], [2, 0, 2, 1, 2]])
    v = torch.tensor([3.0, 4.0, 5.0, 6.0, 7.0])                  # (0, 2) appears twice
    sr = torch.sparse_coo_tensor(i, v, (4, 3))
    s = torch.sparse_coo_tensor(i.to(dev), v.to(dev), (4, 3))
    assert s.is_sparse and s.device.type == "blackwell" and s._nnz() == 5 and s.sparse_dim() == 2
    assert torch.equal(s.to_dense().cpu(), sr.to_dense())
    c, cr = s.coalesce(), sr.coalesce()
    assert c.is_coalesced() and c._nnz() == 4
    assert torch.equal(c.indices().cpu(), cr.indices()) and torch.equal(c.values().cpu(), cr.values())
    d = torch.randn(3, 6)
    assert torch.allclose(torch.sparse.mm(s, d.to(dev)).cpu(), torch.sparse.mm(sr, d), atol=1e-5)
    # values with trailing dense dimensions
    v2 = torch.randn(5, 2)
    s2 = torch.sparse_coo_tensor(i.to(dev), v2.to(dev), (4, 3, 2))
    assert torch.allclose(s2.to_dense().cpu(), torch.sparse_coo_tensor(i, v2, (4, 3, 2)).to_dense())


def test_jagged_nested_tensor(bw, dev):
    """Jagged nested tensors are a wrapper over one packed values tensor: their operators land on this device's
    dense kernels (linear on the GEMM, element-wise and reductions on the substrate)."""
    torch.manual_seed(2)
    parts = [torch.randn(n, 64) for n in (5, 1, 9)]
    w = torch.randn(32, 64)
    nt = torch.nested.nested_tensor([p.to(dev) for p in parts], layout=torch.jagged)
    assert nt.device.type == "blackwell" and nt.is_nested
    out = torch.nn.functional.linear(nt, w.to(dev))
    act = torch.nn.functional.gelu(out) * 2.0
    for got, p in zip(act.unbind(), parts):
        ref = torch.nn.functional.gelu(p @ w.t()) * 2.0
        assert torch.allclose(got.cpu(), ref, atol=2e-2, rtol=2e-2)
    padded = torch.nested.to_padded_tensor(act, 0.0)
    assert tuple(padded.shape) == (3, 9, 32)
    assert torch.allclose(padded[1, 1:].cpu(), torch.zeros(8, 32))
