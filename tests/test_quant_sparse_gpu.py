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
