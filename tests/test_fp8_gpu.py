"""Block-scaled fp8 GEMM (tcgen05 kind::f8f6f4) and the 1x128 quantiser against an fp32 reference built from the
same quantised values."""
import pytest
import torch

pytestmark = pytest.mark.gpu

F8 = torch.float8_e4m3fn


def quant_blocks(x, bm, bk=128):
    """Reference block quantisation on the CPU: returns (fp8 tensor, scales [M/bm, K/bk])."""
    M, K = x.shape
    xb = x.float().view(M // bm, bm, K // bk, bk)
    amax = xb.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / 448.0
    q = (xb / scale[:, None, :, None]).clamp(-448, 448).view(M, K).to(F8)
    return q, scale


def dequant(q, scale, bm, bk=128):
    M, K = q.shape
    return (q.float().view(M // bm, bm, K // bk, bk) * scale[:, None, :, None]).view(M, K)


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (384, 256, 1024), (200, 136, 256)])
def test_blockwise_scaled_mm(bw, dev, m, n, k):
    torch.manual_seed(0)
    a, b = torch.randn(m, k), torch.randn(n, k) * 0.5
    mp, npad = (m + 127) // 128 * 128, (n + 127) // 128 * 128
    qa, sa = quant_blocks(a, 1)                                      # 1 x 128 blocks
    bpad = torch.zeros(npad, k); bpad[:n] = b
    qb_p, sb = quant_blocks(bpad, 128)                               # 128 x 128 blocks
    qb = qb_p[:n].contiguous()
    ref = dequant(qa, sa, 1) @ dequant(qb_p, sb, 128)[:n].t()
    bw.reset_kernel_launch_count()
    y = torch.ops.blackwell.scaled_mm(qa.to(dev), qb.to(dev), sa.to(dev), sb.to(dev), None, None, None, torch.bfloat16)
    assert bw.kernel_launch_count() == 1
    err = (y.float().cpu() - ref).abs().max() / ref.abs().max()
    assert err < 1e-2, float(err)
    bw.synchronize()
    assert bw._C._gemm_status(False) == 0


def test_aten_scaled_mm_layouts(bw, dev):
    torch.manual_seed(1)
    m, n, k = 256, 256, 256
    a, b = torch.randn(m, k), torch.randn(n, k)
    qa, qb = a.clamp(-400, 400).to(F8), b.clamp(-400, 400).to(F8)
    ref = qa.float() @ qb.float().t()
    ad, bd = qa.to(dev), qb.to(dev)
    # tensor-wise
    sa, sb = torch.tensor(0.5, device=dev), torch.tensor(0.25, device=dev)
    y = torch._scaled_mm(ad, bd.t(), sa, sb, out_dtype=torch.float32)
    assert torch.allclose(y.cpu(), ref * 0.125, rtol=1e-3, atol=1e-2)
    # row-wise with bias
    ra, rb = torch.rand(m, 1) + 0.5, torch.rand(1, n) + 0.5
    bias = torch.randn(n).to(torch.bfloat16)
    y = torch._scaled_mm(ad, bd.t(), ra.to(dev), rb.to(dev), bias=bias.to(dev), out_dtype=torch.bfloat16)
    want = ref * ra * rb + bias.float()
    assert ((y.float().cpu() - want).abs().max() / want.abs().max()) < 1e-2


def test_quantize_1x128(bw, dev):
    x = (torch.randn(64, 512) * 3).to(torch.bfloat16)
    q, s = torch.ops.blackwell.quantize_fp8_1x128(x.to(dev))
    q_ref, s_ref = quant_blocks(x.float(), 1)
    assert torch.allclose(s.cpu(), s_ref, rtol=1e-6)
    back = dequant(q.cpu(), s.cpu(), 1)
    assert ((back - x.float()).abs().max() / x.float().abs().max()) < 0.07
    # end to end: quantise on the device, multiply, compare with the bf16 product
    w = (torch.randn(256, 512) * 0.1)
    qw, sw = quant_blocks(w, 128)
    y = torch.ops.blackwell.scaled_mm(q, qw.to(dev), s, sw.to(dev), None, None, None, torch.bfloat16)
    ref = x.float() @ w.t()
    assert ((y.float().cpu() - ref).abs().max() / ref.abs().max()) < 0.08
