"""Quantization support: fused conv / batch-norm / SiLU blocks through torch.ao's eager flow (QAT and post-training)
and the graph lowering, all on the CPU."""
import warnings

import pytest
import torch
from torch import nn

import torch_musa_b200  # noqa: F401
import torch_musa_b200.ao as ao

tq = torch.ao.quantization


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.quant, self.dequant = tq.QuantStub(), tq.DeQuantStub()
        self.conv1, self.bn1, self.act1 = nn.Conv2d(3, 8, 3, padding=1, bias=False), nn.BatchNorm2d(8), nn.SiLU()
        self.conv2, self.act2 = nn.Conv2d(8, 8, 3, padding=1), nn.SiLU()

    def forward(self, x):
        x = self.quant(x)
        x = self.act1(self.bn1(self.conv1(x)))
        return self.dequant(self.act2(self.conv2(x)))


def test_qat_flow_fuses_trains_and_converts():
    warnings.simplefilter("ignore")
    torch.manual_seed(0)
    m = _Net().train()
    m.qconfig = tq.get_default_qat_qconfig("fbgemm")
    tq.fuse_modules_qat(m, [["conv1", "bn1", "act1"], ["conv2", "act2"]], inplace=True)
    assert isinstance(m.conv1, ao.nn.intrinsic.ConvBnSiLU2d) and isinstance(m.conv2, ao.nn.intrinsic.ConvSiLU2d)
    assert isinstance(m.bn1, nn.Identity) and isinstance(m.act1, nn.Identity)
    tq.prepare_qat(m, inplace=True)
    assert type(m.conv1) is ao.nn.qat.ConvBnSiLU2d and type(m.conv2) is ao.nn.qat.ConvSiLU2d
    opt = torch.optim.SGD(m.parameters(), lr=0.01)
    w0 = m.conv1.weight.detach().clone()
    for _ in range(4):
        loss = m(torch.randn(4, 3, 16, 16)).pow(2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert not torch.equal(w0, m.conv1.weight)                       # gradients reach the folded weight
    m.eval()
    x = torch.randn(2, 3, 16, 16)
    want = m(x)                                                       # fake-quantized evaluation
    q = tq.convert(m, inplace=False)
    assert type(q.conv1) is ao.nn.quantized.ConvSiLU2d and type(q.conv2) is ao.nn.quantized.ConvSiLU2d
    assert q.conv1.weight_int8.dtype == torch.int8 and q.conv1.bias is not None    # the folded norm left a bias
    got = q(x)
    assert (got - want).abs().max() <= 2.5 * q.conv2.scale            # within a couple of output quantization steps
    # a fresh converted copy takes the state dict (scales included)
    q2 = tq.convert(m, inplace=False)
    q2.conv2.scale = 123.0
    q2.load_state_dict(q.state_dict())
    assert q2.conv2.scale == q.conv2.scale and torch.equal(q2(x), got)
    # back to float for export: the norm is folded, the activation kept
    f = m.conv1.to_float()
    assert isinstance(f, ao.nn.intrinsic.ConvSiLU2d) and f[0].bias is not None


def test_post_training_flow_and_residual_block():
    warnings.simplefilter("ignore")
    torch.manual_seed(1)
    m = _Net().eval()
    m.qconfig = tq.get_default_qconfig("fbgemm")
    tq.fuse_modules(m, [["conv1", "bn1", "act1"], ["conv2", "act2"]], inplace=True)
    assert isinstance(m.conv1, ao.nn.intrinsic.ConvSiLU2d)            # eval: norm folded at fusion time
    ref = m(torch.randn(2, 3, 16, 16))
    assert torch.isfinite(ref).all()
    tq.prepare(m, inplace=True)
    for _ in range(4):
        m(torch.randn(4, 3, 16, 16))
    x = torch.randn(2, 3, 16, 16)
    want = m(x)
    q = tq.convert(m, inplace=False)
    assert type(q.conv1) is ao.nn.quantized.ConvSiLU2d
    assert (q(x) - want).abs().max() < 0.1 * float(want.abs().max()) + 0.05
    # residual tail: silu(conv(x) + other)
    blk = ao.nn.intrinsic.ConvAddSiLU2d(nn.Conv2d(8, 8, 1), nn.SiLU())
    a, b = torch.randn(2, 8, 5, 5), torch.randn(2, 8, 5, 5)
    assert torch.allclose(blk(a, b), torch.nn.functional.silu(blk[0](a) + b))
    blk.qconfig = tq.get_default_qat_qconfig("fbgemm")
    tq.propagate_qconfig_(blk)
    qat_blk = ao.nn.qat.ConvAddSiLU2d.from_float(blk)
    qat_blk.activation_post_process = blk.qconfig.activation()
    qat_blk.activation_post_process(qat_blk(a, b))
    qb = ao.nn.quantized.ConvAddSiLU2d.from_float(qat_blk)
    got = qb(torch.quantize_per_tensor(a, 0.05, 128, torch.quint8), b).dequantize()
    assert (got - blk(a, b)).abs().max() < 0.15
    with pytest.raises(TypeError):
        ao.nn.intrinsic.ConvSiLU2d(nn.Linear(2, 2), nn.SiLU())


def test_classes_are_published_under_torch_ao():
    import torch.ao.nn.intrinsic as nni

    assert nni.ConvBnSiLU2d is ao.nn.intrinsic.ConvBnSiLU2d and nni.qat.ConvSiLU2d is ao.nn.qat.ConvSiLU2d
    assert nni.quantized.ConvAddSiLU2d is ao.nn.quantized.ConvAddSiLU2d
    ao.register()                                                     # idempotent


class _DequantLinear(nn.Module):
    def __init__(self):
        super().__init__()
        import torch.ao.quantization.fx._decomposed  # noqa: F401  (defines the quantized_decomposed operators)

        self.register_buffer("w", torch.randint(-127, 127, (8, 16), dtype=torch.int8))
        self.register_buffer("b", torch.randn(8))

    def forward(self, x):
        w = torch.ops.quantized_decomposed.dequantize_per_tensor(self.w, 0.02, 0, -128, 127, torch.int8)
        return torch.nn.functional.linear(x, w, self.b * 2.0)


def test_graph_lowering_rewrites_transposes_and_folds_constants():
    m = _DequantLinear().eval()
    ex = (torch.randn(4, 16),)
    low = ao.lower_pt2e_quantized(torch.export.export(m, ex).module(), ex)
    targets = [str(n.target) for n in low.graph.nodes if n.op == "call_function"]
    assert not any("aten.t." in t for t in targets) and any("aten.permute" in t for t in targets)
    assert not any("aten.mul" in t for t in targets)                  # constant arithmetic is folded at lowering
    # the weight's dequantize stays: it is the pattern a quantized-GEMM rewrite downstream matches
    assert sum("dequantize_per_tensor" in t for t in targets) == 1
    assert torch.allclose(low(*ex), m(*ex), atol=1e-5)
