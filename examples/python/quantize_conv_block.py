#!/usr/bin/env python
"""Quantization-aware training of a conv / batch-norm / SiLU block with the backend's torch.ao extensions, then
conversion to the int8-weight block.

    python examples/python/quantize_conv_block.py
"""
from __future__ import annotations

import os
import sys
import warnings

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402
from torch import nn  # noqa: E402

import torch_musa_b200  # noqa: E402,F401  (publishes ConvBnSiLU2d & co. under torch.ao.nn.intrinsic*)

tq = torch.ao.quantization


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.quant, self.dequant = tq.QuantStub(), tq.DeQuantStub()
        self.conv, self.bn, self.act = nn.Conv2d(3, 16, 3, padding=1, bias=False), nn.BatchNorm2d(16), nn.SiLU()

    def forward(self, x):
        return self.dequant(self.act(self.bn(self.conv(self.quant(x)))))


def main() -> float:
    warnings.simplefilter("ignore")
    torch.manual_seed(0)
    m = Block().train()
    m.qconfig = tq.get_default_qat_qconfig("fbgemm")
    tq.fuse_modules_qat(m, [["conv", "bn", "act"]], inplace=True)        # -> intrinsic.ConvBnSiLU2d
    tq.prepare_qat(m, inplace=True)                                       # -> qat.ConvBnSiLU2d (fake-quantized weight)
    opt = torch.optim.SGD(m.parameters(), lr=0.05)
    for _ in range(20):
        loss = (m(torch.randn(8, 3, 16, 16)) - 0.25).pow(2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
    m.eval()
    q = tq.convert(m, inplace=False)                                      # -> quantized.ConvSiLU2d (int8 weights)
    x = torch.randn(2, 3, 16, 16)
    err = float((q(x) - m(x)).abs().max())
    print(f"{type(q.conv).__name__}: int8 weights {tuple(q.conv.weight_int8.shape)}, output scale {q.conv.scale:.4g}, "
          f"max |quantized - fake-quantized| = {err:.4g}")
    return err


if __name__ == "__main__":
    main()
