"""Lowering of a PT2E-quantized graph for this backend.

``lower_pt2e_quantized(model, example_inputs)`` takes the GraphModule that ``convert_pt2e`` produced (quantize /
dequantize nodes around float operators), re-exports it, keeps only the composite-implicit decompositions (the
quantization patterns must survive), rewrites ``aten.t`` as ``aten.permute`` (the pattern matchers downstream know
permute only), and folds what depends on constants alone -- except the dequantize of a quantized weight, which the
folder leaves in place on purpose: ``dequantize -> permute -> addmm`` is the pattern a quantized-GEMM rewrite matches.
The result is an ordinary GraphModule: run it eagerly or hand it to ``torch.compile``.

Parity: reference torch_musa/core/lowering.py:7-60 (installed there over the x86 lowering entry point).
"""
from __future__ import annotations

from typing import Tuple

import torch


def _implicit_only_decompositions():
    """The default export decomposition table restricted to composite-implicit operators."""
    from torch._export.utils import _is_cia_op

    table = torch.export.default_decompositions()
    for op in [op for op in table.keys() if not _is_cia_op(op)]:
        del table[op]
    return table


def _t_to_permute(gm: torch.fx.GraphModule) -> int:
    aten, n = torch.ops.aten, 0
    for node in list(gm.graph.nodes):
        if node.op == "call_function" and node.target == aten.t.default:
            with gm.graph.inserting_before(node):
                new = gm.graph.call_function(aten.permute.default, args=(node.args[0], [1, 0]))
            new.meta = dict(node.meta)
            node.replace_all_uses_with(new)
            gm.graph.erase_node(node)
            n += 1
    if n:
        gm.graph.lint()
        gm.recompile()
    return n


def lower_pt2e_quantized(model: torch.fx.GraphModule, example_inputs: Tuple[torch.Tensor, ...]) -> torch.fx.GraphModule:
    from torch._inductor.constant_folding import constant_fold

    exported = torch.export.export(model, tuple(example_inputs), strict=True)
    lowered = exported.run_decompositions(_implicit_only_decompositions()).module()
    _t_to_permute(lowered)
    constant_fold(lowered)
    return lowered


def install() -> None:
    """Publishes the lowering under ``torch.ao.quantization.pt2e`` for code that looks it up there."""
    try:
        import torch.ao.quantization.pt2e as pt2e

        pt2e.lower_pt2e_quantized_to_blackwell = lower_pt2e_quantized
    except ImportError:  # pragma: no cover - the PT2E package is optional in a PyTorch build
        pass
