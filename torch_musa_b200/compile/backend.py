"""``torch.compile`` for the blackwell device.

``backend="blackwell"`` (also what plain ``torch.compile(model)`` resolves to when the inputs live
on this device): Dynamo traces, AOT-autograd splits forward and backward, and each graph is lowered
by ``compile.lower`` -- GEMM epilogue fusion, element-wise groups turned into generated CUDA kernels,
everything else dispatched to the backend's hand-written kernels -- into a program that a C++ runner
executes without the interpreter.  With ``options={"graphs": True}`` (or ``mode="reduce-overhead"``)
the programs are additionally recorded in graph trees and replayed as CUDA graphs.

Parity: reference torch_musa/_inductor/__init__.py:17-39 (device code generation registered with the
compiler), _dynamo/backend/musagraphs.py:171-322 and _inductor/musagraph_trees.py (graph replay).
"""
from __future__ import annotations

import functools
import os
from typing import Sequence

import torch

from . import graph_trees, lower

stats = {"graphs_lowered": 0, "graphs_fallback": 0, "fused_kernels": 0, "fused_ops": 0, "addmm_epilogues": 0}
last_descriptions = []   # program descriptions of the most recent compilations (introspection, tests)


def _compile_graph(fx_gm: torch.fx.GraphModule, example_inputs, *, graphs: bool, is_backward: bool, fuse: bool):
    try:
        n_epi = lower.fuse_addmm_activation(fx_gm) if fuse else 0
        kernels = lower.partition_pointwise(fx_gm) if fuse else {}
        desc = lower.describe_program(fx_gm, kernels)
        runner = lower.instantiate(desc)
    except lower.Unsupported as e:
        if os.environ.get("B200_COMPILE_DEBUG"):
            print(f"[blackwell compile] interpreter fallback: {e}")
        stats["graphs_fallback"] += 1
        fwd = fx_gm.forward

        def call(args):
            out = fwd(*args)
            return list(out) if isinstance(out, (tuple, list)) else [out]
    else:
        stats["graphs_lowered"] += 1
        stats["fused_kernels"] += len(kernels)
        stats["fused_ops"] += sum(k["n_ops"] for k in kernels.values())
        stats["addmm_epilogues"] += n_epi
        last_descriptions.append(desc)
        del last_descriptions[:-8]
        call = runner.run

    if not graphs:
        def run(args):
            a = list(args)
            args.clear()
            return call(a)
    else:
        fn_id = graph_trees.new_function_id()

        def run(args):
            a = list(args)
            args.clear()
            on_dev = [t for t in a if isinstance(t, torch.Tensor) and t.device.type == "blackwell"]
            if not on_dev:
                return call(a)
            dev = on_dev[0].device.index
            if dev is None:
                import torch_musa_b200 as bw

                dev = bw.current_device()
            return graph_trees.get_manager(dev).run(fn_id, call, a, clone_outputs=is_backward)

    run._boxed_call = True
    return run


def blackwell(gm: torch.fx.GraphModule, example_inputs: Sequence[torch.Tensor], *, graphs: bool = False,
              fuse: bool = True, options: dict = None, mode: str = None):
    """Options (``torch.compile(..., backend="blackwell", options={...})``): ``graphs`` -- record and replay CUDA
    graphs through graph trees (also switched on by ``mode="reduce-overhead"``); ``fuse`` -- run the fusion passes."""
    from torch._dynamo.backends.common import aot_autograd

    options = dict(options or {})
    graphs = bool(options.pop("graphs", graphs)) or mode in ("reduce-overhead", "max-autotune")
    fuse = bool(options.pop("fuse", fuse))
    if options:
        raise ValueError(f"unknown options for the blackwell compiler: {sorted(options)}")

    mk = lambda bwd: functools.partial(_compile_graph, graphs=graphs, is_backward=bwd, fuse=fuse)  # noqa: E731
    return aot_autograd(fw_compiler=mk(False), bw_compiler=mk(True), inference_compiler=mk(False))(gm, example_inputs)


def _on_device(gm: torch.fx.GraphModule, inputs) -> bool:
    for t in inputs:
        if isinstance(t, torch.Tensor) and t.device.type == "blackwell":
            return True
    for n in gm.graph.nodes:
        v = n.meta.get("example_value", n.meta.get("val"))
        if isinstance(v, torch.Tensor) and v.device.type == "blackwell":
            return True
    return False


def register() -> None:
    """Registers ``backend="blackwell"`` and routes the default compiler to it for graphs on this device."""
    try:
        from torch._dynamo import register_backend
        from torch._dynamo.backends.registry import _COMPILER_FNS

        if "blackwell" not in _COMPILER_FNS:
            register_backend(name="blackwell")(blackwell)
    except Exception:  # pragma: no cover
        return
    wrapper = getattr(torch, "_TorchCompileInductorWrapper", None)
    if wrapper is None or getattr(wrapper, "_b200_routed", False):
        return
    stock_call = wrapper.__call__

    def routed(self, model_, inputs_):
        if isinstance(model_, torch.fx.GraphModule) and _on_device(model_, inputs_):
            cfg = getattr(self, "config", {}) or {}
            return blackwell(model_, inputs_, graphs=bool(cfg.get("triton.cudagraphs", False)))
        return stock_call(self, model_, inputs_)

    wrapper.__call__ = routed
    wrapper._b200_routed = True
