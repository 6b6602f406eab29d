"""Ahead-of-time compilation: ``aot_compile`` turns a module into a self-contained package and
``aot_load`` runs it without tracing, Python operator dispatch or a compiler at hand.

The package is a zip with
* ``program.pkl``  -- the lowered program (instruction list over value slots, see ``compile.lower``),
* ``kernels/*.cubin`` + ``kernels/*.cu`` -- the generated fused kernels, compiled for sm_100a at export time,
* ``weights.pt``   -- parameters and buffers in the order the program reads them,
* ``spec.json``    -- input / output tree specs and which outputs are buffer updates.
Loading builds a C++ ``_GraphRunner`` over the program; calling it flattens the arguments, runs the
instructions natively and rebuilds the output structure.

Parity: reference torch_musa/_export/__init__.py:10-39 (aot_compile / aot_load for the device) and
csrc/inductor/aoti_runner/model_container_runner_musa.cpp:6-49 (the native runner behind aot_load).
"""
from __future__ import annotations

import io
import json
import pickle
import zipfile
from typing import Any, Dict, Optional, Sequence, Tuple

import torch
import torch.utils._pytree as pytree

from .compile import lower

FORMAT_VERSION = 1


def aot_compile(model: torch.nn.Module, args: Tuple[Any, ...], path: str, kwargs: Optional[Dict[str, Any]] = None,
                *, fuse: bool = True) -> str:
    """Export ``model`` for the given example inputs and write the package to ``path``."""
    from torch.export.graph_signature import InputKind, OutputKind

    ep = torch.export.export(model, tuple(args), kwargs or {}, strict=False)
    ep = ep.run_decompositions({})
    gm = ep.graph_module
    sig = ep.graph_signature
    state = dict(ep.state_dict)
    state.update(getattr(ep, "constants", {}) or {})
    weights, input_kinds = [], []
    for spec in sig.input_specs:
        if spec.kind == InputKind.USER_INPUT:
            input_kinds.append("user")
        elif spec.kind in (InputKind.PARAMETER, InputKind.BUFFER, InputKind.CONSTANT_TENSOR):
            input_kinds.append("weight")
            weights.append((spec.target, state[spec.target].detach()))
        else:
            raise lower.Unsupported(f"exported input of kind {spec.kind}")
    out_kinds = []
    for spec in sig.output_specs:
        if spec.kind == OutputKind.USER_OUTPUT:
            out_kinds.append(["user", None])
        elif spec.kind == OutputKind.BUFFER_MUTATION:
            out_kinds.append(["buffer", spec.target])
        else:
            raise lower.Unsupported(f"exported output of kind {spec.kind}")
    kernels = {}
    if fuse:
        lower.fuse_addmm_activation(gm)
        kernels = lower.partition_pointwise(gm)
    desc = lower.describe_program(gm, kernels)
    with zipfile.ZipFile(path, "w", zipfile.ZIP_STORED) as z:
        for name, info in desc["kernels"].items():
            k = lower.get_kernel(info)
            z.writestr(f"kernels/{info['entry']}.cubin", bytes(k.cubin))
            z.writestr(f"kernels/{info['entry']}.cu", info["source"])
            info.pop("source", None)
        z.writestr("program.pkl", pickle.dumps(desc))
        buf = io.BytesIO()
        torch.save({"names": [n for n, _ in weights], "tensors": [t.cpu() for _, t in weights]}, buf)
        z.writestr("weights.pt", buf.getvalue())
        call_spec = ep.call_spec
        z.writestr("spec.json", json.dumps({
            "format": FORMAT_VERSION,
            "in_spec": pytree.treespec_dumps(call_spec.in_spec),
            "out_spec": pytree.treespec_dumps(call_spec.out_spec),
            "input_kinds": input_kinds,
            "output_kinds": out_kinds,
            "device": str(next((t.device for _, t in weights), "cpu")),
        }))
    return path


class LoadedModel:
    """Callable returned by ``aot_load``."""

    def __init__(self, runner, weights, names, spec):
        self.runner = runner
        self.weights = weights
        self.names = names
        self.in_spec = pytree.treespec_loads(spec["in_spec"])
        self.out_spec = pytree.treespec_loads(spec["out_spec"])
        self.input_kinds = spec["input_kinds"]
        self.output_kinds = spec["output_kinds"]

    def __call__(self, *args, **kwargs):
        flat, in_spec = pytree.tree_flatten((args, kwargs))
        if in_spec != self.in_spec:
            raise TypeError("arguments do not match the structure the package was compiled for")
        it_w, it_u = iter(self.weights), iter(flat)
        inputs = [next(it_w) if k == "weight" else next(it_u) for k in self.input_kinds]
        with torch.no_grad():
            outs = self.runner.run(inputs)
        user = []
        for (kind, target), o in zip(self.output_kinds, outs):
            if kind == "buffer":
                self.weights[self.names.index(target)].copy_(o)
            else:
                user.append(o)
        return pytree.tree_unflatten(user, self.out_spec)


def aot_load(path: str, device: Optional[Any] = None) -> LoadedModel:
    """Load a package written by ``aot_compile``; weights go to ``device`` (default: where they were exported)."""
    with zipfile.ZipFile(path) as z:
        spec = json.loads(z.read("spec.json"))
        if spec.get("format") != FORMAT_VERSION:
            raise RuntimeError(f"unsupported package format {spec.get('format')}")
        desc = pickle.loads(z.read("program.pkl"))
        for info in desc["kernels"].values():
            info["cubin"] = z.read(f"kernels/{info['entry']}.cubin")
        w = torch.load(io.BytesIO(z.read("weights.pt")), weights_only=True)
    dev = torch.device(device if device is not None else spec["device"])
    weights = [t.to(dev) for t in w["tensors"]]
    runner = lower.instantiate(desc)
    return LoadedModel(runner, weights, w["names"], spec)
