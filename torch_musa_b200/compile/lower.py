"""FX graph -> native program.

1. ``fuse_addmm_activation``: ``relu/gelu(addmm(b, x, w))`` becomes one ``aten._addmm_activation`` call, whose
   epilogue runs inside this backend's GEMM kernel.
2. ``partition_pointwise``: element-wise operators are grouped (capability-based partitioner, so a
   group never closes a cycle) and every valid group is turned into one generated CUDA kernel.
3. ``build_program``: the remaining graph is flattened into instructions for the C++ ``_GraphRunner``
   (boxed dispatcher calls / fused kernels / tuple indexing) with slot lifetimes planned ahead.
"""
from __future__ import annotations

import hashlib
import operator
from typing import Dict, List, Optional

import torch
from torch.fx.passes.infra.partitioner import CapabilityBasedPartitioner
from torch.fx.passes.operator_support import OperatorSupportBase

from . import codegen

aten = torch.ops.aten


class Unsupported(RuntimeError):
    """The graph holds something the native runner cannot express; the caller runs the FX module instead."""


def _C():
    from .. import _C as C

    return C


# ----------------------------------------------------------------- pass 1
def fuse_addmm_activation(gm: torch.fx.GraphModule) -> int:
    n_fused = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_function" or node.target not in (aten.relu.default, aten.gelu.default):
            continue
        src = node.args[0]
        if not (isinstance(src, torch.fx.Node) and src.op == "call_function" and src.target == aten.addmm.default):
            continue
        if len(src.users) != 1 or src.kwargs.get("beta", 1) != 1 or src.kwargs.get("alpha", 1) != 1:
            continue
        val = src.meta.get("val")
        if not isinstance(val, torch.Tensor) or val.device.type != "blackwell" or val.dtype not in (
                torch.bfloat16, torch.float16):
            continue
        if node.target == aten.gelu.default and node.kwargs.get("approximate", "none") != "tanh":
            continue  # the fused epilogue implements the tanh form
        bias = src.args[0]
        bval = bias.meta.get("val") if isinstance(bias, torch.fx.Node) else None
        if not isinstance(bval, torch.Tensor) or bval.dim() != 1:
            continue
        with gm.graph.inserting_before(node):
            new = gm.graph.call_function(aten._addmm_activation.default, (src.args[0], src.args[1], src.args[2]),
                                         {"use_gelu": node.target == aten.gelu.default})
        new.meta = dict(node.meta)
        node.replace_all_uses_with(new)
        gm.graph.erase_node(node)
        gm.graph.erase_node(src)
        n_fused += 1
    if n_fused:
        gm.graph.lint()
        gm.recompile()
    return n_fused


# ----------------------------------------------------------------- pass 2
class _PointwiseSupport(OperatorSupportBase):
    def is_node_supported(self, submodules, node) -> bool:
        return codegen.node_supported(node)


def partition_pointwise(gm: torch.fx.GraphModule, min_ops: int = 2) -> Dict[str, dict]:
    """Replaces fusible groups by ``call_module`` nodes; returns {submodule name: kernel description}."""
    part = CapabilityBasedPartitioner(gm, _PointwiseSupport(), allows_single_node_partition=False)
    partitions = part.propose_partitions()
    keep = []
    for p in partitions:
        nodes = list(p.nodes)
        if len(nodes) < min_ops:
            continue
        node_set = set(nodes)
        outs = [n for n in nodes if any(u not in node_set for u in n.users)]
        shapes = {tuple(n.meta["val"].shape) for n in outs}
        if len(shapes) != 1:
            continue
        shape = next(iter(shapes))
        ok = True
        for n in nodes:
            s = tuple(n.meta["val"].shape)
            if len(s) > len(shape) or any(a != b and a != 1 for a, b in zip(reversed(s), reversed(shape))):
                ok = False
            for a in n.all_input_nodes:
                if a not in node_set:
                    s = tuple(a.meta["val"].shape)
                    if len(s) > len(shape) or any(x != y and x != 1 for x, y in zip(reversed(s), reversed(shape))):
                        ok = False
        n_in = len({a for n in nodes for a in n.all_input_nodes if a not in node_set})
        if not ok or n_in + len(outs) > 12 or n_in == 0:
            continue
        keep.append(p)
    if not keep:
        return {}
    fused = part.fuse_partitions(keep)
    kernels: Dict[str, dict] = {}
    for node in fused.graph.nodes:
        if node.op == "call_module" and node.target.startswith("fused_"):
            sub = getattr(fused, node.target)
            # meta of the sub-graph's placeholders comes from the outer arguments
            phs = [n for n in sub.graph.nodes if n.op == "placeholder"]
            for ph, arg in zip(phs, node.args):
                ph.meta["val"] = arg.meta["val"]
            src, info = codegen.generate(sub, "KERNEL_NAME")
            name = "b200_fused_" + hashlib.sha1(src.encode()).hexdigest()[:16]
            info["source"] = src.replace("KERNEL_NAME", name)
            info["entry"] = name
            kernels[node.target] = info
    if fused is not gm:
        gm.__dict__.update(fused.__dict__)
    return kernels


# ----------------------------------------------------------------- pass 3
_kernel_cache: Dict[str, object] = {}


def get_kernel(info: dict):
    k = _kernel_cache.get(info["entry"])
    if k is None:
        if info.get("cubin") is not None:
            k = _C()._JitKernel.from_cubin(info["cubin"], info["entry"])
        else:
            k = _C()._JitKernel(info["source"], info["entry"])
        _kernel_cache[info["entry"]] = k
    return k


def _normalise(node) -> List[object]:
    """All arguments of an OpOverload call in schema order (defaults filled in)."""
    schema = node.target._schema
    out = []
    for i, arg in enumerate(schema.arguments):
        if i < len(node.args) and not arg.kwarg_only:
            out.append(node.args[i])
        elif arg.name in node.kwargs:
            out.append(node.kwargs[arg.name])
        elif arg.has_default_value():
            out.append(arg.default_value)
        else:
            raise Unsupported(f"{node.format_node()}: no value for argument '{arg.name}'")
    return out


def describe_program(gm: torch.fx.GraphModule, kernels: Dict[str, dict]) -> dict:
    """A picklable description of the program (what ``aot_compile`` stores and ``instantiate`` turns into a runner)."""
    slot: Dict[torch.fx.Node, int] = {}
    nodes = list(gm.graph.nodes)
    last_use: Dict[torch.fx.Node, int] = {}
    for idx, n in enumerate(nodes):
        for a in n.all_input_nodes:
            last_use[a] = idx
    instrs = []
    inputs: List[int] = []
    outputs: List[Optional[int]] = []
    next_slot = 0
    for idx, n in enumerate(nodes):
        dead = lambda: [slot[a] for a in set(n.all_input_nodes) if last_use[a] == idx and a in slot]  # noqa: E731
        if n.op == "placeholder":
            if n.users:
                slot[n] = next_slot
                inputs.append(next_slot)
                next_slot += 1
            else:
                inputs.append(-1)
            continue
        if n.op == "output":
            vals = n.args[0]
            vals = list(vals) if isinstance(vals, (tuple, list)) else [vals]
            for v in vals:
                if v is None:
                    outputs.append(None)
                elif isinstance(v, torch.fx.Node):
                    outputs.append(slot[v])
                else:
                    raise Unsupported("constant graph outputs")
            continue
        if n.op == "get_attr":
            raise Unsupported("graph constants (get_attr)")
        if n in slot:
            continue  # element of a fused kernel's result tuple: it already has its slot
        my = next_slot
        next_slot += 1
        slot[n] = my
        if n.op == "call_module":
            info = kernels.get(n.target)
            if info is None:
                raise Unsupported(f"call_module {n.target}")
            ins = [slot[a] for a in n.args]
            n_out = len(info["out_dtypes"])
            if n_out == 1:
                out_slots = [my]
                instrs.append({"kind": "fused", "kernel": n.target, "in": ins, "out": out_slots, "free": dead(),
                               "label": n.name})
            else:
                # users index the result tuple; give each element a slot of its own
                out_slots = list(range(next_slot, next_slot + n_out))
                next_slot += n_out
                instrs.append({"kind": "fused", "kernel": n.target, "in": ins, "out": out_slots, "free": dead(),
                               "label": n.name})
                for u in list(n.users):
                    if u.op == "call_function" and u.target is operator.getitem:
                        slot[u] = out_slots[u.args[1]]
                    else:
                        raise Unsupported("fused tuple used whole")
            continue
        if n.op != "call_function":
            raise Unsupported(n.format_node())
        if n.target is operator.getitem:
            src = n.args[0]
            if not isinstance(src, torch.fx.Node) or not isinstance(n.args[1], int):
                raise Unsupported("getitem with a computed index")
            instrs.append({"kind": "getitem", "src": slot[src], "index": n.args[1], "out": my, "free": dead()})
            continue
        if not isinstance(n.target, torch._ops.OpOverload):
            raise Unsupported(f"call of {n.target}")
        args = []
        for a in _normalise(n):
            if isinstance(a, torch.fx.Node):
                args.append(("slot", slot[a]))
            elif isinstance(a, (list, tuple)) and any(isinstance(x, torch.fx.Node) for x in a):
                if not all(x is None or isinstance(x, torch.fx.Node) for x in a):
                    raise Unsupported("list argument mixing tensors and constants")
                args.append(("slots", [None if x is None else slot[x] for x in a]))
            else:
                if isinstance(a, (torch.SymInt, torch.SymFloat, torch.SymBool)):
                    raise Unsupported("symbolic shapes")
                args.append(("const", list(a) if isinstance(a, tuple) else a))
        schema = n.target._schema
        ns, opname = schema.name.split("::")
        instrs.append({"kind": "op", "op": schema.name, "overload": schema.overload_name, "args": args, "out": my,
                       "free": dead() + ([my] if not n.users else []), "label": n.name})
    return {"n_slots": next_slot, "inputs": inputs, "outputs": [-1 if o is None else o for o in outputs],
            "instrs": instrs,
            "kernels": {k: {kk: vv for kk, vv in v.items()} for k, v in kernels.items()}}


def instantiate(desc: dict):
    """Builds the C++ runner of a program description (compiling or loading its fused kernels)."""
    r = _C()._GraphRunner()
    r.n_slots = desc["n_slots"]
    r.input_slots = desc["inputs"]
    r.output_slots = desc["outputs"]
    for ins in desc["instrs"]:
        if ins["kind"] == "op":
            r.add_op(ins["op"], ins["overload"], list(ins["args"]), ins["out"], ins["free"], ins.get("label", ""))
        elif ins["kind"] == "getitem":
            r.add_getitem(ins["src"], ins["index"], ins["out"], ins["free"])
        else:
            info = desc["kernels"][ins["kernel"]]
            r.add_fused(get_kernel(info), ins["in"], list(info["shape"]), list(info["out_dtypes"]), ins["out"],
                        info["vec"], ins["free"], ins.get("label", ""))
    return r


def lower(gm: torch.fx.GraphModule, fuse: bool = True):
    """Runs the passes on ``gm`` (in place) and returns ``(runner, description)``."""
    kernels: Dict[str, dict] = {}
    if fuse:
        fuse_addmm_activation(gm)
        kernels = partition_pointwise(gm)
    desc = describe_program(gm, kernels)
    return instantiate(desc), desc
