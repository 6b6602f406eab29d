"""``torch.compile(backend="blackwell_graphs")``: trace with AOT-autograd, run the traced graphs
on the backend's eager kernels, and replay them as CUDA graphs once shapes are stable.

There is deliberately no kernel code generator: the hot operators already are hand-written
sm_100a kernels and the remaining cost of an eager step is launch latency, which graph replay
removes.  Parity: reference torch_musa/_dynamo/backend/musagraphs.py:171-322 and
_inductor/musagraph_trees.py (capture + replay with a private pool per graph).
"""
from __future__ import annotations

from typing import Callable, List, Sequence

import torch


class _GraphedCallable:
    """Wraps an fx callable: warm up on a side stream, capture once per input-shape set, replay afterwards."""

    def __init__(self, fn: Callable, warmup: int = 2):
        self.fn = fn
        self.warmup = warmup
        self.calls = 0
        self.graph = None
        self.static_inputs: List[torch.Tensor] = []
        self.static_outputs = None
        self.key = None

    def _is_device(self, args) -> bool:
        return any(isinstance(a, torch.Tensor) and a.device.type == "blackwell" for a in args)

    def __call__(self, *args):
        import torch_musa_b200 as bw

        if not self._is_device(args) or any(isinstance(a, torch.Tensor) and a.requires_grad for a in args):
            return self.fn(*args)
        key = tuple((tuple(a.shape), a.dtype, tuple(a.stride())) if isinstance(a, torch.Tensor) else a for a in args)
        if self.graph is not None and key == self.key:
            for s, a in zip(self.static_inputs, args):
                if isinstance(a, torch.Tensor) and s.data_ptr() != a.data_ptr():
                    s.copy_(a)
            self.graph.replay()
            return self.static_outputs
        self.calls += 1
        if self.calls <= self.warmup or bw.is_current_stream_capturing():
            return self.fn(*args)
        # capture
        self.key = key
        self.static_inputs = [a.clone() if isinstance(a, torch.Tensor) else a for a in args]
        side = bw.Stream()
        side.wait_stream(bw.current_stream())
        with bw.stream(side):
            self.fn(*self.static_inputs)
        bw.current_stream().wait_stream(side)
        g = bw.BlackwellGraph()
        with bw.graph(g):
            self.static_outputs = self.fn(*self.static_inputs)
        self.graph = g
        self.graph.replay()
        return self.static_outputs


def blackwell_graphs(gm: torch.fx.GraphModule, example_inputs: Sequence[torch.Tensor]):
    from torch._dynamo.backends.common import aot_autograd
    from functorch.compile import make_boxed_func

    def compiler(fx_gm, inputs):
        graphed = _GraphedCallable(fx_gm.forward)

        def run(args):
            out = graphed(*args)
            return out

        run._boxed_call = True
        return run

    return aot_autograd(fw_compiler=compiler, bw_compiler=compiler)(gm, example_inputs)


def register() -> None:
    try:
        from torch._dynamo import register_backend

        register_backend(name="blackwell_graphs")(blackwell_graphs)
    except Exception:  # pragma: no cover
        pass
