"""Graph capture and replay: ``torch.blackwell.BlackwellGraph``, the ``graph`` context
manager, ``graph_pool_handle`` and ``make_graphed_callables``.

A captured graph replays a whole launch-bound region (a decode step, a small
training step) with one driver call.  Memory allocated during capture comes from
a private pool so that addresses baked into the graph stay valid.
Parity: reference torch_musa/musa_graph/graphs.py:12-516.
"""
from __future__ import annotations

import weakref

import gc
from typing import Any, Callable, Optional, Tuple, Union

import torch


def _bw():
    import torch_musa_b200

    return torch_musa_b200


def graph_pool_handle() -> Tuple[int, int]:
    """An opaque token naming a graph memory pool; pass it to several captures to share memory."""
    return tuple(_bw()._C._graph_pool_handle())


class BlackwellGraph:
    """Wrapper around a captured CUDA graph for the blackwell device."""

    _instances = weakref.WeakSet()     # live graphs, for update_graph_with_profile()

    def __init__(self, keep_graph: bool = False):
        self._g = _bw()._C._Graph()
        self._keeps_graph = bool(keep_graph)
        if keep_graph:
            self._g.enable_debug_mode()
        BlackwellGraph._instances.add(self)

    def capture_begin(self, pool: Optional[Tuple[int, int]] = None, capture_error_mode: str = "global") -> None:
        self._g.capture_begin(pool, capture_error_mode)

    def capture_end(self) -> None:
        self._g.capture_end()

    def replay(self) -> None:
        self._g.replay()

    def reset(self) -> None:
        self._g.reset()

    def pool(self) -> Tuple[int, int]:
        return tuple(self._g.pool())

    def enable_debug_mode(self) -> None:
        self._keeps_graph = True
        self._g.enable_debug_mode()

    def debug_dump(self, debug_path: str) -> None:
        self._g.debug_dump(debug_path)

    def reinstantiate_graph(self) -> None:
        self._g.reinstantiate_graph()


class graph:
    """Context manager that captures the work of its body into ``blackwell_graph``.

    Synchronises, collects garbage and empties the allocator cache first (so the capture starts from a
    quiet state), then runs the body on a side stream under capture.
    """

    default_capture_stream = None

    def __init__(self, blackwell_graph: BlackwellGraph, pool: Optional[Tuple[int, int]] = None,
                 stream: Optional[torch.Stream] = None, capture_error_mode: str = "global"):
        bw = _bw()
        if self.__class__.default_capture_stream is None:
            self.__class__.default_capture_stream = bw.Stream()
        self.pool = pool
        self.capture_stream = stream if stream is not None else self.__class__.default_capture_stream
        self.stream_ctx = bw.stream(self.capture_stream)
        self.graph = blackwell_graph
        self.capture_error_mode = capture_error_mode

    def __enter__(self):
        bw = _bw()
        bw.synchronize()
        gc.collect()
        bw.empty_cache()
        self.stream_ctx.__enter__()
        self.graph.capture_begin(self.pool, self.capture_error_mode)

    def __exit__(self, exc_type, exc_value, tb):
        try:
            if exc_type is None:
                self.graph.capture_end()
            else:
                self.graph.reset()
        finally:
            self.stream_ctx.__exit__(exc_type, exc_value, tb)
        return False


def make_graphed_callables(callables, sample_args, num_warmup_iters: int = 3, allow_unused_input: bool = False,
                           pool: Optional[Tuple[int, int]] = None):
    """Graph-captured versions of ``callables`` (functions or ``nn.Module``s) with autograd support.

    Each callable's forward and backward are captured as separate graphs over static input/output
    buffers; the returned callable copies new inputs into the static buffers and replays.
    """
    bw = _bw()
    just_one = False
    if not isinstance(callables, tuple):
        just_one = True
        callables = (callables,)
        sample_args = (sample_args,)

    flat_args = []
    for c, args in zip(callables, sample_args):
        if isinstance(c, torch.nn.Module):
            assert len(c._backward_hooks) == 0 and len(c._forward_hooks) == 0 and len(c._forward_pre_hooks) == 0, (
                "Modules must not have hooks registered at the time they are passed."
            )
            assert all(b.requires_grad is False for b in c.buffers()), "Only parameters may require grad."
        args = tuple(args) if isinstance(args, (tuple, list)) else (args,)
        assert all(isinstance(a, torch.Tensor) for a in args), "sample_args must be tensors"
        flat_args.append(args)

    per_callable_params = [tuple(c.parameters()) if isinstance(c, torch.nn.Module) else () for c in callables]
    per_callable_inputs = [flat_args[i] + per_callable_params[i] for i in range(len(callables))]
    fwd_graphs = [BlackwellGraph() for _ in callables]
    bwd_graphs = [BlackwellGraph() for _ in callables]
    mempool = graph_pool_handle() if pool is None else pool

    # warm-up on a side stream so lazy initialisation does not end up in the capture
    bw.synchronize()
    side = bw.Stream()
    side.wait_stream(bw.current_stream())
    with bw.stream(side):
        for func, args, static_inputs in zip(callables, flat_args, per_callable_inputs):
            for _ in range(num_warmup_iters):
                outs = func(*args)
                outs = (outs,) if isinstance(outs, torch.Tensor) else tuple(outs)
                need = tuple(i for i in static_inputs if i.requires_grad)
                if need:
                    grads = torch.autograd.grad(outputs=tuple(o for o in outs if o.requires_grad), inputs=need,
                                                grad_outputs=tuple(torch.empty_like(o) for o in outs if o.requires_grad),
                                                only_inputs=True, allow_unused=allow_unused_input)
                    del grads
            del outs
    bw.current_stream().wait_stream(side)
    bw.synchronize()

    per_callable_static_outputs, per_callable_output_was_tensor = [], []
    for func, args, g in zip(callables, flat_args, fwd_graphs):
        with graph(g, pool=mempool):
            outs = func(*args)
        per_callable_output_was_tensor.append(isinstance(outs, torch.Tensor))
        per_callable_static_outputs.append((outs,) if isinstance(outs, torch.Tensor) else tuple(outs))

    per_callable_static_grad_outputs, per_callable_static_grad_inputs = [], []
    for static_inputs, static_outputs, g in zip(reversed(per_callable_inputs), reversed(per_callable_static_outputs),
                                                reversed(bwd_graphs)):
        static_grad_outputs = tuple(torch.empty_like(o) if o.requires_grad else None for o in static_outputs)
        need = tuple(i for i in static_inputs if i.requires_grad)
        grad_inputs = ()
        if need:
            with graph(g, pool=mempool):
                grad_inputs = torch.autograd.grad(
                    outputs=tuple(o for o in static_outputs if o.requires_grad), inputs=need,
                    grad_outputs=tuple(o for o in static_grad_outputs if o is not None), only_inputs=True,
                    allow_unused=allow_unused_input)
        static_grad_inputs, k = [], 0
        for a in static_inputs:
            if a.requires_grad:
                static_grad_inputs.append(grad_inputs[k])
                k += 1
            else:
                static_grad_inputs.append(None)
        per_callable_static_grad_outputs.append(static_grad_outputs)
        per_callable_static_grad_inputs.append(tuple(static_grad_inputs))
    per_callable_static_grad_outputs.reverse()
    per_callable_static_grad_inputs.reverse()

    def make_fn(fwd_graph, bwd_graph, n_user_args, static_inputs, static_outputs, static_grad_outputs,
                static_grad_inputs, was_tensor, params):
        class Graphed(torch.autograd.Function):
            @staticmethod
            def forward(ctx, *inputs):
                for i in range(n_user_args):
                    if static_inputs[i].data_ptr() != inputs[i].data_ptr():
                        static_inputs[i].copy_(inputs[i])
                fwd_graph.replay()
                return tuple(o.detach() for o in static_outputs)

            @staticmethod
            @torch.autograd.function.once_differentiable
            def backward(ctx, *grads):
                for g_static, g in zip(static_grad_outputs, grads):
                    if g_static is not None and g is not None and g_static.data_ptr() != g.data_ptr():
                        g_static.copy_(g)
                bwd_graph.replay()
                return tuple(b.detach() if b is not None else b for b in static_grad_inputs)

        def run(*user_args):
            out = Graphed.apply(*(tuple(user_args) + params))
            return out[0] if was_tensor else out

        return run

    ret = []
    for i, func in enumerate(callables):
        graphed = make_fn(fwd_graphs[i], bwd_graphs[i], len(flat_args[i]), per_callable_inputs[i],
                          per_callable_static_outputs[i], per_callable_static_grad_outputs[i],
                          per_callable_static_grad_inputs[i], per_callable_output_was_tensor[i],
                          per_callable_params[i])
        if isinstance(func, torch.nn.Module):
            def wrap(mod, orig_fwd, graphed_fn, training):
                def new_fwd(*a):
                    return graphed_fn(*a) if mod.training == training else orig_fwd(*a)
                return new_fwd
            func.forward = wrap(func, func.forward, graphed, func.training)
            ret.append(func)
        else:
            ret.append(graphed)
    return ret[0] if just_one else tuple(ret)


def update_graph_with_profile() -> int:
    """Re-instantiates the executable of every live graph that kept its captured graph (``keep_graph=True`` or
    ``enable_debug_mode()`` before the capture).  A profiler that attaches after a graph was instantiated does not
    see the kernels inside it; instantiating again under the profiler makes them visible.  Returns the number of
    graphs that were re-instantiated; graphs that did not keep their captured graph are left alone.
    Parity: reference torch_musa/musa_graph/graphs.py:21-28."""
    n = 0
    for g in list(BlackwellGraph._instances):
        if g._keeps_graph:
            try:
                g.reinstantiate_graph()
                n += 1
            except RuntimeError:
                pass        # nothing captured yet
    return n
