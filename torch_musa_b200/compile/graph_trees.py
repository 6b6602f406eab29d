"""Graph trees: CUDA-graph capture and replay for compiled functions that run in sequence.

A training step runs several compiled graphs one after another (forward pieces, then backward
pieces), the later ones reading what the earlier ones produced.  Each distinct sequence is a path in
a tree: a node is one captured graph, its parent is the graph that ran before it while that graph's
outputs were still alive.  All nodes of a tree allocate from one private memory pool, so temporaries
are shared across graphs, while every node's outputs stay allocated for as long as the node exists;
a child is therefore captured with its ancestors' outputs in place and can read them by address.

Inputs whose address is fixed (parameters, buffers, outputs of an ancestor node) are read in place;
their addresses are part of the node's key, so a new address records a new node.  Every other input
is copied into a buffer owned by the node before the replay.

Parity: reference torch_musa/_inductor/musagraph_trees.py:202-2815 (tree of recorded graphs per
device, warm-up / record / replay states, one pool per tree, liveness-driven paths).
"""
from __future__ import annotations

import itertools
import threading
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

_fn_ids = itertools.count()
_DEBUG = bool(__import__("os").environ.get("B200_COMPILE_DEBUG"))


def _bw():
    import torch_musa_b200 as bw

    return bw


class GraphNode:
    def __init__(self, parent: Optional["GraphNode"], key):
        self.parent = parent
        self.key = key
        self.children: Dict[tuple, "GraphNode"] = {}
        self.graph = None
        self.copy_inputs: List[Tuple[int, torch.Tensor]] = []   # (argument index, node-owned buffer)
        self.outputs: List[object] = []                          # node-owned tensors (or None / numbers)
        self.base_use: List[int] = []                            # storage reference counts with no alias handed out
        self.aliased = False                                     # the last run handed out aliases (not clones)
        self.replays = 0

    @staticmethod
    def _use_counts(outputs) -> List[int]:
        count = _bw()._C._storage_use_count
        return [count(t) if isinstance(t, torch.Tensor) else 0 for t in outputs]

    def path_outputs_alive(self) -> bool:
        """Does anything outside the tree still reference memory that this path handed out?  (Reference counts of the
        storages: Python wrappers come and go while autograd keeps the tensors, so weak references would not tell.)"""
        n = self
        while n is not None:
            if n.aliased and any(c > b for c, b in zip(self._use_counts(n.outputs), n.base_use)):
                return True
            n = n.parent
        return False

    def owns(self, ptr: int) -> bool:
        n = self
        while n is not None:
            for t in n.outputs:
                if isinstance(t, torch.Tensor) and t.numel() and t.untyped_storage().data_ptr() <= ptr < (
                        t.untyped_storage().data_ptr() + t.untyped_storage().nbytes()):
                    return True
            n = n.parent
        return False


class GraphTreeManager:
    """One per device.  ``run(fn_id, fn, args, clone_outputs)`` is the only entry point; calls are serialised."""

    def __init__(self, device_index: int, warmup: int = 1, max_recordings: int = 16):
        self.device_index = device_index
        self.pool = _bw().graph_pool_handle()
        self.roots: Dict[tuple, GraphNode] = {}
        self.current: Optional[GraphNode] = None
        self.warmup = warmup
        self.max_recordings = max_recordings
        self.seen: Dict[tuple, int] = {}
        self.recordings: Dict[int, int] = {}
        self.stats = {"warmup_runs": 0, "recorded": 0, "replayed": 0, "eager_runs": 0}
        self._lock = threading.RLock()

    # ------------------------------------------------------------- keys
    @staticmethod
    def _is_fixed(t: torch.Tensor, node: Optional[GraphNode]) -> bool:
        if isinstance(t, torch.nn.Parameter) or getattr(t, "_b200_static", False):
            return True
        return node is not None and t.numel() > 0 and node.owns(t.data_ptr())

    def _key(self, fn_id: int, args: Sequence[object], parent: Optional[GraphNode]):
        parts = [fn_id]
        fixed = []
        for a in args:
            if isinstance(a, torch.Tensor):
                fx = self._is_fixed(a, parent)
                fixed.append(fx)
                parts.append((tuple(a.shape), tuple(a.stride()), a.dtype, a.data_ptr() if fx else None))
            else:
                fixed.append(True)
                parts.append(a)
        return tuple(parts), fixed

    # -------------------------------------------------------------- run
    def run(self, fn_id: int, fn: Callable[[List[object]], List[object]], args: List[object],
            clone_outputs: bool = False) -> List[object]:
        with self._lock:
            return self._run(fn_id, fn, args, clone_outputs)

    def _run(self, fn_id, fn, args, clone_outputs):
        bw = _bw()
        if bw.is_current_stream_capturing() or not any(
                isinstance(a, torch.Tensor) and a.device.type == "blackwell" for a in args):
            self.stats["eager_runs"] += 1
            return fn(list(args))
        # where are we in the tree?  Stay on the current path while something it produced is still in use.
        parent = self.current if (self.current is not None and self.current.path_outputs_alive()) else None
        key, fixed = self._key(fn_id, args, parent)
        table = parent.children if parent is not None else self.roots
        node = table.get(key)
        if node is None and parent is not None:
            # not a continuation of this path: maybe the start of a known one
            rkey, rfixed = self._key(fn_id, args, None)
            if rkey in self.roots:
                parent, key, fixed, table, node = None, rkey, rfixed, self.roots, self.roots[rkey]
        if _DEBUG:
            print(f"[graph trees] fn {fn_id}: parent={'none' if parent is None else id(parent) % 10000} "
                  f"hit={node is not None} seen={self.seen.get(key, 0)} fixed={sum(fixed)}/{len(fixed)}")
        if node is not None:
            return self._replay(node, args, clone_outputs)
        count = self.seen.get(key, 0)
        self.seen[key] = count + 1
        if count < self.warmup or self.recordings.get(fn_id, 0) >= self.max_recordings:
            self.stats["warmup_runs" if count < self.warmup else "eager_runs"] += 1
            self.current = None if parent is None else self.current
            return fn(list(args))
        node = self._record(fn_id, fn, args, fixed, parent, key)
        table[key] = node
        return self._hand_out(node, clone_outputs)

    def _record(self, fn_id, fn, args, fixed, parent, key) -> GraphNode:
        bw = _bw()
        node = GraphNode(parent, key)
        static_args = list(args)
        side = bw.Stream()
        side.wait_stream(bw.current_stream())
        with bw.stream(side):
            for i, (a, fx) in enumerate(zip(args, fixed)):
                if isinstance(a, torch.Tensor) and not fx:
                    buf = torch.empty_strided(a.shape, a.stride(), dtype=a.dtype, device=a.device)
                    buf.copy_(a)
                    node.copy_inputs.append((i, buf))
                    static_args[i] = buf
        bw.current_stream().wait_stream(side)
        g = bw.BlackwellGraph()
        with bw.graph(g, pool=self.pool):
            outs = fn(list(static_args))
        node.graph = g
        node.outputs = list(outs)
        del outs
        node.base_use = GraphNode._use_counts(node.outputs)
        g.replay()
        self.recordings[fn_id] = self.recordings.get(fn_id, 0) + 1
        self.stats["recorded"] += 1
        self.current = node
        return node

    def _replay(self, node: GraphNode, args, clone_outputs) -> List[object]:
        for i, buf in node.copy_inputs:
            a = args[i]
            if a.data_ptr() != buf.data_ptr():
                buf.copy_(a)
        node.graph.replay()
        node.replays += 1
        self.stats["replayed"] += 1
        self.current = node
        return self._hand_out(node, clone_outputs)

    def _hand_out(self, node: GraphNode, clone_outputs: bool) -> List[object]:
        res = []
        for t in node.outputs:
            if isinstance(t, torch.Tensor):
                # a clone leaves the caller free to keep or accumulate into the result across replays (gradients);
                # an alias costs nothing and is overwritten by the node's next replay (activations)
                res.append(t.clone() if clone_outputs else t.detach())
            else:
                res.append(t)
        node.aliased = not clone_outputs
        return res

    def node_count(self) -> int:
        def count(n):
            return 1 + sum(count(c) for c in n.children.values())
        return sum(count(r) for r in self.roots.values())


# One manager per device for the whole process: the backward of a compiled function runs on the autograd
# engine's device thread, and it has to find the tree its forward recorded from the caller's thread.
_managers: Dict[int, GraphTreeManager] = {}
_managers_lock = threading.Lock()


def get_manager(device_index: int) -> GraphTreeManager:
    with _managers_lock:
        m = _managers.get(device_index)
        if m is None:
            m = _managers[device_index] = GraphTreeManager(device_index)
        return m


def reset() -> None:
    """Forget every recorded graph (their pool memory returns to the allocator)."""
    with _managers_lock:
        _managers.clear()


def new_function_id() -> int:
    return next(_fn_ids)


def mark_static(t: torch.Tensor) -> torch.Tensor:
    """Declare that ``t`` keeps its address across calls, so compiled graphs read it in place."""
    t._b200_static = True
    return t
