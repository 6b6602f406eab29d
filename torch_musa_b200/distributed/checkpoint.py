"""Distributed checkpointing (``torch.distributed.checkpoint``) for models sharded on the blackwell device.

``save`` / ``load`` write and read the standard DCP directory format, so a checkpoint taken here loads into a CUDA
run of the same model and the other way round (the device type is not part of the format: tensors are staged through
host memory).  Two things are specific to this backend:

* planning collectives run as ``all_gather_object`` followed by a local reduction on every rank.  DCP's planner
  otherwise gathers the local plans on the coordinator and scatters the global plan back, two object collectives
  that a device backend has to serve with pickled bytes in device tensors and point-to-point sends; one all-gather
  is cheaper and needs no scatter support.  ``use_allgather_planning()`` installs that (idempotent).
* ``sharded_state`` collects a model's and an optimizer's sharded state in the key layout
  ``torch.distributed.checkpoint.state_dict`` uses, including the optimizer facade of the fused FSDP engine.

Parity: reference torch_musa/distributed/dist_wrapper_patch.py:13-62 (the same planning change, as a patch of
``_DistWrapper.reduce_scatter``) and its FSDP2 DCP test (tests/unittest/distributed/fsdp/fsdp_v2/test_fully_shard_dcp.py).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch
import torch.distributed as dist

_installed = False


def use_allgather_planning() -> None:
    """Makes DCP's ``reduce_scatter`` planning step one ``all_gather_object`` plus a local reduction."""
    global _installed
    if _installed:
        return
    from torch.distributed.checkpoint.api import CheckpointException, _wrap_exception
    from torch.distributed.checkpoint.utils import _DistWrapper, _get_failure_dict

    def reduce_scatter(self, step: str, map_fun: Callable[[], Any], reduce_fun: Callable[[List[Any]], List[Any]]):
        try:
            mine = map_fun()
        except BaseException as exc:  # noqa: BLE001  (DCP reports any failure of any rank on all ranks)
            mine = _wrap_exception(exc)
        everyone = self.all_gather_object(mine)
        failures = _get_failure_dict(everyone)
        result = None
        if not failures:
            try:
                # every rank holds every local plan: the (deterministic) reduction runs everywhere, no scatter
                result = reduce_fun(everyone)[self.rank]
            except BaseException as exc:  # noqa: BLE001
                failures[self.rank] = _wrap_exception(exc)
            # a reduction that failed on one rank only must still fail everywhere
            if self.use_dist:
                flags = self.all_gather_object(self.rank in failures)
                for r, bad in enumerate(flags):
                    if bad and r not in failures:
                        failures[r] = _wrap_exception(RuntimeError(f"plan reduction failed on rank {r}"))
        if failures:
            raise CheckpointException(step, failures)
        return result

    _DistWrapper.reduce_scatter = reduce_scatter
    _installed = True


def sharded_state(model: torch.nn.Module, optimizer=None) -> Dict[str, Any]:
    """``{"model": ..., "optim": ...}`` with sharded (DTensor) values, ready for ``save`` / ``load``."""
    out: Dict[str, Any] = {"model": model.state_dict()}
    if optimizer is not None:
        sd = optimizer.state_dict()
        # flatten to string keys: DCP plans over a flat mapping of tensors and small objects
        flat: Dict[str, Any] = {}
        for idx, st in sd["state"].items():
            for k, v in st.items():
                flat[f"state.{idx}.{k}"] = v
        flat["param_groups"] = sd["param_groups"]
        out["optim"] = flat
    return out


def restore_optimizer(optimizer, flat: Dict[str, Any]) -> None:
    """Inverse of the optimizer part of ``sharded_state`` after ``load`` has filled ``flat`` in place."""
    state: Dict[int, Dict[str, Any]] = {}
    for key, v in flat.items():
        if key.startswith("state."):
            _, idx, name = key.split(".", 2)
            state.setdefault(int(idx), {})[name] = v
    optimizer.load_state_dict({"state": state, "param_groups": flat["param_groups"]})


def save(state: Dict[str, Any], checkpoint_id: str, process_group=None, planning: str = "allgather") -> None:
    import torch.distributed.checkpoint as dcp

    if planning == "allgather":
        use_allgather_planning()
    dcp.save(state, checkpoint_id=checkpoint_id, process_group=process_group)


def load(state: Dict[str, Any], checkpoint_id: str, process_group=None, planning: str = "allgather") -> None:
    """Fills the tensors of ``state`` in place (sharded values receive exactly their shard)."""
    import torch.distributed.checkpoint as dcp

    if planning == "allgather":
        use_allgather_planning()
    dcp.load(state, checkpoint_id=checkpoint_id, process_group=process_group)
