"""Helpers shared by the peer-memory ("symmetric memory") users in this package.

A symmetric arena is set up through a key-value store: every member publishes its CUDA IPC record under
``<key>/<group rank>``.  The key must therefore be the same on every member and different for every arena.
A process-local counter does not guarantee that (ranks that belong to different sets of groups count differently),
so the key is counted *per group*, and the store is the group's own prefixed store: two disjoint groups can never
see each other's records.
Parity: the reference exchanges its communicator ids through the group's store in the same way
(reference torch_musa/csrc/distributed/ProcessGroupMCCL.cpp:1950-2010).
"""
from __future__ import annotations

from collections import defaultdict
from typing import Tuple

import torch.distributed as dist

_counters = defaultdict(int)


def group_info(group=None) -> Tuple[int, int]:
    """(rank, world) of ``group``; (0, 1) without an initialised process group."""
    if not (dist.is_available() and dist.is_initialized()):
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def group_store_and_key(group, kind: str):
    """Returns ``(store, key)`` for a new arena of ``kind`` in ``group`` (None: the default group).

    Every member of the group must call this the same number of times per kind, in the same order."""
    if not (dist.is_available() and dist.is_initialized()):
        return dist.HashStore(), f"{kind}/0"
    pg = group if group is not None else dist.group.WORLD
    store = dist.distributed_c10d._world.pg_map[pg][1]
    name = dist.distributed_c10d._world.pg_names.get(pg, "default")
    n = _counters[(name, kind)]
    _counters[(name, kind)] = n + 1
    return store, f"{kind}/{n}"
