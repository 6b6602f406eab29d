"""RNG state API of ``torch.blackwell`` (per-device Philox generators).
Parity: reference torch_musa/core/random.py:28-186."""
from __future__ import annotations

from typing import Any, Iterable, List, Union

import torch

from ._lazy_init import _lazy_init, _lazy_call, _C
from .device import _get_device_index, device_count, current_device


class _DefaultGenerators:
    def __getitem__(self, idx: int) -> torch.Generator:
        _lazy_init()
        return _C()._default_generator(int(idx))

    def __len__(self):
        return device_count()

    def __iter__(self):
        return (self[i] for i in range(len(self)))


default_generators = _DefaultGenerators()


def get_rng_state(device: Any = "blackwell") -> torch.Tensor:
    _lazy_init()
    return default_generators[_get_device_index(device, optional=True)].get_state()


def get_rng_state_all() -> List[torch.Tensor]:
    return [get_rng_state(i) for i in range(device_count())]


def set_rng_state(new_state: torch.Tensor, device: Any = "blackwell") -> None:
    state = new_state.clone(memory_format=torch.contiguous_format)
    idx = _get_device_index(device, optional=True) if not isinstance(device, str) or ":" in device else None

    def cb():
        i = current_device() if idx is None else idx
        default_generators[i].set_state(state)

    _lazy_call(cb)


def set_rng_state_all(new_states: Iterable[torch.Tensor]) -> None:
    for i, s in enumerate(new_states):
        set_rng_state(s, i)


def manual_seed(seed: int) -> None:
    """Seed the current device's generator (and the twin generator that serves long-tail random ops)."""
    seed = int(seed)

    def cb():
        i = current_device()
        default_generators[i].manual_seed(seed)
        _C()._seed_cuda_twin(i, seed)

    _lazy_call(cb)


def manual_seed_all(seed: int) -> None:
    seed = int(seed)

    def cb():
        for i in range(device_count()):
            default_generators[i].manual_seed(seed)
            _C()._seed_cuda_twin(i, seed)

    _lazy_call(cb)


def seed() -> None:
    def cb():
        default_generators[current_device()].seed()

    _lazy_call(cb)


def seed_all() -> None:
    def cb():
        s = 0
        for i in range(device_count()):
            g = default_generators[i]
            if i == 0:
                s = g.seed()
            else:
                g.manual_seed(s)

    _lazy_call(cb)


def initial_seed() -> int:
    _lazy_init()
    return default_generators[current_device()].initial_seed()
