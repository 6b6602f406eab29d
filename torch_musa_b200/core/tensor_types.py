"""Legacy typed tensor classes: ``torch.blackwell.FloatTensor``, ``HalfTensor``, ``BFloat16Tensor``, ...

They behave like ``torch.cuda.FloatTensor``: ``isinstance(t, torch.blackwell.FloatTensor)`` is true for an fp32
tensor on the device, and calling the class builds one (``FloatTensor(2, 3)`` uninitialised, ``FloatTensor([1, 2])``
from data, ``FloatTensor(other_tensor)`` converted).  New code should use ``torch.empty(..., device="blackwell")``.
Parity: reference torch_musa/csrc/core/PythonTensor.cpp:15-410 (the same classes built in C++ against a patched
torch; here a metaclass over the public tensor API is enough).
"""
from __future__ import annotations

import torch

_TYPES = {
    "FloatTensor": torch.float32, "DoubleTensor": torch.float64, "HalfTensor": torch.float16,
    "BFloat16Tensor": torch.bfloat16, "ByteTensor": torch.uint8, "CharTensor": torch.int8,
    "ShortTensor": torch.int16, "IntTensor": torch.int32, "LongTensor": torch.int64, "BoolTensor": torch.bool,
}


class _TypedTensorMeta(type):
    dtype: torch.dtype

    def __instancecheck__(cls, obj) -> bool:
        return isinstance(obj, torch.Tensor) and obj.device.type == "blackwell" and obj.dtype == cls.dtype

    def __call__(cls, *args, device=None):
        from . import device as _dev

        dev = torch.device("blackwell", _dev.current_device() if device is None else torch.device(device).index or 0)
        if len(args) == 0:
            return torch.empty(0, dtype=cls.dtype, device=dev)
        if len(args) == 1 and isinstance(args[0], torch.Tensor):
            return args[0].to(device=dev, dtype=cls.dtype)
        if len(args) == 1 and isinstance(args[0], torch.Size):
            return torch.empty(args[0], dtype=cls.dtype, device=dev)
        if len(args) == 1 and isinstance(args[0], (list, tuple)):
            return torch.tensor(args[0], dtype=cls.dtype).to(dev)
        if all(isinstance(a, int) for a in args):
            return torch.empty(*args, dtype=cls.dtype, device=dev)
        raise TypeError(f"{cls.__name__}(): expected sizes, a sequence or a tensor, got {tuple(type(a).__name__ for a in args)}")

    def __repr__(cls) -> str:
        return f"<class 'torch.blackwell.{cls.__name__}'>"


def make_types() -> dict:
    out = {}
    for name, dt in _TYPES.items():
        out[name] = _TypedTensorMeta(name, (), {"dtype": dt, "is_blackwell": True, "is_sparse": False,
                                                "__module__": "torch.blackwell",
                                                "__doc__": f"{dt} tensors on the blackwell device (legacy typed class)."})
    return out
