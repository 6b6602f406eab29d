"""apex-style ``multi_tensor_applier(op, noop_flag, tensor_lists, *args)``.
Parity: reference torch_musa/multi_tensor_apply/multi_tensor_apply.py:13-37."""
from __future__ import annotations

import torch


class MultiTensorApply:
    available = True

    def __init__(self, chunk_size: int = 65536):
        self.chunk_size = chunk_size

    def __call__(self, op, noop_flag_buffer, tensor_lists, *args):
        return op(self.chunk_size, noop_flag_buffer, tensor_lists, *args)


multi_tensor_applier = MultiTensorApply(65536)


def multi_tensor_l2norm(chunk_size, noop_flag, tensor_lists, per_tensor=False):
    total, per = torch.ops.blackwell.multi_tensor_l2norm(list(tensor_lists[0]), bool(per_tensor))
    return total, per


def multi_tensor_scale(chunk_size, noop_flag, tensor_lists, scale):
    src, dst = tensor_lists
    torch.ops.blackwell.multi_tensor_axpby_(list(dst), list(src), [], float(scale), 0.0)
    return None


def multi_tensor_axpby(chunk_size, noop_flag, tensor_lists, a, b, arg_to_check=-1):
    x, y, out = tensor_lists
    torch.ops.blackwell.multi_tensor_axpby_(list(out), list(x), list(y), float(a), float(b))
    return None
