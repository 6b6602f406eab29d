"""Pipeline parallelism over point-to-point send / recv: one model stage per rank, micro-batches flowing through.

    stage = PipelineStage(my_layers, stage_index, n_stages, group=pp_group)
    loss = stage.run(schedule="1f1b", micro_inputs=[...] if stage.is_first else None,
                     micro_targets=[...] if stage.is_last else None, loss_fn=F.cross_entropy)
    optimizer.step()                      # every rank steps its own stage's parameters

Two schedules: ``"gpipe"`` (all forwards, then all backwards; activation memory grows with the number of
micro-batches) and ``"1f1b"`` (a stage runs at most ``n_stages - stage`` forwards ahead of its backwards, then
alternates one forward with one backward).  Activations and their gradients travel between neighbouring stages as
batched send / receive pairs: in the steady state "activation out + gradient in" and "gradient out + activation in"
are each ONE batch, so the two directions progress together and no rank can block the other with a send queued ahead
of its receive.  Shapes and dtypes are announced once, with the first micro-batch, in a small header message, so a
stage needs no knowledge of its neighbours' layers.  On the blackwell device the transfers are the collective
backend's point-to-point operations (NCCL send / recv over NVLink); the schedules are tested on CPU ranks (gloo).

Parity: the reference offers send / recv only (reference torch_musa/csrc/distributed/ProcessGroupMCCL.cpp:4187-4330)
and tests them in tests/unittest/distributed/test_dist.py; the schedules here are what a user builds on top.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.int32, torch.uint8, torch.bool]


class PipelineStage:
    def __init__(self, module: torch.nn.Module, stage: int, n_stages: int, group=None, device=None):
        if not 0 <= stage < n_stages:
            raise ValueError(f"stage {stage} outside [0, {n_stages})")
        self.module, self.stage, self.n_stages, self.group = module, stage, n_stages, group
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(dist.get_world_size()))
        if len(ranks) != n_stages:
            raise ValueError(f"the group has {len(ranks)} ranks, the pipeline {n_stages} stages")
        self._prev = ranks[stage - 1] if stage > 0 else None          # global ranks of the neighbours
        self._next = ranks[stage + 1] if stage + 1 < n_stages else None
        p = next(module.parameters(), None)
        self.device = torch.device(device) if device is not None else (p.device if p is not None else torch.device("cpu"))
        self._in_meta = None      # (shape, dtype) of the activation this stage receives
        self._meta_sent = False

    is_first = property(lambda self: self.stage == 0)
    is_last = property(lambda self: self.stage == self.n_stages - 1)

    # ------------------------------------------------------------------ transfers
    def _p2p(self, send: Optional[torch.Tensor] = None, send_to: Optional[int] = None, recv: Optional[torch.Tensor] = None,
             recv_from: Optional[int] = None) -> Optional[torch.Tensor]:
        """One send and / or one receive issued as ONE batch: both directions of an exchange between neighbours make
        progress together, whatever order the two ranks reached it in (a lone send queued ahead of the matching
        receive on both sides would block a stream-ordered transport)."""
        ops = []
        if send is not None and send_to is not None:
            ops.append(dist.P2POp(dist.isend, send.contiguous(), send_to, self.group))
        if recv is not None and recv_from is not None:
            ops.append(dist.P2POp(dist.irecv, recv, recv_from, self.group))
        if ops:
            for work in dist.batch_isend_irecv(ops):
                work.wait()
        return recv

    def _send_meta(self, t: torch.Tensor) -> None:
        head = torch.full((10,), -1, dtype=torch.int64)
        head[0], head[1] = t.dim(), _DTYPES.index(t.dtype)
        head[2:2 + t.dim()] = torch.tensor(list(t.shape), dtype=torch.int64)
        self._p2p(send=head.to(self.device), send_to=self._next)
        self._meta_sent = True

    def _input_buffer(self) -> Optional[torch.Tensor]:
        """An empty tensor for the next activation from the previous stage (None on the first stage)."""
        if self.is_first:
            return None
        if self._in_meta is None:
            head = torch.empty(10, dtype=torch.int64, device=self.device)
            self._p2p(recv=head, recv_from=self._prev)
            head = head.cpu().tolist()
            self._in_meta = (tuple(head[2:2 + head[0]]), _DTYPES[head[1]])
        shape, dtype = self._in_meta
        return torch.empty(shape, dtype=dtype, device=self.device)

    def _recv_forward(self) -> Optional[torch.Tensor]:
        return self._p2p(recv=self._input_buffer(), recv_from=self._prev)

    def _send_forward(self, y: Optional[torch.Tensor]) -> None:
        if not self.is_last:
            if not self._meta_sent:
                self._send_meta(y)
            self._p2p(send=y.detach(), send_to=self._next)

    # ------------------------------------------------------------------ one micro-batch
    def _forward(self, i: int, x, micro_inputs, micro_targets, loss_fn, n_micro: int, saved: dict, losses: list):
        """Runs the stage on micro-batch i; returns what goes to the next stage (None on the last stage)."""
        if self.is_first:
            x = micro_inputs[i]
        elif x.dtype.is_floating_point:
            x.requires_grad_()
        y = self.module(x)
        if self.is_last:
            loss = loss_fn(y, micro_targets[i]) / n_micro
            losses.append(loss.detach())
            saved[i] = (x, loss)
            return None
        saved[i] = (x, y)
        return y

    def _backward(self, i: int, g: Optional[torch.Tensor], saved: dict) -> Optional[torch.Tensor]:
        """Backward of micro-batch i given the gradient of its output; returns the gradient for the previous stage."""
        x, out = saved.pop(i)
        if self.is_last:
            out.backward()
        else:
            out.backward(g)
        return None if self.is_first else x.grad

    # ------------------------------------------------------------------ schedules
    def run(self, schedule: str = "1f1b", micro_inputs: Optional[Sequence[torch.Tensor]] = None,
            micro_targets: Optional[Sequence[torch.Tensor]] = None, loss_fn: Optional[Callable] = None,
            n_micro: Optional[int] = None) -> Optional[torch.Tensor]:
        """Forward and backward of ``n_micro`` micro-batches; parameter gradients accumulate in ``.grad`` (the loss of a
        micro-batch is divided by ``n_micro``).  The first stage passes ``micro_inputs``, the last ``micro_targets`` and
        ``loss_fn``; stages in between pass ``n_micro``.  Returns the mean loss on the last stage, None elsewhere."""
        if self.is_first:
            n_micro = len(micro_inputs)
        elif self.is_last:
            n_micro = len(micro_targets)
        if not n_micro:
            raise ValueError("the number of micro-batches is unknown: pass n_micro on a middle stage")
        if self.is_last and loss_fn is None:
            raise ValueError("the last stage needs loss_fn")
        saved, losses = {}, []
        fwd = lambda i, x: self._forward(i, x, micro_inputs, micro_targets, loss_fn, n_micro, saved, losses)  # noqa: E731
        grad_like = lambda i: None if self.is_last else torch.empty_like(saved[i][1])                          # noqa: E731
        if schedule == "gpipe":
            for i in range(n_micro):
                self._send_forward(fwd(i, self._recv_forward()))
            for i in range(n_micro):
                g = self._p2p(recv=grad_like(i), recv_from=self._next)
                self._p2p(send=self._backward(i, g, saved), send_to=self._prev)
        elif schedule == "1f1b":
            warm = min(self.n_stages - self.stage - 1, n_micro)
            steady = n_micro - warm
            for i in range(warm):
                self._send_forward(fwd(i, self._recv_forward()))
            x = self._recv_forward() if steady > 0 else None
            for i in range(steady):
                y = fwd(warm + i, x)
                if y is not None and not self._meta_sent:
                    self._send_meta(y)
                # forward activation out, gradient of the oldest micro-batch in flight in: one exchange with the next stage
                g = self._p2p(send=None if y is None else y.detach(), send_to=self._next, recv=grad_like(i), recv_from=self._next)
                dx = self._backward(i, g, saved)
                if i + 1 < steady:   # gradient out, next activation in: one exchange with the previous stage
                    x = self._p2p(send=dx, send_to=self._prev, recv=self._input_buffer(), recv_from=self._prev)
                else:
                    self._p2p(send=dx, send_to=self._prev)
            for i in range(steady, n_micro):
                g = self._p2p(recv=grad_like(i), recv_from=self._next)
                self._p2p(send=self._backward(i, g, saved), send_to=self._prev)
        else:
            raise ValueError(f"unknown schedule {schedule!r}: 'gpipe' or '1f1b'")
        return torch.stack(losses).sum() if self.is_last else None


def split_into_stages(layers: Sequence[torch.nn.Module], n_stages: int) -> List[torch.nn.Sequential]:
    """Contiguous, near-equal groups of ``layers``, one ``nn.Sequential`` per stage (earlier stages take the extras)."""
    if n_stages < 1 or n_stages > len(layers):
        raise ValueError(f"cannot split {len(layers)} layers into {n_stages} stages")
    base, extra = divmod(len(layers), n_stages)
    out, i = [], 0
    for s in range(n_stages):
        n = base + (1 if s < extra else 0)
        out.append(torch.nn.Sequential(*layers[i:i + n]))
        i += n
    return out
