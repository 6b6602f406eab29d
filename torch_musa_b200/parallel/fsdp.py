"""FSDP2 (``fully_shard``) on the backend's own sharded-parameter kernels.

``install_fused_collectives(model)`` replaces, for every FSDP2 parameter group under ``model``, the five passes
of the library path (cast, copy-in, all-gather, copy-out; copy-in, reduce-scatter) by three kernels over
peer-mapped memory (``csrc/kernels/fsdp_comm.cu``):

* every rank keeps the low-precision copy of its parameter shards (the *shadow*) resident in a symmetric arena; it
  is refreshed by one multi-tensor cast kernel when the master shards changed (``pack``), or by the optimizer
  epilogue of the reduce kernel;
* ``unshard`` launches one ``gather`` kernel that pulls the peers' shadows straight into the final layout of every
  unsharded parameter: no flat all-gather buffer, no ``split_with_sizes_copy``;
* the post-backward hook launches one ``reduce`` kernel that pushes the gradient slices to their owners in the
  gradient dtype (bf16 on the wire, fp32 accumulation: the same sum an fp32 reduce-scatter produces, at half the
  NVLink bytes), and either writes the fp32 gradient shard or -- with ``fused_adamw=...`` -- applies AdamW to the
  fp32 master shard, both moments and the shadow in the same pass, so the reduced gradient never exists in memory
  and the optimizer step of a layer overlaps the backward of the layers before it.

With one rank everything degenerates to local work: the unsharded parameters alias the shadow (no kernel at all
in forward/backward) and the reduce kernel is the optimizer.

Groups the kernels do not cover (more than 40 tensors, sharding on another dimension, CPU offload, HSDP, DTensor
parameters) keep the stock path.  ``FusedFSDP.calls`` counts the kernel launches per kind.

Parity: the reference monkey-patches FSDP2's ``foreach_all_gather`` / ``foreach_reduce`` to call its library
collectives with custom copy kernels and staged overlap levels (reference
torch_musa/distributed/_composable/fsdp/patch.py:60-246, custom_overlap_patch.py:177-305).
"""
from __future__ import annotations

import os
import weakref
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ._symm import group_store_and_key

_MAX_GROUPS = 256
_RING = 2
_patched = False
_engines: "weakref.WeakSet[FusedFSDP]" = weakref.WeakSet()


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


# --------------------------------------------------------------------------------------------- kernel back ends
class _DeviceKernels:
    """The sm_100a kernels over a peer-mapped arena."""

    def __init__(self, group, rank: int, world: int, device: torch.device, arena_bytes: int):
        import torch_musa_b200 as bw

        self.rank, self.world = rank, world
        store, key = group_store_and_key(group, "fsdp_arena")
        self.sm = bw._C._create_symmetric_memory(store, key, rank, world, device.index or 0, arena_bytes)
        if not self.sm.ok:
            raise RuntimeError(f"FSDP arena unavailable: {self.sm.why_not}")
        self._C = bw._C
        w0 = bw._C._comm_user_word0()
        self.flag_word0 = w0                                   # [group][16]
        self.ready_word0 = w0 + _MAX_GROUPS * 16               # [ring][16]
        self.ack_word = self.ready_word0 + 4 * 16              # [16]
        self.counter_word0 = self.ack_word + 16                # [group][4]: pack, reduce (2 words), spare
        assert self.counter_word0 + _MAX_GROUPS * 4 <= bw._C._comm_pad_words()

    def make_layout(self, shard_numel, shard_off, full_numel, total):
        return self._C._FsdpLayout(shard_numel, shard_off, full_numel, total)

    def view(self, byte_off: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        return self.sm.local_tensor(byte_off, [numel], dtype)

    def pack(self, g: "_Group", srcs, n_ctas: int):
        self.sm.fsdp_pack(g.layout, srcs, g.shadow_off, g.shadow_dtype, self.flag_word0 + g.gid * 16, g.version,
                          self.counter_word0 + g.gid * 4, n_ctas)

    def gather(self, g: "_Group", outs, n_ctas: int):
        self.sm.fsdp_gather(g.layout, outs, g.shadow_off, self.flag_word0 + g.gid * 16, g.version, n_ctas)

    def reduce(self, g: "_Group", grads, stage_off: int, scale: float, out32, adam, seq: int, ack_need: int,
               n_ctas: int):
        ring_slot = seq % _RING
        if adam is None:
            p32, m1, m2, hyper, sh_off, sh_ver = [], [], [], [], -1, 0
        else:
            p32, m1, m2, hyper, sh_off, sh_ver = adam
        self.sm.fsdp_reduce(g.layout, grads, stage_off, scale, out32, p32, m1, m2, hyper, sh_off, g.shadow_dtype,
                            self.flag_word0 + g.gid * 16, sh_ver, self.ready_word0 + ring_slot * 16, self.ack_word,
                            seq, ack_need, self.counter_word0 + g.gid * 4 + 1, n_ctas)

    def status(self) -> int:
        return self.sm.take_status()


class _EmulatedKernels:
    """The same data movement with plain tensor operations and the process group's collectives.  Used where the
    device kernels cannot run (CPU ranks over gloo in the unit tests): it exercises the layouts, the hooks and the
    optimizer epilogue, not the transport."""

    def __init__(self, group, rank: int, world: int, device: torch.device, arena_bytes: int):
        self.rank, self.world, self.group, self.device = rank, world, group, device
        self.arena = torch.zeros(arena_bytes, dtype=torch.uint8, device=device)

    def make_layout(self, shard_numel, shard_off, full_numel, total):
        return {"numel": list(shard_numel), "off": list(shard_off), "full": list(full_numel), "total": total}

    def view(self, byte_off: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        # a tensor whose storage STARTS at the given byte (FSDP re-strides unsharded parameters from storage
        # offset 0), over memory owned by the arena
        import ctypes

        nbytes = numel * _itemsize(dtype)
        if nbytes == 0:
            return torch.empty(0, dtype=dtype, device=self.device)
        buf = (ctypes.c_char * nbytes).from_address(self.arena.data_ptr() + byte_off)
        return torch.frombuffer(buf, dtype=dtype, count=numel)

    def pack(self, g: "_Group", srcs, n_ctas: int):
        L = g.layout
        # every view of the arena shares one version counter; the device kernels write memory without touching it
        with torch.autograd._unsafe_preserve_version_counter(g.shadow):
            for src, n, off in zip(srcs, L["numel"], L["off"]):
                g.shadow[off:off + n].copy_(src[:n])

    def gather(self, g: "_Group", outs, n_ctas: int):
        L = g.layout
        if self.world == 1:
            flats = [g.shadow]
        else:
            flats = [torch.empty_like(g.shadow) for _ in range(self.world)]
            dist.all_gather(flats, g.shadow, group=self.group)
        for out, n, off in zip(outs, L["numel"], L["off"]):
            for p in range(self.world):
                out[p * n:(p + 1) * n].copy_(flats[p][off:off + n])

    def reduce(self, g: "_Group", grads, stage_off: int, scale: float, out32, adam, seq: int, ack_need: int,
               n_ctas: int):
        L = g.layout
        W, total = self.world, L["total"]
        flat = torch.zeros(W, total, dtype=torch.float32, device=self.device)
        for grad, n, off, full in zip(grads, L["numel"], L["off"], L["full"]):
            padded = torch.zeros(W * n, dtype=torch.float32, device=self.device)
            padded[:full].copy_(grad.reshape(-1))
            flat[:, off:off + n] = padded.view(W, n)
        if W > 1:
            mine = torch.empty(total, dtype=torch.float32, device=self.device)
            dist.reduce_scatter_tensor(mine, flat.view(-1), group=self.group)
        else:
            mine = flat[0]
        mine = mine * scale
        if adam is None:
            out32[:total].copy_(mine)
            return
        p32, m1, m2, (lr, b1, b2, eps, wd, step), sh_off, _ = adam
        for p, m, v, n, off in zip(p32, m1, m2, L["numel"], L["off"]):
            gr = mine[off:off + n]
            p[:n].mul_(1 - lr * wd)
            m[:n].mul_(b1).add_(gr, alpha=1 - b1)
            v[:n].mul_(b2).addcmul_(gr, gr, value=1 - b2)
            denom = (v[:n].sqrt() / (1 - b2 ** step) ** 0.5).add_(eps)
            p[:n].addcdiv_(m[:n], denom, value=-lr / (1 - b1 ** step))
            if sh_off >= 0:
                with torch.autograd._unsafe_preserve_version_counter(g.shadow):
                    g.shadow[off:off + n].copy_(p[:n])

    def status(self) -> int:
        return 0


# --------------------------------------------------------------------------------------------- per-group state
class _Group:
    """One FSDP2 parameter group on the fused path."""

    def __init__(self, engine: "FusedFSDP", pg, gid: int):
        self.engine, self.pg, self.gid = engine, pg, gid
        self.params = list(pg.fsdp_params)
        W = engine.world
        self.shard_numel = [p.padded_sharded_param_size.numel() for p in self.params]
        self.full_numel = [p._orig_size.numel() for p in self.params]
        offs, off = [], 0
        for n in self.shard_numel:
            offs.append(off)
            off = _align(off + n, 8)
        self.shard_off, self.total = offs, _align(off, 8)
        self.shadow_dtype = self.params[0].param_dtype or self.params[0].orig_dtype
        self.version = 0                 # shadow version published so far (same on every rank)
        self.stale = True                # the master shards changed since the shadow was written
        self.shadow_off = 0              # set by the engine
        self.shadow: Optional[torch.Tensor] = None
        self.layout = None
        self.m: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        self.alias = W == 1


def _group_eligible(pg, max_tensors: int) -> Optional[str]:
    """None when the fused kernels cover this parameter group, else the reason they do not."""
    from torch.distributed.fsdp._fully_shard._fsdp_common import FSDPMeshInfo, HSDPMeshInfo

    if not isinstance(pg.mesh_info, FSDPMeshInfo) or isinstance(pg.mesh_info, HSDPMeshInfo):
        return "not a one-dimensional FSDP mesh"
    if not pg.fsdp_params:
        return "no parameters"
    if len(pg.fsdp_params) > max_tensors:
        return f"more than {max_tensors} tensors"
    dtypes = set()
    for p in pg.fsdp_params:
        if p.fsdp_placement.dim != 0:
            return "sharded on a dimension other than 0"
        if p.offload_to_cpu:
            return "CPU offload"
        if p.is_dtensor:
            return "DTensor parameter"
        if hasattr(p._sharded_local_tensor, "fsdp_pre_all_gather"):
            return "all-gather extension"
        if p.orig_dtype not in (torch.float32, torch.bfloat16, torch.float16):
            return f"dtype {p.orig_dtype}"
        dtypes.add((p.orig_dtype, p.param_dtype or p.orig_dtype))
    if len(dtypes) != 1:
        return "mixed dtypes"
    orig, low = next(iter(dtypes))
    if low not in (torch.bfloat16, torch.float16, torch.float32) or (orig != torch.float32 and orig != low):
        return f"dtype pair {orig}/{low}"
    return None


# --------------------------------------------------------------------------------------------- the engine
class FusedFSDP:
    """Owns the symmetric arena and the per-group state; created by ``install_fused_collectives``."""

    def __init__(self, model: torch.nn.Module, fused_adamw: Optional[dict] = None, gather_ctas: Optional[int] = None,
                 reduce_ctas: Optional[int] = None, emulate: Optional[bool] = None):
        from torch.distributed.fsdp import FSDPModule

        roots = [m for m in model.modules() if isinstance(m, FSDPModule)]
        if not roots:
            raise ValueError("install_fused_collectives: no fully_shard module under the model")
        states = [m._get_fsdp_state() for m in roots]
        states[0]._lazy_init() if states[0]._is_root is None else None
        pgs = [s._fsdp_param_group for s in states if s._fsdp_param_group is not None]
        if not pgs:
            raise ValueError("install_fused_collectives: no parameter group to manage")
        self.device = pgs[0].device
        mesh_pg = pgs[0]._all_gather_process_group
        self.group = mesh_pg
        self.rank, self.world = mesh_pg.rank(), mesh_pg.size()
        self.gather_ctas = int(gather_ctas or os.environ.get("B200_FSDP_GATHER_CTAS", 32))
        # With one rank the reduce kernel is the optimizer pass over the whole model, bound by HBM bandwidth: two CTAs
        # per SM.  With several ranks it shares the SMs with the backward GEMMs while it waits for its peers: fewer.
        self.reduce_ctas = int(reduce_ctas or os.environ.get("B200_FSDP_REDUCE_CTAS", 296 if self.world == 1 else 64))
        self.calls: Dict[str, int] = {"pack": 0, "gather": 0, "reduce": 0, "reduce_adamw": 0}
        self.skipped: Dict[str, str] = {}
        self.seq = 0                      # reduce calls issued so far (same on every rank)
        self.t = 0                        # optimizer steps applied by the fused epilogue
        if emulate is None:
            emulate = self.device.type != "blackwell"
        max_tensors = 40
        if not emulate:
            import torch_musa_b200 as bw

            max_tensors = bw._C._FSDP_MAX_TENSORS
        self.groups: List[_Group] = []
        for pg in pgs:
            pg.lazy_init() if not hasattr(pg, "_orig_dtype") else None
            why = _group_eligible(pg, max_tensors)
            if why is None and pg._all_gather_process_group is not mesh_pg:
                why = "a different shard group"
            if why is not None:
                self.skipped[pg._module_fqn or f"group{len(self.skipped)}"] = why
                continue
            if len(self.groups) >= _MAX_GROUPS:
                self.skipped[pg._module_fqn or "group"] = "group table full"
                continue
            self.groups.append(_Group(self, pg, len(self.groups)))
        if not self.groups:
            raise ValueError(f"install_fused_collectives: no group is covered by the fused kernels: {self.skipped}")

        # ---- arena layout: [shadow of group 0][shadow of group 1]...[staging ring]
        off = 0
        for g in self.groups:
            g.shadow_off = off
            off = _align(off + g.total * _itemsize(g.shadow_dtype), 256)
        grad_bytes = max(_itemsize(g.shadow_dtype) for g in self.groups)
        self.stage_bytes = _align(self.world * max(g.total for g in self.groups) * grad_bytes, 256) if self.world > 1 else 0
        self.stage_off = off
        arena_bytes = off + _RING * self.stage_bytes + 256
        cls = _EmulatedKernels if emulate else _DeviceKernels
        self.k = cls(mesh_pg, self.rank, self.world, self.device, arena_bytes)
        for g in self.groups:
            g.layout = self.k.make_layout(g.shard_numel, g.shard_off, g.full_numel, g.total)
            g.shadow = self.k.view(g.shadow_off, g.total, g.shadow_dtype)
            g.shadow.zero_()
        self.optimizer: Optional[FusedShardedAdamW] = None
        if fused_adamw is not None:
            for g in self.groups:
                if g.params[0].orig_dtype != torch.float32:
                    raise ValueError("fused_adamw needs fp32 master parameters (MixedPrecisionPolicy(param_dtype=...))")
                g.m = [torch.zeros(n, dtype=torch.float32, device=self.device) for n in g.shard_numel]
                g.v = [torch.zeros(n, dtype=torch.float32, device=self.device) for n in g.shard_numel]
            managed = {id(p.sharded_param) for g in self.groups for p in g.params}
            ordered = [p for p in model.parameters() if id(p) in managed]   # torch.optim.AdamW(model.parameters()) order
            self.optimizer = FusedShardedAdamW(self, ordered, **fused_adamw)
        for g in self.groups:
            g.pg._b200 = g
            for p in g.params:
                p._b200_group = g
            if g.alias:
                self._alias_outputs(g)
        if self.world > 1:
            _sync_device(self.device)
            dist.barrier(group=mesh_pg)        # every rank's pad and arena exist before anyone's kernel touches them
        _patch_fsdp()
        _engines.add(self)
        model.register_load_state_dict_post_hook(lambda module, incompatible: self.invalidate())

    # ---- one rank: the unsharded parameters are views of the shadow, for good
    def _alias_outputs(self, g: _Group) -> None:
        item = _itemsize(g.shadow_dtype)
        for p, n, off in zip(g.params, g.shard_numel, g.shard_off):
            p.all_gather_outputs = [self.k.view(g.shadow_off + off * item, n, g.shadow_dtype)]
            p.alloc_all_gather_outputs = _noop
            p.free_unsharded_param = _noop

    # ---- shadow refresh
    def _refresh(self, g: _Group, stream) -> None:
        if not g.stale:
            return
        g.version += 1
        with self._stream(stream):
            self.k.pack(g, [p._sharded_param_data for p in g.params], self.gather_ctas)
        g.stale = False
        self.calls["pack"] += 1

    def invalidate(self) -> None:
        """Marks every shadow out of date: the next unshard of a group casts its master shards again.  Called after
        every optimizer step and ``load_state_dict``; call it yourself after writing to parameters any other way.
        Every rank must call it at the same point of the program."""
        for g in self.groups:
            g.stale = True

    def _stream(self, stream):
        return self.groups[0].pg.device_handle.stream(stream)

    # ---- unshard / wait (called from the patched FSDPParamGroup methods)
    def unshard(self, g: _Group, async_op: bool) -> None:
        from torch.distributed.fsdp._fully_shard._fsdp_collectives import AllGatherResult

        pg = g.pg
        copy_in_stream, ag_stream = pg.comm_ctx.get_all_gather_streams(async_op, pg._training_state)
        self._refresh(g, copy_in_stream)
        if g.alias:
            ag_stream.wait_stream(copy_in_stream)
            event = ag_stream.record_event()
        else:
            compute = pg.device_handle.current_stream()
            ag_stream.wait_stream(copy_in_stream)
            with self._stream(ag_stream):
                # The outputs come from the all-gather stream's pool so that the pull can run ahead of the compute
                # stream; record_stream keeps a freed block away from later pulls until the compute work queued at
                # the time of the free has finished with it.
                outs = []
                for p, n in zip(g.params, g.shard_numel):
                    p.init_all_gather_outputs([n], [g.shadow_dtype], self.world, self.device)
                    p.alloc_all_gather_outputs()
                    out = p.all_gather_outputs[0]
                    if self.device.type != "cpu" and ag_stream != compute:
                        out.record_stream(compute)
                    outs.append(out)
                # the backward pull rewrites tensors that the forward saved for its own backward: same values
                with torch.autograd._unsafe_preserve_version_counter(tuple(outs)):
                    self.k.gather(g, outs, self.gather_ctas)
                event = ag_stream.record_event()
            self.calls["gather"] += 1
        pg._all_gather_result = AllGatherResult(pg._all_gather_output, event, None, [], [], [])

    def wait_for_unshard(self, g: _Group) -> None:
        from torch.distributed.fsdp._fully_shard._fsdp_param_group import TrainingState

        pg = g.pg
        result = pg._all_gather_result
        if pg._training_state == TrainingState.FORWARD:
            if prev := pg.comm_ctx.all_gather_state:   # a stock group ran before this one
                pg._wait_all_gather_streams_on_event(prev.event)
                pg.comm_ctx.all_gather_state = None
        if result.all_gather_event is not None:
            pg.device_handle.current_stream().wait_event(result.all_gather_event)
        for p in g.params:
            p.init_unsharded_param()
        pg._to_unsharded()
        pg._all_gather_result = None

    # ---- gradient reduce (called from the patched foreach_reduce)
    def reduce(self, g: _Group, fsdp_params, unsharded_grads, reduce_scatter_stream, orig_dtype,
               gradient_divide_factor):
        pg = g.pg
        handle = pg.device_handle
        current = handle.current_stream()
        grads = [gr if gr.is_contiguous() else gr.contiguous() for gr in unsharded_grads]
        unsharded_grads.clear()
        reduce_scatter_stream.wait_stream(current)
        scale = 1.0 / (gradient_divide_factor if gradient_divide_factor is not None else self.world)
        self.seq += 1
        seq = self.seq
        ack_need = max(0, seq - _RING)
        stage_off = self.stage_off + (seq % _RING) * self.stage_bytes
        opt = self.optimizer
        with handle.stream(reduce_scatter_stream):
            if opt is not None:
                if g.stale:
                    raise RuntimeError("fused_adamw: parameters were modified outside the engine after the last "
                                       "unshard; run a forward pass (or call engine.invalidate() earlier)")
                g.version += 1
                adam = ([p._sharded_param_data for p in g.params], g.m, g.v, opt._hyper(g, self.t + 1), g.shadow_off,
                        g.version)
                self.k.reduce(g, grads, stage_off, scale, None, adam, seq, ack_need, self.reduce_ctas)
                # the epilogue rewrites the master shards and the shadow together: nothing to pack afterwards
                g.stale = False
                opt._note_reduced(g)
                self.calls["reduce_adamw"] += 1
                reduce_scatter_event = reduce_scatter_stream.record_event()
                post_reduce_event = reduce_scatter_event
            else:
                out32 = torch.empty(g.total, dtype=torch.float32, device=self.device)
                self.k.reduce(g, grads, stage_off, scale, out32, None, seq, ack_need, self.reduce_ctas)
                self.calls["reduce"] += 1
                reduce_scatter_event = reduce_scatter_stream.record_event()
                reduce_output = out32 if orig_dtype in (None, torch.float32) else out32.to(orig_dtype)
                for p, off in zip(g.params, g.shard_off):
                    new_grad = torch.as_strided(reduce_output, size=p.sharded_size, stride=p.contiguous_sharded_stride,
                                                storage_offset=off)
                    if p.sharded_param.grad is not None:
                        p.sharded_param.grad._local_tensor += new_grad
                    else:
                        p.sharded_param.grad = p.to_sharded_dtensor(new_grad)
                    for hook in (getattr(p.sharded_param, "_post_accumulate_grad_hooks", {}) or {}).values():
                        hook(p.sharded_param)
                post_reduce_event = reduce_scatter_stream.record_event()
        # the gradients are read by the kernel on the reduce-scatter stream: the caller keeps this list until the
        # compute stream has waited for reduce_scatter_event
        return grads, reduce_scatter_event, post_reduce_event, None, None, None

    def check(self) -> None:
        """Raises if a kernel of this engine gave up on a bounded wait since the last call."""
        st = self.k.status()
        if st:
            raise RuntimeError(f"an FSDP kernel gave up waiting for rank {st - 1}")

    @property
    def fused_collective_count(self) -> int:
        return self.calls["gather"] + self.calls["reduce"] + self.calls["reduce_adamw"]


def _noop(*a, **k):
    return None


def _itemsize(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def _sync_device(device: torch.device) -> None:
    if device.type == "blackwell":
        import torch_musa_b200 as bw

        bw.synchronize()
    elif device.type == "cuda":
        torch.cuda.synchronize()


# --------------------------------------------------------------------------------------------- optimizer facade
class FusedShardedAdamW:
    """What the training loop holds when the AdamW update runs inside the gradient reduce kernel.

    ``step()`` does not launch anything: by the time ``backward()`` returns every group's update has been applied
    (fp32 master shard, both moments, the low-precision shadow).  It advances the step count that the next
    backward's bias correction uses.  ``param_groups`` has the usual single group so that learning-rate
    schedulers work; ``state_dict()`` / ``load_state_dict()`` use ``torch.optim.AdamW``'s format with sharded
    DTensor moments, so checkpoints are interchangeable with the stock optimizer over the same ``fully_shard`` model.
    Every backward applies one update: gradient accumulation needs the unfused mode.
    Parity: reference torch_musa/optim/fused_adamw.py (a separate multi-tensor pass after the reduce-scatter)."""

    def __init__(self, engine: FusedFSDP, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2):
        self.engine = engine
        params = list(params)
        assert len(params) == sum(len(g.params) for g in engine.groups)
        self.param_groups = [{"params": params, "lr": lr, "betas": tuple(betas), "eps": eps,
                              "weight_decay": weight_decay}]
        self.defaults = {"lr": lr, "betas": tuple(betas), "eps": eps, "weight_decay": weight_decay}
        self._reduced = set()

    def _hyper(self, g: _Group, step: int):
        pgp = self.param_groups[0]
        lr = pgp["lr"]
        lr = float(lr) if not isinstance(lr, torch.Tensor) else float(lr.item())
        return [lr, pgp["betas"][0], pgp["betas"][1], pgp["eps"], pgp["weight_decay"], float(step)]

    def _note_reduced(self, g: _Group) -> None:
        self._reduced.add(g.gid)

    def step(self, closure=None):
        loss = closure() if closure is not None else None
        if self._reduced:
            self.engine.t += 1
            self._reduced.clear()
        return loss

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.param_groups[0]["params"]:
            p.grad = None

    @property
    def state(self):
        out = {}
        for g in self.engine.groups:
            for p, m, v in zip(g.params, g.m, g.v):
                n = p.sharded_size.numel()
                out[p.sharded_param] = {
                    "step": torch.tensor(float(self.engine.t)),
                    "exp_avg": p.to_sharded_dtensor(m[:n].view(p.sharded_size)),
                    "exp_avg_sq": p.to_sharded_dtensor(v[:n].view(p.sharded_size)),
                }
        return out

    def state_dict(self) -> dict:
        st = self.state
        params = self.param_groups[0]["params"]
        packed = {k: v for k, v in self.param_groups[0].items() if k != "params"}
        packed["params"] = list(range(len(params)))
        return {"state": {i: st[p] for i, p in enumerate(params)}, "param_groups": [packed]}

    def load_state_dict(self, sd: dict) -> None:
        params = self.param_groups[0]["params"]
        by_param = {}
        for g in self.engine.groups:
            for p, m, v in zip(g.params, g.m, g.v):
                by_param[id(p.sharded_param)] = (p, m, v)
        step = None
        for i, st in sd["state"].items():
            p, m, v = by_param[id(params[int(i)])]
            n = p.sharded_size.numel()
            for key, dst in (("exp_avg", m), ("exp_avg_sq", v)):
                src = st[key]
                src = src._local_tensor if hasattr(src, "_local_tensor") else src
                dst[:n].copy_(src.reshape(-1))
            step = float(st["step"])
        if step is not None:
            self.engine.t = int(step)
        for k, v in sd["param_groups"][0].items():
            if k != "params":
                self.param_groups[0][k] = tuple(v) if k == "betas" else v


# --------------------------------------------------------------------------------------------- hooks into FSDP2
def _patch_fsdp() -> None:
    """Routes ``FSDPParamGroup.unshard`` / ``wait_for_unshard`` and ``foreach_reduce`` through the engine for the
    groups it manages; every other group keeps torch's implementation."""
    global _patched
    if _patched:
        return
    from torch.distributed.fsdp._fully_shard import _fsdp_param_group as mod

    PG = mod.FSDPParamGroup
    orig_unshard, orig_wait, orig_reduce = PG.unshard, PG.wait_for_unshard, mod.foreach_reduce

    def unshard(self, async_op: bool = False):
        g = getattr(self, "_b200", None)
        if g is None:
            return orig_unshard(self, async_op)
        if self._all_gather_result is not None or self.is_unsharded:
            return
        if not self.unshard_in_backward and self._training_state == mod.TrainingState.PRE_BACKWARD:
            return
        if self._reshard_after_forward_event is not None:
            self._wait_all_gather_streams_on_event(self._reshard_after_forward_event)
            self._reshard_after_forward_event = None
        with torch.no_grad():
            g.engine.unshard(g, async_op)

    def wait_for_unshard(self):
        g = getattr(self, "_b200", None)
        if g is None:
            return orig_wait(self)
        if not self._all_gather_result:
            return
        with torch.no_grad():
            g.engine.wait_for_unshard(g)

    def foreach_reduce(fsdp_params, unsharded_grads, reduce_scatter_group, reduce_scatter_stream, reduce_scatter_comm,
                       orig_dtype, reduce_dtype, device, gradient_divide_factor, all_reduce_group, all_reduce_stream,
                       all_reduce_grads, partial_reduce_output, all_reduce_hook, force_sum_reduction_for_comms=False):
        g = getattr(fsdp_params[0], "_b200_group", None) if fsdp_params else None
        ok = (g is not None and all_reduce_group is None and all_reduce_hook is None and partial_reduce_output is None
              and len(fsdp_params) == len(g.params) and all(a is b for a, b in zip(fsdp_params, g.params))
              and len({gr.dtype for gr in unsharded_grads}) == 1 and unsharded_grads[0].dtype == g.shadow_dtype
              and not (g.engine.optimizer is not None and any(p.sharded_param.grad is not None for p in g.params)))
        if not ok:
            return orig_reduce(fsdp_params, unsharded_grads, reduce_scatter_group, reduce_scatter_stream,
                               reduce_scatter_comm, orig_dtype, reduce_dtype, device, gradient_divide_factor,
                               all_reduce_group, all_reduce_stream, all_reduce_grads, partial_reduce_output,
                               all_reduce_hook, force_sum_reduction_for_comms)
        with torch.no_grad():
            return g.engine.reduce(g, fsdp_params, unsharded_grads, reduce_scatter_stream, orig_dtype,
                                   gradient_divide_factor)

    PG.unshard = unshard
    PG.wait_for_unshard = wait_for_unshard
    mod.foreach_reduce = foreach_reduce

    def after_any_optimizer_step(optimizer, args, kwargs):
        # the engine's own optimizer facade is not a torch.optim.Optimizer: this fires for ordinary optimizers only
        for e in list(_engines):
            e.invalidate()

    from torch.optim.optimizer import register_optimizer_step_post_hook

    register_optimizer_step_post_hook(after_any_optimizer_step)
    _patched = True


def install_fused_collectives(model: torch.nn.Module, fused_adamw: Optional[dict] = None, **kw) -> FusedFSDP:
    """Puts every FSDP2 parameter group under ``model`` that the kernels cover on the fused path.

    Call it after ``fully_shard`` has been applied, the parameters live on the device and have their initial values
    (the first forward packs them), and before the first forward.  ``fused_adamw``: ``dict(lr=..., betas=..., eps=...,
    weight_decay=...)`` moves the AdamW update into the gradient reduce kernel; the returned engine's ``optimizer``
    then replaces ``torch.optim.AdamW`` in the training loop.  Returns the engine (``engine.calls``,
    ``engine.skipped``, ``engine.check()``)."""
    return FusedFSDP(model, fused_adamw=fused_adamw, **kw)


def fused_collective_count(group=None) -> int:
    """How many collectives of ``group`` ran on the process group's own peer-memory kernels so far."""
    import torch_musa_b200 as bw

    pg = (group or dist.group.WORLD)._get_backend(torch.device("blackwell"))
    return int(bw._C._pg_fused_count(pg))
