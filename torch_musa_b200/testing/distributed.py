"""Multi-process test harness: spawn ``world_size`` ranks as child processes for a test body (gloo on CPU, bccl on
GPUs), collect a traceback or OK from every rank through a queue, and fail the calling test with all tracebacks.
``MultiProcessTestCase`` wraps it for ``unittest``-style suites; ``FSDPTest`` adds what sharded-training suites share
(mesh plans incl. hybrid sharding, ``run_subtests`` inside one set of ranks, ``check_sharded_parity`` against a replicated
twin, ``skip_if_lt_x_gpu``); ``spawn_isolated_test`` runs one function in a fresh interpreter (for tests that must own
process-wide state such as the allocator backend).

Parity: reference torch_musa/testing/common_fsdp.py:29-245 (FSDPTest: per-rank processes, exit-code protocol) and
torch_musa/testing/common_utils.py:194-254 (spawn_isolated_test).
"""
import os
import socket
import sys
import traceback

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, backend, fn, args, q, env):
    try:
        os.environ.update(env)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"] = str(rank), str(world), str(rank)
        if ROOT not in sys.path:
            sys.path.insert(0, ROOT)
        import torch.distributed as dist
        import torch_musa_b200 as bw

        if backend == "bccl":
            bw.set_device(rank)
        import datetime

        dist.init_process_group(backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
        try:
            fn(rank, world, *args)
        finally:
            try:
                dist.destroy_process_group()
            except Exception:
                pass
        q.put((rank, None))
    except Exception:
        q.put((rank, traceback.format_exc()))


def run_ranks(fn, world, backend="gloo", args=(), env=None, timeout=300):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, backend, fn, args, q, env or {})) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            r, err = q.get(timeout=timeout)
            results[r] = err
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()  # our own child, by handle
    errs = {r: e for r, e in results.items() if e}
    assert not errs, "\n".join(f"--- rank {r} ---\n{e}" for r, e in errs.items())
    assert len(results) == world


class MultiProcessTestCase:
    """Base class for suites whose tests run on every rank: subclasses set ``world_size`` / ``backend`` and call
    ``self.run_on_ranks(fn, *args)`` with a module-level function ``fn(rank, world, *args)``."""

    world_size = 2
    backend = "gloo"
    env = None
    timeout = 300

    def run_on_ranks(self, fn, *args):
        run_ranks(fn, self.world_size, self.backend, args=args, env=self.env, timeout=self.timeout)


def _isolated_entry(fn, args, q):
    try:
        if ROOT not in sys.path:
            sys.path.insert(0, ROOT)
        q.put((fn(*args), None))
    except Exception:
        q.put((None, traceback.format_exc()))


def spawn_isolated_test(fn, *args, timeout=300):
    """Runs ``fn(*args)`` (a module-level function) in a fresh interpreter and returns its result; raises with the
    child's traceback if it failed."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_isolated_entry, args=(fn, args, q))
    p.start()
    try:
        result, err = q.get(timeout=timeout)
    finally:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()  # our own child, by handle
    assert err is None, err
    return result


# ---------------------------------------------------------------------------------------------- sharded-training suites
def skip_if_lt_x_gpu(n: int):
    """pytest / unittest decorator: skip when fewer than ``n`` devices are visible."""
    import unittest

    import torch_musa_b200 as bw

    have = bw.device_count() if bw.is_available() else 0
    return unittest.skipIf(have < n, f"needs {n} GPUs, {have} visible")


def run_subtests(subtest_config, test_fn, *test_args, **test_kwargs):
    """Calls ``test_fn(*test_args, **test_kwargs, **combo)`` for every combination of the value lists in
    ``subtest_config`` inside ONE set of rank processes (spawning ranks and creating the process group is the
    expensive part of a distributed test), with a barrier between combinations; a failure names its combination."""
    import itertools

    import torch.distributed as dist

    keys = list(subtest_config)
    for values in itertools.product(*(subtest_config[k] for k in keys)):
        combo = dict(zip(keys, values))
        try:
            test_fn(*test_args, **test_kwargs, **combo)
        except Exception as e:
            raise AssertionError(f"subtest {combo} failed: {e}") from e
        if dist.is_initialized():
            dist.barrier()


def check_sharded_parity(replicated: torch.nn.Module, sharded: torch.nn.Module, prefixes_to_ignore=(), rtol=1e-5,
                         atol=1e-6) -> None:
    """Every parameter (and gradient) of a ``fully_shard``-ed module equals the matching shard of its replicated
    twin: the replicated tensor is distributed with the sharded parameter's own mesh and placements and the local
    shards are compared."""
    from torch.distributed.tensor import DTensor, Shard, distribute_tensor

    rep, sh = list(replicated.named_parameters()), list(sharded.named_parameters())
    assert len(rep) == len(sh), f"{len(rep)} replicated parameters against {len(sh)} sharded ones"
    for (rn, rp), (sn, sp) in zip(rep, sh):
        for prefix in prefixes_to_ignore:
            sn = sn.replace(prefix, "")
        assert rn == sn, f"parameter order differs: {rn} vs {sn}"
        assert isinstance(sp, DTensor), f"{sn} is not sharded"
        if tuple(sp.placements) == (Shard(0), Shard(0)):
            raise AssertionError("a (Shard(0), Shard(0)) layout cannot be reproduced with distribute_tensor")
        want = distribute_tensor(rp.detach(), sp.device_mesh, sp.placements).to_local()
        torch.testing.assert_close(sp.to_local().detach(), want, rtol=rtol, atol=atol, msg=lambda m: f"{rn}: {m}")
        if rp.grad is None:
            assert sp.grad is None, f"{sn} has a gradient, its replicated twin has none"
            continue
        assert sp.grad is not None and isinstance(sp.grad, DTensor), f"{sn}: missing or unsharded gradient"
        want_g = distribute_tensor(rp.grad, sp.device_mesh, sp.placements).to_local()
        torch.testing.assert_close(sp.grad.to_local(), want_g, rtol=rtol, atol=atol, msg=lambda m: f"{rn}.grad: {m}")


class FSDPTest(MultiProcessTestCase):
    """Suite base for sharded-data-parallel tests: rank processes as in ``MultiProcessTestCase`` plus the helpers
    such suites share.  ``device_mesh_plan`` gives the 1-D mesh (or the replicate x shard mesh of hybrid sharding)
    over the ranks of the calling process group."""

    world_size = 2

    @staticmethod
    def device_type() -> str:
        import torch.distributed as dist

        return "cpu" if dist.get_backend() == "gloo" else "blackwell"

    @classmethod
    def device_mesh_plan(cls, hybrid_shard: bool = False):
        import torch.distributed as dist
        from torch.distributed.device_mesh import init_device_mesh

        world = dist.get_world_size()
        if not hybrid_shard:
            return init_device_mesh(cls.device_type(), (world,))
        assert world % 2 == 0, "hybrid sharding needs an even number of ranks"
        return init_device_mesh(cls.device_type(), (2, world // 2), mesh_dim_names=("replicate", "shard"))

    run_subtests = staticmethod(run_subtests)
    check_sharded_parity = staticmethod(check_sharded_parity)
