"""Multi-process test harness: spawn ``world_size`` ranks as child processes for a test body (gloo on CPU, bccl on
GPUs), collect a traceback or OK from every rank through a queue, and fail the calling test with all tracebacks.
``MultiProcessTestCase`` wraps it for ``unittest``-style suites; ``spawn_isolated_test`` runs one function in a fresh
interpreter (for tests that must own process-wide state such as the allocator backend).

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
