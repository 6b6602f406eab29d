"""Spawns world_size ranks as child processes for a test body (gloo on CPU, bccl on GPUs).
Each rank reports OK or a traceback through a queue; the parent asserts all succeeded.
(The reference's FSDPTest does the same with an exit-code protocol: reference
torch_musa/testing/common_fsdp.py:29-245.)"""
import os
import socket
import sys
import traceback

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


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
