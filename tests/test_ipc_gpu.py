"""Device tensors across processes (torch.multiprocessing), with cudaMalloc segments and with
expandable segments; expandable segments and pool checkpoints on the device.
Mirrors reference tests/unittest/core/test_multiprocess.py:155-584 and test_memory.py (expandable
segment / mempool cases)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run_worker(conf):
    env = dict(os.environ)
    env["PYTORCH_BLACKWELL_ALLOC_CONF"] = conf
    r = subprocess.run([sys.executable, os.path.join(HERE, "_ipc_worker.py")], env=env, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().endswith("OK"), r.stdout + r.stderr
    return r.stdout


def test_share_tensor_between_processes():
    out = _run_worker("expandable_segments:False")
    assert "expandable_segments {False}" in out


def test_share_tensor_between_processes_expandable_segments():
    out = _run_worker("expandable_segments:True")
    assert "expandable_segments {True}" in out


_EXPANDABLE = r"""
import torch, torch_musa_b200 as bw
MiB = 1 << 20
dev = "blackwell"
xs = []
for i in range(6):
    xs.append(torch.full((32 * MiB // 4,), float(i), device=dev))
st = bw.memory_stats()
assert st["segment.all.current"] <= 2, st["segment.all.current"]       # one large (+ maybe one small) segment
snap = bw.memory_snapshot()
assert all(s["is_expandable"] for s in snap)
addr = sorted(x.data_ptr() for x in xs)
assert all(b - a == 32 * MiB for a, b in zip(addr, addr[1:]))           # grown in place, contiguous
assert [float(x.sum().cpu()) / x.numel() for x in xs] == [0., 1., 2., 3., 4., 5.]
y = torch.randn(1024, 1024, device=dev, dtype=torch.bfloat16)
ref = (y.cpu().float() @ y.cpu().float()).to(torch.bfloat16)
assert torch.allclose((y @ y).cpu().float(), ref.float(), rtol=2e-2, atol=2.0)
reserved = bw.memory_reserved()
del xs[1:5]
bw.empty_cache()
assert bw.memory_reserved() <= reserved - 120 * MiB                      # whole units went back to the driver
z = torch.ones(100 * MiB // 4, device=dev)                               # re-fills the hole
assert float(z.sum().cpu()) == z.numel()
del xs, z, y
bw.empty_cache()
assert bw.memory_reserved() == 0
print("OK")
"""


def test_expandable_segments_on_device():
    env = dict(os.environ, PYTORCH_BLACKWELL_ALLOC_CONF="expandable_segments:True")
    r = subprocess.run([sys.executable, "-c", _EXPANDABLE], env=env, capture_output=True, text=True, timeout=300,
                       cwd=os.path.dirname(HERE))
    assert r.returncode == 0 and r.stdout.strip().endswith("OK"), r.stdout + r.stderr


def test_pool_checkpoint_restore_on_device(bw):
    pool = bw.MemPool()
    with bw.use_mem_pool(pool):
        a = torch.full((1 << 20,), 3.0, device="blackwell")
        b = torch.full((1 << 20,), 4.0, device="blackwell")
    dev = bw.current_device()
    state = bw.get_pool_checkpoint(dev, pool.id)
    assert sorted(state.live_pointers) == sorted([a.data_ptr(), b.data_ptr()])
    pa, nbytes = a.data_ptr(), a.numel() * 4
    with bw.use_mem_pool(pool):
        c = torch.zeros(1 << 18, device="blackwell")
    pc = c.data_ptr()
    del a                                   # dies after the checkpoint: the restore brings its block back
    torch.blackwell.synchronize()
    freed, created = bw.set_pool_checkpoint(dev, state, stale=[c])
    assert freed == [pc] and sorted(created) == sorted([pa, b.data_ptr()])
    a2 = bw.adopt_allocation(dev, pa, nbytes).view(torch.float32)
    assert a2.data_ptr() == pa and float(a2.sum().cpu()) == 3.0 * (1 << 20)   # contents untouched
    assert float(b.sum().cpu()) == 4.0 * (1 << 20)
    with pytest.raises(RuntimeError, match="already has an owner"):
        bw.adopt_allocation(dev, b.data_ptr(), 16)
    del c, b, a2
    bw.empty_cache()
    assert pool.snapshot() == []
