"""The fused FSDP2 engine on the device kernels (pack / gather / reduce, csrc/kernels/fsdp_comm.cu): a small model
with shard sizes that divide neither by the world size nor by the 16-byte packet must train exactly like stock
``fully_shard`` + ``torch.optim.AdamW`` on 1, 2, 4 and 8 GPUs, in both modes (fp32 gradient shard / AdamW inside the
reduce kernel), and the kernels' own entry points must match an fp32 reference on ragged layouts.
Parity: reference tests/unittest/distributed/fsdp/fsdp_v2/test_fully_shard_training.py:48-90."""
import pytest
import torch

from _dist_utils import run_ranks
from test_fsdp_cpu import _body

pytestmark = pytest.mark.gpu


def _ngpu():
    import torch_musa_b200 as bw

    return bw.device_count()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("mode", ["plain", "adamw"])
def test_fused_fsdp_matches_stock(world, mode):
    if _ngpu() < world:
        pytest.skip(f"needs {world} GPUs")
    env = {"BCCL_DEVICE_WAIT_MS": "20000", "NCCL_NVLS_ENABLE": "0"}
    run_ranks(_body, world, "bccl", args=(mode, True, "blackwell"), env=env)


def _kernel_body(rank, world):
    """Drives pack / gather / reduce directly on a ragged layout and checks them against plain tensor math."""
    import torch.distributed as dist
    import torch_musa_b200 as bw
    from torch_musa_b200.parallel._symm import group_store_and_key

    dev = torch.device("blackwell", rank)
    shard = [1031, 8, 40000, 3]                      # padded shard elements per tensor (odd sizes on purpose)
    full = [world * 1031 - 5, world * 8, world * 40000 - 17, world * 3 - 2] if world > 1 else shard
    offs, off = [], 0
    for n in shard:
        offs.append(off)
        off = (off + n + 7) // 8 * 8
    total = off
    lay = bw._C._FsdpLayout(shard, offs, full, total)
    stage = world * total * 2
    store, key = group_store_and_key(None, "fsdp_test")
    sm = bw._C._create_symmetric_memory(store, key, rank, world, rank, total * 2 + 256 + 2 * stage + 512)
    assert sm.ok, sm.why_not
    w0 = bw._C._comm_user_word0()
    flag, ready, ack, ctr = w0, w0 + 64, w0 + 128, w0 + 160
    if world > 1:
        bw.synchronize()
        dist.barrier()
    g = torch.Generator().manual_seed(7)
    masters_all = [[torch.randn(n, generator=g) for n in shard] for _ in range(world)]
    masters = [t.to(dev) for t in masters_all[rank]]
    stage_off = (total * 2 + 255) // 256 * 256
    for version in (1, 2):
        sm.fsdp_pack(lay, masters, 0, torch.bfloat16, flag, version, ctr, 8)
        outs = [torch.empty(world * n, dtype=torch.bfloat16, device=dev) for n in shard]
        sm.fsdp_gather(lay, outs, 0, flag, version, 8)
        bw.synchronize()
        for i, n in enumerate(shard):
            want = torch.cat([masters_all[r][i].bfloat16() for r in range(world)])
            assert torch.equal(outs[i].cpu(), want), (version, i)
    # reduce: every rank contributes grads = (rank + 1) * base
    base = [torch.randn(f, generator=g).bfloat16() for f in full]
    grads = [(b.float() * (rank + 1)).bfloat16().to(dev) for b in base]
    want_sum = [sum((b.float() * (r + 1)).bfloat16().float() for r in range(world)) / world for b in base]
    for seq in (1, 2, 3):
        out32 = torch.full((total,), float("nan"), device=dev)
        sm.fsdp_reduce(lay, grads, stage_off + (seq % 2) * ((stage + 255) // 256 * 256), 1.0 / world, out32, [], [], [],
                       [], -1, torch.bfloat16, flag, 0, ready + (seq % 2) * 16, ack, seq, max(0, seq - 2), ctr + 1, 8)
        bw.synchronize()
        got = out32.cpu()
        for i, n in enumerate(shard):
            padded = torch.zeros(world * n)
            padded[:full[i]] = want_sum[i]
            want = padded[rank * n:(rank + 1) * n]
            assert torch.allclose(got[offs[i]:offs[i] + n], want, atol=1e-6, rtol=1e-6), (seq, i)
    # AdamW epilogue against plain tensor math
    p32 = [t.clone() for t in masters]
    m = [torch.zeros_like(t) for t in masters]
    v = [torch.zeros_like(t) for t in masters]
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    sm.fsdp_reduce(lay, grads, stage_off, 1.0 / world, None, p32, m, v, [lr, b1, b2, eps, wd, 1.0], 0, torch.bfloat16,
                   flag, 3, ready, ack, 4, 2, ctr + 1, 8)
    bw.synchronize()
    shadow = sm.local_tensor(0, [total], torch.bfloat16).cpu()
    for i, n in enumerate(shard):
        padded = torch.zeros(world * n)
        padded[:full[i]] = want_sum[i]
        gr = padded[rank * n:(rank + 1) * n]
        p = masters_all[rank][i].clone() * (1 - lr * wd)
        mm = (1 - b1) * gr
        vv = (1 - b2) * gr * gr
        p = p - (lr / (1 - b1)) * mm / (vv.sqrt() / (1 - b2) ** 0.5 + eps)
        assert torch.allclose(p32[i].cpu(), p, atol=1e-5, rtol=1e-5), i
        assert torch.allclose(m[i].cpu(), mm, atol=1e-6, rtol=1e-5), i
        assert torch.equal(shadow[offs[i]:offs[i] + n], p32[i].cpu().bfloat16()), i
    assert sm.take_status() == 0


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_fsdp_kernels_ragged_layout(world):
    if _ngpu() < world:
        pytest.skip(f"needs {world} GPUs")
    run_ranks(_kernel_body, world, "bccl", env={"BCCL_DEVICE_WAIT_MS": "20000", "NCCL_NVLS_ENABLE": "0"})


def _timeout_body(rank, world):
    """A gather whose flag nobody raises must give up after the configured limit, report through the status word
    and leave the device usable (the bounded-wait form of failure detection: no fault, no hang)."""
    import time

    import torch_musa_b200 as bw
    from torch_musa_b200.parallel._symm import group_store_and_key

    dev = torch.device("blackwell", rank)
    lay = bw._C._FsdpLayout([64], [0], [64 * world], 64)
    store, key = group_store_and_key(None, "fsdp_timeout")
    sm = bw._C._create_symmetric_memory(store, key, rank, world, rank, 4096)
    assert sm.ok, sm.why_not
    import torch.distributed as dist

    bw.synchronize()
    dist.barrier()
    old = bw._C._comm_get_wait_ms()
    bw._C._comm_set_wait_ms(5.0)
    try:
        out = [torch.zeros(64 * world, dtype=torch.bfloat16, device=dev)]
        t0 = time.time()
        sm.fsdp_gather(lay, out, 0, bw._C._comm_user_word0(), 1, 2)   # version 1 was never published
        bw.synchronize()
        assert time.time() - t0 < 5.0
        st = sm.take_status()
        assert st != 0, "the wait should have run out"
        assert st - 1 != rank
    finally:
        bw._C._comm_set_wait_ms(old)
    # the context is still usable
    x = torch.ones(1024, device=dev)
    assert float((x + x).sum().cpu()) == 2048.0
    dist.barrier()


def test_device_wait_times_out_and_reports():
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_timeout_body, 2, "bccl", env={"NCCL_NVLS_ENABLE": "0"})
