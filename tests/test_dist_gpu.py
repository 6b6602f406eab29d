"""Collectives of the bccl backend on real GPUs (2, 4 and 8 ranks, as many as the box has): closed-form expected values for every
collective (reference tests/unittest/distributed/test_dist.py:29-300), the peer-memory kernels
against NCCL, DDP and FSDP2 training parity, the watchdog."""
import pytest
import torch

from _dist_utils import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

WORLDS = [2, 4, 8]


def _need(world):
    import torch_musa_b200 as bw

    if bw.device_count() < world:
        pytest.skip(f"needs {world} GPUs")


def _collectives_body(rank, world):
    import torch.distributed as dist
    import torch_musa_b200 as bw

    dev = torch.device("blackwell", rank)
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        x = torch.full((1024,), float(rank + 1), dtype=dt, device=dev)
        dist.all_reduce(x)
        assert torch.all(x.float().cpu() == sum(range(1, world + 1)))
        x = torch.full((1024,), float(rank + 1), dtype=dt, device=dev)
        dist.all_reduce(x, op=dist.ReduceOp.AVG)
        assert torch.allclose(x.float().cpu(), torch.full((1024,), (world + 1) / 2))
        x = torch.full((8,), float(rank), dtype=dt, device=dev)
        dist.broadcast(x, src=1)
        assert torch.all(x.float().cpu() == 1.0)
        out = torch.empty(world * 512, dtype=dt, device=dev)
        dist.all_gather_into_tensor(out, torch.full((512,), float(rank), dtype=dt, device=dev))
        assert torch.equal(out.float().cpu(), torch.arange(world).repeat_interleave(512).float())
        lst = [torch.empty(16, dtype=dt, device=dev) for _ in range(world)]
        dist.all_gather(lst, torch.full((16,), float(rank), dtype=dt, device=dev))
        assert all(torch.all(t.float().cpu() == i) for i, t in enumerate(lst))
        rs = torch.empty(512, dtype=dt, device=dev)
        dist.reduce_scatter_tensor(rs, torch.arange(world * 512, device=dev).to(dt) * 0 + (rank + 1))
        assert torch.all(rs.float().cpu() == sum(range(1, world + 1)))
        r = torch.full((8,), float(rank + 1), dtype=dt, device=dev)
        dist.reduce(r, dst=0)
        if rank == 0:
            assert torch.all(r.float().cpu() == sum(range(1, world + 1)))
    # all_to_all_single
    inp = (torch.arange(world * 4, device=dev) + rank * 100).float()
    out = torch.empty(world * 4, device=dev)
    dist.all_to_all_single(out, inp)
    exp = torch.cat([torch.arange(rank * 4, rank * 4 + 4).float() + s * 100 for s in range(world)])
    assert torch.equal(out.cpu(), exp)
    # gather / scatter / send / recv / barrier / objects
    g = [torch.empty(4, device=dev) for _ in range(world)] if rank == 0 else None
    dist.gather(torch.full((4,), float(rank), device=dev), g, dst=0)
    if rank == 0:
        assert all(torch.all(t.cpu() == i) for i, t in enumerate(g))
    sc = torch.empty(4, device=dev)
    dist.scatter(sc, [torch.full((4,), float(i), device=dev) for i in range(world)] if rank == 0 else None, src=0)
    assert torch.all(sc.cpu() == rank)
    if rank == 0:
        dist.send(torch.arange(10, device=dev).float(), dst=1)
    elif rank == 1:
        t = torch.empty(10, device=dev)
        dist.recv(t, src=0)
        assert torch.equal(t.cpu(), torch.arange(10).float())
    dist.barrier()
    objs = [None] * world
    dist.all_gather_object(objs, {"rank": rank})
    assert [o["rank"] for o in objs] == list(range(world))
    b = torch.tensor([True, False], device=dev) if rank == 0 else torch.tensor([False, False], device=dev)
    dist.all_reduce(b)
    assert b.cpu().tolist() == [True, False]
    # scale-then-sum in one pass (gradient averaging with an arbitrary divisor)
    x = torch.full((4096,), float(rank + 1), device=dev)
    dist.all_reduce(x, op=dist._make_nccl_premul_sum(0.25))
    assert torch.allclose(x.cpu(), torch.full((4096,), 0.25 * sum(range(1, world + 1))))
    rs = torch.empty(256, dtype=torch.bfloat16, device=dev)
    dist.reduce_scatter_tensor(rs, torch.ones(world * 256, dtype=torch.bfloat16, device=dev),
                               op=dist._make_nccl_premul_sum(0.5))
    assert torch.all(rs.float().cpu() == 0.5 * world)
    # complex tensors travel as pairs of reals
    z = torch.full((64,), complex(rank + 1, -(rank + 1)), dtype=torch.complex64, device=dev)
    dist.all_reduce(z)
    tot = sum(range(1, world + 1))
    assert torch.allclose(torch.view_as_real(z).cpu(), torch.tensor([float(tot), -float(tot)]).repeat(64, 1))
    pg = dist.group.WORLD._get_backend(dev)
    dump = bw._C._pg_dump_flight_recorder(pg)
    assert "all_gather_into_tensor" in dump
    assert '"stack"' in dump                    # BCCL_TRACE_CPP_STACK=1: every record carries its caller's backtrace
    assert bw._C._event_cache_stats()[0] > 0    # events of finished collectives were reused


@pytest.mark.parametrize("world", WORLDS)
def test_collectives_closed_form(world):
    _need(world)
    run_ranks(_collectives_body, world, "bccl", env={"BCCL_TRACE_CPP_STACK": "1"})


def _fused_vs_nccl_body(rank, world):
    import torch.distributed as dist
    import torch_musa_b200 as bw

    dev = torch.device("blackwell", rank)
    pg = dist.group.WORLD._get_backend(dev)
    sm = bw._C._pg_symmetric_memory(pg, rank)
    assert sm.ok, sm.why_not
    torch.manual_seed(rank)
    for dt in (torch.float32, torch.bfloat16):
        for n in (2048, 1 << 20, (6 << 20) + 8 * 13):
            x = torch.randn(n).to(dt)
            before = bw._C._pg_fused_count(pg)
            a = x.to(dev)
            dist.all_reduce(a, op=dist.ReduceOp.AVG)
            assert bw._C._pg_fused_count(pg) == before + 1, "all-reduce did not take the peer-memory kernel"
            bw._C._pg_set_fused(pg, False)
            b = x.to(dev)
            dist.all_reduce(b, op=dist.ReduceOp.AVG)
            bw._C._pg_set_fused(pg, True)
            tol = 1e-6 if dt == torch.float32 else 2e-2
            assert torch.allclose(a.float().cpu(), b.float().cpu(), atol=tol, rtol=tol)
            # all-gather
            out_f = torch.empty(world * n, dtype=dt, device=dev)
            dist.all_gather_into_tensor(out_f, x.to(dev))
            bw._C._pg_set_fused(pg, False)
            out_n = torch.empty(world * n, dtype=dt, device=dev)
            dist.all_gather_into_tensor(out_n, x.to(dev))
            bw._C._pg_set_fused(pg, True)
            assert torch.equal(out_f.cpu(), out_n.cpu())
            # reduce-scatter (+ fused fp32 output for bf16 input)
            big = torch.randn(world * n).to(dt)
            rs_f = torch.empty(n, dtype=dt, device=dev)
            dist.reduce_scatter_tensor(rs_f, big.to(dev), op=dist.ReduceOp.AVG)
            bw._C._pg_set_fused(pg, False)
            rs_n = torch.empty(n, dtype=dt, device=dev)
            dist.reduce_scatter_tensor(rs_n, big.to(dev), op=dist.ReduceOp.AVG)
            bw._C._pg_set_fused(pg, True)
            assert torch.allclose(rs_f.float().cpu(), rs_n.float().cpu(), atol=tol, rtol=tol)
    assert sm.take_status() == 0
    bw.synchronize()


@pytest.mark.parametrize("world", WORLDS)
def test_peer_memory_kernels_match_nccl(world):
    _need(world)
    run_ranks(_fused_vs_nccl_body, world, "bccl", env={"NCCL_NVLS_ENABLE": "0"})


def _ddp_body(rank, world):
    import torch.distributed as dist
    import torch_musa_b200 as bw
    from torch_musa_b200.parallel import wrap_ddp

    dev = torch.device("blackwell", rank)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.ReLU(), torch.nn.Linear(512, 10))
    ref = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.ReLU(), torch.nn.Linear(512, 10))
    ref.load_state_dict(model.state_dict())
    ddp = wrap_ddp(model.to(dev), device_ids=[rank])
    gens = [torch.Generator().manual_seed(r) for r in range(world)]
    data = [(torch.randn(32, 256, generator=g), torch.randint(0, 10, (32,), generator=g)) for g in gens]
    X, Y = torch.cat([d[0] for d in data]), torch.cat([d[1] for d in data])
    x, y = data[rank]
    torch.nn.functional.cross_entropy(ddp(x.to(dev)), y.to(dev)).backward()
    torch.nn.functional.cross_entropy(ref(X), Y).backward()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p.grad.cpu(), q.grad, atol=1e-5), (p.grad.cpu() - q.grad).abs().max()
    bw.synchronize()


@pytest.mark.parametrize("world", WORLDS)
def test_ddp_matches_single_process(world):
    _need(world)
    run_ranks(_ddp_body, world, "bccl")


def _fsdp_body(rank, world):
    import torch.distributed as dist
    import torch_musa_b200 as bw
    from torch.distributed.fsdp import fully_shard, MixedPrecisionPolicy
    from torch_musa_b200.models import Llama, llama_tiny_config

    dev = torch.device("blackwell", rank)
    cfg = llama_tiny_config()
    torch.manual_seed(0)
    ref = Llama(cfg)
    ref.reset_parameters(seed=3)
    model = Llama(cfg)
    model.load_state_dict(ref.state_dict())
    model = model.to(dev)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for layer in model.layers:
        fully_shard(layer, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, fused=True)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-3)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, cfg.vocab_size, (world * 2, 65), generator=g)
    mine = toks[rank * 2:(rank + 1) * 2].to(dev)
    losses, rlosses = [], []
    for _ in range(4):
        loss = model(mine[:, :-1], mine[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad()
        lt = loss.detach().float().clone()
        dist.all_reduce(lt, op=dist.ReduceOp.AVG)
        losses.append(float(lt.cpu()))
        rl = ref(toks[:, :-1], toks[:, 1:])
        rl.backward()
        ropt.step()
        ropt.zero_grad()
        rlosses.append(float(rl))
    for a, b in zip(losses, rlosses):
        assert abs(a - b) < 0.08, (losses, rlosses)
    assert losses[-1] < losses[0]
    pg = dist.group.WORLD._get_backend(dev)
    assert bw._C._pg_fused_count(pg) > 0
    bw.synchronize()


@pytest.mark.parametrize("world", WORLDS)
def test_fsdp2_tracks_single_process_reference(world):
    _need(world)
    run_ranks(_fsdp_body, world, "bccl")


def _watchdog_body(rank, world):
    import datetime
    import time
    import torch.distributed as dist
    import torch_musa_b200 as bw

    dev = torch.device("blackwell", rank)
    pg = dist.group.WORLD._get_backend(dev)
    w = bw._C._pg_make_test_work(pg, datetime.timedelta(milliseconds=300))
    time.sleep(1.0)
    assert w.is_completed() and not w.is_success()
    with pytest.raises(Exception, match="did not finish"):
        w.wait()
    assert "timed_out" in bw._C._pg_dump_flight_recorder(pg)
    assert bw._C._pg_error(pg) != 0


@pytest.mark.parametrize("world", WORLDS)
def test_watchdog_reports_timeout(world):
    _need(world)
    run_ranks(_watchdog_body, world, "bccl")


def _fused_ag_matmul_body(rank, world):
    import torch_musa_b200 as bw
    from torch_musa_b200.parallel import tensor_parallel as TP
    from torch_musa_b200.parallel.fused_tp import FusedTensorParallel

    dev = torch.device("blackwell", rank)
    ctx = FusedTensorParallel(max_shard_bytes=1024 * 1024 * 2, max_rows=2048 * world, device=dev, copier_pairs=4)
    for rows, K, N in [(256, 512, 384), (512, 1024, 512), (1024, 256, 136)]:
        torch.manual_seed(100 + rank)
        x = (torch.randn(rows, K) * 0.5).to(torch.bfloat16).to(dev)
        torch.manual_seed(7)
        w = (torch.randn(N, K) * 0.1).to(torch.bfloat16).to(dev)
        x_full_ref = TP.all_gather_rows(x)
        ref = (x_full_ref.float() @ w.float().t()).cpu()
        for wt in (w, w.t().contiguous().t()):            # K-major and N-major weight layouts
            out = ctx.ag_matmul(x, wt, None)
            assert out is not None, "shape should be covered by the fused kernel"
            y, x_full = out
            assert torch.equal(x_full.cpu(), x_full_ref.cpu())
            err = (y.float().cpu() - ref).abs().max() / ref.abs().max()
            assert err < 2e-2, float(err)
    # through autograd with the fused forward installed
    ctx.install()
    try:
        x = (torch.randn(256, 512) * 0.5).to(torch.bfloat16).to(dev).requires_grad_()
        w = (torch.randn(384, 512) * 0.1).to(torch.bfloat16).to(dev).requires_grad_()
        before = ctx.calls
        y = TP.ag_matmul(x, w)
        y.float().pow(2).sum().backward()
        assert ctx.calls == before + 1
        TP.FUSED_AG_MATMUL = None
        x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
        y2 = TP.ag_matmul(x2, w2)
        y2.float().pow(2).sum().backward()
        assert torch.allclose(y.float(), y2.float(), atol=2e-2, rtol=2e-2)
        assert torch.allclose(x.grad.float(), x2.grad.float(), atol=0.5, rtol=5e-2)
        assert torch.allclose(w.grad.float(), w2.grad.float(), atol=0.5, rtol=5e-2)
    finally:
        ctx.uninstall()
    bw.synchronize()
    ctx.check()


@pytest.mark.parametrize("world", WORLDS)
def test_fused_allgather_gemm_matches_unfused(world):
    _need(world)
    run_ranks(_fused_ag_matmul_body, world, "bccl", env={"NCCL_NVLS_ENABLE": "0"})


def _fused_matmul_rs_body(rank, world):
    import torch_musa_b200 as bw
    from torch_musa_b200.parallel import tensor_parallel as TP
    from torch_musa_b200.parallel.fused_tp import FusedTensorParallel

    dev = torch.device("blackwell", rank)
    sc = world // 2                       # row counts must divide by 256 x world
    ctx = FusedTensorParallel(max_shard_bytes=1 << 21, max_rows=4096 * sc, device=dev, copier_pairs=4,
                              max_partial_bytes=2048 * 1024 * 2 * sc, reducer_pairs=4)
    for M, K, N in [(512 * sc, 256, 256), (1024 * sc, 520, 512), (2048 * sc, 136, 1024), (512 * sc, 256, 256)]:
        torch.manual_seed(200 + rank)
        x = (torch.randn(M, K) * 0.5).to(torch.bfloat16).to(dev)
        w = (torch.randn(N, K) * 0.1).to(torch.bfloat16).to(dev)
        ref = TP.reduce_scatter_rows((x.float() @ w.float().t())).cpu()
        for wt in (w, w.t().contiguous().t()):
            y = ctx.matmul_rs(x, wt, None)
            assert y is not None
            err = (y.float().cpu() - ref).abs().max() / ref.abs().max()
            assert err < 3e-2, (M, K, N, float(err))
    ctx.install()
    try:
        x = (torch.randn(512 * sc, 256) * 0.5).to(torch.bfloat16).to(dev).requires_grad_()
        w = (torch.randn(256, 256) * 0.1).to(torch.bfloat16).to(dev).requires_grad_()
        y = TP.matmul_rs(x, w)
        y.float().pow(2).sum().backward()
        assert ctx.rs_calls >= 9 and ctx.calls >= 1      # backward of matmul_rs ran the fused all-gather GEMM
        TP.FUSED_AG_MATMUL = TP.FUSED_MATMUL_RS = None
        x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
        y2 = TP.matmul_rs(x2, w2)
        y2.float().pow(2).sum().backward()
        assert torch.allclose(y.float(), y2.float(), atol=3e-2, rtol=3e-2)
        assert torch.allclose(x.grad.float(), x2.grad.float(), atol=0.5, rtol=5e-2)
        assert torch.allclose(w.grad.float(), w2.grad.float(), atol=0.5, rtol=5e-2)
    finally:
        ctx.uninstall()
    bw.synchronize()
    ctx.check()


@pytest.mark.parametrize("world", WORLDS)
def test_fused_gemm_reduce_scatter_matches_unfused(world):
    _need(world)
    run_ranks(_fused_matmul_rs_body, world, "bccl", env={"NCCL_NVLS_ENABLE": "0"})


def _sharded_adamw_body(rank, world):
    import torch_musa_b200 as bw
    from torch_musa_b200.parallel.zero import ShardedFusedAdamW

    dev = torch.device("blackwell", rank)
    torch.manual_seed(0)
    shapes = [(256, 128), (128,), (512, 256), (64, 64)]
    base = [torch.randn(*s) * 0.1 for s in shapes]
    results = []
    for fused in (True, False):
        params = [torch.nn.Parameter(b.to(torch.bfloat16).to(dev)) for b in base]
        opt = ShardedFusedAdamW(params, lr=1e-2, weight_decay=0.1, bucket_mb=1, fused=fused)
        assert opt.fused == fused
        for it in range(3):
            opt.zero_grad()
            torch.manual_seed(100 * it + rank)                    # every rank its own gradients
            for p in params:
                p.grad.copy_((torch.randn(p.shape) * 0.05).to(torch.bfloat16).to(dev))
            opt.step()
        bw.synchronize()
        opt.check()
        results.append([p.detach().float().cpu() for p in params])
    for a, b in zip(*results):
        assert torch.allclose(a, b, atol=2e-2, rtol=2e-2), (a - b).abs().max()
    # closed form for the first step direction: the update moves against the averaged gradient
    assert all(torch.isfinite(a).all() for a in results[0])


@pytest.mark.parametrize("world", WORLDS)
def test_fused_reduce_scatter_adamw_matches_unfused(world):
    _need(world)
    run_ranks(_sharded_adamw_body, world, "bccl", env={"NCCL_NVLS_ENABLE": "0"})


def _remote_error_body(rank, world):
    import datetime
    import time
    import torch.distributed as dist
    import torch_musa_b200 as bw

    dev = torch.device("blackwell", rank)
    t = torch.ones(8, device=dev)
    dist.all_reduce(t)                      # communicators are up; nothing is in flight afterwards
    bw.synchronize()
    pg = dist.group.WORLD._get_backend(dev)
    if rank == 1:
        bw._C._pg_make_test_work(pg, datetime.timedelta(milliseconds=200))     # a collective that never completes
    deadline = time.time() + 8.0
    while time.time() < deadline and bw._C._pg_error(pg) == 0:
        time.sleep(0.2)
    # rank 1 sees its own time-out, rank 0 learns of it through the store (no GPU involved on either side)
    assert bw._C._pg_error(pg) != 0, f"rank {rank} never learned of the failure"


@pytest.mark.parametrize("world", WORLDS)
def test_failure_on_one_rank_is_propagated_through_the_store(world):
    _need(world)
    run_ranks(_remote_error_body, world, "bccl", env={"NCCL_NVLS_ENABLE": "0"})


def _dtensor_tp_body(rank, world):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Shard, distribute_tensor
    import torch_musa_b200 as bw
    from torch_musa_b200.models import Llama, llama_tiny_config
    from torch_musa_b200.ops import functional as BF
    from torch_musa_b200.parallel.dtensor_tp import parallelize_llama

    dev = torch.device("blackwell", rank)
    mesh = init_device_mesh("blackwell", (world,))
    cfg = llama_tiny_config(fused_qkv=False, fused_gate_up=False, n_heads=8, n_kv_heads=8, vocab_size=512)
    torch.manual_seed(0)
    full = Llama(cfg)
    full.reset_parameters(seed=3)
    tp = Llama(cfg)
    tp.load_state_dict(full.state_dict())
    tp = tp.to(dev).to(torch.bfloat16)
    full = full.to(torch.bfloat16)
    parallelize_llama(tp, mesh, loss_parallel=True)
    torch.manual_seed(11)
    toks = torch.randint(0, cfg.vocab_size, (2, 33))
    loss_ref = full(toks[:, :-1], toks[:, 1:])
    loss_ref.backward()
    loss = tp(toks[:, :-1].to(dev), toks[:, 1:].to(dev))
    loss.backward()
    assert abs(float(loss) - float(loss_ref)) < 5e-2, (float(loss), float(loss_ref))
    g = tp.layers[0].attn.wq.weight.grad.to_local().float().cpu()
    rows = g.shape[0]
    ref = full.layers[0].attn.wq.weight.grad[rank * rows:(rank + 1) * rows].float()
    assert (g - ref).abs().max() <= 0.05 * ref.abs().max() + 1e-3
    # a custom kernel called on DTensors: the registered rule keeps the shards where they are
    a = distribute_tensor(torch.randn(4, 16, 64).to(torch.bfloat16).to(dev), mesh, [Shard(1)])
    b = distribute_tensor(torch.randn(4, 16, 64).to(torch.bfloat16).to(dev), mesh, [Shard(1)])
    out = torch.ops.blackwell.silu_mul(a, b)
    assert isinstance(out, DTensor) and out.placements == (Shard(1),)
    ref = torch.nn.functional.silu(a.full_tensor().float()) * b.full_tensor().float()
    assert (out.full_tensor().float() - ref).abs().max() < 0.1


@pytest.mark.parametrize("world", [2, 4])
def test_dtensor_tensor_parallel_on_device(world):
    _need(world)
    run_ranks(_dtensor_tp_body, world, "bccl")


def _fsdp1_body(rank, world):
    import torch.distributed as dist
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
    import torch_musa_b200 as bw  # noqa: F401

    dev = torch.device("blackwell", rank)
    torch.manual_seed(0)
    ref = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 32))
    model = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 32))
    model.load_state_dict(ref.state_dict())
    fsdp = FSDP(model.to(dev), device_id=dev, use_orig_params=True)
    opt = torch.optim.SGD(fsdp.parameters(), lr=0.1)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    for step in range(3):
        torch.manual_seed(100 + step)
        xs = torch.randn(world, 16, 64)
        loss = fsdp(xs[rank].to(dev)).pow(2).mean()
        loss.backward()
        opt.step()
        opt.zero_grad()
        rloss = sum(ref(xs[r]).pow(2).mean() for r in range(world)) / world
        rloss.backward()
        ropt.step()
        ropt.zero_grad()
        tot = loss.detach().clone()
        dist.all_reduce(tot)
        assert abs(float(tot) / world - float(rloss)) < 1e-3, (step, float(tot) / world, float(rloss))
    with FSDP.summon_full_params(fsdp):
        for (n, p), (_, q) in zip(fsdp.named_parameters(), ref.named_parameters()):
            assert torch.allclose(p.detach().cpu(), q.detach(), atol=1e-4), n


def test_fsdp1_wrapper_trains_on_device():
    """The flat-parameter FSDP wrapper (device handle, streams, all-gather / reduce-scatter on bccl) at 2 ranks."""
    _need(2)
    run_ranks(_fsdp1_body, 2, "bccl")


def test_data_parallel_comm_on_devices(bw=None):
    """broadcast / scatter / gather / reduce_add between two GPUs of one process, and the DataParallel wrapper."""
    import torch_musa_b200 as bw
    from torch_musa_b200.parallel import data_parallel as dp

    _need(2)
    d0, d1 = torch.device("blackwell", 0), torch.device("blackwell", 1)
    x = torch.arange(24, dtype=torch.float32).view(6, 4)
    copies = dp.broadcast(x.to(d0), [0, 1])
    assert [c.device.index for c in copies] == [0, 1] and all(torch.equal(c.cpu(), x) for c in copies)
    parts = dp.scatter(x.to(d0), [0, 1])
    assert parts[1].device.index == 1 and torch.equal(parts[1].cpu(), x[3:])
    assert torch.equal(dp.gather(parts, 0, destination=0).cpu(), x)
    assert torch.equal(dp.reduce_add([x.to(d0), (2 * x).to(d1)], destination=1).cpu(), 3 * x)
    torch.manual_seed(0)
    m = torch.nn.Linear(4, 3)
    wrapped = dp.DataParallel(torch.nn.Linear(4, 3).to(d0), device_ids=[0, 1])
    wrapped.module.load_state_dict(m.state_dict())
    out = wrapped(x.to(d0))
    assert out.device.index == 0 and torch.allclose(out.cpu(), m(x), atol=1e-5)
    bw.synchronize()


def _tp_decode_graph_body(rank, world):
    import copy
    import torch.distributed as dist
    import torch_musa_b200 as bw
    from torch_musa_b200.models import Llama, llama_tiny_config
    from torch_musa_b200.models.decode import LlamaDecoder, shard_for_tensor_parallel

    dev = torch.device("blackwell", rank)
    cfg = llama_tiny_config(fused_qkv=False, fused_gate_up=False, n_heads=8, n_kv_heads=4, dim=1024, ffn_dim=1024)
    torch.manual_seed(0)
    full = Llama(cfg).eval()
    prompt = torch.randint(0, cfg.vocab_size, (4, 9))
    shard = shard_for_tensor_parallel(copy.deepcopy(full), rank, world).to(dev)
    eager = LlamaDecoder(shard, 4, 64, device=dev, tp_group=dist.group.WORLD)
    eager.prefill(prompt.to(dev))
    want = eager.decode(8).cpu()
    graphed = LlamaDecoder(shard, 4, 64, device=dev, tp_group=dist.group.WORLD)
    graphed.prefill(prompt.to(dev))
    graphed.capture()                     # the all-reduces of the step are recorded into the graph
    got = graphed.decode(8).cpu()
    bw.synchronize()
    assert torch.equal(got, want)
    single = LlamaDecoder(copy.deepcopy(full).to(dev), 4, 64, device=dev)
    single.prefill(prompt.to(dev))
    ref = single.decode(8).cpu()
    assert (got == ref).float().mean() > 0.9          # fp32 sums in a different order: ties aside, the same tokens
    x = torch.ones(8, device=dev)
    dist.all_reduce(x)                                # the group still works eagerly after the capture
    assert float(x[0]) == world


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_decode_captured_in_a_graph(world):
    _need(world)
    run_ranks(_tp_decode_graph_body, world, "bccl")
