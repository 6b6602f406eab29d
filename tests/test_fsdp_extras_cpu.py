"""Sharded training utilities on CPU ranks (gloo): the sharded gradient scaler, distributed checkpointing of a
``fully_shard`` model with the fused engine's optimizer, HSDP meshes (which keep torch's collectives) and a
two-stage pipeline over send/recv.
Parity: reference torch_musa/distributed/fsdp/sharded_grad_scaler.py, tests/unittest/distributed/fsdp/fsdp_v2/
test_fully_shard_dcp.py, tests/unittest/distributed/test_dist.py (send/recv)."""
import copy
import os
import tempfile

import pytest
import torch

from _dist_utils import run_ranks
from test_fsdp_cpu import _Net, _shard


def _scaler_body(rank, world):
    import torch.distributed as dist
    from torch.distributed.fsdp import MixedPrecisionPolicy
    from torch_musa_b200.parallel import ShardedGradScaler

    torch.manual_seed(0)
    model = _shard(_Net(), MixedPrecisionPolicy())
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    scaler = ShardedGradScaler(device="cpu", init_scale=1024.0, growth_interval=2)
    before = [p._local_tensor.clone() for p in model.parameters()]
    x = torch.randn(4, 16)
    # step 1: finite gradients -> parameters move, gradients were unscaled
    scaler.scale(model(x).sum()).backward()
    scaler.unscale_(opt)
    ref = _shard(_Net(), MixedPrecisionPolicy())   # same seed? no: rebuild with the same weights below
    scaler.step(opt)
    scaler.update()
    assert scaler.get_scale() == 1024.0
    assert any(not torch.equal(a, p._local_tensor) for a, p in zip(before, model.parameters()))
    opt.zero_grad()
    # step 2: finite again -> growth interval reached, scale doubles
    scaler.scale(model(x).sum()).backward()
    scaler.step(opt)
    scaler.update()
    assert scaler.get_scale() == 2048.0
    opt.zero_grad()
    # step 3: ONE rank sees an overflow in ONE shard -> every rank skips the step and backs off
    scaler.scale(model(x).sum()).backward()
    if rank == 1:
        next(p for p in model.parameters() if p.grad._local_tensor.numel())
        for p in model.parameters():
            if p.grad._local_tensor.numel():
                p.grad._local_tensor.view(-1)[0] = float("inf")
                break
    snap = [p._local_tensor.clone() for p in model.parameters()]
    scaler.step(opt)
    scaler.update()
    assert scaler.get_scale() == 1024.0
    for a, p in zip(snap, model.parameters()):
        assert torch.equal(a, p._local_tensor), "a rank stepped although another rank overflowed"
    sd = scaler.state_dict()
    other = ShardedGradScaler(device="cpu")
    other.load_state_dict(sd)
    assert other.get_scale() == 1024.0 and other.get_growth_interval() == 2


def test_sharded_grad_scaler_agrees_across_ranks():
    run_ranks(_scaler_body, 2, "gloo")


def _dcp_body(rank, world, path):
    import torch.distributed as dist
    from torch.distributed.fsdp import MixedPrecisionPolicy
    from torch_musa_b200.distributed import checkpoint as ckpt
    from torch_musa_b200.parallel import fsdp as bw_fsdp

    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    torch.manual_seed(0)
    base = _Net()
    a = _shard(copy.deepcopy(base), MixedPrecisionPolicy())
    eng_a = bw_fsdp.install_fused_collectives(a, fused_adamw=hp, emulate=True)
    g = torch.Generator().manual_seed(5 + rank)
    xs = [torch.randn(8, 16, generator=g) for _ in range(4)]
    for x in xs[:2]:
        a(x).sum().backward()
        eng_a.optimizer.step()
    ckpt.save(ckpt.sharded_state(a, eng_a.optimizer), path)
    dist.barrier()
    # a fresh model (different weights) resumes from the checkpoint and must continue identically
    torch.manual_seed(123)
    b = _shard(_Net(), MixedPrecisionPolicy())
    eng_b = bw_fsdp.install_fused_collectives(b, fused_adamw=hp, emulate=True)
    state = ckpt.sharded_state(b, eng_b.optimizer)
    ckpt.load(state, path)
    b.load_state_dict(state["model"])
    ckpt.restore_optimizer(eng_b.optimizer, state["optim"])
    assert eng_b.t == 2
    for x in xs[2:]:
        for m, e in ((a, eng_a), (b, eng_b)):
            m(x).sum().backward()
            e.optimizer.step()
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        assert torch.allclose(p._local_tensor, q._local_tensor, atol=1e-6), n


def test_dcp_round_trip_with_fused_optimizer():
    with tempfile.TemporaryDirectory() as d:
        run_ranks(_dcp_body, 2, "gloo", args=(os.path.join(d, "ckpt"),))


def _hsdp_body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    from torch_musa_b200.parallel import fsdp as bw_fsdp

    torch.manual_seed(0)
    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("replicate", "shard"))
    model = _Net()
    for l in model.layers:
        fully_shard(l, mesh=mesh)
    fully_shard(model, mesh=mesh)
    with pytest.raises(ValueError, match="no group is covered"):
        bw_fsdp.install_fused_collectives(model, emulate=True)      # HSDP keeps torch's collectives
    ref = _Net()
    torch.manual_seed(0)
    ref = _Net()
    x = torch.randn(8, 16)
    model(x).sum().backward()
    ref(x).sum().backward()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p.grad.full_tensor(), q.grad, atol=1e-5)


def test_hsdp_mesh_runs_on_stock_collectives():
    run_ranks(_hsdp_body, 4, "gloo")


def _pipeline_body(rank, world):
    """Two stages, two micro-batches, activations and gradients over send / recv."""
    import torch.distributed as dist

    torch.manual_seed(0)
    full = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
    ref = copy.deepcopy(full)
    stage = full[:2] if rank == 0 else full[2:]
    xs = [torch.randn(3, 8, generator=torch.Generator().manual_seed(i)) for i in range(2)]
    if rank == 0:
        acts = []
        for x in xs:
            a = stage(x)
            dist.send(a.detach(), dst=1)
            acts.append(a)
        for a in acts:
            g = torch.empty_like(a)
            dist.recv(g, src=1)
            a.backward(g)
    else:
        # all forwards, then all backwards (the order in which stage 0 sends and receives)
        acts = []
        for _ in xs:
            a = torch.empty(3, 16)
            dist.recv(a, src=0)
            acts.append(a.requires_grad_())
        for a in acts:
            stage(a).sum().backward()
            dist.send(a.grad, dst=0)
    for x in xs:
        ref(x).sum().backward()
    mine = list(stage.parameters())
    theirs = list(ref[:2].parameters()) if rank == 0 else list(ref[2:].parameters())
    for p, q in zip(mine, theirs):
        assert torch.allclose(p.grad, q.grad, atol=1e-6)


def test_two_stage_pipeline_over_send_recv():
    run_ranks(_pipeline_body, 2, "gloo")


def _fsdp_suite_body(rank, world):
    import copy

    import torch
    import torch.distributed as dist
    from torch.distributed.fsdp import fully_shard
    from torch_musa_b200.testing.distributed import FSDPTest

    seen = []

    def one(lr, hybrid):
        torch.manual_seed(0)
        ref = torch.nn.Sequential(torch.nn.Linear(12, 20), torch.nn.ReLU(), torch.nn.Linear(20, 6))
        model = copy.deepcopy(ref)
        mesh = FSDPTest.device_mesh_plan(hybrid_shard=hybrid)
        for layer in model:
            fully_shard(layer, mesh=mesh)
        fully_shard(model, mesh=mesh)
        torch.manual_seed(100 + rank)
        x = torch.randn(4, 12)
        for m in (ref, model):
            m(x).pow(2).mean().backward()
        for p in ref.parameters():                       # what data parallelism averages
            dist.all_reduce(p.grad)
            p.grad /= world
        FSDPTest.check_sharded_parity(ref, model, atol=1e-5)
        seen.append((lr, hybrid))

    FSDPTest.run_subtests({"lr": [0.1], "hybrid": [False, True]}, one)
    assert seen == [(0.1, False), (0.1, True)]
    # a failing combination is reported with its parameters
    try:
        FSDPTest.run_subtests({"k": [1]}, lambda k: (_ for _ in ()).throw(ValueError("boom")))
    except AssertionError as e:
        assert "{'k': 1}" in str(e) and "boom" in str(e)
    else:
        raise AssertionError("run_subtests swallowed a failure")


def test_fsdp_suite_helpers_on_cpu_ranks():
    from torch_musa_b200.testing.distributed import FSDPTest

    class Suite(FSDPTest):
        world_size = 4

    Suite().run_on_ranks(_fsdp_suite_body)


def _pipeline_schedule_body(rank, world, schedule):
    import torch
    import torch.nn.functional as F
    from torch_musa_b200.parallel.pipeline import PipelineStage, split_into_stages

    torch.manual_seed(0)
    layers = [torch.nn.Linear(16, 16) if i % 2 == 0 else torch.nn.Tanh() for i in range(9)] + [torch.nn.Linear(16, 5)]
    full = torch.nn.Sequential(*layers)
    stages = split_into_stages(layers, world)           # the same modules: stage r trains its slice in place
    n_micro = 5
    xs = [torch.randn(3, 16) for _ in range(n_micro)]
    ys = [torch.randint(0, 5, (3,)) for _ in range(n_micro)]
    # single-process oracle on a copy
    import copy

    ref = copy.deepcopy(full)
    ref_loss = sum(F.cross_entropy(ref(x), y) for x, y in zip(xs, ys)) / n_micro
    ref_loss.backward()
    stage = PipelineStage(stages[rank], rank, world)
    for _ in range(2):                                   # the second round reuses the announced shapes
        for p in stages[rank].parameters():
            p.grad = None
        loss = stage.run(schedule, micro_inputs=xs if stage.is_first else None, micro_targets=ys if stage.is_last else None,
                         loss_fn=F.cross_entropy, n_micro=n_micro)
        if stage.is_last:
            assert abs(float(loss) - float(ref_loss)) < 1e-5
        else:
            assert loss is None
        mine = dict(stages[rank].named_parameters())
        offset = sum(len(s) for s in stages[:rank])
        for name, p in mine.items():
            idx, leaf = name.split(".", 1)
            want = dict(ref.named_parameters())[f"{offset + int(idx)}.{leaf}"].grad
            assert torch.allclose(p.grad, want, atol=1e-6), name


def test_pipeline_schedules_match_single_process():
    import pytest as _pytest

    for schedule, world in (("gpipe", 2), ("1f1b", 4)):
        run_ranks(_pipeline_schedule_body, world, "gloo", args=(schedule,))
    from torch_musa_b200.parallel.pipeline import split_into_stages

    with _pytest.raises(ValueError):
        split_into_stages([torch.nn.ReLU()], 2)


def _sharded_scaler_body(rank, world):
    """A non-finite gradient on ONE rank skips the step on EVERY rank (and only the scale changes)."""
    from torch_musa_b200.parallel.zero import ShardedFusedAdamW

    torch.manual_seed(0)
    ps = [torch.nn.Parameter((torch.randn(64, 8) * 0.1).to(torch.bfloat16)), torch.nn.Parameter(torch.zeros(8, dtype=torch.bfloat16))]
    opt = ShardedFusedAdamW(ps, lr=1e-2, bucket_mb=1)
    scaler = torch.amp.GradScaler("cpu", init_scale=64.0, growth_interval=100)
    before = [p.detach().clone() for p in ps]
    for p in ps:
        p.grad.fill_(0.5 * 64.0)
    if rank == 1:
        ps[0].grad[3, 3] = float("nan")
    assert opt.step_with_scaler(scaler) is False and scaler.get_scale() == 32.0
    assert all(torch.equal(a, b) for a, b in zip(before, ps))
    opt.zero_grad()
    for p in ps:
        p.grad.fill_(0.5 * 32.0)
    assert opt.step_with_scaler(scaler) is True
    assert all(not torch.equal(a, b) for a, b in zip(before, ps))
    # every rank holds the same updated parameters
    flat = torch.cat([p.detach().float().reshape(-1) for p in ps])
    ref = flat.clone()
    torch.distributed.broadcast(ref, src=0)
    assert torch.equal(flat, ref)


def test_sharded_adamw_loss_scaling_skips_on_every_rank():
    run_ranks(_sharded_scaler_body, 2, "gloo")
