"""Host-side distributed logic on CPU ranks (gloo, world_size 2): DDP plumbing with the package's
communication hook (gradients equal a single-process run of the combined batch), the
vocabulary-parallel cross entropy, and failure detection driven from the host."""
import pytest
import torch

from _dist_utils import run_ranks


def _mlp():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(784, 1024), torch.nn.ReLU(), torch.nn.Linear(1024, 10))


def _data(rank):
    g = torch.Generator().manual_seed(0 + rank)
    return torch.randn(64, 784, generator=g), torch.randint(0, 10, (64,), generator=g)


def _ddp_body(rank, world):
    import torch.distributed as dist
    from torch_musa_b200.parallel import wrap_ddp

    model = _mlp()
    ddp = wrap_ddp(model)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.01, momentum=0.9)
    # single-process oracle on the concatenated batch
    ref = _mlp()
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.01, momentum=0.9)
    xs, ys = zip(*[_data(r) for r in range(world)])
    X, Y = torch.cat(xs), torch.cat(ys)
    x, y = _data(rank)
    for step in range(10):
        opt.zero_grad()
        torch.nn.functional.cross_entropy(ddp(x), y).backward()
        ref_opt.zero_grad()
        torch.nn.functional.cross_entropy(ref(X), Y).backward()
        for p, q in zip(model.parameters(), ref.parameters()):
            assert (p.grad - q.grad).abs().max() <= 1e-5, (step, (p.grad - q.grad).abs().max())
        opt.step()
        ref_opt.step()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=1e-5)


def test_ddp_gloo_matches_single_process():
    run_ranks(_ddp_body, 2, "gloo")


def _vp_ce_body(rank, world):
    from torch_musa_b200.parallel import parallel_fused_cross_entropy

    torch.manual_seed(1)
    T, V = 37, 64
    logits = torch.randn(T, V)
    target = torch.randint(0, V, (T,))
    target[::5] = -100
    shard = logits[:, rank * (V // world):(rank + 1) * (V // world)].clone().requires_grad_()
    loss = parallel_fused_cross_entropy(shard, target)
    loss.backward()
    full = logits.clone().requires_grad_()
    ref = torch.nn.functional.cross_entropy(full, target)
    ref.backward()
    assert abs(float(loss) - float(ref)) < 1e-5
    assert torch.allclose(shard.grad, full.grad[:, rank * (V // world):(rank + 1) * (V // world)], atol=1e-6)


def test_vocab_parallel_cross_entropy_gloo():
    run_ranks(_vp_ce_body, 2, "gloo")


def _failing_rank_body(rank, world):
    """A rank that raises before joining a collective must surface as an error on the others
    (short process-group timeout), not as a hang."""
    import datetime
    import torch.distributed as dist

    pg = dist.new_group(ranks=list(range(world)), backend="gloo", timeout=datetime.timedelta(seconds=3))
    t = torch.ones(4)
    dist.all_reduce(t, group=pg)  # healthy round
    assert float(t[0]) == world
    if rank == 1:
        return  # leaves between steps without joining the next collective
    with pytest.raises(Exception):
        dist.all_reduce(t, group=pg)


def test_missing_rank_is_detected_gloo():
    run_ranks(_failing_rank_body, 2, "gloo", timeout=120)
