"""The fused FSDP2 engine on CPU ranks (gloo, world_size 2) with its emulated kernels: the layouts, the patched
unshard / reduce hooks and the optimizer epilogue must reproduce stock ``fully_shard`` + ``torch.optim.AdamW``
step for step.  (The device kernels behind the same engine are covered by the GPU tests.)
Parity: reference tests/unittest/distributed/fsdp/fsdp_v2/test_fully_shard_training.py:48-90."""
import copy

import pytest
import torch

from _dist_utils import run_ranks


class _Block(torch.nn.Module):
    def __init__(self, d, h):
        super().__init__()
        self.norm = torch.nn.LayerNorm(d)
        self.up = torch.nn.Linear(d, h, bias=False)
        self.down = torch.nn.Linear(h, d, bias=True)

    def forward(self, x):
        return x + self.down(torch.nn.functional.gelu(self.up(self.norm(x))))


class _Net(torch.nn.Module):
    # 37 and 53 do not divide by the world size or by 8: padded shards and unaligned tails are exercised
    def __init__(self, d=37, h=53, layers=3):
        super().__init__()
        self.inp = torch.nn.Linear(16, d)
        self.layers = torch.nn.ModuleList([_Block(d, h) for _ in range(layers)])
        self.out = torch.nn.Linear(d, 5)

    def forward(self, x):
        x = self.inp(x)
        for l in self.layers:
            x = l(x)
        return self.out(x)


def _shard(model, mp):
    from torch.distributed.fsdp import fully_shard

    for l in model.layers:
        fully_shard(l, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    return model


def _body(rank, world, mode, low, device="cpu"):
    import torch.distributed as dist
    from torch.distributed.fsdp import MixedPrecisionPolicy
    from torch_musa_b200.parallel import fsdp as bw_fsdp

    emulate = device == "cpu"
    dev = torch.device(device if emulate else f"{device}:{rank}")
    torch.manual_seed(0)
    base = _Net().to(dev)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32) if low else MixedPrecisionPolicy()
    ref = _shard(copy.deepcopy(base), mp)
    ours = _shard(copy.deepcopy(base), mp)
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref_opt = torch.optim.AdamW(ref.parameters(), **hp)
    if mode == "adamw":
        eng = bw_fsdp.install_fused_collectives(ours, fused_adamw=hp, emulate=emulate)
        opt = eng.optimizer
    else:
        eng = bw_fsdp.install_fused_collectives(ours, emulate=emulate)
        opt = torch.optim.AdamW(ours.parameters(), **hp)
    assert not eng.skipped, eng.skipped
    assert len(eng.groups) == 4
    g = torch.Generator().manual_seed(100 + rank)
    tol = 2e-2 if low else 1e-5
    for step in range(4):
        x = torch.randn(8, 16, generator=g).to(dev)
        y = torch.randn(8, 5, generator=g).to(dev)
        for m in (ref, ours):
            torch.nn.functional.mse_loss(m(x).float(), y).backward()
        if mode != "adamw":
            for p, q in zip(ref.parameters(), ours.parameters()):
                assert torch.allclose(p.grad._local_tensor.cpu(), q.grad._local_tensor.cpu(), atol=tol, rtol=tol), step
        for o in (ref_opt, opt):
            o.step()
            o.zero_grad()
        for (n, p), q in zip(ref.named_parameters(), ours.parameters()):
            a, b = p._local_tensor.cpu(), q._local_tensor.cpu()
            assert torch.allclose(a, b, atol=tol, rtol=tol), (step, n, (a - b).abs().max())
    if world > 1:
        assert eng.calls["gather"] > 0
    assert eng.calls["reduce_adamw" if mode == "adamw" else "reduce"] == 4 * 4
    eng.check()
    if mode == "adamw":
        # optimizer state round trip in torch.optim.AdamW's format
        sd = opt.state_dict()
        ref_sd = ref_opt.state_dict()
        assert set(sd["state"].keys()) == set(ref_sd["state"].keys())
        for i in sd["state"]:
            a, b = sd["state"][i]["exp_avg"]._local_tensor.cpu(), ref_sd["state"][i]["exp_avg"]._local_tensor.cpu()
            assert torch.allclose(a, b, atol=tol, rtol=tol)
            assert float(sd["state"][i]["step"]) == float(ref_sd["state"][i]["step"])
        ref_opt2 = torch.optim.AdamW(ref.parameters(), **hp)
        ref_opt2.load_state_dict(sd)          # the stock optimizer accepts the engine's state
        opt.load_state_dict(ref_sd)           # and the other way round
        assert eng.t == 4


@pytest.mark.parametrize("mode", ["plain", "adamw"])
@pytest.mark.parametrize("low", [False, True])
def test_fused_fsdp_matches_stock_two_ranks(mode, low):
    run_ranks(_body, 2, "gloo", args=(mode, low))


def test_fused_fsdp_single_rank_aliases_shadow():
    run_ranks(_body, 1, "gloo", args=("adamw", False))


def test_fused_fsdp_matches_stock_eight_ranks():
    """The engine's layouts at the largest world size of one node (shards of 1/8, padded tails, eight staging slots)."""
    run_ranks(_body, 8, "gloo", args=("adamw", True))
