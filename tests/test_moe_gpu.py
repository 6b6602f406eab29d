"""Expert-parallel token exchange: the fused peer-memory kernels against the sort + all_to_all reference,
single device (all experts local) and across two GPUs."""
import pytest
import torch

from _dist_utils import run_ranks

pytestmark = pytest.mark.gpu


def _roundtrip(dev, ex_fused, ex_ref, T=96, d=64, E=4, K=2, seed=0):
    """dispatch -> per-expert scaling -> combine, forward values and all gradients, fused vs reference."""
    g = torch.Generator().manual_seed(seed)
    x0 = torch.randn(T, d, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    top, idx = torch.topk(logits, K, dim=-1)
    gates0 = torch.softmax(top, -1)
    scale = torch.arange(1, E + 1, dtype=torch.float32)           # expert e multiplies its rows by (e + 1)
    outs = []
    for ex in (ex_fused, ex_ref):
        x = x0.to(dev).requires_grad_()
        gates = gates0.to(dev).requires_grad_()
        recv, rows, ctx = ex.dispatch(x, idx.to(dev), 0)
        if isinstance(rows, torch.Tensor):         # counts left on the device: the whole receive buffer comes back
            rows = rows.tolist()
            recv = recv[:sum(rows)]
        assert recv.shape[0] == sum(rows)
        e0 = ex.rank * ex.E_local
        per_row = torch.repeat_interleave(scale[e0:e0 + ex.E_local].to(dev), torch.tensor(rows, device=dev))
        y = (recv.float() * per_row.unsqueeze(1)).to(torch.bfloat16)
        out = ex.combine(y, gates, ctx, 0)
        (out.float() * torch.linspace(0.5, 1.5, d, device=dev)).sum().backward()
        outs.append((out.detach().float().cpu(), x.grad.float().cpu(), gates.grad.float().cpu(), sorted(rows)))
    (o1, gx1, gg1, r1), (o2, gx2, gg2, r2) = outs
    assert r1 == r2
    assert torch.allclose(o1, o2, atol=3e-2, rtol=3e-2), (o1 - o2).abs().max()
    assert torch.allclose(gx1, gx2, atol=6e-2, rtol=3e-2), (gx1 - gx2).abs().max()
    assert torch.allclose(gg1, gg2, atol=0.5, rtol=3e-2), (gg1 - gg2).abs().max()
    # closed form as well: out[t] = sum_k gate * (idx + 1) * x[t]
    ref = (x0.float().unsqueeze(1) * (gates0 * (idx + 1).float()).unsqueeze(-1)).sum(1)
    assert torch.allclose(o1, ref, atol=5e-2, rtol=3e-2)


def test_fused_exchange_single_device(bw, dev):
    from torch_musa_b200.parallel.moe import FusedExpertExchange, ReferenceExpertExchange

    fused = FusedExpertExchange(4, 64, cap_rows=96 * 2, slots=1, device=dev)
    _roundtrip(dev, fused, ReferenceExpertExchange(4))
    fused.check()


def test_moe_model_step_matches_reference(bw, dev):
    from torch_musa_b200.models import MoETransformer, moe_tiny_config
    from torch_musa_b200.parallel.moe import make_expert_exchange, ReferenceExpertExchange

    cfg = moe_tiny_config()
    torch.manual_seed(0)
    model = MoETransformer(cfg).to(dev).to(torch.bfloat16)
    tok = torch.randint(0, cfg.vocab_size, (2, 33)).to(dev)
    losses = []
    for ex in (make_expert_exchange(cfg.n_experts, cfg.dim, 2 * 32, cfg.top_k, slots=cfg.n_layers, device=dev),
               ReferenceExpertExchange(cfg.n_experts)):
        model.zero_grad()
        model.set_exchange(ex)
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        losses.append((float(loss), model.layers[0].moe.experts.w13.grad.float().norm().item(),
                       model.layers[0].moe.router.weight.grad.float().norm().item()))
    (l1, a1, b1), (l2, a2, b2) = losses
    assert abs(l1 - l2) < 2e-2 and abs(a1 - a2) / max(a2, 1e-6) < 5e-2 and abs(b1 - b2) / max(b2, 1e-6) < 0.1


def _multi_rank_body(rank, world):
    import torch_musa_b200 as bw
    from torch_musa_b200.parallel.moe import FusedExpertExchange, ReferenceExpertExchange

    dev = torch.device("blackwell", rank)
    E = 8                                       # divisible by every world size tested
    fused = FusedExpertExchange(E, 64, cap_rows=world * 2 * 96, slots=1, device=dev)
    _roundtrip(dev, fused, ReferenceExpertExchange(E), E=E, seed=rank)
    _roundtrip(dev, fused, ReferenceExpertExchange(E), E=E, T=64 + 8 * rank, seed=10 + rank)   # uneven token counts
    bw.synchronize()
    fused.check()


@pytest.mark.multigpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_exchange_multi_gpu(bw, world):
    if bw.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    # plain peer loads/stores only (no NVLS) so that a failing rank cannot disturb its peers' GPUs
    run_ranks(_multi_rank_body, world, "bccl", env={"NCCL_NVLS_ENABLE": "0"})
