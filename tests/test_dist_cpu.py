"""Host-side distributed logic on CPU ranks (gloo, world_size 2): DDP plumbing with the package's
communication hook (gradients equal a single-process run of the combined batch), the
vocabulary-parallel cross entropy, and failure detection driven from the host."""
import pytest
import torch

import torch.distributed as dist

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


def _tp_llama_body(rank, world):
    from torch_musa_b200.models.llama import llama_tiny_config
    from torch_musa_b200.models.llama_tp import TPLlama
    cfg = llama_tiny_config(n_kv_heads=2)
    torch.manual_seed(0)
    full = TPLlama(cfg, 1)
    torch.manual_seed(1)
    tok = torch.randint(0, cfg.vocab_size, (2, 33))
    loss_ref = full(tok[:, :-1], tok[:, 1:]); loss_ref.backward()
    tp = TPLlama(cfg, world)
    hd, h, kv = cfg.head_dim, cfg.n_heads, cfg.kv_heads
    def rows(w, n_units, unit):  # take this rank's block of n_units/world units of `unit` rows
        per = n_units // world
        return w[rank * per * unit:(rank + 1) * per * unit]
    with torch.no_grad():
        tp.tok_emb.weight.copy_(full.tok_emb.weight); tp.norm.weight.copy_(full.norm.weight)
        tp.lm_head.weight.copy_(rows(full.lm_head.weight, cfg.vocab_size, 1))
        for a, b in zip(tp.layers, full.layers):
            a.attn_norm.weight.copy_(b.attn_norm.weight); a.ffn_norm.weight.copy_(b.ffn_norm.weight)
            W = b.attn.wqkv.weight
            q, k, v = W[:h * hd], W[h * hd:(h + kv) * hd], W[(h + kv) * hd:]
            a.attn.wqkv.weight.copy_(torch.cat([rows(q, h, hd), rows(k, kv, hd), rows(v, kv, hd)]))
            per = h * hd // world
            a.attn.wo.weight.copy_(b.attn.wo.weight[:, rank * per:(rank + 1) * per])
            W13 = b.ffn.w13.weight; f = cfg.ffn_dim; pf = f // world
            a.ffn.w13.weight.copy_(torch.cat([W13[rank * pf:(rank + 1) * pf], W13[f + rank * pf:f + (rank + 1) * pf]]))
            a.ffn.w2.weight.copy_(b.ffn.w2.weight[:, rank * pf:(rank + 1) * pf])
    loss = tp(tok[:, :-1], tok[:, 1:]); loss.backward()
    for p in tp.replicated_parameters():
        dist.all_reduce(p.grad)
    assert abs(float(loss) - float(loss_ref)) < 1e-4, (float(loss), float(loss_ref))
    assert torch.allclose(tp.tok_emb.weight.grad, full.tok_emb.weight.grad, atol=1e-5)
    per = h * hd // world
    if cfg.n_layers > 0: assert torch.allclose(tp.layers[0].attn.wo.weight.grad, full.layers[0].attn.wo.weight.grad[:, rank * per:(rank + 1) * per], atol=1e-5)
    if cfg.n_layers > 1: assert torch.allclose(tp.layers[1].attn_norm.weight.grad, full.layers[1].attn_norm.weight.grad, atol=1e-5)



def test_tensor_parallel_llama_matches_single_process():
    """TP=2 Llama (column/row-parallel layers, sequence-parallel norms, vocabulary-parallel loss) over gloo:
    loss and gradients equal the unsharded model's."""
    run_ranks(_tp_llama_body, 2, "gloo")


def _moe_ep_body(rank, world):
    from torch_musa_b200.models import MoETransformer, moe_tiny_config
    from torch_musa_b200.parallel.moe import ReferenceExpertExchange

    cfg = moe_tiny_config()
    torch.manual_seed(0)
    full = MoETransformer(cfg, 1)
    full.set_exchange(ReferenceExpertExchange.__new__(ReferenceExpertExchange))
    solo = full.layers[0].moe._exchange[0]
    solo.E, solo.group, solo.rank, solo.world, solo.E_local = cfg.n_experts, None, 0, 1, cfg.n_experts
    ep = MoETransformer(cfg, world)
    ep.set_exchange(ReferenceExpertExchange(cfg.n_experts))
    n_local = cfg.n_experts // world
    with torch.no_grad():
        sd = {k: v for k, v in full.state_dict().items() if "experts" not in k}
        ep.load_state_dict(sd, strict=False)
        for a, b in zip(ep.layers, full.layers):
            a.moe.experts.w13.copy_(b.moe.experts.w13[rank * n_local:(rank + 1) * n_local])
            a.moe.experts.w2.copy_(b.moe.experts.w2[rank * n_local:(rank + 1) * n_local])
    torch.manual_seed(7)
    toks = torch.randint(0, cfg.vocab_size, (world, 2, 17))
    # the unsharded model sees every rank's tokens; each EP rank its own
    loss_ref = sum(full(toks[r][:, :-1], toks[r][:, 1:]) for r in range(world)) / world
    loss_ref.backward()
    loss = ep(toks[rank][:, :-1], toks[rank][:, 1:])
    loss.backward()
    total = loss.detach().clone()
    dist.all_reduce(total)
    assert abs(float(total) / world - float(loss_ref)) < 1e-4
    g = ep.layers[0].moe.experts.w2.grad / world          # expert gradients: summed over source ranks already
    gr = full.layers[0].moe.experts.w2.grad[rank * n_local:(rank + 1) * n_local]
    assert torch.allclose(g, gr, atol=1e-5), (g - gr).abs().max()
    rg = ep.layers[0].moe.router.weight.grad.clone()
    dist.all_reduce(rg)
    assert torch.allclose(rg / world, full.layers[0].moe.router.weight.grad, atol=1e-5)


def test_expert_parallel_moe_matches_single_process():
    """EP=2 MoE decoder with the sort + all_to_all exchange over gloo against the same model with all experts local."""
    run_ranks(_moe_ep_body, 2, "gloo")


def _dtensor_tp_body(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch_musa_b200.models import Llama, llama_tiny_config
    from torch_musa_b200.parallel.dtensor_tp import parallelize_llama

    cfg = llama_tiny_config(fused_qkv=False, fused_gate_up=False, fused_loss=False)
    torch.manual_seed(0)
    full = Llama(cfg)
    full.reset_parameters(seed=3)
    tp = Llama(cfg)
    tp.load_state_dict(full.state_dict())
    mesh = init_device_mesh("cpu", (world,))
    parallelize_llama(tp, mesh, loss_parallel=True)
    torch.manual_seed(11)
    toks = torch.randint(0, cfg.vocab_size, (2, 17))
    loss_ref = full(toks[:, :-1], toks[:, 1:])
    loss_ref.backward()
    loss = tp(toks[:, :-1], toks[:, 1:])
    loss.backward()
    assert abs(float(loss) - float(loss_ref)) < 1e-4, (float(loss), float(loss_ref))
    # column-parallel weight: this rank's rows of the full gradient; sequence-parallel norm: partial sums to reduce
    g = tp.layers[0].attn.wq.weight.grad.to_local()
    rows = g.shape[0]
    assert torch.allclose(g, full.layers[0].attn.wq.weight.grad[rank * rows:(rank + 1) * rows], atol=1e-5)
    g = tp.layers[0].ffn.w2.weight.grad.to_local()
    cols = g.shape[1]
    assert torch.allclose(g, full.layers[0].ffn.w2.weight.grad[:, rank * cols:(rank + 1) * cols], atol=1e-5)
    gn = tp.layers[1].attn_norm.weight.grad.full_tensor()
    assert torch.allclose(gn, full.layers[1].attn_norm.weight.grad, atol=1e-5)
    ge = tp.tok_emb.weight.grad.full_tensor()
    assert torch.allclose(ge, full.tok_emb.weight.grad, atol=1e-5)


def test_dtensor_tensor_parallel_llama_matches_single_process():
    """The DTensor plan (Colwise/Rowwise/SequenceParallel + vocabulary-parallel loss) at TP=2 over gloo."""
    run_ranks(_dtensor_tp_body, 2, "gloo")


def test_custom_op_sharding_rules_are_registered():
    from torch_musa_b200.distributed import tensor_ops
    from torch.distributed.tensor import DTensor

    tensor_ops.register()
    table = DTensor._op_dispatcher.sharding_propagator.op_strategy_funcs
    for name in ("silu_mul", "swiglu", "rope", "rms_norm_residual", "cross_entropy_fwd"):
        assert getattr(torch.ops.blackwell, name).default in table, name


def _tp_decode_body(rank, world):
    import copy
    from torch_musa_b200.models import Llama, llama_tiny_config
    from torch_musa_b200.models.decode import LlamaDecoder, shard_for_tensor_parallel

    cfg = llama_tiny_config(fused_qkv=False, fused_gate_up=False, n_kv_heads=2)
    torch.manual_seed(0)
    full = Llama(cfg).eval()
    prompt = torch.randint(0, cfg.vocab_size, (3, 6))
    single = LlamaDecoder(copy.deepcopy(full), 3, 32)
    single.prefill(prompt)
    want = single.decode(6)
    shard = shard_for_tensor_parallel(copy.deepcopy(full), rank, world)
    assert shard.layers[0].attn.wq.weight.shape[0] == full.layers[0].attn.wq.weight.shape[0] // world
    dec = LlamaDecoder(shard, 3, 32, tp_group=dist.group.WORLD)
    assert dec.k_cache.shape[2] == cfg.kv_heads // world        # each rank caches its own heads only
    dec.prefill(prompt)
    got = dec.decode(6)
    assert torch.equal(got, want), (got, want)


def test_tensor_parallel_decode_matches_single_process():
    """KV-cache decode with heads and cache sharded over 2 ranks produces the tokens of the unsharded decoder."""
    run_ranks(_tp_decode_body, 2, "gloo")
