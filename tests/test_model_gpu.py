"""End-to-end: a small Llama trains on the device and tracks the CPU fp32 run; graphs replay."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_llama_loss_parity_and_training(bw, dev):
    from torch_musa_b200.models import Llama, llama_tiny_config

    torch.manual_seed(0)
    cfg = llama_tiny_config()
    ref = Llama(cfg)
    ref.reset_parameters(seed=1)
    model = Llama(cfg)
    model.load_state_dict(ref.state_dict())
    model = model.to(dev).to(torch.bfloat16)
    tok = torch.randint(0, cfg.vocab_size, (4, 64))
    l_ref = ref(tok, tok)
    bw.reset_kernel_launch_count()
    l_dev = model(tok.to(dev), tok.to(dev))
    assert abs(float(l_dev) - float(l_ref)) < 0.05, (float(l_dev), float(l_ref))
    l_ref.backward()
    l_dev.backward()
    assert bw.kernel_launch_count() > 30
    gr = ref.layers[0].ffn.w2.weight.grad
    gd = model.layers[0].ffn.w2.weight.grad.float().cpu()
    cos = torch.nn.functional.cosine_similarity(gr.flatten(), gd.flatten(), dim=0)
    assert cos > 0.99, float(cos)
    opt = bw.optim.FusedAdamW(model.parameters(), lr=3e-3)
    losses = []
    for _ in range(8):
        opt.zero_grad(set_to_none=True)
        loss = model(tok.to(dev), tok.to(dev))
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0] - 0.5, losses


def test_graph_capture_replay(bw, dev):
    lin = torch.nn.Linear(256, 256).to(dev).to(torch.bfloat16)
    static_x = torch.randn(64, 256, device=dev, dtype=torch.bfloat16)
    s = bw.Stream()
    s.wait_stream(bw.current_stream())
    with bw.stream(s):
        for _ in range(2):
            lin(static_x)
    bw.current_stream().wait_stream(s)
    g = bw.BlackwellGraph()
    with bw.graph(g):
        static_y = torch.nn.functional.silu(lin(static_x))
    for _ in range(3):
        x = torch.randn(64, 256, device=dev, dtype=torch.bfloat16)
        static_x.copy_(x)
        g.replay()
        bw.synchronize()
        ref = torch.nn.functional.silu(lin(x))
        assert torch.allclose(static_y.float().cpu(), ref.float().cpu(), atol=1e-2, rtol=1e-2)
    pool = g.pool()
    assert isinstance(pool, tuple) and len(pool) == 2
    g.reset()
    # a graph that kept its captured graph can be instantiated again (what a profiler attached later needs)
    k = bw.BlackwellGraph(keep_graph=True)
    with bw.graph(k):
        static_z = lin(static_x) * 2
    assert bw.update_graph_with_profile() >= 1
    k.replay()
    bw.synchronize()
    assert torch.allclose(static_z.float().cpu(), (lin(static_x) * 2).float().cpu(), atol=1e-2, rtol=1e-2)


def test_graph_rng_advances(bw, dev):
    x = torch.ones(4096, device=dev)
    g = bw.BlackwellGraph()
    with bw.graph(g):
        y = torch.nn.functional.dropout(x, 0.5, training=True)
    g.replay(); bw.synchronize(); a = y.clone()
    g.replay(); bw.synchronize(); b = y.clone()
    assert not torch.equal(a.cpu(), b.cpu()), "replays must draw fresh random numbers"


def test_graph_captured_decode_matches_eager_and_cpu(bw, dev):
    """KV-cache decode: the graph replay produces the tokens of the eager step loop, and (in fp32) of a full
    recomputation on the CPU."""
    from torch_musa_b200.models import Llama, llama_tiny_config
    from torch_musa_b200.models.decode import LlamaDecoder

    cfg = llama_tiny_config(n_kv_heads=2)
    torch.manual_seed(0)
    ref_model = Llama(cfg).eval()
    prompt = torch.randint(0, cfg.vocab_size, (4, 7))
    seq, want = prompt.clone(), []
    with torch.no_grad():
        for _ in range(8):
            nxt = ref_model(seq)[:, -1].argmax(-1, keepdim=True)
            want.append(nxt)
            seq = torch.cat([seq, nxt], 1)
    want = torch.cat(want, 1)
    import copy

    model = copy.deepcopy(ref_model).to(dev)
    eager = LlamaDecoder(model, 4, 64, device=dev)
    eager.prefill(prompt.to(dev))
    got_eager = eager.decode(8).cpu()
    graphed = LlamaDecoder(model, 4, 64, device=dev)
    graphed.prefill(prompt.to(dev))
    graphed.capture()
    got_graph = graphed.decode(8).cpu()
    assert torch.equal(got_graph, got_eager)
    assert (got_eager == want).float().mean() > 0.9      # fp32 on both sides: ties aside, the same tokens
