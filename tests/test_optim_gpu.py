"""Fused optimizers / AMP kernels against torch's reference optimizers on the CPU, step by step
(reference tests/unittest/optim/test_fused_adamw.py:52-227 strategy)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def make_params(dt, seed=0):
    g = torch.Generator().manual_seed(seed)
    shapes = [(1,), (17,), (128, 33), (300, 257), (70000,), (512, 1024)]
    return [torch.randn(*s, generator=g).to(dt) for s in shapes]


def run_pair(bw, dev, make_dev_opt, make_ref_opt, dt, steps=4, tol=None):
    ps = make_params(dt)
    dev_p = [p.to(dev).detach().clone().requires_grad_() for p in ps]
    ref_p = [p.float().detach().clone().requires_grad_() for p in ps]
    od, orf = make_dev_opt(dev_p), make_ref_opt(ref_p)
    g = torch.Generator().manual_seed(1)
    for _ in range(steps):
        for a, b in zip(dev_p, ref_p):
            gr = torch.randn(b.shape, generator=g).to(dt)
            a.grad = gr.to(dev)
            b.grad = gr.float()
        od.step()
        orf.step()
    atol, rtol = tol or ((1e-5, 1e-5) if dt == torch.float32 else (3e-2, 3e-2))
    for a, b in zip(dev_p, ref_p):
        assert torch.allclose(a.detach().float().cpu(), b.detach(), atol=atol, rtol=rtol), (
            a.shape, (a.detach().float().cpu() - b.detach()).abs().max())


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("amsgrad", [False, True])
@pytest.mark.parametrize("wd", [0.0, 0.1])
def test_fused_adamw(bw, dev, dt, amsgrad, wd):
    bw.reset_kernel_launch_count()
    run_pair(bw, dev, lambda p: bw.optim.FusedAdamW(p, lr=1e-2, weight_decay=wd, amsgrad=amsgrad),
             lambda p: torch.optim.AdamW(p, lr=1e-2, weight_decay=wd, amsgrad=amsgrad), dt)
    assert bw.kernel_launch_count() >= 4


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_fused_adam(bw, dev, dt):
    run_pair(bw, dev, lambda p: bw.optim.FusedAdam(p, lr=1e-2, weight_decay=0.05),
             lambda p: torch.optim.Adam(p, lr=1e-2, weight_decay=0.05), dt)


def test_torch_adamw_fused_flag_and_tensor_lr(bw, dev):
    run_pair(bw, dev, lambda p: torch.optim.AdamW(p, lr=torch.tensor(1e-2), fused=True),
             lambda p: torch.optim.AdamW(p, lr=1e-2), torch.float32)


@pytest.mark.parametrize("momentum,nesterov,wd", [(0.0, False, 0.0), (0.9, False, 1e-4), (0.9, True, 1e-4)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_fused_sgd(bw, dev, dt, momentum, nesterov, wd):
    run_pair(bw, dev, lambda p: bw.optim.FusedSGD(p, lr=0.05, momentum=momentum, nesterov=nesterov, weight_decay=wd),
             lambda p: torch.optim.SGD(p, lr=0.05, momentum=momentum, nesterov=nesterov, weight_decay=wd), dt,
             tol=None if dt == torch.float32 else (6e-2, 6e-2))


def test_fused_lamb_matches_reference(bw, dev):
    ps = make_params(torch.float32)
    dev_p = [p.to(dev).detach().clone().requires_grad_() for p in ps]
    ref_p = [p.clone().requires_grad_() for p in ps]
    od = bw.optim.FusedLAMB(dev_p, lr=1e-2, weight_decay=0.01)
    orf = bw.optim.FusedLAMB(ref_p, lr=1e-2, weight_decay=0.01)  # CPU path = plain PyTorch formulation
    g = torch.Generator().manual_seed(3)
    for _ in range(3):
        for a, b in zip(dev_p, ref_p):
            gr = torch.randn(b.shape, generator=g)
            a.grad, b.grad = gr.to(dev), gr.clone()
        od.step()
        orf.step()
    for a, b in zip(dev_p, ref_p):
        assert torch.allclose(a.detach().cpu(), b.detach(), atol=1e-5, rtol=1e-4)


def test_state_dict_roundtrip(bw, dev):
    p = [torch.randn(64, 64, device=dev, requires_grad=True)]
    o = bw.optim.FusedAdamW(p, lr=1e-3)
    p[0].grad = torch.randn(64, 64, device=dev)
    o.step()
    sd = copy.deepcopy(o.state_dict())
    o2 = bw.optim.FusedAdamW(p, lr=1e-3)
    o2.load_state_dict(sd)
    assert float(o2.state[p[0]]["step"]) == 1.0
    assert o2.state[p[0]]["exp_avg"].device.type == "blackwell"


def test_grad_scaler_and_clip(bw, dev):
    model = torch.nn.Linear(32, 32).to(dev)
    opt = bw.optim.FusedAdamW(model.parameters(), lr=1e-3)
    scaler = bw.amp.GradScaler(init_scale=1024.0, growth_interval=2)
    w0 = model.weight.detach().clone()
    for i in range(3):
        opt.zero_grad()
        with bw.amp.autocast(dtype=torch.bfloat16):
            loss = model(torch.randn(8, 32, device=dev)).float().pow(2).mean()
        scaler.scale(loss).backward()
        if i == 1:
            model.weight.grad[0, 0] = float("inf")  # this step must be skipped and the scale backed off
        scaler.unscale_(opt)
        bw.optim.clip_grad_norm_(model.parameters(), 1.0)
        before = model.weight.detach().clone()
        scaler.step(opt)
        scaler.update()
        if i == 1:
            assert torch.equal(before.cpu(), model.weight.detach().cpu())
            assert scaler.get_scale() == 512.0
    assert not torch.equal(w0.cpu(), model.weight.detach().cpu())


def test_clip_grad_norm(bw, dev):
    ps = [torch.randn(1000, device=dev, requires_grad=True), torch.randn(33, 7, device=dev, requires_grad=True)]
    for p in ps:
        p.grad = torch.randn_like(p) * 10
    ref = torch.stack([p.grad.cpu().norm() for p in ps]).norm()
    total = bw.optim.clip_grad_norm_(ps, 1.0)
    assert float(total) == pytest.approx(float(ref), rel=1e-4)
    new = torch.stack([p.grad.cpu().norm() for p in ps]).norm()
    assert float(new) == pytest.approx(1.0, rel=1e-3)
    # torch's own utility resolves to the device kernels too
    t2 = torch.nn.utils.clip_grad_norm_(ps, 0.5)
    assert float(t2) == pytest.approx(1.0, rel=1e-3)
