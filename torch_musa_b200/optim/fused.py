from __future__ import annotations

from typing import Iterable, List, Optional, Tuple, Union

import torch
from torch.optim.optimizer import Optimizer

from ..ops.functional import multi_tensor_l2norm


class FusedAdamW(torch.optim.AdamW):
    """AdamW whose step is ``aten::_fused_adamw_`` -> the backend's multi-tensor kernel.

    Unlike the reference's FusedAdamW (reference torch_musa/optim/fused_adam.py:497-503, which keeps step
    counters on the CPU and reads ``found_inf`` back every step), counters live on the device and a skipped
    step under a GradScaler is handled inside the kernel."""

    def __init__(self, params, lr: Union[float, torch.Tensor] = 1e-3, betas: Tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 1e-2, amsgrad: bool = False, *, maximize: bool = False,
                 capturable: bool = False):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad,
                         maximize=maximize, capturable=capturable, fused=True)


class FusedAdam(torch.optim.Adam):
    """Adam (L2-regularisation form of weight decay) on the multi-tensor kernel."""

    def __init__(self, params, lr: Union[float, torch.Tensor] = 1e-3, betas: Tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.0, amsgrad: bool = False, *, maximize: bool = False,
                 capturable: bool = False):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad,
                         maximize=maximize, capturable=capturable, fused=True)


class FusedSGD(torch.optim.SGD):
    """SGD (momentum / nesterov / dampening) on the multi-tensor kernel."""

    def __init__(self, params, lr: Union[float, torch.Tensor] = 1e-3, momentum: float = 0.0, dampening: float = 0.0,
                 weight_decay: float = 0.0, nesterov: bool = False, *, maximize: bool = False):
        super().__init__(params, lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                         nesterov=nesterov, maximize=maximize, fused=True)


class FusedLAMB(Optimizer):
    """LAMB: Adam moments + layer-wise trust ratio, in two multi-tensor stages plus two norm passes.

    Arguments follow apex's FusedLAMB (reference torch_musa/optim/fused_lamb.py:12-240)."""

    def __init__(self, params, lr: float = 1e-3, bias_correction: bool = True, betas=(0.9, 0.999), eps: float = 1e-6,
                 weight_decay: float = 0.01, amsgrad: bool = False, adam_w_mode: bool = True,
                 grad_averaging: bool = True, max_grad_norm: float = 1.0, use_nvlamb: bool = False):
        if amsgrad:
            raise RuntimeError("FusedLAMB does not support the AMSGrad variant.")
        defaults = dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps, weight_decay=weight_decay,
                        grad_averaging=grad_averaging, max_grad_norm=max_grad_norm)
        super().__init__(params, defaults)
        self.adam_w_mode = adam_w_mode
        self.use_nvlamb = use_nvlamb

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        all_grads = [p.grad for g in self.param_groups for p in g["params"] if p.grad is not None]
        if not all_grads:
            return loss
        # global gradient norm over every group and dtype
        by_dtype = {}
        for g in all_grads:
            by_dtype.setdefault((g.device, g.dtype), []).append(g)
        norms = [multi_tensor_l2norm(v)[0] for v in by_dtype.values()]
        global_norm = torch.stack([n.reshape(()) for n in norms]).norm(2).reshape(1) if len(norms) > 1 else norms[0]

        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            group["step"] = group.get("step", 0) + 1
            buckets = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("FusedLAMB does not support sparse gradients")
                st = self.state[p]
                if len(st) == 0:
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                b = buckets.setdefault((p.device, p.dtype), ([], [], [], []))
                b[0].append(p); b[1].append(p.grad); b[2].append(st["exp_avg"]); b[3].append(st["exp_avg_sq"])
            for (dev, dt), (ps, gs, ms, vs) in buckets.items():
                if dev.type == "blackwell":
                    torch.ops.blackwell.multi_tensor_lamb_(ps, gs, ms, vs, float(group["lr"]), beta1, beta2,
                                                           group["eps"], group["weight_decay"], group["step"],
                                                           bool(group["bias_correction"]), bool(group["grad_averaging"]),
                                                           self.adam_w_mode, float(group["max_grad_norm"]),
                                                           self.use_nvlamb, global_norm.to(dev))
                else:
                    _lamb_reference(ps, gs, ms, vs, group, self.adam_w_mode, self.use_nvlamb, global_norm)
        return loss


def _lamb_reference(ps, gs, ms, vs, group, adam_w_mode, use_nvlamb, global_norm):
    beta1, beta2 = group["betas"]
    step, eps, wd, lr = group["step"], group["eps"], group["weight_decay"], group["lr"]
    clip = 1.0
    if group["max_grad_norm"] > 0:
        gn = float(global_norm)
        clip = gn / group["max_grad_norm"] if gn > group["max_grad_norm"] else 1.0
    bc1 = 1 - beta1 ** step if group["bias_correction"] else 1.0
    bc2 = 1 - beta2 ** step if group["bias_correction"] else 1.0
    b3 = 1 - beta1 if group["grad_averaging"] else 1.0
    for p, g, m, v in zip(ps, gs, ms, vs):
        gf = g.float() / clip
        pf = p.float()
        if not adam_w_mode:
            gf = gf + wd * pf
        m.copy_((beta1 * m.float() + b3 * gf).to(m.dtype))
        v.copy_((beta2 * v.float() + (1 - beta2) * gf * gf).to(v.dtype))
        upd = (m.float() / bc1) / ((v.float() / bc2).sqrt() + eps)
        if adam_w_mode:
            upd = upd + wd * pf
        ratio = 1.0
        if use_nvlamb or wd != 0:
            pn, un = pf.norm(2), upd.norm(2)
            ratio = float(pn / un) if float(pn) != 0 and float(un) != 0 else 1.0
        p.copy_((pf - lr * ratio * upd).to(p.dtype))


@torch.no_grad()
def clip_grad_norm_(parameters: Iterable[torch.Tensor], max_norm: float, norm_type: float = 2.0,
                    error_if_nonfinite: bool = False) -> torch.Tensor:
    """Gradient clipping whose norm and scaling each take a handful of multi-tensor launches."""
    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]
    grads = [p.grad for p in parameters if p.grad is not None]
    if not grads:
        return torch.tensor(0.0)
    if norm_type != 2.0 or grads[0].device.type != "blackwell":
        return torch.nn.utils.clip_grad_norm_(parameters if not isinstance(parameters, list) else parameters,
                                              max_norm, norm_type, error_if_nonfinite)
    by_dtype = {}
    for g in grads:
        by_dtype.setdefault(g.dtype, []).append(g)
    norms = [multi_tensor_l2norm(v)[0].reshape(()) for v in by_dtype.values()]
    total = torch.stack(norms).norm(2) if len(norms) > 1 else norms[0]
    if error_if_nonfinite and not bool(torch.isfinite(total)):
        raise RuntimeError(f"The total norm of order {norm_type} for gradients is non-finite, so it cannot be clipped.")
    coef = (max_norm / (total + 1e-6)).clamp(max=1.0).to(torch.float32).reshape(1)
    found = torch.zeros(1, dtype=torch.float32, device=grads[0].device)
    for v in by_dtype.values():
        torch.ops.blackwell.multi_tensor_scale_(v, coef, 1.0, found)
    return total
