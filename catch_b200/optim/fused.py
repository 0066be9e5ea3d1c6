"""Fused multi-tensor SGD-momentum and AdamW.

One kernel launch updates up to 48 parameter tensors (fp32 master weights and
state, any floating gradient dtype).  The per-parameter state uses the same
keys as ``torch.optim.SGD`` / ``torch.optim.AdamW`` (``momentum_buffer``,
``exp_avg``, ``exp_avg_sq``, ``step``) so ``state_dict()`` stays interchangeable
with the stock optimizers.  The reference has no fused optimizer; stock
``torch.optim`` issues many small element-wise launches per parameter.
"""
from __future__ import annotations

from typing import Iterable

import torch
from torch.optim import Optimizer


def _grad_like(p: torch.Tensor) -> torch.Tensor:
    """The gradient of ``p`` laid out in memory exactly like ``p`` (the kernels are element-wise)."""
    g = p.grad
    if g.stride() == p.stride():
        return g
    return torch.empty_like(p, dtype=g.dtype).copy_(g)


def _group_by_device_dtype(params, grads, *states):
    buckets = {}
    for i, (p, g) in enumerate(zip(params, grads)):
        key = (p.device, g.dtype)
        buckets.setdefault(key, []).append(i)
    for idx in buckets.values():
        yield ([params[i] for i in idx], [grads[i] for i in idx]) + tuple([s[i] for i in idx] for s in states)


class FusedSGD(Optimizer):
    """SGD with momentum / weight decay / Nesterov, one fused kernel per step."""

    def __init__(self, params: Iterable, lr: float = 1e-3, momentum: float = 0.0, dampening: float = 0.0,
                 weight_decay: float = 0.0, nesterov: bool = False, grad_scale: float = 1.0):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        defaults = dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay, nesterov=nesterov,
                        grad_scale=grad_scale)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            fresh, fresh_g, fresh_b = [], [], []
            seen, seen_g, seen_b = [], [], []
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = _grad_like(p)
                st = self.state[p]
                if group["momentum"] != 0 and "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p)
                    fresh.append(p); fresh_g.append(g); fresh_b.append(st["momentum_buffer"])
                else:
                    seen.append(p); seen_g.append(g)
                    if group["momentum"] != 0:
                        seen_b.append(st["momentum_buffer"])
            for first, (ps, gs, bs) in ((True, (fresh, fresh_g, fresh_b)), (False, (seen, seen_g, seen_b))):
                if not ps:
                    continue
                if group["momentum"] != 0:
                    parts = _group_by_device_dtype(ps, gs, bs)
                else:
                    parts = ((a, b, []) for a, b in _group_by_device_dtype(ps, gs))
                for p_, g_, b_ in parts:
                    torch.ops.catch_b200.fused_sgd_step(p_, g_, b_, [], group["lr"], group["momentum"],
                                                        group["dampening"], group["weight_decay"], group["nesterov"],
                                                        first, group["grad_scale"])
        return loss


class FusedAdamW(Optimizer):
    """AdamW (decoupled weight decay), one fused kernel per step."""

    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, grad_scale: float = 1.0, adam_l2_mode: bool = False):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, grad_scale=grad_scale,
                        adam_l2_mode=adam_l2_mode)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            by_step = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "step" not in st:
                    st["step"] = torch.tensor(0.0)
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                st["step"] += 1
                by_step.setdefault(int(st["step"].item()), []).append(p)
            b1, b2 = group["betas"]
            for step, ps in by_step.items():
                gs = [_grad_like(p) for p in ps]
                m1 = [self.state[p]["exp_avg"] for p in ps]
                m2 = [self.state[p]["exp_avg_sq"] for p in ps]
                for p_, g_, a_, v_ in _group_by_device_dtype(ps, gs, m1, m2):
                    torch.ops.catch_b200.fused_adamw_step(p_, g_, a_, v_, [], group["lr"], b1, b2, group["eps"],
                                                          group["weight_decay"], step, group["grad_scale"],
                                                          group["adam_l2_mode"])
        return loss
