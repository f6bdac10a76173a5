"""Fused AdamW: one sm_100a kernel launch per parameter tensor updates p, m and v in a single pass
(mixed bf16 / fp32 storage, fp32 math).  Same update rule as the reference's Triton kernel
(opss/kernels/fused_adamw.py:58-93): the decay term uses the pre-update parameter,
``p - lr * (m_hat / (sqrt(v_hat) + eps) + wd * p)``; ``amsgrad`` keeps the running maximum of v (:95-133).
"""
from __future__ import annotations

from typing import Callable, Iterable, Optional

import torch

from ..ops import kernels, reference as ref


class YvFusedAdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, amsgrad: bool = False, state_dtype: Optional[torch.dtype] = None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad))
        self.state_dtype = state_dtype
        self.grad_scale = 1.0

    @torch.no_grad()
    def step(self, closure: Optional[Callable[[], torch.Tensor]] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    dt = self.state_dtype or (torch.float32 if p.dtype == torch.float32 else p.dtype)
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=dt)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=dt)
                    if group["amsgrad"]:
                        st["max_exp_avg_sq"] = torch.zeros_like(p, dtype=dt)
                st["step"] += 1
                if p.is_cuda and not group["amsgrad"] and p.dtype in (torch.bfloat16, torch.float32) \
                        and p.grad.dtype in (torch.bfloat16, torch.float32):
                    kernels().adamw(p.data, p.grad.contiguous(), st["exp_avg"], st["exp_avg_sq"], group["lr"], b1, b2,
                                    group["eps"], group["weight_decay"], st["step"], self.grad_scale)
                elif group["amsgrad"]:
                    g = p.grad.float() * self.grad_scale
                    m, v, vmax = st["exp_avg"], st["exp_avg_sq"], st["max_exp_avg_sq"]
                    m.mul_(b1).add_(g.to(m.dtype), alpha=1 - b1)
                    v.mul_(b2).add_((g * g).to(v.dtype), alpha=1 - b2)
                    torch.maximum(vmax, v, out=vmax)
                    mh = m.float() / (1 - b1 ** st["step"])
                    vh = vmax.float() / (1 - b2 ** st["step"])
                    upd = mh / (vh.sqrt() + group["eps"]) + group["weight_decay"] * p.data.float()
                    p.data.add_((-group["lr"] * upd).to(p.dtype))
                else:
                    ref.adamw_step(p.data, p.grad.to(p.dtype) * self.grad_scale, st["exp_avg"], st["exp_avg_sq"],
                                   group["lr"], b1, b2, group["eps"], group["weight_decay"], st["step"])
        return loss


PiscesLxFusedAdamW = YvFusedAdamW
