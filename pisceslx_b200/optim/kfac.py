"""Kronecker-factored curvature preconditioner for linear layers (reference opss/optim/kfac.py: running input and
output-gradient covariances per layer, damped inverses refreshed every few steps, gradients preconditioned as
``G^-1 dW A^-1`` before the base optimizer's step).

Works on modules that expose a 2-D ``weight`` and are called as ``module(x)``: forward pre-hooks record the input
covariance ``A = E[x x^T]``, full backward hooks the output-gradient covariance ``G = E[g g^T]``."""
from __future__ import annotations

from typing import Dict, Iterable, List

import torch
import torch.nn as nn


class PiscesLxKFACPreconditioner:
    def __init__(self, modules: Iterable[nn.Module], damping: float = 1e-3, ema: float = 0.95, update_every: int = 10,
                 max_dim: int = 8192):
        self.modules: List[nn.Module] = [m for m in modules if getattr(m, "weight", None) is not None
                                         and m.weight.dim() == 2 and max(m.weight.shape) <= max_dim]
        self.damping, self.ema, self.update_every = damping, ema, update_every
        self.A: Dict[nn.Module, torch.Tensor] = {}
        self.G: Dict[nn.Module, torch.Tensor] = {}
        self.Ainv: Dict[nn.Module, torch.Tensor] = {}
        self.Ginv: Dict[nn.Module, torch.Tensor] = {}
        self.steps = 0
        self._handles = []
        for m in self.modules:
            self._handles.append(m.register_forward_pre_hook(self._fwd))
            self._handles.append(m.register_full_backward_hook(self._bwd))

    def _acc(self, store: Dict, m: nn.Module, x: torch.Tensor) -> None:
        x = x.detach().reshape(-1, x.shape[-1]).float()
        c = x.t() @ x / max(1, x.shape[0])
        store[m] = c if m not in store else store[m].mul_(self.ema).add_(c, alpha=1 - self.ema)

    def _fwd(self, m: nn.Module, args) -> None:
        if m.training and torch.is_grad_enabled():
            self._acc(self.A, m, args[0])

    def _bwd(self, m: nn.Module, gin, gout) -> None:
        if gout[0] is not None:
            g = gout[0]
            self._acc(self.G, m, g * g.shape[0] if g.dim() > 1 else g)

    @staticmethod
    def _damped_inverse(c: torch.Tensor, damping: float) -> torch.Tensor:
        d = damping * (c.diagonal().mean().clamp_min(1e-12))
        eye = torch.eye(c.shape[0], device=c.device, dtype=c.dtype)
        return torch.linalg.inv(c + d * eye)

    @torch.no_grad()
    def precondition(self) -> None:
        """Call after backward and before the optimizer step: rewrites ``weight.grad`` in place."""
        refresh = self.steps % self.update_every == 0
        for m in self.modules:
            if m.weight.grad is None or m not in self.A or m not in self.G:
                continue
            if refresh or m not in self.Ainv:
                self.Ainv[m] = self._damped_inverse(self.A[m], self.damping)
                self.Ginv[m] = self._damped_inverse(self.G[m], self.damping)
            g = m.weight.grad
            ng = self.Ginv[m] @ g.float() @ self.Ainv[m]
            # keep the step length of the raw gradient (the base optimizer owns the learning rate)
            ng.mul_(g.float().norm() / ng.norm().clamp_min(1e-12))
            g.copy_(ng.to(g.dtype))
        self.steps += 1

    def close(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles.clear()
