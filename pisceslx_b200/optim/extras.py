"""Further optimizers and training aids (reference opss/optim: ``PiscesLxGaLoreOperator``, ``PiscesLxROOTOptimizer``
(root.py), ``PiscesLxTERAIOManager`` offload planner; opss/train: ``PiscesLxMoEGradientOperator`` (moe_gradient.py),
multi-task uncertainty weighting, modality learning-rate scheduler, Chinchilla scaler)."""
from __future__ import annotations

import math
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch


class PiscesLxGaLoreProjector:
    """Gradient low-rank projection: every ``update_gap`` steps the top-``rank`` left (or right) singular vectors of
    the gradient are refreshed; optimizer moments live in the projected space."""

    def __init__(self, rank: int = 128, update_gap: int = 200, scale: float = 0.25):
        self.rank, self.update_gap, self.scale = rank, update_gap, scale
        self.basis: Optional[torch.Tensor] = None
        self.left = True
        self.step = 0

    def project(self, g: torch.Tensor) -> torch.Tensor:
        if self.basis is None or self.step % self.update_gap == 0:
            self.left = g.shape[0] <= g.shape[1]
            u, _, vh = torch.linalg.svd(g.float(), full_matrices=False)
            r = min(self.rank, u.shape[1])
            self.basis = (u[:, :r] if self.left else vh[:r].t()).contiguous()
        self.step += 1
        return self.basis.t() @ g.float() if self.left else g.float() @ self.basis

    def project_back(self, low: torch.Tensor) -> torch.Tensor:
        return self.scale * (self.basis @ low if self.left else low @ self.basis.t())


class PiscesLxGaLoreAdamW(torch.optim.Optimizer):
    """AdamW whose 2-D parameters keep their moments in the GaLore-projected space."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, rank=128, update_gap=200,
                 scale=0.25):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, rank=rank,
                                      update_gap=update_gap, scale=scale))

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                grad = p.grad
                if p.dim() == 2 and min(p.shape) > g["rank"]:
                    proj = st.setdefault("proj", PiscesLxGaLoreProjector(g["rank"], g["update_gap"], g["scale"]))
                    grad = proj.project(grad)
                else:
                    proj = None
                    grad = grad.float()
                if "m" not in st or st["m"].shape != grad.shape:
                    st["m"], st["v"], st["t"] = torch.zeros_like(grad), torch.zeros_like(grad), 0
                st["t"] += 1
                st["m"].mul_(b1).add_(grad, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                upd = (st["m"] / (1 - b1 ** st["t"])) / ((st["v"] / (1 - b2 ** st["t"])).sqrt() + g["eps"])
                if proj is not None:
                    upd = proj.project_back(upd)
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(upd.to(p.dtype), alpha=-g["lr"])
    def state_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for s in self.state.values() for t in s.values() if torch.is_tensor(t))


class PiscesLxROOTMomentumOptimizer(torch.optim.Optimizer):
    """The momentum-only form of the robust orthogonalised optimizer (``optim.root.PiscesLxROOTOptimizer`` is the
    configured form with Adam moments, soft threshold and spectral clip): momentum -> outlier clipping of the update by a soft threshold (a proximal
    step that removes gradient spikes) -> Newton-Schulz orthogonalisation with shape-adapted scaling."""

    def __init__(self, params, lr=2e-4, momentum=0.95, weight_decay=0.0, ns_steps=5, outlier_quantile=0.99):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, ns_steps=ns_steps,
                                      outlier_quantile=outlier_quantile))

    @torch.no_grad()
    def step(self, closure=None):
        from ..ops.reference import MUON_NS_COEFFS, newton_schulz
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                buf = st.setdefault("momentum", torch.zeros_like(p, dtype=torch.float32))
                buf.mul_(g["momentum"]).add_(p.grad.float())
                upd = buf.clone()
                if p.dim() == 2:
                    flat = upd.abs().flatten()
                    k = max(1, int(g["outlier_quantile"] * flat.numel()))
                    thr = flat.kthvalue(min(k, flat.numel())).values
                    upd = upd.clamp(-thr, thr)                                    # soft-threshold the spikes
                    upd = newton_schulz(upd, MUON_NS_COEFFS[-g["ns_steps"]:]) * math.sqrt(max(1.0, p.shape[0] / p.shape[1]))
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(upd.to(p.dtype), alpha=-g["lr"])


PiscesLxROOTOptimizer = PiscesLxROOTMomentumOptimizer           # the name this class had before optim/root.py existed


class PiscesLxTERAIOManager:
    """Offload planner: given tensor sizes and the step at which each is next needed, choose what to move to the host
    so that resident bytes stay under the budget, evicting the tensors needed furthest in the future first."""

    def __init__(self, budget_bytes: int):
        self.budget = budget_bytes

    def plan(self, tensors: Dict[str, Tuple[int, int]]) -> Dict[str, str]:
        """tensors: name -> (bytes, next_use_step).  Returns name -> 'gpu' | 'host'."""
        placement = {n: "gpu" for n in tensors}
        resident = sum(b for b, _ in tensors.values())
        for name, (b, _) in sorted(tensors.items(), key=lambda kv: -kv[1][1]):
            if resident <= self.budget:
                break
            placement[name] = "host"
            resident -= b
        return placement


class PiscesLxMoEGradientOperator:
    """Per-expert gradient conditioning for stacked expert weights [E, ...]: clip each expert's gradient to
    ``max_norm`` separately (one noisy expert does not shrink the others) and rescale rarely used experts."""

    def __init__(self, max_norm: float = 1.0, min_count_scale: float = 0.1):
        self.max_norm, self.min_count_scale = max_norm, min_count_scale

    @torch.no_grad()
    def apply(self, grad: torch.Tensor, counts: Optional[torch.Tensor] = None) -> torch.Tensor:
        E = grad.shape[0]
        norms = grad.float().flatten(1).norm(dim=1)
        coef = (self.max_norm / (norms + 1e-6)).clamp(max=1.0)
        if counts is not None:
            share = counts.float() / counts.float().mean().clamp_min(1e-6)
            coef = coef * share.clamp(min=self.min_count_scale, max=1.0)
        grad.mul_(coef.view(E, *([1] * (grad.dim() - 1))).to(grad.dtype))
        return norms


class PiscesLxMultiTaskUncertainty(torch.nn.Module):
    """Homoscedastic-uncertainty weighting: L = sum_i exp(-s_i) L_i + s_i with learned log-variances s_i."""

    def __init__(self, n_tasks: int):
        super().__init__()
        self.log_var = torch.nn.Parameter(torch.zeros(n_tasks))

    def forward(self, losses: List[torch.Tensor]) -> torch.Tensor:
        return sum(torch.exp(-self.log_var[i]) * l + self.log_var[i] for i, l in enumerate(losses))


class PiscesLxModalityLRScheduler:
    """Per-modality learning-rate multipliers by parameter-name prefix (e.g. a slower vision tower)."""

    def __init__(self, optimizer: torch.optim.Optimizer, named_params: Iterable[Tuple[str, torch.nn.Parameter]],
                 multipliers: Dict[str, float]):
        self.mult = {id(p): next((m for k, m in multipliers.items() if k in n), 1.0) for n, p in named_params}
        self.optimizer = optimizer

    def scales(self) -> List[float]:
        return [max((self.mult.get(id(p), 1.0) for p in g["params"]), default=1.0) for g in self.optimizer.param_groups]

    def apply(self, base_lr: float) -> None:
        for g, s in zip(self.optimizer.param_groups, self.scales()):
            g["lr"] = base_lr * s


def chinchilla_optimal(compute_flops: float, a: float = 0.5, tokens_per_param: float = 20.0) -> Dict[str, float]:
    """Compute-optimal split C = 6 N D with D = tokens_per_param * N."""
    n = math.sqrt(compute_flops / (6.0 * tokens_per_param))
    return {"params": n, "tokens": tokens_per_param * n}
