"""ROOT, the robust orthogonalised optimizer, as a configured operator, an optimizer and its schedule (reference
opss/optim/root.py:77-815).

One step on a matrix parameter: Adam moments -> orthogonalise the first moment (Newton-Schulz) -> soft-threshold the
small entries away -> clip the spectral norm -> divide by the root of the second moment -> bias-corrected step.

Built for the device:
* matrices of one shape are stacked and orthogonalised as ONE batched Newton-Schulz chain (a transformer has a handful
  of distinct shapes, so a step is a handful of batched GEMM chains instead of one chain per parameter);
* the spectral norm comes from a power iteration whose vector is kept in the optimizer state, so two matrix-vector
  products per step track it (the reference restarts ten iterations from a random vector each step, root.py:418-455);
* the clip is a ``torch.where`` on the device and the statistics stay tensors - the reference reads every parameter's
  spectral norm and kept ratio back with ``.item()`` (root.py:285-300), one stream synchronisation per parameter per step.

Three departures, each because the reference's form cannot do what it says: its orthogonalisation ends in
``torch.linalg.matrix_power(I + M, 0.5)``, which raises for a fractional power and is caught by a bare ``except`` that
returns the momentum unchanged (root.py:362-372) - here the quintic Newton-Schulz iteration of ``ops.reference`` is
used; and its soft threshold is an absolute 0.1 although an orthogonalised n x m update has entries of size about
1 / sqrt(max(n, m)), so every entry of a large matrix would be zeroed - here the threshold is relative to the update's
root mean square; and an orthogonalised matrix has unit singular values whatever the size of the gradient, so dividing
it by the root of the second moment (which does scale with the gradient) gives steps that grow without bound as the
gradient shrinks - here the orthogonalised moment is rescaled to the Frobenius norm of the moment it came from, so the
step keeps Adam's size and only its direction is equalised across singular directions."""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn
from torch.optim import Optimizer

from ..ops.reference import MUON_NS_COEFFS, newton_schulz
from ..utils.opsc import PiscesLxOperatorInterface


@dataclass
class PiscesLxROOTConfig:
    name: str = "root"
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    orthogonalization_steps: int = 5
    soft_threshold: float = 0.1                  # x the update's root mean square
    spectral_norm_clip: float = 1.0
    use_orthogonalization: bool = True
    use_soft_threshold: bool = True
    min_dim_for_ortho: int = 16
    amsgrad: bool = False
    maximize: bool = False
    power_iterations: int = 2

    def __post_init__(self) -> None:
        if self.lr < 0:
            raise ValueError(f"Invalid learning rate: {self.lr}")
        if not 0 <= self.beta1 < 1:
            raise ValueError(f"Invalid beta1: {self.beta1}")
        if not 0 <= self.beta2 < 1:
            raise ValueError(f"Invalid beta2: {self.beta2}")
        if self.orthogonalization_steps < 1:
            raise ValueError("orthogonalization_steps must be at least 1")

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


def orthogonalize_momentum(momentum: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Nearest (semi-)orthogonal matrix of a [*, n, m] stack by the quintic Newton-Schulz iteration; vectors pass through,
    tensors of more than two axes are flattened to [first, rest] unless they are already a stack of matrices."""
    if momentum.dim() < 2:
        return momentum
    coeffs = MUON_NS_COEFFS[-steps:] if steps <= len(MUON_NS_COEFFS) else tuple(MUON_NS_COEFFS) + (MUON_NS_COEFFS[-1],) * (steps - len(MUON_NS_COEFFS))
    return newton_schulz(momentum, coeffs).to(momentum.dtype)


def soft_threshold_denoise(update: torch.Tensor, threshold: float = 0.1) -> Tuple[torch.Tensor, torch.Tensor]:
    """sign(u) max(|u| - t rms(u), 0) per matrix of a stack; also the share of entries kept (a tensor)."""
    dims = tuple(range(-min(update.dim(), 2), 0))
    t = threshold * update.float().pow(2).mean(dims, keepdim=True).sqrt()
    mag = update.abs().float() - t
    return (torch.sign(update) * mag.clamp_min(0).to(update.dtype)), (mag > 0).float().mean()


def compute_spectral_norm(matrix: torch.Tensor, num_iterations: int = 10, u: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Largest singular value of every matrix of a [*, n, m] stack by power iteration from ``u`` [*, n] (a fixed vector
    when none is given, so the result is reproducible); returns (sigma [*], u) for the next call to start from."""
    if matrix.dim() == 1:
        return matrix.norm(), matrix
    x = matrix.float()
    if u is None:
        u = torch.ones(x.shape[:-1], device=x.device, dtype=torch.float32)
        u = u + 0.01 * torch.arange(x.shape[-2], device=x.device, dtype=torch.float32)       # not orthogonal to a sign-balanced vector
    u = u / u.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    v = None
    for _ in range(max(num_iterations, 1)):
        v = torch.einsum("...nm,...n->...m", x, u)
        v = v / v.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        u = torch.einsum("...nm,...m->...n", x, v)
        sigma = u.norm(dim=-1)
        u = u / sigma.unsqueeze(-1).clamp_min(1e-12)
    return sigma, u


def _root_update_stack(exp_avg: torch.Tensor, cfg: PiscesLxROOTConfig, u: Optional[torch.Tensor]) -> Tuple[torch.Tensor, Dict[str, torch.Tensor], Optional[torch.Tensor]]:
    """The shaping of the first moment for a [k, n, m] stack (or a single tensor of fewer than two axes)."""
    stats: Dict[str, torch.Tensor] = {}
    upd = exp_avg
    is_matrix = upd.dim() >= 3
    if is_matrix and cfg.use_orthogonalization and min(upd.shape[-2:]) >= cfg.min_dim_for_ortho:
        norm = upd.float().flatten(-2).norm(dim=-1)
        upd = orthogonalize_momentum(upd, cfg.orthogonalization_steps)
        upd = upd * (norm / upd.float().flatten(-2).norm(dim=-1).clamp_min(1e-30)).view(-1, 1, 1).to(upd.dtype)   # direction changes, size stays
        stats["orthogonalized"] = torch.full((), float(upd.shape[0]), device=upd.device)
    if cfg.use_soft_threshold:
        upd, stats["kept"] = soft_threshold_denoise(upd, cfg.soft_threshold)
    if is_matrix and cfg.spectral_norm_clip > 0:
        sigma, u = compute_spectral_norm(upd, cfg.power_iterations if u is not None else 10, u)
        stats["spectral_norm"] = sigma.mean()
        scale = torch.where(sigma > cfg.spectral_norm_clip, cfg.spectral_norm_clip / sigma.clamp_min(1e-12), torch.ones_like(sigma))
        upd = upd * scale.view(-1, 1, 1).to(upd.dtype)
    return upd, stats, u


class PiscesLxROOTOptimizer(Optimizer):
    """``PiscesLxROOTOptimizer(model.parameters(), lr=1e-3)``; every keyword of ``PiscesLxROOTConfig`` is accepted, and
    ``betas=(b1, b2)`` as in Adam."""

    def __init__(self, params: Iterable, lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 orthogonalization_steps: int = 5, soft_threshold: float = 0.1, spectral_norm_clip: float = 1.0, use_orthogonalization: bool = True,
                 use_soft_threshold: bool = True, min_dim_for_ortho: int = 16, amsgrad: bool = False, maximize: bool = False, power_iterations: int = 2):
        cfg = PiscesLxROOTConfig(lr=lr, beta1=betas[0], beta2=betas[1], eps=eps, weight_decay=weight_decay, orthogonalization_steps=orthogonalization_steps,
                                 soft_threshold=soft_threshold, spectral_norm_clip=spectral_norm_clip, use_orthogonalization=use_orthogonalization,
                                 use_soft_threshold=use_soft_threshold, min_dim_for_ortho=min_dim_for_ortho, amsgrad=amsgrad, maximize=maximize,
                                 power_iterations=power_iterations)
        d = cfg.to_dict()
        d.pop("name")
        d["betas"] = (d.pop("beta1"), d.pop("beta2"))
        super().__init__(params, d)
        self.last_stats: Dict[str, torch.Tensor] = {}

    @classmethod
    def from_config(cls, params: Iterable, config: PiscesLxROOTConfig) -> "PiscesLxROOTOptimizer":
        d = config.to_dict()
        d.pop("name")
        return cls(params, betas=(d.pop("beta1"), d.pop("beta2")), **d)

    @staticmethod
    def _group_cfg(g: Dict[str, Any]) -> PiscesLxROOTConfig:
        d = {k: v for k, v in g.items() if k in PiscesLxROOTConfig.__dataclass_fields__}
        return PiscesLxROOTConfig(beta1=g["betas"][0], beta2=g["betas"][1], **d)

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        agg: Dict[str, List[torch.Tensor]] = {}
        for g in self.param_groups:
            cfg = self._group_cfg(g)
            buckets: Dict[Tuple, List[nn.Parameter]] = {}
            for p in g["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("ROOT does not support sparse gradients")
                shape = tuple(p.shape) if p.dim() <= 2 else (p.shape[0], p.numel() // p.shape[0])
                buckets.setdefault((shape, p.dtype, p.device), []).append(p)
            for (shape, _, _), ps in buckets.items():
                grads = []
                for p in ps:
                    st = self.state[p]
                    if not st:
                        st["step"] = 0
                        st["exp_avg"] = torch.zeros(shape, device=p.device, dtype=torch.float32)
                        st["exp_avg_sq"] = torch.zeros(shape, device=p.device, dtype=torch.float32)
                        if cfg.amsgrad:
                            st["max_exp_avg_sq"] = torch.zeros(shape, device=p.device, dtype=torch.float32)
                    st["step"] += 1
                    gr = p.grad.float().reshape(shape)
                    gr = -gr if cfg.maximize else gr
                    if cfg.weight_decay:
                        gr = gr.add(p.float().reshape(shape), alpha=cfg.weight_decay)
                    grads.append(gr)
                m = [self.state[p]["exp_avg"] for p in ps]
                v = [self.state[p]["exp_avg_sq"] for p in ps]
                torch._foreach_mul_(m, cfg.beta1)
                torch._foreach_add_(m, grads, alpha=1 - cfg.beta1)
                torch._foreach_mul_(v, cfg.beta2)
                torch._foreach_addcmul_(v, grads, grads, value=1 - cfg.beta2)
                if cfg.amsgrad:
                    mx = [self.state[p]["max_exp_avg_sq"] for p in ps]
                    torch._foreach_maximum_(mx, v)
                    v = mx
                matrix = len(shape) == 2
                stack = torch.stack(m) if matrix else None
                if matrix:
                    u = self.state[ps[0]].get("u_stack")
                    if u is not None and u.shape[0] != len(ps):
                        u = None
                    upd, stats, u = _root_update_stack(stack, cfg, u)
                    if u is not None:
                        self.state[ps[0]]["u_stack"] = u
                    upds = list(upd.unbind(0))
                else:
                    upds, stats = [], {}
                    for t in m:
                        u1, s1, _ = _root_update_stack(t, cfg, None)
                        upds.append(u1)
                        stats = s1 or stats
                for k, val in stats.items():
                    agg.setdefault(k, []).append(val)
                for p, u_, v_ in zip(ps, upds, v):
                    t = self.state[p]["step"]
                    step_size = g["lr"] * math.sqrt(1 - cfg.beta2 ** t) / (1 - cfg.beta1 ** t)
                    p.add_((u_ / (v_.sqrt() + cfg.eps)).reshape(p.shape).to(p.dtype), alpha=-step_size)
        self.last_stats = {k: (torch.stack([x.float().reshape(()) for x in v]).sum() if k == "orthogonalized" else torch.stack([x.float().reshape(()) for x in v]).mean())
                           for k, v in agg.items()}
        return loss

    def get_config(self) -> Dict[str, Any]:
        return {k: v for k, v in self.param_groups[0].items() if k != "params"}


class PiscesLxROOTOperator(PiscesLxOperatorInterface):
    """One functional step over a model's named parameters: ``run({"model", "gradients"?, "config"?, "optimizer_state"?})``
    returns the model, the state to pass to the next call and statistics (tensors)."""

    name = "root"
    version = "1.0.0"

    orthogonalize_momentum = staticmethod(orthogonalize_momentum)
    soft_threshold_denoise = staticmethod(soft_threshold_denoise)

    @staticmethod
    def compute_spectral_norm(matrix: torch.Tensor, num_iterations: int = 10) -> torch.Tensor:
        return compute_spectral_norm(matrix, num_iterations)[0]

    @staticmethod
    def _should_orthogonalize(param: torch.Tensor, config: PiscesLxROOTConfig) -> bool:
        return param.dim() >= 2 and min(param.shape[0], param.numel() // param.shape[0]) >= config.min_dim_for_ortho

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs.get("model"), nn.Module)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        model: nn.Module = inputs["model"]
        cfg: PiscesLxROOTConfig = inputs.get("config") or PiscesLxROOTConfig()
        state = inputs.get("optimizer_state") or {}
        opt: Optional[PiscesLxROOTOptimizer] = state.get("optimizer")
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        if opt is None or state.get("model_id") != id(model):
            opt = PiscesLxROOTOptimizer.from_config([p for _, p in named], cfg)
            state = {"optimizer": opt, "model_id": id(model), "config": cfg}
        for gdict in opt.param_groups:
            gdict["lr"] = cfg.lr
        grads = inputs.get("gradients") or {}
        for n, p in named:
            if n in grads:
                p.grad = grads[n]
        opt.step()
        ortho = sum(1 for _, p in named if p.grad is not None and cfg.use_orthogonalization and self._should_orthogonalize(p, cfg))
        s = opt.last_stats
        stats = {"orthogonalized_params": ortho, "total_params": len(named),
                 "avg_spectral_norm": s.get("spectral_norm", torch.zeros(())), "avg_threshold_ratio": s.get("kept", torch.ones(()))}
        return {"model": model, "optimizer_state": state, "statistics": stats, "orthogonalized_ratio": ortho / max(len(named), 1)}


class PiscesLxROOTScheduler:
    """Linear warm-up, then cosine / linear / exponential decay to ``min_lr`` (or a constant); every group keeps its own
    base rate."""

    def __init__(self, optimizer: Optimizer, warmup_steps: int = 1000, total_steps: int = 100000, min_lr: float = 1e-6, decay_type: str = "cosine"):
        if decay_type not in ("cosine", "linear", "exponential", "constant"):
            raise ValueError(f"unknown decay type {decay_type}")
        self.optimizer, self.warmup_steps, self.total_steps, self.min_lr, self.decay_type = optimizer, warmup_steps, total_steps, min_lr, decay_type
        self.current_step = 0
        self.base_lrs = [g["lr"] for g in optimizer.param_groups]

    @property
    def base_lr(self) -> float:
        return self.base_lrs[0]

    def _compute_lr(self, base: Optional[float] = None) -> float:
        base = self.base_lrs[0] if base is None else base
        if self.current_step < self.warmup_steps:
            return base * self.current_step / max(self.warmup_steps, 1)
        p = min((self.current_step - self.warmup_steps) / max(self.total_steps - self.warmup_steps, 1), 1.0)
        lo = min(self.min_lr, base)
        if self.decay_type == "cosine":
            return lo + 0.5 * (base - lo) * (1 + math.cos(math.pi * p))
        if self.decay_type == "linear":
            return base - p * (base - lo)
        if self.decay_type == "exponential":
            return base * (max(lo, 1e-30) / base) ** p if base > 0 else 0.0
        return base

    def step(self) -> float:
        self.current_step += 1
        for g, b in zip(self.optimizer.param_groups, self.base_lrs):
            g["lr"] = self._compute_lr(b)
        return self.optimizer.param_groups[0]["lr"]

    def state_dict(self) -> Dict[str, Any]:
        return {"current_step": self.current_step, "base_lrs": list(self.base_lrs), "warmup_steps": self.warmup_steps,
                "total_steps": self.total_steps, "min_lr": self.min_lr, "decay_type": self.decay_type}

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        self.current_step = state_dict["current_step"]
        self.base_lrs = list(state_dict.get("base_lrs", [state_dict.get("base_lr", self.base_lrs[0])] * len(self.base_lrs)))
        self.warmup_steps, self.total_steps = state_dict["warmup_steps"], state_dict["total_steps"]
        self.min_lr, self.decay_type = state_dict["min_lr"], state_dict["decay_type"]
