"""Gradient conditioning for mixture-of-experts training (reference opss/train/moe_gradient.py:131-1057): expert and
non-expert parameters have gradient scales that differ by orders of magnitude (an expert sees a fraction of the
tokens), so experts are clipped against their own adaptive threshold, optionally renormalised against the dense
parameters, and the routing gets auxiliary balance / importance losses.

Differences from the reference, on purpose:

  * Stacked expert tensors.  This framework stores the routed experts of a layer as ``[E, ...]`` tensors, so "per
    expert" means per leading index: each expert is clipped separately (one spiking expert does not shrink the other
    127) with one vectorised norm over the flattened trailing dimensions.  Unstacked per-expert parameters are handled
    per tensor.
  * No host read-back in the step.  Norms come from one multi-tensor ``torch._foreach_norm`` call, the clip
    coefficients are tensors, the adaptive threshold is a quantile of a ring buffer kept on the device; the reference
    calls ``.item()`` per parameter and runs numpy percentiles each step (moe_gradient.py:503-590).
  * The auxiliary losses are differentiable tensors to be ADDED to the loss.  The reference returns Python floats
    (``.item()``), which cannot train anything (moe_gradient.py:629-721)."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..utils.opsc import PiscesLxOperatorInterface


class PiscesLxMoEExpertType(str, Enum):
    FFN = "ffn"
    ATTENTION = "attention"
    EMBEDDING = "embedding"
    CROSS_MODAL = "cross_modal"
    UNIFIED = "unified"


@dataclass
class PiscesLxMoEGradientConfig:
    expert_clip_threshold: float = 0.1          # upper bound of a single expert's gradient norm
    expert_norm_factor: float = 1.0             # target ratio expert-norm / dense-norm after normalisation
    enable_adaptive_clip: bool = True
    enable_gradient_normalization: bool = False
    load_balancing_weight: float = 0.01
    importance_weight: float = 0.01
    utilization_weight: float = 0.01
    detect_expert_patterns: List[str] = field(default_factory=lambda: ["experts", "expert", "moe", "experts_w13", "experts_w2",
                                                                       "w1", "w2", "w3", "gate_proj", "up_proj", "down_proj"])
    exclude_patterns: List[str] = field(default_factory=lambda: ["norm", "embed", "head", "shared"])
    gating_patterns: List[str] = field(default_factory=lambda: ["router", "routing", "gate.weight", "expert_bias"])
    warmup_steps: int = 100
    clip_history_window: int = 100
    clip_percentile: float = 95.0
    min_history: int = 10

    def __post_init__(self) -> None:
        if not 0 < self.clip_percentile <= 100:
            raise ValueError("clip_percentile must be in (0, 100]")
        if self.expert_clip_threshold <= 0:
            raise ValueError("expert_clip_threshold must be positive")


class PiscesLxExpertGradientClipper:
    """Clips a set of parameters by their joint norm (the plain case) and returns the norm as a tensor."""

    def __init__(self, max_norm: float = 1.0, norm_type: float = 2.0):
        self.max_norm, self.norm_type = max_norm, norm_type

    @torch.no_grad()
    def clip(self, parameters: Iterable[torch.nn.Parameter]) -> torch.Tensor:
        grads = [p.grad for p in parameters if p.grad is not None]
        if not grads:
            return torch.zeros(())
        total = torch.linalg.vector_norm(torch.stack(torch._foreach_norm(grads, self.norm_type)).float(), self.norm_type)
        coef = (self.max_norm / (total + 1e-6)).clamp(max=1.0)
        torch._foreach_mul_(grads, coef.to(grads[0].dtype) if len({g.dtype for g in grads}) == 1 else coef)
        return total


class PiscesLxMoEGradientOperator(PiscesLxOperatorInterface):
    """``classify(model)`` once, then after every backward ``process(model)``:

      1. per-expert clipping against min(configured threshold, 1.2 x the ``clip_percentile`` quantile of the recent
         per-expert norms) - after ``warmup_steps`` and ``min_history`` observations, the configured threshold before;
      2. optional normalisation: scale all expert gradients so that their joint norm is ``expert_norm_factor`` x the
         dense parameters' norm;
      3. statistics (tensors; ``get_gradient_statistics()`` converts them when asked).

    ``auxiliary_losses(router_probs, expert_index)`` gives the balance, importance and utilisation terms."""

    name = "moe_gradient_optimizer"

    def __init__(self, config: Optional[PiscesLxMoEGradientConfig] = None):
        self.config = config or PiscesLxMoEGradientConfig()
        self.expert_params: List[str] = []
        self.non_expert_params: List[str] = []
        self.gating_params: List[str] = []
        self._types: Dict[str, PiscesLxMoEExpertType] = {}
        self._history: Optional[torch.Tensor] = None
        self._hist_n = 0
        self.steps = 0
        self._last: Dict[str, torch.Tensor] = {}

    # -- classification ---------------------------------------------------------------------------------------------------------
    def _detect_expert_parameter(self, param_name: str) -> Tuple[bool, PiscesLxMoEExpertType]:
        n, c = param_name.lower(), self.config
        if any(p in n for p in c.gating_patterns):
            return False, PiscesLxMoEExpertType.UNIFIED
        if any(p in n for p in c.exclude_patterns):
            return False, PiscesLxMoEExpertType.UNIFIED
        if not any(p in n for p in c.detect_expert_patterns):
            return False, PiscesLxMoEExpertType.UNIFIED
        if any(p in n for p in ("attn", "attention")):
            return True, PiscesLxMoEExpertType.ATTENTION
        if any(p in n for p in ("cross", "multimodal")):
            return True, PiscesLxMoEExpertType.CROSS_MODAL
        return True, PiscesLxMoEExpertType.FFN

    def classify(self, model: nn.Module) -> Dict[str, Any]:
        self.expert_params, self.non_expert_params, self.gating_params, self._types = [], [], [], {}
        out: Dict[str, Any] = {"expert": {t.value: [] for t in PiscesLxMoEExpertType}, "non_expert": [], "gating": []}
        for name, _ in model.named_parameters():
            if any(p in name.lower() for p in self.config.gating_patterns):
                self.gating_params.append(name)
                self.non_expert_params.append(name)
                out["gating"].append(name)
                out["non_expert"].append(name)
                continue
            is_e, t = self._detect_expert_parameter(name)
            if is_e:
                self.expert_params.append(name)
                self._types[name] = t
                out["expert"][t.value].append(name)
            else:
                self.non_expert_params.append(name)
                out["non_expert"].append(name)
        return out

    _classify_parameters = classify

    def get_expert_parameters(self) -> List[str]:
        return list(self.expert_params)

    def get_non_expert_parameters(self) -> List[str]:
        return list(self.non_expert_params)

    # -- the step ---------------------------------------------------------------------------------------------------------------
    @staticmethod
    def _is_stacked(p: torch.Tensor) -> bool:
        return p.dim() >= 3

    @staticmethod
    def _per_expert_norms(g: torch.Tensor, stacked: bool) -> torch.Tensor:
        return g.float().flatten(1).norm(dim=1) if stacked else g.float().norm().reshape(1)

    def _threshold(self, device: torch.device) -> torch.Tensor:
        c = self.config
        base = torch.tensor(c.expert_clip_threshold, device=device)
        if not c.enable_adaptive_clip or self._history is None or self._hist_n < c.min_history or self.steps <= c.warmup_steps:
            return base
        h = self._history[: min(self._hist_n, self._history.numel())].to(device)
        return torch.minimum(base, 1.2 * torch.quantile(h, c.clip_percentile / 100.0))

    def _remember(self, norms: torch.Tensor) -> None:
        w = self.config.clip_history_window
        if self._history is None:
            self._history = torch.zeros(w, device=norms.device)
        v = norms.detach().float().max().reshape(1)                 # the worst expert of this step
        self._history[self._hist_n % w] = v.to(self._history.device)[0]
        self._hist_n += 1

    @torch.no_grad()
    def process(self, model: nn.Module) -> Dict[str, torch.Tensor]:
        if not self.expert_params and not self.non_expert_params:
            self.classify(model)
        self.steps += 1
        params = dict(model.named_parameters())
        experts = [(n, params[n]) for n in self.expert_params if n in params and params[n].grad is not None]
        dense = [params[n].grad for n in self.non_expert_params if n in params and params[n].grad is not None]
        dev = experts[0][1].grad.device if experts else (dense[0].device if dense else torch.device("cpu"))
        dense_norm = torch.stack(torch._foreach_norm(dense)).float().norm() if dense else torch.zeros((), device=dev)
        thr = self._threshold(dev)
        all_norms, clipped = [], torch.zeros((), device=dev)
        for _, p in experts:
            st = self._is_stacked(p)
            norms = self._per_expert_norms(p.grad, st)
            coef = (thr / (norms + 1e-8)).clamp(max=1.0)
            p.grad.mul_(coef.view(-1, *([1] * (p.grad.dim() - 1))).to(p.grad.dtype) if st else coef.to(p.grad.dtype))
            clipped = clipped + (coef < 1.0).sum()
            all_norms.append(norms)
        if all_norms:
            cat = torch.cat(all_norms)
            self._remember(cat)
            expert_norm = cat.norm()
        else:
            cat, expert_norm = torch.zeros(1, device=dev), torch.zeros((), device=dev)
        if self.config.enable_gradient_normalization and experts and dense:
            after = torch.stack(torch._foreach_norm([p.grad for _, p in experts])).float().norm()
            scale = torch.where((after > 0) & (dense_norm > 0), self.config.expert_norm_factor * dense_norm / after.clamp_min(1e-12),
                                torch.ones_like(after))
            torch._foreach_mul_([p.grad for _, p in experts], scale)
        final = torch.stack(torch._foreach_norm([p.grad for _, p in experts])).float().norm() if experts else expert_norm
        self._last = {"expert_grad_norm": expert_norm, "expert_grad_norm_after": final, "non_expert_grad_norm": dense_norm,
                      "num_clipped": clipped, "clip_threshold": thr, "max_expert_norm": cat.max(),
                      "scale_gap": dense_norm / expert_norm.clamp_min(1e-12)}
        return dict(self._last)

    # -- auxiliary losses ---------------------------------------------------------------------------------------------------------
    def _compute_load_balancing_loss(self, router_probs: Optional[torch.Tensor] = None,
                                     expert_index: Optional[torch.Tensor] = None, num_experts: Optional[int] = None) -> torch.Tensor:
        """E x sum_e f_e P_e (switch form) when both the probabilities [T, E] and the chosen indices [T, k] are given -
        f_e the share of assignments, P_e the mean probability; its minimum 1 is subtracted so that a balanced router
        scores 0.  With probabilities only: the squared deviation of the mean probability from uniform."""
        w = self.config.load_balancing_weight
        if router_probs is None and expert_index is None:
            return torch.zeros(())
        if router_probs is not None:
            E = router_probs.shape[-1]
            P = router_probs.float().reshape(-1, E).mean(0)
            if expert_index is not None:
                f = torch.bincount(expert_index.reshape(-1).long(), minlength=E).float()
                f = f / f.sum().clamp_min(1.0)
                return w * (E * (f.detach() * P).sum() - 1.0)
            return w * ((P - 1.0 / E) ** 2).sum() * E
        E = int(num_experts or int(expert_index.max()) + 1)
        f = torch.bincount(expert_index.reshape(-1).long(), minlength=E).float()
        f = f / f.sum().clamp_min(1.0)
        return w * ((f - 1.0 / E) ** 2).sum() * E                  # indices carry no gradient: a monitor, not a loss

    def _compute_importance_loss(self, router_probs: torch.Tensor) -> torch.Tensor:
        """Squared coefficient of variation of the experts' total probability mass."""
        imp = router_probs.float().reshape(-1, router_probs.shape[-1]).sum(0)
        return self.config.importance_weight * imp.var(unbiased=False) / imp.mean().pow(2).clamp_min(1e-12)

    def _compute_utilization_loss(self, router_probs: torch.Tensor) -> torch.Tensor:
        """Penalises experts whose best probability over the batch stays low (dead experts): mean of (1 - max_t p)."""
        p = router_probs.float().reshape(-1, router_probs.shape[-1])
        return self.config.utilization_weight * (1.0 - p.max(0).values).mean()

    def auxiliary_losses(self, router_probs: Optional[torch.Tensor] = None, expert_index: Optional[torch.Tensor] = None,
                         num_experts: Optional[int] = None) -> Dict[str, torch.Tensor]:
        lb = self._compute_load_balancing_loss(router_probs, expert_index, num_experts)
        if router_probs is None:
            z = lb.new_zeros(())
            return {"load_balancing": lb, "importance": z, "utilization": z, "total": lb}
        imp, ut = self._compute_importance_loss(router_probs), self._compute_utilization_loss(router_probs)
        return {"load_balancing": lb, "importance": imp, "utilization": ut, "total": lb + imp + ut}

    # -- front --------------------------------------------------------------------------------------------------------------------
    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs.get("model"), nn.Module)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        out: Dict[str, Any] = self.process(inputs["model"])
        if inputs.get("router_probs") is not None or inputs.get("expert_index") is not None:
            out["auxiliary"] = self.auxiliary_losses(inputs.get("router_probs"), inputs.get("expert_index"), inputs.get("num_experts"))
        return out

    def get_gradient_statistics(self) -> Dict[str, float]:
        return {k: float(v) for k, v in self._last.items()} | {"steps": float(self.steps), "history": float(min(self._hist_n, self.config.clip_history_window))}

    def reset(self) -> None:
        self._history, self._hist_n, self.steps, self._last = None, 0, 0, {}


class PiscesLxMoEGradientFacade:
    """``f = PiscesLxMoEGradientFacade(model, expert_clip_threshold=...)``; after backward ``f.process()``; inside the
    forward ``loss = loss + f.get_auxiliary_losses(probs, idx)["total"]``."""

    def __init__(self, model: nn.Module, config: Optional[PiscesLxMoEGradientConfig] = None, **overrides: Any):
        self.model = model
        self.operator = PiscesLxMoEGradientOperator(config or PiscesLxMoEGradientConfig(**overrides))
        self.classification = self.operator.classify(model)

    def process(self) -> Dict[str, torch.Tensor]:
        return self.operator.process(self.model)

    def get_auxiliary_losses(self, router_probs: Optional[torch.Tensor] = None, expert_index: Optional[torch.Tensor] = None,
                             num_experts: Optional[int] = None) -> Dict[str, torch.Tensor]:
        return self.operator.auxiliary_losses(router_probs, expert_index, num_experts)

    def get_statistics(self) -> Dict[str, float]:
        return self.operator.get_gradient_statistics()
