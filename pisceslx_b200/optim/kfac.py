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


# ---------------------------------------------------------------------------------------------------------------------------
# The operator form (reference opss/train/kfac.py:128-1128): configuration, layer types, eigenbasis preconditioning,
# adaptive damping, statistics, and a facade for training loops.
# ---------------------------------------------------------------------------------------------------------------------------
import fnmatch
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Optional, Tuple

from ..utils.opsc import PiscesLxOperatorInterface


class PiscesLxKFacLayerType(str, Enum):
    LINEAR = "linear"            # nn.Linear: hooks on the module
    EMBEDDING = "embedding"      # nn.Embedding: diagonal input factor (token counts)
    FUNCTIONAL = "functional"    # a 2-D parameter used through a functional linear: captured by ``capture()``
    UNSUPPORTED = "unsupported"


@dataclass
class PiscesLxKFacConfig:
    damping: float = 1e-3
    update_freq: int = 100
    diag_first: bool = False            # keep only the diagonal of the input factor (memory of O(n) instead of O(n^2))
    adaptive_damping: bool = True
    damping_upper_bound: float = 1.0
    damping_lower_bound: float = 1e-8
    damping_scale_factor: float = 0.95
    momentum: float = 0.95
    include_bias: bool = True
    include_embedding: bool = False
    clip_gradients: bool = True
    grad_clip_norm: float = 1.0
    use_eigen_decomp: bool = True
    layer_selection: List[str] = field(default_factory=list)
    layer_exclusion: List[str] = field(default_factory=list)
    warmup_steps: int = 100
    max_dim: int = 8192
    keep_gradient_norm: bool = True     # rescale the preconditioned gradient to the raw gradient's norm

    def __post_init__(self) -> None:
        if not 0 <= self.momentum < 1:
            raise ValueError("momentum must be in [0, 1)")
        if not self.damping_lower_bound <= self.damping <= self.damping_upper_bound:
            raise ValueError("damping must lie inside its bounds")
        if not 0 < self.damping_scale_factor < 1:
            raise ValueError("damping_scale_factor must be in (0, 1)")


class PiscesLxKFacOperator(PiscesLxOperatorInterface):
    """Kronecker-factored natural gradient.  For a layer y = W a (+ b) the Fisher block is approximated by G (x) A with
    A = E[a a^T] (inputs, with a constant 1 appended when the bias is included) and G = E[g g^T] (gradients with
    respect to y).  The preconditioned gradient is the EXACT damped inverse of that Kronecker product, applied in the
    eigenbasis:  Q_G [ (Q_G^T dW Q_A) / (lambda_G lambda_A^T + damping) ] Q_A^T.

    The reference divides by ``(lambda_G + damping)`` row-wise only and rotates with the input basis on both sides
    (kfac.py:705-712); that is not an inverse of the curvature.

    Layers: ``register_hooks(model)`` covers ``nn.Linear`` (and ``nn.Embedding`` when enabled); parameters that are used
    through a functional linear - this framework's own layers hold bare ``nn.Parameter`` weights - are registered with
    ``register_functional({name: parameter})`` and observed inside ``with op.capture(): loss = model(...)``.

    Adaptive damping: after every preconditioning the ratio of the gradient norms (after / before, measured before the
    optional rescaling) is compared with 1: an update that shrank below half asks for less damping, one that more than
    doubled for more; the value stays inside its bounds."""

    name = "kfac"

    def __init__(self, config: Optional[PiscesLxKFacConfig] = None):
        self.config = config or PiscesLxKFacConfig()
        self.damping = self.config.damping
        self.layer_info: Dict[str, Dict[str, Any]] = {}
        self.cov_a: Dict[str, torch.Tensor] = {}
        self.cov_g: Dict[str, torch.Tensor] = {}
        self.eigen_a: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.eigen_g: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._handles: List[Any] = []
        self._functional: Dict[int, str] = {}
        self.steps = 0
        self._stats = {"updates": 0, "preconditioned_layers": 0, "norm_before": 0.0, "norm_after": 0.0, "eig_refreshes": 0}

    # -- selection ------------------------------------------------------------------------------------------------------------
    def _selected(self, name: str) -> bool:
        c = self.config
        if c.layer_selection and not any(fnmatch.fnmatch(name, p) or p in name for p in c.layer_selection):
            return False
        return not any(fnmatch.fnmatch(name, p) or p in name for p in c.layer_exclusion)

    def _detect_layer_type(self, module: Any) -> PiscesLxKFacLayerType:
        if isinstance(module, nn.Linear):
            return PiscesLxKFacLayerType.LINEAR if max(module.weight.shape) <= self.config.max_dim else PiscesLxKFacLayerType.UNSUPPORTED
        if isinstance(module, nn.Embedding):
            return PiscesLxKFacLayerType.EMBEDDING if self.config.include_embedding else PiscesLxKFacLayerType.UNSUPPORTED
        return PiscesLxKFacLayerType.UNSUPPORTED

    # -- statistics collection ------------------------------------------------------------------------------------------------
    def _ema(self, store: Dict[str, torch.Tensor], key: str, value: torch.Tensor) -> None:
        m = self.config.momentum
        store[key] = value if key not in store else store[key].mul_(m).add_(value, alpha=1 - m)

    def _observe_input(self, key: str, a: torch.Tensor, bias: bool, diag: bool) -> None:
        a = a.detach().reshape(-1, a.shape[-1]).float()
        if bias:
            a = torch.cat([a, a.new_ones(a.shape[0], 1)], 1)
        n = max(a.shape[0], 1)
        self._ema(self.cov_a, key, (a * a).sum(0) / n if diag else a.t() @ a / n)

    def _observe_grad(self, key: str, g: torch.Tensor) -> None:
        g = g.detach().reshape(-1, g.shape[-1]).float()
        n = max(g.shape[0], 1)
        g = g * n                                           # a mean-reduced loss scales every row's gradient by 1 / n
        self._ema(self.cov_g, key, g.t() @ g / n)

    def register_hooks(self, model: nn.Module) -> List[Any]:
        c = self.config
        for name, m in model.named_modules():
            kind = self._detect_layer_type(m)
            if kind is PiscesLxKFacLayerType.UNSUPPORTED or not self._selected(name):
                continue
            bias = c.include_bias and getattr(m, "bias", None) is not None and kind is PiscesLxKFacLayerType.LINEAR
            self.layer_info[name] = {"module": m, "type": kind, "bias": bias, "weight": m.weight}

            def fwd(mod, args, _n=name, _k=kind, _b=bias):
                if not (mod.training and torch.is_grad_enabled()):
                    return
                if _k is PiscesLxKFacLayerType.EMBEDDING:
                    cnt = torch.bincount(args[0].reshape(-1), minlength=mod.num_embeddings).float() / max(args[0].numel(), 1)
                    self._ema(self.cov_a, _n, cnt)
                else:
                    self._observe_input(_n, args[0], _b, c.diag_first)

            def bwd(mod, gin, gout, _n=name):
                if gout[0] is not None:
                    self._observe_grad(_n, gout[0])
            self._handles += [m.register_forward_pre_hook(fwd), m.register_full_backward_hook(bwd)]
        return list(self._handles)

    def register_functional(self, params: Dict[str, torch.nn.Parameter]) -> int:
        n = 0
        for name, p in params.items():
            if p.dim() == 2 and max(p.shape) <= self.config.max_dim and self._selected(name):
                self.layer_info[name] = {"module": None, "type": PiscesLxKFacLayerType.FUNCTIONAL, "bias": False, "weight": p}
                self._functional[id(p)] = name
                n += 1
        return n

    def capture(self):
        """Context manager: while active, every ``ops.functional.linear(x, w)`` whose ``w`` was registered records the
        input factor and hooks the output for the gradient factor."""
        from ..ops import functional as F_
        op = self

        class _Capture:
            def __enter__(self_inner):
                self_inner.orig = F_.linear

                def linear(x, w, *a, **k):
                    y = self_inner.orig(x, w, *a, **k)
                    name = op._functional.get(id(w))
                    if name is not None and torch.is_grad_enabled() and y.requires_grad:
                        op._observe_input(name, x, False, op.config.diag_first)
                        y.register_hook(lambda g, _n=name: op._observe_grad(_n, g))
                    return y
                F_.linear = linear
                return op

            def __exit__(self_inner, *exc):
                F_.linear = self_inner.orig
                return False
        return _Capture()

    # -- inverses ---------------------------------------------------------------------------------------------------------------
    @staticmethod
    def _compute_eigen_decomposition(c: torch.Tensor) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        if c.dim() == 1:
            return c.clamp_min(0), None
        sym = 0.5 * (c + c.t())
        vals, vecs = torch.linalg.eigh(sym.double())
        return vals.clamp_min(0).float(), vecs.float()

    def update_matrices(self, force: bool = False) -> int:
        """Refresh the eigendecompositions (every ``update_freq`` steps, or now with ``force``); returns how many layers
        were refreshed."""
        if not force and self.steps % max(self.config.update_freq, 1) != 0 and self.eigen_a:
            return 0
        n = 0
        for key in self.layer_info:
            if key in self.cov_a and key in self.cov_g:
                self.eigen_a[key] = self._compute_eigen_decomposition(self.cov_a[key])
                self.eigen_g[key] = self._compute_eigen_decomposition(self.cov_g[key])
                n += 1
        self._stats["eig_refreshes"] += int(n > 0)
        return n

    def _precondition_one(self, key: str, grad: torch.Tensor, bias_grad: Optional[torch.Tensor]) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        la, qa = self.eigen_a[key]
        lg, qg = self.eigen_g[key]
        g = grad.float()
        if bias_grad is not None:
            g = torch.cat([g, bias_grad.float().unsqueeze(1)], 1)
        kind = self.layer_info[key]["type"]
        if kind is PiscesLxKFacLayerType.EMBEDDING:           # weight [V, D]: rows indexed by tokens (diag A), columns by G
            t = g @ qg
            t = t / (la[:, None] * lg[None, :] + self.damping)
            out = t @ qg.t()
        elif qa is None:                                       # diagonal input factor
            t = qg.t() @ g
            t = t / (lg[:, None] * la[None, :] + self.damping)
            out = qg @ t
        else:
            t = qg.t() @ g @ qa
            t = t / (lg[:, None] * la[None, :] + self.damping)
            out = qg @ t @ qa.t()
        if bias_grad is not None:
            return out[:, :-1], out[:, -1]
        return out, None

    @torch.no_grad()
    def precondition_gradients(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Rewrite the gradients of every observed layer in place; returns (norm before, norm after) as tensors.  During
        the warm-up steps only the statistics are collected."""
        c = self.config
        self.steps += 1
        zero = torch.zeros(())
        if self.steps <= c.warmup_steps:
            return zero, zero
        self.update_matrices()
        before, after, n = [], [], 0
        for key, info in self.layer_info.items():
            w = info["weight"]
            if w.grad is None or key not in self.eigen_a or key not in self.eigen_g:
                continue
            b = info["module"].bias if info["bias"] else None
            bg = b.grad if b is not None and b.grad is not None else None
            if info["bias"] and bg is None:
                continue
            new_w, new_b = self._precondition_one(key, w.grad, bg)
            nb = w.grad.float().norm()
            na = new_w.norm()
            if c.keep_gradient_norm:
                s = nb / na.clamp_min(1e-12)
                new_w = new_w * s
                new_b = new_b * s if new_b is not None else None
            w.grad.copy_(new_w.to(w.grad.dtype))
            if new_b is not None:
                b.grad.copy_(new_b.to(b.grad.dtype))
            before.append(nb)
            after.append(na)
            n += 1
        if not n:
            return zero, zero
        nb_t, na_t = torch.stack(before).norm(), torch.stack(after).norm()
        self._update_adaptive_damping(nb_t, na_t)
        if c.clip_gradients and c.grad_clip_norm > 0:
            torch.nn.utils.clip_grad_norm_([i["weight"] for i in self.layer_info.values() if i["weight"].grad is not None], c.grad_clip_norm)
        s = self._stats
        s["updates"] += 1
        s["preconditioned_layers"] = n
        s["norm_before"], s["norm_after"] = nb_t, na_t
        return nb_t, na_t

    def _update_adaptive_damping(self, norm_before: torch.Tensor, norm_after: torch.Tensor) -> None:
        c = self.config
        if not c.adaptive_damping:
            return
        ratio = float(norm_after / norm_before.clamp_min(1e-12))
        if ratio < 0.5:
            self.damping = max(self.damping * c.damping_scale_factor, c.damping_lower_bound)
        elif ratio > 2.0:
            self.damping = min(self.damping / c.damping_scale_factor, c.damping_upper_bound)

    def _compute_curvature_factor(self) -> float:
        """Mean over layers of mean( lambda / (lambda + damping) ) over the Kronecker spectrum: near 1 the curvature
        dominates the damping (a natural-gradient step), near 0 the step is plain gradient descent."""
        vals = []
        for k in self.eigen_a:
            if k in self.eigen_g:
                prod = self.eigen_g[k][0][:, None] * self.eigen_a[k][0][None, :]
                vals.append((prod / (prod + self.damping)).mean())
        return float(torch.stack(vals).mean()) if vals else 0.0

    # -- operator front -----------------------------------------------------------------------------------------------------------
    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return inputs.get("action", "precondition") in ("register", "precondition", "update", "statistics", "reset")

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        a = inputs.get("action", "precondition")
        if a == "register":
            return {"hooks": len(self.register_hooks(inputs["model"])), "layers": len(self.layer_info)}
        if a == "precondition":
            nb, na = self.precondition_gradients()
            return {"norm_before": nb, "norm_after": na, "damping": self.damping, "step": self.steps}
        if a == "update":
            return {"refreshed": self.update_matrices(force=True)}
        if a == "reset":
            self.reset()
            return {}
        return self.get_statistics()

    def get_covariance_matrices(self) -> Dict[str, Dict[str, torch.Tensor]]:
        return {k: {"A": self.cov_a[k], "G": self.cov_g[k]} for k in self.layer_info if k in self.cov_a and k in self.cov_g}

    def get_statistics(self) -> Dict[str, Any]:
        s = dict(self._stats)
        s.update(steps=self.steps, damping=self.damping, layers=len(self.layer_info), observed=len(self.get_covariance_matrices()),
                 curvature_factor=self._compute_curvature_factor(),
                 norm_before=float(s["norm_before"]), norm_after=float(s["norm_after"]))
        return s

    def reset(self) -> None:
        self.cov_a.clear(), self.cov_g.clear(), self.eigen_a.clear(), self.eigen_g.clear()
        self.steps, self.damping = 0, self.config.damping

    def remove_hooks(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles.clear()


class PiscesLxKFacFacade:
    """For a training loop:  ``k = PiscesLxKFacFacade(model, damping=...)`` once;  after ``loss.backward()`` call
    ``k.precondition_gradients()``, then the optimizer's step.  ``cleanup()`` removes the hooks."""

    def __init__(self, model: Optional[nn.Module] = None, config: Optional[PiscesLxKFacConfig] = None, **overrides: Any):
        cfg = config or PiscesLxKFacConfig(**overrides)
        self.operator = PiscesLxKFacOperator(cfg)
        if model is not None:
            self.register_hooks(model)

    def register_hooks(self, model: nn.Module) -> None:
        self.operator.register_hooks(model)

    def precondition_gradients(self) -> Dict[str, Any]:
        nb, na = self.operator.precondition_gradients()
        return {"norm_before": float(nb), "norm_after": float(na), "damping": self.operator.damping}

    def update_matrices(self, force: bool = True) -> Dict[str, Any]:
        return {"refreshed": self.operator.update_matrices(force)}

    def get_statistics(self) -> Dict[str, Any]:
        return self.operator.get_statistics()

    def cleanup(self) -> None:
        self.operator.remove_hooks()
