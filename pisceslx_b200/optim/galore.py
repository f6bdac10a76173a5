"""GaLore as a configured operator and a training-loop adapter (reference opss/optim/galore.py:60-520; Zhao et al.,
"GaLore: Memory-Efficient LLM Training by Gradient Low-Rank Projection", arXiv:2403.03507).

Two modes:
* ``filter`` (what the reference operator does, galore.py:388-430): the gradient is replaced by its projection onto the
  top-``rank`` subspace and back, G P P^T x scale, and whatever optimizer follows sees the filtered gradient.  Its
  moments stay full size, so this saves nothing by itself.
* ``lowrank`` (the method of the paper): Adam moments are kept for the PROJECTED gradient [n, r] only and the update is
  projected back, which is where the memory goes away: 2 n m floats of state become 2 n r + m r.

The basis: the reference calls ``torch.svd_lowrank`` / a full SVD per matrix.  Here the default is a randomised range
finder with subspace iteration - G^T (G Omega), re-orthonormalised by a thin QR of an [m, r] matrix - which is GEMM work
on the gradient plus a small factorisation, against a full SVD of a 4096 x 11008 matrix; ``proj_type="std"`` keeps the
exact SVD.  A refresh starts from the previous basis (one iteration from a warm start tracks a slowly turning subspace).

The stored basis can be 8-bit (a scale per column) or 4-bit (two codes per byte, a scale per column); the reference keeps
one scale for the whole matrix and stores 4-bit codes one per int8 byte (galore.py:374-386).

The rank adapts from the share of the gradient's energy the basis captures, looked at every ``rank_adapt_interval``
steps (the only host read, since a new rank changes shapes)."""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from ..utils.opsc import PiscesLxOperatorInterface
from .ink_extras import pack_nibbles, unpack_nibbles

QuantBasis = Tuple[torch.Tensor, torch.Tensor, int, int]          # codes, per-column scale, bits, rows


@dataclass
class PiscesLxGaLoreConfig:
    name: str = "galore"
    rank: int = 128
    update_proj_gap: int = 50
    scale: float = 1.0
    proj_type: str = "rand"                 # "rand": randomised subspace iteration; "std": exact SVD
    quantization_bits: int = 8              # 0 keeps the basis in the gradient's dtype; 8 / 4 store codes
    lr_ratio: float = 1.0
    min_rank: int = 32
    max_rank: int = 512
    rank_adapt_interval: int = 1000
    rank_adapt_threshold: float = 0.1
    memory_efficient: bool = False
    moe_expert_only: bool = False
    use_int4_projection: bool = False       # shorthand for quantization_bits = 4
    adaptive_rank_update: bool = True
    convergence_threshold: float = 0.01
    mode: str = "filter"                    # "filter" | "lowrank"
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    subspace_iterations: int = 1
    min_dim: int = 2                        # matrices whose short side is not above the rank are left alone

    def __post_init__(self) -> None:
        if self.rank <= 0 or self.update_proj_gap <= 0 or self.scale <= 0:
            raise ValueError("rank, update_proj_gap and scale must be positive")
        if self.proj_type not in ("rand", "std"):
            raise ValueError(f"unknown proj_type {self.proj_type}")
        if self.mode not in ("filter", "lowrank"):
            raise ValueError(f"unknown mode {self.mode}")
        if self.use_int4_projection:
            self.quantization_bits = 4
        if self.quantization_bits not in (0, 4, 8):
            raise ValueError("quantization_bits must be 0, 4 or 8")

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


def quantize_basis(p: torch.Tensor, bits: int) -> QuantBasis:
    qmax = 127 if bits == 8 else 7
    scale = p.float().abs().amax(0, keepdim=True).clamp_min(1e-12) / qmax
    q = (p.float() / scale).round().clamp(-qmax - 1, qmax).to(torch.int8)
    if bits == 4:
        flat = q.flatten()
        if flat.numel() % 2:
            flat = torch.cat([flat, flat.new_zeros(1)])
        return pack_nibbles(flat), scale, 4, p.shape[0]
    return q, scale, 8, p.shape[0]


def dequantize_basis(b: Union[torch.Tensor, QuantBasis], dtype: torch.dtype = torch.float32) -> torch.Tensor:
    if isinstance(b, torch.Tensor):
        return b.to(dtype)
    codes, scale, bits, rows = b
    cols = scale.shape[-1]
    if bits == 4:
        q = unpack_nibbles(codes)[: rows * cols].view(rows, cols).float()
    else:
        q = codes.float()
    return (q * scale).to(dtype)


def basis_bytes(b: Union[torch.Tensor, QuantBasis, None]) -> int:
    if b is None:
        return 0
    if isinstance(b, torch.Tensor):
        return b.numel() * b.element_size()
    return b[0].numel() * b[0].element_size() + b[1].numel() * b[1].element_size()


class PiscesLxGaLoreOperator(PiscesLxOperatorInterface):
    name = "galore"
    version = "1.0.0"

    # -- which parameters ----------------------------------------------------------------------------------------------------------
    @staticmethod
    def _eligible(name: str, p: torch.Tensor, cfg: PiscesLxGaLoreConfig, rank: int) -> bool:
        if p.dim() < 2 or min(p.shape[-1], p.numel() // p.shape[-1]) <= max(rank, cfg.min_dim - 1):
            return False
        return (not cfg.moe_expert_only) or ("expert" in name)

    def _initialize_galore_state(self, model: nn.Module, config: PiscesLxGaLoreConfig) -> Dict[str, Any]:
        return {"step": 0, "rank": config.rank, "update_proj_gap": config.update_proj_gap, "proj_matrices": {}, "last_update_steps": {},
                "moments": {}, "energy": {}, "model_id": id(model)}

    def _should_update_projection(self, param_name: str, state: Dict[str, Any]) -> bool:
        last = state["last_update_steps"].get(param_name)
        return last is None or (state["step"] - last) >= state["update_proj_gap"]

    # -- basis ---------------------------------------------------------------------------------------------------------------------
    def _compute_projection_matrix(self, gradient: torch.Tensor, rank: int, config: Optional[PiscesLxGaLoreConfig] = None,
                                   previous: Optional[torch.Tensor] = None) -> Union[torch.Tensor, QuantBasis]:
        """Orthonormal basis [m, r] of the gradient's top right-singular subspace (the gradient is taken as [-1, m])."""
        cfg = config or PiscesLxGaLoreConfig()
        g = gradient.reshape(-1, gradient.shape[-1]).float()
        r = min(rank, g.shape[0], g.shape[1])
        if cfg.proj_type == "std":
            p = torch.linalg.svd(g, full_matrices=False)[2][:r].t().contiguous()
        else:
            if previous is not None and previous.shape == (g.shape[1], r):
                q = previous.float()
                iters = max(cfg.subspace_iterations, 1)
            else:
                gen = torch.Generator(device="cpu").manual_seed(g.shape[0] * 7919 + g.shape[1])
                q = torch.randn(g.shape[1], r, generator=gen).to(g.device)
                iters = max(cfg.subspace_iterations, 1) + 2
            for _ in range(iters):
                q = torch.linalg.qr(g.t() @ (g @ q)).Q
            p = q.contiguous()
        if cfg.quantization_bits:
            return quantize_basis(p, cfg.quantization_bits)
        return p.to(gradient.dtype)

    def _quantize_projection_int4(self, matrix: torch.Tensor) -> QuantBasis:
        return quantize_basis(matrix, 4)

    # -- the two modes -----------------------------------------------------------------------------------------------------------
    def _apply_galore_transform(self, gradient: torch.Tensor, proj_matrix: Union[None, torch.Tensor, QuantBasis], config: PiscesLxGaLoreConfig) -> torch.Tensor:
        if proj_matrix is None or gradient.dim() < 2:
            return gradient
        p = dequantize_basis(proj_matrix, torch.float32)
        g = gradient.reshape(-1, gradient.shape[-1]).float()
        return ((g @ p) @ p.t() * config.scale).view_as(gradient).to(gradient.dtype)

    def _lowrank_adam(self, name: str, param: torch.Tensor, gradient: torch.Tensor, basis: Union[torch.Tensor, QuantBasis],
                      cfg: PiscesLxGaLoreConfig, state: Dict[str, Any], previous: Optional[torch.Tensor] = None) -> None:
        """``previous`` is the basis that was just replaced (None when it was not): the first moment is carried into the new
        basis by the rotation previous^T p; the second moment has no such map and is kept as it is."""
        p = dequantize_basis(basis, torch.float32)
        low = gradient.reshape(-1, gradient.shape[-1]).float() @ p                     # [n, r]
        st = state["moments"].get(name)
        if st is None or st["m"].shape != low.shape:
            st = state["moments"][name] = {"m": torch.zeros_like(low), "v": torch.zeros_like(low), "t": 0}
        elif previous is not None and previous.shape == p.shape:
            st["m"] = st["m"] @ (previous.float().t() @ p)
        st["t"] += 1
        st["m"].mul_(cfg.beta1).add_(low, alpha=1 - cfg.beta1)
        st["v"].mul_(cfg.beta2).addcmul_(low, low, value=1 - cfg.beta2)
        upd = (st["m"] / (1 - cfg.beta1 ** st["t"])) / ((st["v"] / (1 - cfg.beta2 ** st["t"])).sqrt() + cfg.eps)
        full = (upd @ p.t()).view_as(param) * cfg.scale
        lr = cfg.lr * cfg.lr_ratio
        if cfg.weight_decay:
            param.mul_(1 - lr * cfg.weight_decay)
        param.add_(full.to(param.dtype), alpha=-lr)

    def _adapt_rank(self, state: Dict[str, Any], cfg: PiscesLxGaLoreConfig) -> None:
        if not state["energy"]:
            return
        captured = float(torch.stack(list(state["energy"].values())).mean())          # one read every rank_adapt_interval steps
        lost = 1.0 - captured
        r = state["rank"]
        if lost > cfg.rank_adapt_threshold:
            r = min(cfg.max_rank, r * 2)
        elif lost < cfg.rank_adapt_threshold * 0.25:
            r = max(cfg.min_rank, r // 2)
        if r != state["rank"]:
            state["rank"] = r
            state["proj_matrices"].clear()
            state["last_update_steps"].clear()
            state["moments"].clear()
        state["captured_energy"] = captured

    @torch.no_grad()
    def _perform_galore_step(self, model: nn.Module, gradients: Dict[str, torch.Tensor], config: PiscesLxGaLoreConfig,
                             state: Dict[str, Any]) -> Tuple[nn.Module, Dict[str, Any], Dict[str, Any]]:
        state["step"] += 1
        projected = refreshed_n = 0
        state["updated_names"] = []
        for name, param in model.named_parameters():
            if not param.requires_grad:
                continue
            grad = gradients.get(name, param.grad) if gradients else param.grad
            if grad is None:
                continue
            if not self._eligible(name, param, config, state["rank"]):
                if config.mode == "filter" and name in gradients:
                    param.grad = grad
                continue
            prev_fp = None
            if self._should_update_projection(name, state):
                prev = state["proj_matrices"].get(name)
                prev_fp = dequantize_basis(prev) if prev is not None else None
                state["proj_matrices"][name] = self._compute_projection_matrix(grad, state["rank"], config, prev_fp)
                state["last_update_steps"][name] = state["step"]
                refreshed_n += 1
                if config.adaptive_rank_update:
                    p = dequantize_basis(state["proj_matrices"][name])
                    g2 = grad.reshape(-1, grad.shape[-1]).float()
                    state["energy"][name] = (g2 @ p).pow(2).sum() / g2.pow(2).sum().clamp_min(1e-30)
            basis = state["proj_matrices"][name]
            if config.mode == "filter":
                param.grad = self._apply_galore_transform(grad, basis, config)
            else:
                self._lowrank_adam(name, param, grad, basis, config, state, prev_fp)
                state["updated_names"].append(name)
            projected += 1
        if config.adaptive_rank_update and state["step"] % config.rank_adapt_interval == 0:
            self._adapt_rank(state, config)
        full = sum(2 * p.numel() * 4 for n, p in model.named_parameters() if n in state["proj_matrices"])
        low = sum(basis_bytes(b) for b in state["proj_matrices"].values()) + sum(2 * s["m"].numel() * 4 for s in state["moments"].values())
        stats = {"step": state["step"], "active_projections": len(state["proj_matrices"]), "projected_this_step": projected,
                 "refreshed_this_step": refreshed_n, "total_parameters": sum(1 for _ in model.parameters()), "rank": state["rank"],
                 "basis_bytes": sum(basis_bytes(b) for b in state["proj_matrices"].values()),
                 "state_bytes_full_adam": full, "state_bytes_lowrank": low if config.mode == "lowrank" else None}
        return model, state, stats

    # -- front -------------------------------------------------------------------------------------------------------------------
    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs.get("model"), nn.Module)

    def validate_config(self, config: Any) -> bool:
        return isinstance(config, PiscesLxGaLoreConfig) and config.rank > 0 and config.update_proj_gap > 0 and config.scale > 0

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        model = inputs["model"]
        cfg = inputs.get("config") or PiscesLxGaLoreConfig()
        state = inputs.get("optimizer_state") or {}
        if not state or state.get("model_id") != id(model):
            state = self._initialize_galore_state(model, cfg)
        model, state, stats = self._perform_galore_step(model, inputs.get("gradients") or {}, cfg, state)
        return {"model": model, "optimizer_state": state, "statistics": stats}


class PiscesLxGaLoreOptimizerAdapter:
    """``adapter.step(model, gradients)`` after ``loss.backward()``: in ``filter`` mode the model's ``.grad`` fields now hold
    the filtered gradients for the optimizer that follows; in ``lowrank`` mode the eligible matrices have been updated and
    their ``.grad`` is cleared so that a following optimizer only touches the rest."""

    def __init__(self, config: PiscesLxGaLoreConfig):
        self.operator, self.config, self.state = PiscesLxGaLoreOperator(), config, {}

    def step(self, model: nn.Module, gradients: Optional[Dict[str, torch.Tensor]] = None) -> Tuple[nn.Module, Dict[str, Any]]:
        res = self.operator.execute({"model": model, "gradients": gradients or {}, "config": self.config, "optimizer_state": self.state})
        if not res.is_success():
            raise RuntimeError(f"GaLore optimization failed: {res.error or 'unknown error'}")
        self.state = res.output["optimizer_state"]
        if self.config.mode == "lowrank":
            done = set(self.state["updated_names"])
            for n, p in model.named_parameters():
                if n in done:
                    p.grad = None
        return res.output["model"], res.output["statistics"]

    def state_dict(self) -> Dict[str, Any]:
        return {k: v for k, v in self.state.items() if k != "model_id"}

    def load_state_dict(self, sd: Dict[str, Any], model: nn.Module) -> None:
        self.state = dict(sd, model_id=id(model))
