"""Model growth as classes with an operator front (reference opss/train/growth.py:75-688) and the scaling-law
operator (reference opss/scaling/__init__.py:53-341).

The growth primitives of ``engine/alignment.py`` (``grow_depth``, ``grow_experts``, ``grow_expert_width``) do the tensor
surgery on this framework's stacked expert weights; the classes here choose what to grow from a
``PiscesLxModelGrowthConfig`` and add the missing dimension, ``grow_hidden``: a FUNCTION-PRESERVING growth of the
hidden size.  New residual channels start at exactly zero (embedding columns, output rows of every projection that
writes the residual stream), every projection that reads the stream gets small random columns for them (they multiply
zeros until training moves the channels), and the RMSNorm weights of the old channels are scaled by
sqrt(old / new) because the mean square is now taken over more channels.  The model computes the same logits right
after growing.  (The reference pads only the input side of the attention projections with noise, leaves the norms,
the experts and the output sides untouched and so breaks the model's shapes, growth.py:392-424.)

The scaler uses this framework's own parameter count (``YvConfig.param_counts``) and takes the sustained throughput
of the hardware as an argument, where the reference hard-codes an A100 figure and an approximate 12 h^2 per layer."""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..utils.opsc import PiscesLxOperatorInterface
from .alignment import grow_depth, grow_expert_width, grow_experts


class PiscesLxGrowthType(str, Enum):
    DEPTH = "depth"
    WIDTH = "width"
    EXPERT = "expert"
    HYBRID = "hybrid"


@dataclass
class PiscesLxModelGrowthConfig:
    growth_type: str = "depth"
    num_new_layers: int = 4
    new_hidden_size: Optional[int] = None
    new_expert_ffn: Optional[int] = None
    num_new_experts: int = 8
    preserve_knowledge: bool = True
    init_noise_scale: float = 0.01
    layer_copy_strategy: str = "last"            # "last" | "middle" | "uniform" | "interleave"

    def __post_init__(self) -> None:
        self.growth_type = PiscesLxGrowthType(getattr(self.growth_type, "value", self.growth_type)).value
        if self.layer_copy_strategy not in ("last", "middle", "uniform", "interleave"):
            raise ValueError(f"unknown layer_copy_strategy {self.layer_copy_strategy!r}")


def _layers(model: nn.Module) -> nn.ModuleList:
    trunk = getattr(model, "model", model)
    if not hasattr(trunk, "layers"):
        raise ValueError("the model has no .layers / .model.layers")
    return trunk.layers


class PiscesLxDepthGrower:
    """Adds ``num_new_layers`` blocks as copies of existing ones placed right after their source: after the last block
    ("last"), after the middle one ("middle"), after blocks spread evenly over the depth ("uniform" / "interleave").
    With ``preserve_knowledge`` the copies' output projections are zero, so each copy adds nothing to the residual
    stream at first and the model's function is unchanged; without it the copies keep their weights plus noise."""

    def __init__(self, config: PiscesLxModelGrowthConfig):
        self.config = config

    def positions(self, n_existing: int) -> List[int]:
        c, k = self.config, self.config.num_new_layers
        if c.layer_copy_strategy == "last":
            return [n_existing - 1] * k
        if c.layer_copy_strategy == "middle":
            return [n_existing // 2] * k
        return [min(n_existing - 1, int((i + 0.5) * n_existing / k)) for i in range(k)]

    def grow(self, model: nn.Module) -> nn.Module:
        c = self.config
        n = len(_layers(model))
        pos = self.positions(n)
        if c.preserve_knowledge:
            grow_depth(model, pos)                          # one zero-output copy per listed index
        else:
            layers = list(_layers(model))
            for p in sorted(pos, reverse=True):
                clone = copy.deepcopy(layers[p])
                with torch.no_grad():
                    for q in clone.parameters():
                        q.add_(torch.randn_like(q) * c.init_noise_scale)
                layers.insert(p + 1, clone)
            for i, blk in enumerate(layers):
                blk.layer_idx = i
                if hasattr(blk, "attention"):
                    blk.attention.layer_idx = i
            trunk = getattr(model, "model", model)
            trunk.layers = nn.ModuleList(layers)
            trunk.layer_hi = len(layers)
            model.cfg.n_layer = len(layers)
        return model


def _pad_last(w: torch.Tensor, new: int, std: float) -> torch.Tensor:
    out = torch.zeros(*w.shape[:-1], new, dtype=w.dtype, device=w.device)
    out[..., : w.shape[-1]] = w
    if std > 0:
        out[..., w.shape[-1]:].normal_(std=std)
    return out


def _pad_dim(w: torch.Tensor, dim: int, new: int) -> torch.Tensor:
    shape = list(w.shape)
    shape[dim] = new
    out = torch.zeros(shape, dtype=w.dtype, device=w.device)
    out.narrow(dim, 0, w.shape[dim]).copy_(w)
    return out


@torch.no_grad()
def grow_hidden(model: nn.Module, new_hidden: int, init_noise_scale: float = 0.01) -> nn.Module:
    """Function-preserving growth of the hidden size of a ``YvModelForCausalLM`` with standard attention blocks (the
    head dimension and the head counts stay, so the attention inner width is unchanged).  See the module docstring for
    the rule per tensor.  Optional components that carry their own hidden-size tensors (FiLM fields, SSM branch,
    multimodal encoders, latent attention) are not handled and raise."""
    cfg = model.cfg
    old = cfg.hidden_size
    if new_hidden <= old:
        raise ValueError(f"new_hidden ({new_hidden}) must exceed the current hidden size ({old})")
    trunk = model.model
    for attr in ("subconscious", "block_field", "vision_encoder", "video_encoder", "audio_encoder", "modal_fusion"):
        if getattr(trunk, attr, None) is not None:
            raise NotImplementedError(f"grow_hidden does not handle the attached component {attr!r}")
    ratio = math.sqrt(old / new_hidden)
    P = nn.Parameter
    s = init_noise_scale

    def norm(n: nn.Module) -> None:
        w = torch.ones(new_hidden, dtype=n.weight.dtype, device=n.weight.device)
        w[:old] = n.weight * ratio
        n.weight = P(w)
        for a in ("dim", "hidden", "normalized_shape"):
            if isinstance(getattr(n, a, None), int):
                setattr(n, a, new_hidden)

    if hasattr(trunk, "embed"):
        trunk.embed.weight = P(_pad_last(trunk.embed.weight, new_hidden, 0.0))
        trunk.embed.embedding_dim = new_hidden
    for blk in trunk.layers:
        att, mlp = blk.attention, blk.mlp
        if not (hasattr(att, "qkv_proj") and hasattr(att, "o_proj")) or getattr(blk, "ssm", None) is not None:
            raise NotImplementedError("grow_hidden handles the standard attention block only")
        norm(blk.norm_attention)
        norm(blk.norm_mlp)
        att.qkv_proj = P(_pad_last(att.qkv_proj, new_hidden, s))            # reads the stream
        att.o_proj = P(_pad_dim(att.o_proj, 0, new_hidden))                # writes the stream: new rows zero
        if hasattr(mlp, "experts_w13"):
            mlp.experts_w13 = P(_pad_last(mlp.experts_w13, new_hidden, s))
            mlp.experts_w2 = P(_pad_dim(mlp.experts_w2, 1, new_hidden))
            if getattr(mlp, "num_shared", 0):
                mlp.shared_w13 = P(_pad_last(mlp.shared_w13, new_hidden, s))
                mlp.shared_w2 = P(_pad_dim(mlp.shared_w2, 0, new_hidden))
            g = mlp.router.gate
            ng = nn.Linear(new_hidden, g.out_features, bias=False).to(g.weight.device, g.weight.dtype)
            ng.weight.copy_(_pad_last(g.weight, new_hidden, 0.0))
            mlp.router.gate = ng
            mlp.router.__dict__.pop("_gate_bf16", None)
        else:
            mlp.w13 = P(_pad_last(mlp.w13, new_hidden, s))
            mlp.w2 = P(_pad_dim(mlp.w2, 0, new_hidden))
            mlp.hidden = new_hidden
    if hasattr(trunk, "norm"):
        norm(trunk.norm)
    if hasattr(model, "lm_head"):
        model.lm_head = P(_pad_last(model.lm_head, new_hidden, s))
    for i in range(len(getattr(model, "mtp_heads", []))):
        model.mtp_heads[i] = P(_pad_last(model.mtp_heads[i], new_hidden, s))
    cfg.hidden_size = new_hidden
    return model


class PiscesLxWidthGrower:
    """Hidden size (``new_hidden_size``) and / or the experts' feed-forward width (``new_expert_ffn``), both function
    preserving."""

    def __init__(self, config: PiscesLxModelGrowthConfig):
        self.config = config

    def grow(self, model: nn.Module) -> nn.Module:
        c = self.config
        if c.new_hidden_size is None and c.new_expert_ffn is None:
            raise ValueError("width growth needs new_hidden_size or new_expert_ffn")
        if c.new_expert_ffn is not None:
            for blk in _layers(model):
                if hasattr(blk.mlp, "experts_w13"):
                    grow_expert_width(blk.mlp, c.new_expert_ffn)
            model.cfg.moe_expert_intermediate_size = c.new_expert_ffn
        if c.new_hidden_size is not None:
            grow_hidden(model, c.new_hidden_size, c.init_noise_scale)
        return model


class PiscesLxExpertGrower:
    """Adds ``num_new_experts`` routed experts to every MoE layer as noisy copies of existing ones with copied router
    rows.  The top-k stays, so a token whose best expert now has a twin takes the twin as its second choice and drops
    the expert that used to be second: this growth is NOT function preserving (depth and width growth are); the loss
    rises a little and recovers within a few hundred steps as the twins drift apart."""

    def __init__(self, config: PiscesLxModelGrowthConfig):
        self.config = config

    def grow(self, model: nn.Module) -> nn.Module:
        c = self.config
        grown = 0
        for blk in _layers(model):
            if hasattr(blk.mlp, "experts_w13"):
                grow_experts(blk.mlp, blk.mlp.experts_w13.shape[0] + c.num_new_experts, c.init_noise_scale if not c.preserve_knowledge else min(c.init_noise_scale, 1e-3))
                grown = blk.mlp.experts_w13.shape[0]
        if grown:
            model.cfg.moe_num_experts = grown
        return model


class PiscesLxModelGrowthOperator(PiscesLxOperatorInterface):
    """inputs: {"model": module, optional "config": PiscesLxModelGrowthConfig or dict}; output: parameter counts before
    and after and what was grown.  "hybrid" applies depth, then experts, then width."""

    name = "model_growth"

    def __init__(self, config: Optional[PiscesLxModelGrowthConfig] = None):
        self.config = config or PiscesLxModelGrowthConfig()

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs.get("model"), nn.Module)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        cfg = inputs.get("config", self.config)
        if isinstance(cfg, dict):
            cfg = PiscesLxModelGrowthConfig(**cfg)
        model = inputs["model"]
        count = lambda: sum(p.numel() for p in model.parameters())
        before = count()
        steps = {"depth": [PiscesLxDepthGrower], "width": [PiscesLxWidthGrower], "expert": [PiscesLxExpertGrower],
                 "hybrid": [PiscesLxDepthGrower, PiscesLxExpertGrower, PiscesLxWidthGrower]}[cfg.growth_type]
        done = []
        for g in steps:
            if g is PiscesLxWidthGrower and cfg.new_hidden_size is None and cfg.new_expert_ffn is None:
                continue
            g(cfg).grow(model)
            done.append(g.__name__)
        return {"model": model, "parameters_before": before, "parameters_after": count(), "applied": done,
                "layers": len(_layers(model)), "hidden_size": model.cfg.hidden_size}

    def grow(self, model: nn.Module, config: Optional[PiscesLxModelGrowthConfig] = None) -> nn.Module:
        r = self.execute({"model": model, "config": config or self.config})
        if not r.is_success():
            raise RuntimeError(r.error)
        return r.output["model"]


# ---------------------------------------------------------------------------------------------------------------- scaling laws
@dataclass
class PiscesLxScalingConfig:
    compute_budget: float = 1e21
    budget_unit: str = "flops"                   # "flops" | "gpu_hours"
    tokens_per_parameter: float = 20.0
    sustained_flops_per_gpu: float = 1.4e15      # bf16 dense GEMM throughput of one B200 under its power cap
    model_flops_utilization: float = 0.4
    enable_memory_correction: bool = True


@dataclass
class PiscesLxScalingResult:
    optimal_parameters: float
    optimal_tokens: float
    compute_efficiency: float
    recommended_config: Optional[Dict[str, Any]] = None
    memory_correction: Optional[float] = None
    gpu_hours: Optional[float] = None


class PiscesLxChinchillaScaler:
    """C = 6 N D with D = r N (r tokens per parameter, 20 by default): N = sqrt(C / (6 r)), D = r N.  For
    mixture-of-experts models N is the ACTIVE parameter count (what a token's FLOPs pay for)."""

    def __init__(self, config: Optional[PiscesLxScalingConfig] = None):
        self.config = config or PiscesLxScalingConfig()

    def to_flops(self, budget: float, unit: str = "flops") -> float:
        c = self.config
        return budget * 3600.0 * c.sustained_flops_per_gpu * c.model_flops_utilization if unit == "gpu_hours" else budget

    def optimal_nd(self, c_budget: float, unit: str = "flops") -> Tuple[float, float]:
        r = self.config.tokens_per_parameter
        n = math.sqrt(self.to_flops(c_budget, unit) / (6.0 * r))
        return n, r * n

    @staticmethod
    def estimate_params(cfg: Any) -> Dict[str, float]:
        """Total and active parameter counts of a ``YvConfig`` (its own accounting)."""
        pc = cfg.count_parameters() if hasattr(cfg, "count_parameters") else None
        if isinstance(pc, dict):
            return {"total": float(pc.get("total", 0)), "active": float(pc.get("active", pc.get("total", 0)))}
        if isinstance(pc, (tuple, list)) and len(pc) >= 2:
            return {"total": float(pc[0]), "active": float(pc[1])}
        raise ValueError("the configuration does not report parameter counts")

    def get_config_for_params(self, target_active_params: float, presets: Optional[Dict[str, Any]] = None) -> Tuple[str, Any, Dict[str, float]]:
        """The preset whose active parameter count is closest (in log space) to the target."""
        if presets is None:
            from ..config import YvConfig
            presets = {}
            for nm in ("get_small", "get_base", "get_large", "get_xl", "yv_7b_moe", "flagship"):
                f = getattr(YvConfig, nm, None)
                if callable(f):
                    try:
                        presets[nm] = f()
                    except TypeError:
                        continue
        best = min(presets.items(), key=lambda kv: abs(math.log(max(self.estimate_params(kv[1])["active"], 1.0) / target_active_params)))
        return best[0], best[1], self.estimate_params(best[1])

    @staticmethod
    def chinchilla_memory_correction(base_memory: float, enabled: bool, optimal_params: float, original_params: float) -> float:
        """A model trimmed towards the compute-optimal size needs proportionally less state: scale the estimate by the
        parameter ratio, never below a tenth (activations and buffers do not shrink with the parameters)."""
        if not enabled or original_params <= 0 or optimal_params >= original_params:
            return base_memory
        return base_memory * max(0.1, optimal_params / original_params)

    def plan(self, c_budget: Optional[float] = None, unit: Optional[str] = None) -> PiscesLxScalingResult:
        c = self.config
        budget, unit = c.compute_budget if c_budget is None else c_budget, unit or c.budget_unit
        n, d = self.optimal_nd(budget, unit)
        name, cfg, counts = self.get_config_for_params(n)
        flops = self.to_flops(budget, unit)
        spent = 6.0 * counts["active"] * d
        return PiscesLxScalingResult(n, d, min(flops, spent) / max(flops, spent),
                                     {"preset": name, "layers": cfg.n_layer, "hidden_size": cfg.hidden_size,
                                      "total_params": counts["total"], "active_params": counts["active"]},
                                     None, flops / (3600.0 * c.sustained_flops_per_gpu * c.model_flops_utilization))


class PiscesLxScalingOperator(PiscesLxOperatorInterface):
    """operation "optimal" (budget -> N, D, nearest preset, GPU hours), "estimate" (config -> parameter counts),
    "memory" (base memory, original and optimal parameters -> corrected memory)."""

    name = "scaling"

    def __init__(self, config: Optional[PiscesLxScalingConfig] = None):
        self.config = config or PiscesLxScalingConfig()
        self.scaler = PiscesLxChinchillaScaler(self.config)

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return inputs.get("operation", "optimal") in ("optimal", "estimate", "memory")

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        op = inputs.get("operation", "optimal")
        if op == "optimal":
            r = self.scaler.plan(inputs.get("compute_budget"), inputs.get("budget_unit"))
            return {"optimal_parameters": r.optimal_parameters, "optimal_tokens": r.optimal_tokens,
                    "compute_efficiency": r.compute_efficiency, "recommended_config": r.recommended_config, "gpu_hours": r.gpu_hours}
        if op == "estimate":
            return self.scaler.estimate_params(inputs["config"])
        return {"memory_correction": self.scaler.chinchilla_memory_correction(
            float(inputs["base_memory"]), bool(inputs.get("chinchilla_enabled", self.config.enable_memory_correction)),
            float(inputs["optimal_params"]), float(inputs["original_params"]))}
