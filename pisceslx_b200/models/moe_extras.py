"""Expert variants and MoE training aids (reference model/moe/expert.py: ``YvStandardExpert`` / ``YvGeGLUExpert`` /
``YvMultiLayerExpert`` + factory :384-746, ``YvExpertMode.PURE_LOOKUP`` :264-272; model/moe/expert_init.py
``YvGradientClusterInitializer`` and ``YvExpertEvolution``; model/moe/regularization.py
``YvExpertDiversityRegularizer``; model/moe/layer.py ``YvDynamicMoELayer`` :519-963)."""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as F_
from .moe import YvSwiGLUExpert


class YvStandardExpert(nn.Module):
    def __init__(self, hidden: int, inner: int, activation: str = "gelu", std: float = 0.02):
        super().__init__()
        self.w1 = nn.Parameter(torch.empty(inner, hidden).normal_(std=std))
        self.w2 = nn.Parameter(torch.empty(hidden, inner).normal_(std=std))
        self.act = {"gelu": F.gelu, "relu": F.relu, "silu": F.silu}[activation]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F_.linear(self.act(F_.linear(x, self.w1)), self.w2)


class YvGeGLUExpert(nn.Module):
    def __init__(self, hidden: int, inner: int, std: float = 0.02):
        super().__init__()
        self.w13 = nn.Parameter(torch.empty(2 * inner, hidden).normal_(std=std))
        self.w2 = nn.Parameter(torch.empty(hidden, inner).normal_(std=std))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        g, u = F_.linear(x, self.w13).chunk(2, -1)
        return F_.linear(F.gelu(g) * u, self.w2)


class YvMultiLayerExpert(nn.Module):
    def __init__(self, hidden: int, inner: int, depth: int = 2, std: float = 0.02):
        super().__init__()
        self.layers = nn.ModuleList([YvStandardExpert(hidden, inner, "silu", std) for _ in range(depth)])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for l in self.layers:
            x = x + l(x)
        return x


class YvExpertFactory:
    KINDS = {"swiglu": lambda h, i, s: YvSwiGLUExpert(h, i, s), "standard": lambda h, i, s: YvStandardExpert(h, i, std=s),
             "geglu": lambda h, i, s: YvGeGLUExpert(h, i, s), "multilayer": lambda h, i, s: YvMultiLayerExpert(h, i, std=s)}

    @classmethod
    def create(cls, kind: str, hidden: int, inner: int, std: float = 0.02, pure_lookup: bool = False) -> nn.Module:
        m = cls.KINDS[kind](hidden, inner, std)
        if pure_lookup:                                   # frozen expert used as a lookup table
            for p in m.parameters():
                p.requires_grad_(False)
        return m


class YvDynamicMoELayer(nn.Module):
    """MoE layer over a ``ModuleList`` of arbitrary experts (any kind from the factory), routed by a plain top-k gate.
    This is the flexible form; the trunk's ``YvDeepSeekMoELayer`` keeps SwiGLU experts stacked for the grouped GEMM."""

    def __init__(self, hidden: int, inner: int, num_experts: int, top_k: int = 2, kind: str = "swiglu",
                 num_shared: int = 0, std: float = 0.02):
        super().__init__()
        self.top_k = top_k
        self.gate = nn.Parameter(torch.empty(num_experts, hidden).normal_(std=std))
        self.experts = nn.ModuleList([YvExpertFactory.create(kind, hidden, inner, std) for _ in range(num_experts)])
        self.shared = nn.ModuleList([YvExpertFactory.create(kind, hidden, inner, std) for _ in range(num_shared)])
        self.shared_mix = nn.Parameter(torch.zeros(num_shared)) if num_shared else None

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        probs = torch.softmax(F_.linear(x2, self.gate.to(x2.dtype)).float(), -1)
        w, idx = probs.topk(self.top_k, -1)
        w = w / w.sum(-1, keepdim=True)
        out = torch.zeros_like(x2)
        for e, expert in enumerate(self.experts):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel():
                out.index_add_(0, tok, (w[tok, slot, None].to(x2.dtype) * expert(x2[tok])))
        if self.shared_mix is not None:
            mix = torch.softmax(self.shared_mix, 0)
            for m, s in zip(mix, self.shared):
                out = out + m.to(x2.dtype) * s(x2)
        load = torch.zeros(len(self.experts), device=x.device).index_add_(0, idx.flatten(), torch.ones(idx.numel(), device=x.device))
        aux = len(self.experts) * (load / idx.numel() * probs.mean(0)).sum()
        return out.view(shape), aux


class YvExpertDiversityRegularizer:
    """Penalises pairwise cosine similarity between the experts' (flattened) weights."""

    def __init__(self, weight: float = 1e-3):
        self.weight = weight

    def __call__(self, stacked: torch.Tensor) -> torch.Tensor:
        """stacked [E, ...] expert weights -> scalar."""
        f = F.normalize(stacked.flatten(1).float(), dim=1)
        sim = f @ f.t()
        off = sim - torch.diag(torch.diag(sim))
        E = stacked.shape[0]
        return self.weight * off.pow(2).sum() / max(E * (E - 1), 1)


class YvGateClusterInitializer:
    """The gate-only form (``models/expert_init.YvGradientClusterInitializer`` is the full one: streamed gradient
    statistics per parameter, elbow choice of k, experts displaced by cluster).  Initialises experts from k-means centroids of per-token gradient (or activation) features so that experts start
    specialised on different clusters."""

    def __init__(self, num_experts: int, iters: int = 10, seed: int = 0):
        self.E, self.iters, self.seed = num_experts, iters, seed

    def cluster(self, feats: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        g = torch.Generator(device="cpu").manual_seed(self.seed)
        f = feats.float()
        cent = f[torch.randperm(f.shape[0], generator=g)[: self.E]].clone()
        assign = torch.zeros(f.shape[0], dtype=torch.long)
        for _ in range(self.iters):
            assign = torch.cdist(f, cent).argmin(1)
            for e in range(self.E):
                m = assign == e
                if m.any():
                    cent[e] = f[m].mean(0)
        return cent, assign

    def init_gate(self, gate_weight: torch.Tensor, feats: torch.Tensor) -> None:
        cent, _ = self.cluster(feats)
        with torch.no_grad():
            gate_weight.copy_(F.normalize(cent, dim=1).to(gate_weight.dtype) * gate_weight.float().norm(dim=1).mean())


YvGradientClusterInitializer = YvGateClusterInitializer        # the name this class had before models/expert_init.py existed


class YvExpertEvolution:
    """Usage-driven expert maintenance: the least used expert is re-seeded from the most used one plus noise."""

    def __init__(self, noise: float = 0.01, min_share: float = 0.1):
        self.noise, self.min_share = noise, min_share

    @torch.no_grad()
    def step(self, stacked_weights: List[torch.Tensor], counts: torch.Tensor) -> Optional[Tuple[int, int]]:
        share = counts.float() / counts.sum().clamp_min(1)
        lo, hi = int(share.argmin()), int(share.argmax())
        if share[lo] * len(share) >= self.min_share or lo == hi:
            return None
        for w in stacked_weights:
            w[lo].copy_(w[hi] + self.noise * w[hi].float().std().to(w.dtype) * torch.randn_like(w[hi]))
        return lo, hi


# ------------------------------------------------------------------------------------------------ configured experts
class YvExpertType(str, Enum):
    STANDARD = "standard"
    SWIGLU = "swiglu"
    GEGLU = "geglu"
    MULTI_LAYER = "multi_layer"
    SHARED = "shared"
    ATTENTION = "attention"


class YvExpertMode(str, Enum):
    PURE_COMPUTE = "pure_compute"      # a trainable feed-forward expert
    PURE_LOOKUP = "pure_lookup"        # frozen: static knowledge storage beside the reasoning experts


@dataclass
class YvExpertConfig:
    hidden_size: int = 2048
    intermediate_size: int = 5632
    expert_type: YvExpertType = YvExpertType.SWIGLU
    dropout: float = 0.0
    use_bias: bool = False
    activation: str = "silu"
    mode: YvExpertMode = YvExpertMode.PURE_COMPUTE
    num_layers: int = 2                # multi-layer experts
    num_heads: int = 4                 # attention experts
    init_std: float = 0.02

    def __post_init__(self) -> None:
        self.expert_type = YvExpertType(getattr(self.expert_type, "value", self.expert_type))
        self.mode = YvExpertMode(getattr(self.mode, "value", self.mode))
        if self.activation not in ("silu", "gelu", "relu"):
            raise ValueError(f"unknown activation {self.activation}")


class YvExpertBase(nn.Module):
    """An expert built from a ``YvExpertConfig`` (reference model/moe/expert.py:231-290): ``forward(x)`` keeps the shape of
    ``x`` ([tokens, hidden] or [batch, sequence, hidden]); a ``PURE_LOOKUP`` expert is frozen after construction."""

    def __init__(self, config: YvExpertConfig, mode: Optional[YvExpertMode] = None):
        super().__init__()
        self.config = config
        self.mode = YvExpertMode(getattr(mode, "value", mode)) if mode is not None else config.mode
        self.drop = nn.Dropout(config.dropout) if config.dropout > 0 else nn.Identity()

    def _freeze_if_lookup(self) -> None:
        if self.mode is YvExpertMode.PURE_LOOKUP:
            for p in self.parameters():
                p.requires_grad_(False)

    def body(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError("an expert implements body(x)")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.drop(self.body(x))


class _WrappedExpert(YvExpertBase):
    def __init__(self, config: YvExpertConfig, core: nn.Module, mode: Optional[YvExpertMode] = None):
        super().__init__(config, mode)
        self.core = core
        self._freeze_if_lookup()

    def body(self, x: torch.Tensor) -> torch.Tensor:
        return self.core(x)


class YvSharedExpert(YvExpertBase):
    """The always-on expert beside the routed ones: a SwiGLU block whose output is scaled by a learned sigmoid gate of the
    token (so the layer can learn how much every token leans on shared knowledge)."""

    def __init__(self, config: YvExpertConfig, mode: Optional[YvExpertMode] = None):
        super().__init__(config, mode)
        self.core = YvSwiGLUExpert(config.hidden_size, config.intermediate_size, config.init_std)
        self.gate = nn.Parameter(torch.zeros(1, config.hidden_size))
        self._freeze_if_lookup()

    def body(self, x: torch.Tensor) -> torch.Tensor:
        return torch.sigmoid(F_.linear(x, self.gate.to(x.dtype))) * 2.0 * self.core(x)


class YvAttentionExpert(YvExpertBase):
    """An expert that mixes along the sequence: causal self-attention over the tokens it is given, then a projection.  It needs
    [batch, sequence, hidden] input; a flat [tokens, hidden] input is treated as one sequence."""

    def __init__(self, config: YvExpertConfig, mode: Optional[YvExpertMode] = None):
        super().__init__(config, mode)
        h = config.hidden_size
        if h % config.num_heads:
            raise ValueError("hidden_size must be a multiple of num_heads")
        self.qkv = nn.Parameter(torch.empty(3 * h, h).normal_(std=config.init_std))
        self.o = nn.Parameter(torch.empty(h, h).normal_(std=config.init_std))
        self._freeze_if_lookup()

    def body(self, x: torch.Tensor) -> torch.Tensor:
        flat = x.dim() == 2
        x3 = x.unsqueeze(0) if flat else x
        B, T, H = x3.shape
        nh = self.config.num_heads
        q, k, v = F_.linear(x3, self.qkv.to(x.dtype)).view(B, T, 3, nh, H // nh).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=T > 1).transpose(1, 2).reshape(B, T, H)
        out = F_.linear(a, self.o.to(x.dtype))
        return out[0] if flat else out


def _core_for(c: YvExpertConfig) -> nn.Module:
    t = c.expert_type
    if t is YvExpertType.SWIGLU:
        return YvSwiGLUExpert(c.hidden_size, c.intermediate_size, c.init_std)
    if t is YvExpertType.GEGLU:
        return YvGeGLUExpert(c.hidden_size, c.intermediate_size, c.init_std)
    if t is YvExpertType.STANDARD:
        return YvStandardExpert(c.hidden_size, c.intermediate_size, c.activation, c.init_std)
    if t is YvExpertType.MULTI_LAYER:
        return YvMultiLayerExpert(c.hidden_size, c.intermediate_size, c.num_layers, c.init_std)
    raise ValueError(f"no feed-forward core for {t}")


_EXPERT_REGISTRY: Dict[YvExpertType, Callable[[YvExpertConfig, Optional[YvExpertMode]], YvExpertBase]] = {
    YvExpertType.SHARED: YvSharedExpert, YvExpertType.ATTENTION: YvAttentionExpert}


def create_expert(config: YvExpertConfig, mode: Optional[YvExpertMode] = None) -> YvExpertBase:
    """The configured-expert constructor (``YvExpertFactory.create`` builds bare cores from sizes)."""
    maker = _EXPERT_REGISTRY.get(config.expert_type)
    return maker(config, mode) if maker is not None else _WrappedExpert(config, _core_for(config), mode)


def register_expert(expert_type: YvExpertType, expert_class: Callable[[YvExpertConfig, Optional[YvExpertMode]], YvExpertBase]) -> None:
    _EXPERT_REGISTRY[YvExpertType(getattr(expert_type, "value", expert_type))] = expert_class


YvExpertFactory.create_from_config = staticmethod(create_expert)
YvExpertFactory.register = staticmethod(register_expert)
