"""Typed views of the model configuration: architecture / layer / attention / block / cache / modality / token enumerations and
the per-component configuration records, plus the memory-fusion and memory-separation layers (reference model/core/model.py:
247-374, attention.py:179-318, blocks.py:208-327, cache.py, memory_attention.py:38-52, multimodal/types.py, tokenizer/special_tokens.py,
moe/regularization.py).

The framework itself is driven by one flat ``YvConfig``; every record here has ``from_config(cfg)`` that reads its fields from it
(with the record's defaults where the flat configuration has no such field), so that code written against the reference's
per-component records works on top of the same source of truth.

``YvMemoryFusionGate`` and ``YvMemorySeparationLayer`` are empty shells in the reference (``forward`` returns ``None``,
memory_attention.py:38-52); here they compute: the gate mixes retrieved memory into the stream through a per-token, per-channel
sigmoid that starts closed, and the separation layer splits the stream into a reasoning part and a lookup query with an
orthogonality penalty between the two."""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from enum import Enum
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class YvModelType(str, Enum):
    DECODER_ONLY = "decoder_only"
    ENCODER_DECODER = "encoder_decoder"
    ENCODER_ONLY = "encoder_only"
    HYBRID = "hybrid"


class YvLayerType(str, Enum):
    ATTENTION = "attention"
    SSM = "ssm"
    HYBRID = "hybrid"
    MOE = "moe"
    RECURRENT = "recurrent"


class YvAttentionBackend(str, Enum):
    STANDARD = "standard"
    FLASH = "flash"
    SDPA = "sdpa"
    LINEAR = "linear"
    SPARSE = "sparse"
    PAGED = "paged"
    RING = "ring"
    SLIDING_WINDOW = "sliding_window"
    CIRCULANT = "circulant"
    CIRCULAR = "circular"


class YvBlockType(str, Enum):
    STANDARD = "standard"
    PARALLEL = "parallel"
    DEEPNORM = "deepnorm"
    CROSS_ATTENTION = "cross_attention"
    ADAPTIVE = "adaptive"
    MIXTURE_OF_DEPTHS = "mixture_of_depths"


class YvCacheType(str, Enum):
    STANDARD = "standard"
    PAGED = "paged"
    QUANTIZED = "quantized"
    SLIDING_WINDOW = "sliding_window"
    H2O = "h2o"
    STREAMING = "streaming"
    COMPRESSED = "compressed"


class YvModality(str, Enum):
    TEXT = "text"
    IMAGE = "image"
    AUDIO = "audio"
    VIDEO = "video"
    DOCUMENT = "document"
    AGENTIC = "agentic"


class YvSpecialTokenType(str, Enum):
    CONTROL = "control"
    ROLE = "role"
    MULTIMODAL = "multimodal"
    REASONING = "reasoning"
    TOOL = "tool"
    PADDING = "padding"


def _pick(cls: type, cfg: Any, **extra: Any) -> Any:
    """A record of type ``cls`` whose fields are read from ``cfg`` (attributes, then ``cfg.extra``), defaults otherwise."""
    ex = getattr(cfg, "extra", None) or {}
    kw = {}
    for f in fields(cls):
        if f.name in extra:
            kw[f.name] = extra[f.name]
        elif hasattr(cfg, f.name) and getattr(cfg, f.name) is not None:
            kw[f.name] = getattr(cfg, f.name)
        elif f.name in ex:
            kw[f.name] = ex[f.name]
    return cls(**kw)


@dataclass
class YvLayerConfig:
    layer_idx: int
    layer_type: YvLayerType = YvLayerType.ATTENTION
    use_checkpoint: bool = False
    use_moe: bool = False
    num_experts: int = 8
    expert_capacity: float = 1.25

    def __post_init__(self) -> None:
        self.layer_type = YvLayerType(getattr(self.layer_type, "value", self.layer_type))

    @classmethod
    def from_config(cls, cfg: Any, layer_idx: int) -> "YvLayerConfig":
        pattern = list(getattr(cfg, "layer_types", None) or (getattr(cfg, "extra", {}) or {}).get("layer_types", []) or [])
        kind = pattern[layer_idx % len(pattern)] if pattern else "attention"
        n_exp = int(getattr(cfg, "moe_num_experts", 0) or 0)
        first_dense = int(getattr(cfg, "moe_first_dense_layers", getattr(cfg, "first_k_dense", 0)) or 0)
        moe = n_exp > 0 and layer_idx >= first_dense
        lt = YvLayerType(kind) if kind in YvLayerType._value2member_map_ else YvLayerType.ATTENTION
        return cls(layer_idx, lt, bool(getattr(cfg, "use_gradient_checkpointing", False)), moe, n_exp or 8, float(getattr(cfg, "moe_capacity_factor", 1.25) or 1.25))


@dataclass
class YvAttentionConfig:
    hidden_size: int = 4096
    n_head: int = 32
    n_kv_head: int = 8
    head_dim: Optional[int] = None
    max_position_embeddings: int = 10485760
    rope_theta: float = 10000.0
    attention_dropout: float = 0.0
    use_flash_attention: bool = True
    use_alibi: bool = False
    use_attention_sink: bool = True
    sliding_window: int = 0
    use_linear_attention: bool = False
    linear_attention_dim: int = 64
    sparse_attention_pattern: str = "none"
    sparse_block_size: int = 64
    paged_attention_block_size: int = 16
    use_ring_attention: bool = False
    ring_attention_size: int = 4
    attention_scale: Optional[float] = None
    use_qk_norm: bool = True
    use_gqa_residual: bool = True
    compression_ratio: int = 8
    streaming_window: int = 16384
    fused_qkv: bool = True
    sdpa_prefer_flash: bool = True
    use_sliding_window: bool = False
    use_mla: bool = True
    kv_lora_rank: int = 512
    q_lora_rank: Optional[int] = None
    use_circulant_attention: bool = False
    circulant_fft_threshold: int = 4096
    circulant_fft_dim: str = "auto"

    def __post_init__(self) -> None:
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.n_head
        if self.n_head % max(self.n_kv_head, 1):
            raise ValueError("n_head must be a multiple of n_kv_head")

    @classmethod
    def from_config(cls, cfg: Any) -> "YvAttentionConfig":
        return _pick(cls, cfg)

    @property
    def scale(self) -> float:
        return self.attention_scale if self.attention_scale is not None else self.head_dim ** -0.5

    def backend(self) -> YvAttentionBackend:
        if self.use_ring_attention:
            return YvAttentionBackend.RING
        if self.use_circulant_attention:
            return YvAttentionBackend.CIRCULANT
        if self.use_linear_attention:
            return YvAttentionBackend.LINEAR
        if self.sparse_attention_pattern != "none":
            return YvAttentionBackend.SPARSE
        if self.use_sliding_window or self.sliding_window > 0:
            return YvAttentionBackend.SLIDING_WINDOW
        return YvAttentionBackend.FLASH if self.use_flash_attention else YvAttentionBackend.STANDARD

    def kv_bytes_per_token(self, bytes_per_element: int = 2) -> int:
        return (self.kv_lora_rank if self.use_mla else 2 * self.n_kv_head * self.head_dim) * bytes_per_element


@dataclass
class YvBlockConfig:
    hidden_size: int = 4096
    intermediate_size: int = 11008
    n_layer: int = 32
    n_head: int = 32
    n_kv_head: int = 8
    block_type: str = "standard"
    activation: str = "silu"
    use_deepnorm: bool = False
    use_parallel: bool = False
    use_layerscale: bool = True
    layerscale_init: float = 1e-5
    use_swiglu: bool = True
    use_geglu: bool = False
    residual_dropout: float = 0.1
    use_checkpoint: bool = True
    adaptive_checkpointing: bool = True
    use_lora: bool = False
    lora_rank: int = 8
    lora_alpha: float = 16.0
    use_dora: bool = False
    mixture_of_depths: bool = False
    mod_routing_weight: float = 0.1
    use_attn_res: bool = False
    attn_res_block_size: int = 8
    attn_res_use_two_phase: bool = True
    attn_res_use_online_softmax: bool = True
    attn_res_cache_pipeline: bool = True
    attn_res_max_blocks: int = 32
    attn_res_learnable_query: bool = True
    attn_res_use_rmsnorm: bool = True

    def __post_init__(self) -> None:
        self.block_type = YvBlockType(getattr(self.block_type, "value", self.block_type)).value

    @classmethod
    def from_config(cls, cfg: Any) -> "YvBlockConfig":
        return _pick(cls, cfg)

    def resolved_type(self) -> YvBlockType:
        if self.mixture_of_depths:
            return YvBlockType.MIXTURE_OF_DEPTHS
        if self.use_parallel:
            return YvBlockType.PARALLEL
        if self.use_deepnorm:
            return YvBlockType.DEEPNORM
        return YvBlockType(self.block_type)

    def deepnorm_constants(self) -> Tuple[float, float]:
        """(alpha for the residual, beta for the initialisation) of DeepNorm for a decoder of ``n_layer`` layers."""
        return (2.0 * self.n_layer) ** 0.25, (8.0 * self.n_layer) ** -0.25


@dataclass
class YvCacheBlock:
    """One block of a paged cache: which physical block, how many of its slots are filled, how many sequences share it."""
    block_id: int
    block_size: int = 64
    filled: int = 0
    ref_count: int = 1
    last_access: int = 0
    token_hash: Optional[int] = None

    @property
    def is_full(self) -> bool:
        return self.filled >= self.block_size

    @property
    def free_slots(self) -> int:
        return self.block_size - self.filled

    def append(self, n: int = 1) -> int:
        """Fills up to ``n`` slots; returns how many did not fit."""
        take = min(n, self.free_slots)
        self.filled += take
        return n - take

    def share(self) -> "YvCacheBlock":
        self.ref_count += 1
        return self

    def release(self) -> bool:
        """True when nobody holds the block any more."""
        self.ref_count = max(self.ref_count - 1, 0)
        return self.ref_count == 0


@dataclass
class YvRegularizationConfig:
    diversity_weight: float = 0.01
    orthogonality_weight: float = 0.0
    load_balance_weight: float = 0.01
    z_loss_weight: float = 1e-3
    entropy_weight: float = 0.0
    dropout: float = 0.0
    warmup_steps: int = 0

    def weight_at(self, name: str, step: int) -> float:
        w = float(getattr(self, f"{name}_weight"))
        return w * min(1.0, (step + 1) / self.warmup_steps) if self.warmup_steps > 0 else w


class YvNorms:
    """Normalisation layers by name."""

    @staticmethod
    def create(kind: str, dim: int, eps: float = 1e-6) -> nn.Module:
        from .norms import YvRMSNorm
        k = kind.lower()
        if k in ("rms", "rmsnorm"):
            return YvRMSNorm(dim, eps)
        if k in ("layer", "layernorm", "ln"):
            return nn.LayerNorm(dim, eps=eps)
        if k in ("none", "identity"):
            return nn.Identity()
        raise ValueError(f"unknown normalisation {kind}")

    @staticmethod
    def available() -> List[str]:
        return ["rmsnorm", "layernorm", "identity"]


# ---- memory layers --------------------------------------------------------------------------------------------------------------
class YvMemoryFusionGate(nn.Module):
    """h + g * W m with g = sigmoid(W_g [h; m] + b): per token and channel.  ``b`` starts at ``gate_init`` (negative: closed), so a model
    that gets this layer attached computes what it computed before until training opens the gate."""

    def __init__(self, cfg: Any = None, hidden_size: Optional[int] = None, memory_size: Optional[int] = None, gate_init: float = -4.0, device=None, dtype=None):
        super().__init__()
        h = int(hidden_size or getattr(cfg, "hidden_size"))
        m = int(memory_size or getattr(cfg, "memory_size", None) or h)
        self.proj = nn.Linear(m, h, bias=False, device=device, dtype=dtype)
        self.gate = nn.Linear(h + m, h, device=device, dtype=dtype)
        nn.init.zeros_(self.gate.weight)
        nn.init.constant_(self.gate.bias, gate_init)
        self.last_gate_mean: Optional[torch.Tensor] = None

    def forward(self, hidden: torch.Tensor, memory: Optional[torch.Tensor], memory_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """hidden [B, T, H]; memory [B, T, M] (aligned) or [B, M] (one vector per sequence); mask [B, T] or [B] marks where memory exists."""
        if memory is None:
            return hidden
        if memory.dim() == 2:
            memory = memory.unsqueeze(1).expand(-1, hidden.shape[1], -1)
        g = torch.sigmoid(self.gate(torch.cat([hidden, memory.to(hidden.dtype)], -1)))
        if memory_mask is not None:
            mm = memory_mask.to(g.dtype)
            g = g * (mm.unsqueeze(-1) if mm.dim() == 2 else mm.view(-1, 1, 1))
        self.last_gate_mean = g.detach().mean()
        return hidden + g * self.proj(memory.to(hidden.dtype))


class YvMemorySeparationLayer(nn.Module):
    """Splits the stream into a reasoning part (returned as the new hidden state) and a lookup query (what the knowledge store is asked
    with): two projections of the normalised input.  ``separation_loss`` is the squared cosine between the two parts, so training pushes
    facts-to-look-up and reasoning into different directions."""

    def __init__(self, cfg: Any = None, hidden_size: Optional[int] = None, query_size: Optional[int] = None, device=None, dtype=None):
        super().__init__()
        h = int(hidden_size or getattr(cfg, "hidden_size"))
        q = int(query_size or getattr(cfg, "memory_query_size", None) or h)
        self.norm = nn.LayerNorm(h, device=device, dtype=dtype)
        self.reason = nn.Linear(h, h, bias=False, device=device, dtype=dtype)
        self.lookup = nn.Linear(h, q, bias=False, device=device, dtype=dtype)
        with torch.no_grad():
            self.reason.weight.copy_(torch.eye(h, dtype=self.reason.weight.dtype))       # starts as the identity on the stream
        self.separation_loss: Optional[torch.Tensor] = None

    def forward(self, hidden: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        x = self.norm(hidden)
        r, q = self.reason(x), self.lookup(x)
        n = min(r.shape[-1], q.shape[-1])
        self.separation_loss = F.cosine_similarity(r[..., :n].float(), q[..., :n].float(), dim=-1).pow(2).mean()
        return hidden + (r - x), q
