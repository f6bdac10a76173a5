"""YvConfig: the single source of model hyper-parameters.

Field names and defaults follow the reference's ``YvConfig`` dataclass (model/config.py:214-1007) for
every field this framework consumes, so the reference's YAML presets (configs/model/*.yaml) load
unchanged.  Keys this framework does not know are kept in ``extra`` instead of being dropped
(the reference drops them silently, model/config.py:1155-1157), so a config survives a round trip.

Parallel-layout fields (``tensor_parallel`` .. ``context_parallel``) and the product-quantised
Subconscious field (``pq_*``) have no counterpart in the reference dataclass; they describe features
the reference only documents (README.md:70-78) or stubs (opss/train/parallel_3d.py:237-268).
"""
from __future__ import annotations

import copy
import dataclasses
import json
import math
from dataclasses import dataclass, field
from enum import Enum
from pathlib import Path
from typing import Any, Dict, List, Optional

import yaml


class YvAttentionType(str, Enum):
    """Attention variants selectable by ``attention_type`` (reference model/config.py:124-160)."""
    STANDARD = "standard"
    GQA = "gqa"
    MLA = "mla"
    EG_MLA = "eg_mla"
    SLIDING_WINDOW = "sliding_window"
    LINEAR = "linear"
    H2O = "h2o"
    PAGED = "paged"
    RING = "ring"


class YvPositionEmbeddingType(str, Enum):
    ROPE = "rope"
    YARN = "yarn"
    DYNAMIC_NTK = "dynamic_ntk"
    MR_ROPE = "mr_rope"
    ALIBI = "alibi"
    ROPE_3D = "rope_3d"
    NONE = "none"


class YvActivationType(str, Enum):
    SILU = "silu"
    GELU = "gelu"
    RELU = "relu"
    SWIGLU = "swiglu"
    GEGLU = "geglu"


@dataclass
class YvConfig:
    # ---- identity / sizes -------------------------------------------------------------------
    model_type: str = "piscesl1"
    vocab_size: int = 151646
    hidden_size: int = 2048
    n_layer: int = 24
    n_head: int = 16
    n_kv_head: int = 4
    head_dim: Optional[int] = None
    intermediate_size: int = 5632
    max_position_embeddings: int = 8192
    max_context_length: int = 1048576
    # ---- MoE -----------------------------------------------------------------------------------
    moe_num_experts: int = 128
    moe_top_k: int = 8
    moe_capacity_factor: float = 1.0
    moe_min_capacity: int = 4
    moe_load_balance_alpha: float = 0.01
    moe_aux_loss_weight: float = 1.0
    moe_z_loss_alpha: float = 1e-4
    moe_noise_std: float = 0.1
    moe_prediction_horizon: int = 8
    moe_layers: List[int] = field(default_factory=list)
    moe_shared_experts: int = 1
    moe_fine_grained: bool = True
    moe_num_sub_experts: int = 4
    moe_aux_loss_free: bool = True
    moe_bias_update_rate: float = 0.05
    moe_bias_update_freq: int = 50
    moe_bias_in_combine: bool = True
    moe_routing_temperature: float = 1.0
    moe_dropout: float = 0.0
    moe_expert_intermediate_size: Optional[int] = None
    moe_shared_intermediate_size: Optional[int] = None
    moe_gate_type: str = "stable"          # "stable" (YvStableMoEGate) | "lean" (YvMoEGate) | "research" (YvResearchMoEGate)
    moe_use_load_predictor: bool = False    # optional LSTM load predictor of YvStableMoEGate
    moe_drop_tokens: bool = False           # capacity dropping (lowest score dropped by zeroing)
    moe_skip_prev_shared: bool = False      # the 0.1 * previous shared output skip term
    expert_init_method: str = "normal"
    diversity_weight: float = 0.0
    use_fused_moe: bool = True
    backbone_allow_legacy_blocks: bool = True
    use_path_moe: bool = False
    # ---- attention / position ---------------------------------------------------------------------
    attention_type: str = "gqa"
    rope_theta: float = 1e6
    use_rotary_pos_emb: bool = True
    use_partial_rope: bool = False
    partial_rope_dim: int = 64
    use_qk_norm: bool = False
    use_mla: bool = False
    kv_lora_rank: int = 512
    mla_q_lora_rank: Optional[int] = None
    mla_rope_dim: int = 64
    use_enhanced_mla: bool = False           # decoupled RoPE: a shared rotary key slice decompressed from the latent
    attention_output_gate: bool = False      # per-head sigmoid gate on the attention output, computed from the input
    attention_sink_tokens: int = 0           # learned sink tokens prepended to every sequence while training
    use_flash_attention: bool = True
    use_sliding_window: bool = False
    streaming_window: int = 16384
    use_alibi: bool = False
    use_dynamic_yarn: bool = False
    use_mr_rope: bool = False
    linear_rope_scale: float = 1.0
    rope_scaling_factor: float = 1.0
    use_3d_spatio_temporal_rope: bool = False
    max_temporal_frames: int = 64
    use_ring_attention: bool = True
    ring_attention_threshold: int = 32768
    ring_attention_size: int = 4
    ring_attention_distributed: bool = False
    attention_dropout: float = 0.0
    learnable_attention_scale: bool = False
    use_h2o_attention: bool = False
    use_mamba3: bool = False
    mamba3_d_state: int = 128
    mamba3_d_conv: int = 4
    mamba3_expand: int = 2
    # ---- norms / init / misc -----------------------------------------------------------------------
    layer_norm_eps: float = 1e-6
    use_rms_norm: bool = True
    initializer_range: float = 0.02
    use_scaled_init: bool = True
    dropout: float = 0.0
    activation_type: str = "silu"
    use_swiglu: bool = True
    swiglu_clamp: bool = False
    tie_word_embeddings: bool = True
    use_cache: bool = True
    use_gradient_checkpointing: bool = True
    label_smoothing: float = 0.0
    bos_token_id: int = 1
    eos_token_id: int = 2
    pad_token_id: int = 0
    unk_token_id: int = 3
    # ---- multi-token prediction -------------------------------------------------------------------
    num_mtp_heads: int = 0
    mtp_loss_weight: float = 0.5
    mtp_share_embeddings: bool = True
    # ---- KV cache / long context ---------------------------------------------------------------------
    kv_cache_block_size: int = 64
    max_cache_size: int = 8192
    cache_quantization: bool = False
    use_oomb_context: bool = False
    oomb_chunk_size: int = 32768
    use_reform: bool = False
    reform_compression_ratio: int = 4
    # ---- Subconscious (FiLM) -------------------------------------------------------------------------
    use_subconscious: bool = False
    use_dual_inject: bool = False
    subconscious_knowledge_dim: int = 1024
    subconscious_state_dim: int = 1024
    use_subconscious_blocks: bool = False
    block_count: int = 628
    block_rank: int = 512
    block_memory_rows: int = 0
    block_pool_slots: int = 2
    block_gamma_max: float = 0.5
    block_beta_bound: float = 0.25
    block_inject_alpha: float = 0.1
    block_min_dwell_tokens: int = 17
    # product-quantised knowledge field (README.md:70-78 of the reference; not in its code)
    use_pq_field: bool = False
    pq_num_codebooks: int = 16
    pq_codebook_size: int = 131072
    pq_entry_dim: int = 128
    pq_init_std: float = 0.02
    pq_nav_hidden: int = 2048
    pq_film_interval: int = 4
    # ---- multimodal ---------------------------------------------------------------------------------------
    image_patch: int = 14
    image_tokens: int = 256
    audio_tokens: int = 512
    video_tokens: int = 128
    mm_tokens: int = 256
    modal_token_count: int = 8
    native_fusion_output_tokens: int = 8
    native_fusion_num_layers: int = 2
    enable_dynamic_fusion: bool = True
    fusion_dropout: float = 0.1
    vision_hidden_size: Optional[int] = None   # None -> tied to the LM width as in the reference
    vision_n_layer: Optional[int] = None
    vision_n_head: Optional[int] = None
    vision_native_resolution: bool = False
    audio_sampling_rate: int = 16000
    audio_n_mels: int = 128
    audio_n_fft: int = 1024
    audio_hop_length: int = 512
    # ---- generation ------------------------------------------------------------------------------------------
    generation_max_tokens: int = 1024
    generation_temperature: float = 1.0
    generation_top_p: float = 0.95
    generation_top_k: int = 50
    enable_speculative_decoding: bool = False
    speculative_draft_length: int = 5
    speculative_acceptance_threshold: float = 0.8
    use_dspark: bool = False
    dspark_draft_len: int = 5
    dspark_markov_order: int = 3
    # ---- low precision -------------------------------------------------------------------------------------------
    use_fp8: bool = False
    fp8_block_size: int = 128
    use_fp4: bool = False
    fp4_block_size: int = 16
    # ---- task heads ---------------------------------------------------------------------------------------------
    task_classes: int = 256
    classifier_dropout: float = 0.1
    # ---- parallel layout (new) -----------------------------------------------------------------------------
    tensor_parallel: int = 1
    expert_parallel: int = 1
    pipeline_parallel: int = 1
    context_parallel: int = 1
    context_parallel_mode: str = "allgather"   # "ring": K/V blocks travel round the ranks (O(S/cp) K/V memory per rank)
    sequence_parallel: bool = True
    tp_split_head: bool = False             # training: every tensor-parallel rank runs LM head + loss on ITS token shard only
    zero_stage: int = 1
    fused_comm: bool = True                 # peer-memory fused kernels (False = NCCL baseline mode)
    expert_fp8: Optional[str] = None        # "mx": routed experts' forward products in block-scaled e4m3 (single GPU path)
    # ---- anything else found in a config file -----------------------------------------------------------------
    extra: Dict[str, Any] = field(default_factory=dict)

    # ------------------------------------------------------------------------------------------------
    def __post_init__(self) -> None:
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.n_head
        if self.n_kv_head is None or self.n_kv_head <= 0:
            self.n_kv_head = self.n_head
        if self.moe_expert_intermediate_size is None:
            # Fine-grained experts split a dense FFN into ``moe_num_sub_experts`` slices
            # (reference model/moe/layer.py:262-515 keeps sub-expert ids; here each routed expert
            # simply is one slice).
            div = self.moe_num_sub_experts if self.moe_fine_grained else 1
            self.moe_expert_intermediate_size = max(64, self.intermediate_size // max(div, 1))
        if self.moe_shared_intermediate_size is None:
            self.moe_shared_intermediate_size = self.intermediate_size
        if isinstance(self.attention_type, Enum):
            self.attention_type = self.attention_type.value

    # ---- derived ------------------------------------------------------------------------------------
    @property
    def num_key_value_groups(self) -> int:
        return self.n_head // self.n_kv_head

    @property
    def q_dim(self) -> int:
        return self.n_head * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_head * self.head_dim

    def is_moe_layer(self, i: int) -> bool:
        if self.moe_num_experts <= 0:
            return False
        return (not self.moe_layers) or (i in self.moe_layers)

    def validate(self) -> List[str]:
        """Return a list of problems (empty = valid); mirrors reference model/config.py:1267."""
        errs: List[str] = []
        if self.hidden_size <= 0 or self.n_layer <= 0:
            errs.append("hidden_size and n_layer must be positive")
        if self.n_head % self.n_kv_head != 0:
            errs.append(f"n_head {self.n_head} not divisible by n_kv_head {self.n_kv_head}")
        if self.moe_num_experts > 0 and not (0 < self.moe_top_k <= self.moe_num_experts):
            errs.append("moe_top_k must be in (0, moe_num_experts]")
        if self.head_dim % 2 != 0:
            errs.append("head_dim must be even for rotary embeddings")
        if self.moe_num_experts % max(self.expert_parallel, 1) != 0:
            errs.append("moe_num_experts must divide by expert_parallel")
        if self.n_kv_head % max(self.tensor_parallel, 1) != 0:
            errs.append("n_kv_head must divide by tensor_parallel")
        if self.vocab_size <= 0:
            errs.append("vocab_size must be positive")
        return errs

    # ---- parameter / memory estimates --------------------------------------------------------------------
    def count_parameters(self) -> Dict[str, int]:
        H = self.hidden_size
        attn = H * self.q_dim + 2 * H * self.kv_dim + self.q_dim * H
        routed = self.moe_num_experts * 3 * H * self.moe_expert_intermediate_size
        shared = self.moe_shared_experts * 3 * H * self.moe_shared_intermediate_size
        gate = H * self.moe_num_experts
        dense_ffn = 3 * H * self.intermediate_size
        per_layer_moe = attn + routed + shared + gate + 2 * H
        per_layer_dense = attn + dense_ffn + 2 * H
        n_moe = sum(1 for i in range(self.n_layer) if self.is_moe_layer(i))
        n_dense = self.n_layer - n_moe
        emb = self.vocab_size * H * (1 if self.tie_word_embeddings else 2)
        total = n_moe * per_layer_moe + n_dense * per_layer_dense + emb + H
        active_layer = attn + self.moe_top_k * 3 * H * self.moe_expert_intermediate_size + shared + gate
        active = n_moe * active_layer + n_dense * per_layer_dense + self.vocab_size * H
        return {"total": int(total), "active": int(active), "embedding": int(emb),
                "per_layer": int(per_layer_moe if n_moe else per_layer_dense)}

    def estimate_memory_usage(self, batch: int = 1, seq: int = 4096, bytes_per_param: int = 2,
                              optimizer_bytes_per_param: int = 2, world: int = 1) -> Dict[str, float]:
        """Rough per-GPU bytes (reference model/config.py:1911 offers the same kind of estimate)."""
        p = self.count_parameters()["total"]
        w = p * bytes_per_param / world
        o = p * optimizer_bytes_per_param / world
        act = batch * seq * self.hidden_size * 2 * (self.n_layer + 8)
        return {"weights_gb": w / 1e9, "optimizer_gb": o / 1e9, "activations_gb": act / 1e9,
                "total_gb": (w + o + act) / 1e9}

    def flops_per_token(self, seq: int, training: bool = True, recompute: bool = False) -> float:
        act = self.count_parameters()["active"]
        mm = 2.0 * act
        attn = 2.0 * 2.0 * seq * self.q_dim * self.n_layer / 2.0     # causal QK^T and PV
        fwd = mm + attn
        if not training:
            return fwd
        return fwd * (4.0 if recompute else 3.0)

    # ---- (de)serialisation ------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "YvConfig":
        d = dict(d or {})
        names = {f.name for f in dataclasses.fields(cls)}
        known = {k: v for k, v in d.items() if k in names and k != "extra"}
        extra = dict(d.get("extra") or {})
        extra.update({k: v for k, v in d.items() if k not in names})
        cfg = cls(**known)
        cfg.extra = extra
        return cfg

    @classmethod
    def from_yaml(cls, path: str | Path) -> "YvConfig":
        text = Path(path).read_text()
        try:
            from configs.version import VERSION  # type: ignore
        except Exception:
            VERSION = "0.0.0"
        text = text.replace("{{VERSION}}", str(VERSION))
        return cls.from_dict(yaml.safe_load(text) or {})

    @classmethod
    def from_json(cls, path: str | Path) -> "YvConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(dataclasses.asdict(self))

    def to_json(self, path: Optional[str | Path] = None) -> str:
        s = json.dumps(self.to_dict(), indent=2, default=str)
        if path is not None:
            Path(path).write_text(s)
        return s

    def to_yaml(self, path: Optional[str | Path] = None) -> str:
        s = yaml.safe_dump(self.to_dict(), sort_keys=False)
        if path is not None:
            Path(path).write_text(s)
        return s

    def replace(self, **kw: Any) -> "YvConfig":
        d = self.to_dict()
        d.update(kw)
        if "hidden_size" in kw or "n_head" in kw:
            if "head_dim" not in kw:
                d["head_dim"] = None
        return YvConfig.from_dict(d)

    # ---- presets -----------------------------------------------------------------------------------------------
    @classmethod
    def tiny_text_moe(cls, vocab_size: int = 154856) -> "YvConfig":
        """4 layers, hidden 256, 4q/2kv heads, 8 routed experts (FFN 256, top-2) + 1 shared (FFN 512)."""
        return cls(vocab_size=vocab_size, hidden_size=256, n_layer=4, n_head=4, n_kv_head=2, head_dim=64,
                   rope_theta=1e4, moe_num_experts=8, moe_top_k=2, moe_shared_experts=1,
                   moe_expert_intermediate_size=256, moe_shared_intermediate_size=512,
                   intermediate_size=512, tie_word_embeddings=False, max_position_embeddings=4096)

    @classmethod
    def yv_7b_moe(cls, vocab_size: int = 154856, **kw: Any) -> "YvConfig":
        """32 layers, hidden 4096, 32q/8kv heads (hd 128), 64 routed experts (FFN 1408, top-6) + 2 shared (2816)."""
        base = dict(vocab_size=vocab_size, hidden_size=4096, n_layer=32, n_head=32, n_kv_head=8, head_dim=128,
                    rope_theta=1e4, moe_num_experts=64, moe_top_k=6, moe_shared_experts=2,
                    moe_expert_intermediate_size=1408, moe_shared_intermediate_size=2816,
                    intermediate_size=11264, tie_word_embeddings=False, max_position_embeddings=131072)
        base.update(kw)
        return cls(**base)

    @classmethod
    def get_small(cls) -> "YvConfig":
        return cls(hidden_size=512, n_layer=8, n_head=8, n_kv_head=2, moe_num_experts=8, moe_top_k=2,
                   intermediate_size=1408)

    @classmethod
    def get_base(cls) -> "YvConfig":
        return cls(hidden_size=1024, n_layer=16, n_head=16, n_kv_head=4, moe_num_experts=16, moe_top_k=2,
                   intermediate_size=2816)

    @classmethod
    def get_large(cls) -> "YvConfig":
        return cls(hidden_size=2048, n_layer=24, n_head=16, n_kv_head=4, moe_num_experts=32, moe_top_k=4,
                   intermediate_size=5632)

    @classmethod
    def get_xl(cls) -> "YvConfig":
        return cls.yv_7b_moe()


def chinchilla_tokens(n_params: float, ratio: float = 20.0) -> float:
    """Compute-optimal token budget (reference opss/scaling/__init__.py, Chinchilla scaler)."""
    return ratio * n_params


def log2_ceil(x: int) -> int:
    return int(math.ceil(math.log2(max(x, 1))))
