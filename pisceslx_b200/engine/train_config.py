"""The training configuration tree (reference tools/train/config.py:120-900): stage enumeration, optimizer / scheduler /
data / LoRA sections and the root ``PiscesLxTrainingConfig`` with stage files, dotted overrides and the mapping onto this
framework's trainer.

The quantisation and evolution SECTIONS here carry the trainer-side switches (is it on, which method, how many steps per
phase); ``to_pipeline_config()`` turns each into the configuration of the component that does the work
(``quant/pipeline.PiscesLxQuantizationConfig``, ``engine/operators.PiscesLxEvolutionConfig``)."""
from __future__ import annotations

import copy
from dataclasses import asdict, dataclass, field, fields, is_dataclass
from enum import Enum
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple, Union



class PiscesLxTrainingStage(str, Enum):
    PRETRAIN = "pretrain"
    CONTINUED_PRETRAIN = "continued_pretrain"
    SFT = "sft"
    ALIGNMENT_DPO = "alignment_dpo"
    ALIGNMENT_PPO = "alignment_ppo"
    ALIGNMENT_ORPO = "alignment_orpo"
    SPECIALIZED = "specialized"
    RL_GRPO = "rl_grpo"
    RL_RLVR = "rl_rlvr"
    RL_DAPO = "rl_dapo"
    RL_SELF_PLAY = "rl_self_play"
    RL_MEMSEP = "rl_memsep"

    @property
    def loss_type(self) -> str:
        return {"alignment_dpo": "dpo", "alignment_ppo": "ppo", "alignment_orpo": "orpo", "rl_grpo": "grpo", "rl_rlvr": "rlvr",
                "rl_dapo": "dapo", "rl_self_play": "spin", "rl_memsep": "lm"}.get(self.value, "lm")

    @property
    def needs_reference_model(self) -> bool:
        return self.value in ("alignment_dpo", "alignment_ppo", "rl_grpo", "rl_dapo", "rl_rlvr", "rl_self_play")


GLOBAL_DEFAULTS: Dict[str, Any] = {"mixed_precision": "bf16", "gradient_checkpointing": True, "flash_attention": True, "distributed": False,
                                   "world_size": 1, "gradient_accumulation_steps": 1, "moe_gradient": {"enabled": True}}


@dataclass
class PiscesLxOptimizerConfig:
    name: str = "adamw"
    learning_rate: float = 1e-4
    weight_decay: float = 0.01
    betas: Tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    max_grad_norm: float = 1.0
    sparse_gate_lr_multiplier: float = 1.0
    use_galore: bool = False
    galore_rank: int = 128
    galore_update_proj_gap: int = 200
    galore_quantization_bits: int = 8
    galore_lr_ratio: float = 1.0
    galore_min_rank: int = 32
    galore_max_rank: int = 512
    galore_rank_adapt_interval: int = 1000
    galore_rank_adapt_threshold: float = 0.1
    galore_memory_efficient: bool = False
    galore_moe_expert_only: bool = False
    galore_multimodal_modules: List[str] = field(default_factory=lambda: ["vision_encoder", "audio_encoder", "multimodal_fusion"])
    galore_sequence_threshold: int = 1024
    galore_gradient_accumulation_sync: bool = True
    use_fp4: bool = False
    fp4_block_size: int = 16
    fp4_stochastic_rounding: bool = True
    fp4_master_weights_dtype: str = "fp32"
    use_fused_adamw: bool = False

    def __post_init__(self) -> None:
        self.betas = tuple(self.betas)
        if self.learning_rate < 0:
            raise ValueError("learning_rate must not be negative")

    def galore_config(self, mode: str = "lowrank"):
        """The ``optim.galore.PiscesLxGaLoreConfig`` these fields describe."""
        from ..optim.galore import PiscesLxGaLoreConfig
        return PiscesLxGaLoreConfig(rank=self.galore_rank, update_proj_gap=self.galore_update_proj_gap, quantization_bits=self.galore_quantization_bits,
                                    lr_ratio=self.galore_lr_ratio, min_rank=self.galore_min_rank, max_rank=self.galore_max_rank,
                                    rank_adapt_interval=self.galore_rank_adapt_interval, rank_adapt_threshold=self.galore_rank_adapt_threshold,
                                    memory_efficient=self.galore_memory_efficient, moe_expert_only=self.galore_moe_expert_only, mode=mode,
                                    lr=self.learning_rate, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, weight_decay=self.weight_decay)

    def resolved_name(self) -> str:
        """The name ``optim.build_optimizer`` takes."""
        if self.use_fused_adamw and self.name == "adamw":
            return "fused_adamw"
        return self.name


@dataclass
class PiscesLxSchedulerConfig:
    name: str = "cosine"
    warmup_steps: int = 1000
    warmup_ratio: float = 0.1
    min_lr_ratio: float = 0.0
    decay_steps: Optional[int] = None

    def resolved_warmup(self, max_steps: int) -> int:
        """``warmup_steps`` when positive, else ``warmup_ratio`` of the run; never more than the run."""
        w = self.warmup_steps if self.warmup_steps > 0 else int(self.warmup_ratio * max_steps)
        return max(0, min(w, max_steps))


@dataclass
class PiscesLxDataConfig:
    batch_size: int = 32
    sequence_length: int = 2048
    num_workers: int = 4
    pin_memory: bool = True
    prefetch_factor: int = 2
    datasets: List[Dict[str, Any]] = field(default_factory=list)

    def normalized_weights(self) -> Dict[str, float]:
        w = {d.get("name", f"dataset{i}"): float(d.get("weight", 1.0)) for i, d in enumerate(self.datasets)}
        s = sum(w.values())
        return {k: v / s for k, v in w.items()} if s > 0 else w


@dataclass
class PiscesLxTrainingQuantizationConfig:
    enable_quantization: bool = False
    quant_method: str = "nf4"            # int4 | int8 | fp8 | nf4
    bits: int = 4
    group_size: int = 128
    symmetric: bool = False
    enable_fp8_linear: bool = False

    def __post_init__(self) -> None:
        if self.quant_method not in ("int4", "int8", "fp8", "nf4"):
            raise ValueError(f"unknown quant_method {self.quant_method}")
        if self.quant_method == "int8" and self.bits == 4:
            self.bits = 8

    def to_pipeline_config(self):
        from ..quant.pipeline import PiscesLxQuantizationConfig
        return PiscesLxQuantizationConfig(bits=8 if self.quant_method in ("int8", "fp8") else self.bits, group_size=self.group_size)


@dataclass
class PiscesLxTrainingEvolutionConfig:
    enabled: bool = False
    seed_size: str = "0.5B"
    target_size: str = "7B"
    distill_steps: int = 2000
    evolution_steps: int = 1000
    w2s_steps: int = 2000
    growth_stages: List[Dict[str, Any]] = field(default_factory=lambda: [
        {"type": "depth", "num_layers": 4, "train_steps": 500}, {"type": "width", "hidden_size": 2048, "train_steps": 500},
        {"type": "experts", "num_experts": 16, "train_steps": 500}, {"type": "depth", "num_layers": 8, "train_steps": 1000}])
    confidence_threshold: float = 0.7
    use_curriculum: bool = True
    use_self_correction: bool = True
    correction_weight: float = 0.3

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    def total_steps(self) -> int:
        return self.distill_steps + self.evolution_steps + self.w2s_steps + sum(int(g.get("train_steps", 0)) for g in self.growth_stages)

    def to_pipeline_config(self, current_layers: int = 0):
        """Growth stages the evolution pipeline can run: expert count, expert width (``intermediate_size``) and depth
        (``num_layers`` new layers, duplicates of the last layers of a model that has ``current_layers`` now); a ``width``
        stage of the hidden size goes through ``engine.growth.grow_hidden`` and is returned separately."""
        from .operators import PiscesLxEvolutionConfig, PiscesLxGrowthStage
        stages, hidden = [], []
        for g in self.growth_stages:
            t, steps = g.get("type"), int(g.get("train_steps", 0))
            if t == "experts":
                stages.append(PiscesLxGrowthStage("experts", int(g["num_experts"]), steps))
            elif t == "depth":
                n = int(g["num_layers"])
                take = min(n, current_layers) if current_layers else n
                stages.append(PiscesLxGrowthStage("depth", list(range(max(current_layers - take, 0), max(current_layers, take))), steps))
                current_layers += take
            elif t == "width" and "intermediate_size" in g:
                stages.append(PiscesLxGrowthStage("expert_width", int(g["intermediate_size"]), steps))
            elif t == "width":
                hidden.append({"hidden_size": int(g["hidden_size"]), "train_steps": steps})
        return PiscesLxEvolutionConfig(growth=tuple(stages)), hidden


class PiscesLxLoRALinear:
    """Factory: an ``nn.Linear`` as ``models.block_variants.YvLoRA`` with its bias kept."""

    def __new__(cls, lin: Any, r: int, alpha: float, dropout: float):
        import torch.nn.functional as F
        from ..models.block_variants import YvLoRA

        class _WithBias(YvLoRA):
            def forward(self, x):
                y = super().forward(x)
                return y if self.bias is None else y + self.bias.to(y.dtype)

        m = _WithBias(lin.weight, rank=r, alpha=float(alpha), dropout=dropout)
        m.bias = lin.bias
        m.in_features, m.out_features = lin.in_features, lin.out_features
        return m


@dataclass
class PiscesLxLoRAConfig:
    enabled: bool = False
    r: int = 8
    lora_alpha: int = 16
    lora_dropout: float = 0.05
    target_modules: Optional[List[str]] = None
    bias: str = "none"
    task_type: str = "CAUSAL_LM"

    def __post_init__(self) -> None:
        if self.r < 1:
            raise ValueError("LoRA rank must be at least 1")
        if self.bias not in ("none", "all", "lora_only"):
            raise ValueError(f"unknown bias mode {self.bias}")

    @property
    def scaling(self) -> float:
        return self.lora_alpha / self.r

    def matches(self, module_name: str) -> bool:
        targets = self.target_modules or ["q_proj", "k_proj", "v_proj", "o_proj"]
        leaf = module_name.rsplit(".", 1)[-1]
        return any(t == leaf or module_name.endswith(t) for t in targets)

    def apply(self, model: Any) -> int:
        """Wraps every matching ``nn.Linear`` in ``models.block_variants.YvLoRA`` and freezes the rest; returns how many."""
        if not self.enabled:
            return 0
        import torch.nn as nn
        hits = [(n, m) for n, m in model.named_modules() if isinstance(m, nn.Linear) and self.matches(n)]
        for p in model.parameters():
            p.requires_grad_(False)
        for name, lin in hits:
            parent = model
            *path, leaf = name.split(".")
            for part in path:
                parent = getattr(parent, part)
            setattr(parent, leaf, PiscesLxLoRALinear(lin, self.r, self.lora_alpha, self.lora_dropout))
        if self.bias == "all":
            for n, p in model.named_parameters():
                if n.endswith("bias"):
                    p.requires_grad_(True)
        return len(hits)


_SECTIONS = {"optimizer": PiscesLxOptimizerConfig, "scheduler": PiscesLxSchedulerConfig, "data": PiscesLxDataConfig,
             "quantization": PiscesLxTrainingQuantizationConfig, "lora": PiscesLxLoRAConfig, "evolution": PiscesLxTrainingEvolutionConfig}


def _section_from(cls: type, d: Any) -> Any:
    if isinstance(d, cls):
        return d
    names = {f.name for f in fields(cls)} if is_dataclass(cls) else set()
    return cls(**{k: v for k, v in (d or {}).items() if k in names})


@dataclass
class PiscesLxTrainingConfig:
    model_name: str = "pisceslx-base"
    output_dir: str = ".pisceslx/ckpt"
    memory_budget_gb: Optional[float] = None
    enable_expert_evolution: bool = True
    active_modalities: List[str] = field(default_factory=list)
    ddp_static_graph: bool = True
    early_stopping_patience: Optional[int] = None
    task_weights: Optional[Dict[str, float]] = None
    seed: Optional[int] = None
    max_steps: int = 100000
    save_steps: int = 1000
    eval_steps: int = 500
    log_steps: int = 10
    stage_declared_keys: List[str] = field(default_factory=list)
    device: str = "cuda"
    mixed_precision: str = "bf16"
    gradient_checkpointing: bool = True
    flash_attention: bool = True
    distributed: bool = False
    world_size: int = 1
    local_rank: int = -1
    gradient_accumulation_steps: int = 4
    optimizer: PiscesLxOptimizerConfig = field(default_factory=PiscesLxOptimizerConfig)
    scheduler: PiscesLxSchedulerConfig = field(default_factory=PiscesLxSchedulerConfig)
    data: PiscesLxDataConfig = field(default_factory=PiscesLxDataConfig)
    quantization: PiscesLxTrainingQuantizationConfig = field(default_factory=PiscesLxTrainingQuantizationConfig)
    lora: PiscesLxLoRAConfig = field(default_factory=PiscesLxLoRAConfig)
    evolution: PiscesLxTrainingEvolutionConfig = field(default_factory=PiscesLxTrainingEvolutionConfig)
    stage: Optional[PiscesLxTrainingStage] = None
    loss_type: str = "lm"
    response_only_loss: bool = False
    beta: float = 0.1
    reference_free: bool = False
    ppo_epochs: int = 4
    clip_range: float = 0.2
    kl_coef: float = 0.1
    lambda_orpo: float = 0.1
    packing: bool = False
    moe_gradient: Dict[str, Any] = field(default_factory=lambda: {"enabled": True})
    moe: Dict[str, Any] = field(default_factory=lambda: {"routing_temperature": 1.30, "temperature_min": 0.80, "temperature_max": 3.00,
                                                         "expert_temperature_max": 5.00, "expert_load_balance_threshold": 0.15})
    kfac: Dict[str, Any] = field(default_factory=lambda: {"enabled": True})
    multitask: Dict[str, Any] = field(default_factory=lambda: {"enabled": True})
    ink_optimizer: Dict[str, Any] = field(default_factory=dict)
    modality_scheduler: Dict[str, Any] = field(default_factory=lambda: {"enabled": True})
    enable_dpo: bool = True
    enable_sft: bool = True
    enable_pref_align: bool = True
    enable_multitask: bool = True
    enable_distillation: bool = False
    distill_teacher_path: Optional[str] = None
    distill_teacher_name: Optional[str] = None
    distill_teacher_api_key: Optional[str] = None
    distill_teacher_type: str = "local"
    distill_alpha: float = 0.5
    distill_temperature: float = 2.0
    parallel_3d: Dict[str, Any] = field(default_factory=lambda: {"enabled": True, "dp_size": 1, "tp_size": 1, "pp_size": 1, "sequence_parallel": True,
                                                                 "num_micro_batches": 4, "overlap_communication": True,
                                                                 "gradient_checkpointing": False, "zero_stage": 0})
    fsdp: Dict[str, Any] = field(default_factory=lambda: {"enabled": True, "sharding_strategy": "full_shard", "mixed_precision": True, "cpu_offload": False})
    fp8: Dict[str, Any] = field(default_factory=lambda: {"enabled": True, "format": "e4m3", "amax_history_len": 1024, "amax_compute_algo": "max"})

    STAGE_KEY_ALIASES = {
        "training": ("max_steps", "save_steps", "eval_steps", "log_steps", "packing", "mixed_precision", "flash_attention",
                     "gradient_checkpointing", "gradient_accumulation_steps", "memory_budget_gb", "seed"),
        "data": ("batch_size", "sequence_length", "num_workers", "pin_memory", "prefetch_factor"),
        "optimizer": ("learning_rate", "weight_decay", "max_grad_norm"),
        "scheduler": ("warmup_steps", "warmup_ratio", "min_lr_ratio"),
    }

    def __post_init__(self) -> None:
        for name, cls in _SECTIONS.items():
            setattr(self, name, _section_from(cls, getattr(self, name)))
        if self.stage is not None and not isinstance(self.stage, PiscesLxTrainingStage):
            self.stage = PiscesLxTrainingStage(self.stage)
        if self.mixed_precision not in ("fp32", "fp16", "bf16", "fp8"):
            raise ValueError(f"unknown mixed_precision {self.mixed_precision}")

    # -- construction -------------------------------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PiscesLxTrainingConfig":
        names = {f.name for f in fields(cls)}
        cfg = cls(**{k: copy.deepcopy(v) for k, v in d.items() if k in names})
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["stage"] = self.stage.value if self.stage is not None else None
        return d

    def resolved_output_dir(self) -> str:
        """``output_dir`` under the framework's home directory when it is relative (``PISCESLX_HOME`` moves the home)."""
        p = Path(self.output_dir)
        if p.is_absolute():
            return str(p)
        import os
        home = os.environ.get("PISCESLX_HOME")
        return str(Path(home) / p) if home else str(p)

    # -- stage files and overrides --------------------------------------------------------------------------------------------------
    def _apply_stage_file_config(self, stage_config: Dict[str, Any]) -> List[str]:
        """Applies a stage file: either sectioned (``training:`` / ``data:`` / ``optimizer:`` / ``scheduler:``, whose keys are
        the aliases above) or flat field names; returns the keys it set (kept in ``stage_declared_keys``, so that a later
        default does not override what the stage declared)."""
        declared: List[str] = []
        for key, val in (stage_config or {}).items():
            if key in self.STAGE_KEY_ALIASES and isinstance(val, dict):
                target = self if key == "training" else getattr(self, key)
                for k, v in val.items():
                    if k in ("lr",) and key == "optimizer":
                        k = "learning_rate"
                    if k == "type" and key == "scheduler":
                        k = "name"
                    if hasattr(target, k):
                        setattr(target, k, v)
                        declared.append(k if key == "training" else f"{key}.{k}")
            elif key in _SECTIONS and isinstance(val, dict):
                sec = getattr(self, key)
                for k, v in val.items():
                    if hasattr(sec, k):
                        setattr(sec, k, v)
                        declared.append(f"{key}.{k}")
            elif hasattr(self, key) and key != "stage":
                cur = getattr(self, key)
                if isinstance(cur, dict) and isinstance(val, dict):
                    cur.update(val)
                else:
                    setattr(self, key, val)
                declared.append(key)
        self.stage_declared_keys = sorted(set(self.stage_declared_keys) | set(declared))
        return declared

    def load_stage_config(self, stage: Union[str, PiscesLxTrainingStage], path: Optional[str] = None) -> List[str]:
        """Reads ``configs/train/<stage>.yaml`` (or ``path``) when it exists and applies it; a missing file only sets the stage."""
        self.stage = PiscesLxTrainingStage(getattr(stage, "value", stage))
        self.loss_type = self.stage.loss_type
        import yaml
        from .loader import REPO_ROOT
        p = Path(path) if path else REPO_ROOT / "configs" / "train" / f"{self.stage.value}.yaml"
        if not p.exists():
            return []
        return self._apply_stage_file_config(yaml.safe_load(p.read_text()) or {})

    def apply_overrides(self, overrides: Dict[str, Any]) -> None:
        """Dotted keys: ``{"optimizer.learning_rate": 3e-5, "max_steps": 10, "moe.routing_temperature": 1.1}``."""
        for key, val in overrides.items():
            obj: Any = self
            *path, leaf = key.split(".")
            for part in path:
                obj = obj[part] if isinstance(obj, dict) else getattr(obj, part)
            if isinstance(obj, dict):
                obj[leaf] = val
            elif hasattr(obj, leaf):
                setattr(obj, leaf, val)
            else:
                raise KeyError(f"unknown configuration key {key}")

    def validate(self) -> List[str]:
        """Problems as sentences (an empty list when there are none)."""
        out = []
        if self.max_steps <= 0:
            out.append("max_steps must be positive")
        if self.gradient_accumulation_steps < 1:
            out.append("gradient_accumulation_steps must be at least 1")
        if self.data.batch_size < 1 or self.data.sequence_length < 1:
            out.append("data.batch_size and data.sequence_length must be positive")
        p = self.parallel_3d
        if p.get("enabled") and self.distributed and p["dp_size"] * p["tp_size"] * p["pp_size"] not in (1, self.world_size):
            out.append(f"parallel_3d sizes multiply to {p['dp_size'] * p['tp_size'] * p['pp_size']}, world_size is {self.world_size}")
        if self.stage is not None and self.stage.needs_reference_model and self.reference_free and self.stage is not PiscesLxTrainingStage.ALIGNMENT_DPO:
            out.append(f"stage {self.stage.value} needs a reference model")
        if self.enable_distillation and not self.distill_teacher_path:
            out.append("enable_distillation needs distill_teacher_path")
        return out

    # -- onto this framework's trainer --------------------------------------------------------------------------------------------
    def effective_batch_size(self) -> int:
        dp = self.parallel_3d.get("dp_size", 1) if self.distributed else 1
        return self.data.batch_size * self.gradient_accumulation_steps * max(dp, 1)

    def to_trainer_config(self):
        """``engine.trainer.YvTrainerConfig``: the trainer takes the whole step's batch and splits it into micro-batches, so
        its ``micro_batch_size`` is ``data.batch_size`` and a step's batch is ``batch_size x gradient_accumulation_steps``."""
        from .trainer import YvTrainerConfig
        o, s = self.optimizer, self.scheduler
        kw: Dict[str, Any] = {}
        if o.resolved_name() in ("adamw", "fused_adamw"):
            kw = {"betas": tuple(o.betas), "eps": o.eps}
        zero = int(self.parallel_3d.get("zero_stage", 0))
        sharding = "full_shard" if (zero >= 3 or (self.fsdp.get("enabled") and self.fsdp.get("sharding_strategy") == "full_shard" and self.distributed)) else "zero1"
        return YvTrainerConfig(micro_batch_size=self.data.batch_size, optimizer=o.resolved_name(), lr=o.learning_rate, weight_decay=o.weight_decay,
                               scheduler=s.name, warmup_steps=s.resolved_warmup(self.max_steps), max_steps=self.max_steps,
                               min_lr_ratio=s.min_lr_ratio, clip_grad_norm=o.max_grad_norm, log_steps=self.log_steps, save_steps=self.save_steps,
                               output_dir=self.resolved_output_dir(), sharding=sharding, optimizer_kwargs=kw)
