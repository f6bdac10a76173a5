"""The inference configuration tree (reference tools/infer/config.py:73-1000): model / generation / acceleration /
quantisation / sampling / MoE sections under ``PiscesLxInferenceConfig``, the service configuration with its OPSS and
run sections, model specifications by size, and the mappings onto this framework's engine.

Serialisation is generic over the dataclass tree (the reference spells every field of every section out twice, once in
``to_dict`` and once in ``from_dict``, config.py:361-550).  Model specifications are read from the preset files under
``configs/model`` instead of a second hand-kept table, so a preset and its specification cannot drift apart."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field, fields, is_dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional, Union, get_type_hints


def _from_dict(cls: type, d: Optional[Dict[str, Any]]) -> Any:
    """A dataclass of type ``cls`` from a dictionary: nested dataclass fields are built recursively, unknown keys dropped."""
    d = d or {}
    hints = get_type_hints(cls)
    kw = {}
    for f in fields(cls):
        if f.name not in d:
            continue
        v, t = d[f.name], hints.get(f.name)
        args = getattr(t, "__args__", ())
        sub = t if is_dataclass(t) else next((a for a in args if is_dataclass(a)), None)
        kw[f.name] = _from_dict(sub, v) if (sub is not None and isinstance(v, dict)) else v
    return cls(**kw)


@dataclass
class PiscesLxModelConfig:
    model_path: str = ""
    model_type: str = "auto"
    tokenizer_path: Optional[str] = None
    trust_remote_code: bool = False


@dataclass
class PiscesLxGenerationConfig:
    max_new_tokens: int = 512
    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 50
    repetition_penalty: float = 1.0
    do_sample: bool = True
    num_beams: int = 1
    early_stopping: bool = False

    def __post_init__(self) -> None:
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if self.temperature < 0 or not 0 < self.top_p <= 1:
            raise ValueError("temperature must not be negative and top_p must lie in (0, 1]")


@dataclass
class PiscesLxAccelerationConfig:
    use_vllm: bool = False                         # the paged batch engine (this framework's own; no external engine is loaded)
    use_speculative_decoding: bool = False
    spec_gamma: int = 4
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    gpu_memory_utilization: float = 0.9
    enforce_eager: bool = False                    # True switches the CUDA-graph decode replay off
    use_torch_compile: bool = False                # accepted and ignored: the hot path is hand-written kernels under CUDA graphs
    max_num_seqs: int = 256
    min_new_tokens: int = 16
    use_ring_attention: bool = False
    ring_block_size: int = 4096
    max_sequence_length: int = 1048576
    use_mamba: bool = False


@dataclass
class PiscesLxInferQuantizationConfig:
    enable_quantization: bool = False
    quant_method: str = "awq"                      # awq | gptq | squeezellm | fp8 | rtn | smoothquant
    bits: int = 4
    group_size: int = 128
    symmetric: bool = True
    zero_point: bool = True

    def to_pipeline_config(self):
        from ..quant.pipeline import PiscesLxQuantizationConfig, PiscesLxQuantizationMethod
        m = {"awq": "awq", "gptq": "gptq", "smoothquant": "smoothquant"}.get(self.quant_method, "rtn")
        return PiscesLxQuantizationConfig(method=PiscesLxQuantizationMethod(m), bits=8 if self.quant_method == "fp8" else self.bits, group_size=self.group_size)


@dataclass
class PiscesLxSamplingConfig:
    use_advanced_sampling: bool = True
    nucleus_sampling: bool = True
    contrastive_search: bool = False
    beam_search: bool = False
    diverse_beam_search: bool = False


@dataclass
class PiscesLxMoEConfig:
    enable_moe: bool = False
    routing_temp: float = 1.12
    top_k: int = 2
    capacity_factor: float = 1.0
    min_capacity: int = 4
    enable_expert_caching: bool = True
    expert_cache_size: int = 10000
    enable_load_balancing: bool = True
    load_balance_alpha: float = 0.01
    enable_adaptive_temp: bool = True
    adaptive_temp_step: float = 0.03
    adaptive_temp_interval: int = 16
    adaptive_temp_cap: float = 1.30
    enable_prefix_caching: bool = True
    priority_routing: bool = False
    drop_tokens: bool = True

    def to_runtime_config(self):
        from .moe_runtime import PiscesLxMoERuntimeConfig
        return PiscesLxMoERuntimeConfig(routing_strategy="priority" if self.priority_routing else "adaptive", routing_temp=self.routing_temp, top_k=self.top_k,
                                        capacity_factor=self.capacity_factor, min_capacity=self.min_capacity, enable_expert_cache=self.enable_expert_caching,
                                        expert_cache_size=self.expert_cache_size, enable_load_balancing=self.enable_load_balancing,
                                        load_balance_alpha=self.load_balance_alpha, enable_adaptive_temp=self.enable_adaptive_temp,
                                        adaptive_temp_step=self.adaptive_temp_step, adaptive_temp_interval=self.adaptive_temp_interval,
                                        adaptive_temp_cap=self.adaptive_temp_cap, drop_tokens=self.drop_tokens)


@dataclass
class PiscesLxInferenceConfig:
    model: PiscesLxModelConfig = field(default_factory=PiscesLxModelConfig)
    generation: PiscesLxGenerationConfig = field(default_factory=PiscesLxGenerationConfig)
    device: str = "cuda"
    dtype: str = "auto"
    memory_limit: Optional[int] = None             # MB
    acceleration: PiscesLxAccelerationConfig = field(default_factory=PiscesLxAccelerationConfig)
    quantization: PiscesLxInferQuantizationConfig = field(default_factory=PiscesLxInferQuantizationConfig)
    sampling: PiscesLxSamplingConfig = field(default_factory=PiscesLxSamplingConfig)
    moe: PiscesLxMoEConfig = field(default_factory=PiscesLxMoEConfig)
    batch_size: int = 1
    max_batch_size: int = 32
    enable_prefix_caching: bool = True
    enable_chunked_prefill: bool = True
    enable_monitoring: bool = True
    log_level: str = "INFO"
    metrics_export_interval: int = 10

    def __post_init__(self) -> None:
        if self.dtype not in ("auto", "float16", "bfloat16", "float32", "fp16", "bf16", "fp32"):
            raise ValueError(f"unknown dtype {self.dtype}")

    # -- serialisation -------------------------------------------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    @classmethod
    def from_dict(cls, config_dict: Dict[str, Any]) -> "PiscesLxInferenceConfig":
        return _from_dict(cls, config_dict)

    def save_to_json(self, filepath: str) -> None:
        Path(filepath).parent.mkdir(parents=True, exist_ok=True)
        Path(filepath).write_text(json.dumps(self.to_dict(), indent=2))

    @classmethod
    def load_from_json(cls, filepath: str) -> "PiscesLxInferenceConfig":
        return cls.from_dict(json.loads(Path(filepath).read_text()))

    def save_to_yaml(self, filepath: str) -> None:
        import yaml
        Path(filepath).parent.mkdir(parents=True, exist_ok=True)
        Path(filepath).write_text(yaml.safe_dump(self.to_dict(), sort_keys=False))

    @classmethod
    def load_from_yaml(cls, filepath: str) -> "PiscesLxInferenceConfig":
        import yaml
        return cls.from_dict(yaml.safe_load(Path(filepath).read_text()) or {})

    def apply_cli_overrides(self, args: Dict[str, Any]) -> None:
        """The command line's inference switches (``infer_mode``, ``speculative``, ``spec_gamma``, ``min_new_tokens``, ``quant`` /
        ``no_quant`` / ``force_quant`` / ``quant_bits``, ``max_new_tokens``, ``temperature``, ``top_p``, ``top_k``, ``device``,
        ``dtype``, ``model_path``, ``tp``).  Values that do not parse are left alone."""
        def num(key: str, cast):
            v = args.get(key)
            if v is None:
                return None
            try:
                return cast(v)
            except (TypeError, ValueError):
                return None
        mode = args.get("infer_mode")
        if mode in ("vllm", "standard"):
            self.acceleration.use_vllm = mode == "vllm"
        if args.get("speculative"):
            self.acceleration.use_speculative_decoding = True
        for key, target, name, cast in (("spec_gamma", self.acceleration, "spec_gamma", int), ("min_new_tokens", self.acceleration, "min_new_tokens", int),
                                        ("tp", self.acceleration, "tensor_parallel_size", int), ("quant_bits", self.quantization, "bits", int),
                                        ("max_new_tokens", self.generation, "max_new_tokens", int), ("temperature", self.generation, "temperature", float),
                                        ("top_p", self.generation, "top_p", float), ("top_k", self.generation, "top_k", int)):
            v = num(key, cast)
            if v is not None:
                setattr(target, name, v)
        if args.get("no_quant"):
            self.quantization.enable_quantization = False
        if args.get("quant") or args.get("force_quant"):
            self.quantization.enable_quantization = True
        for key, target, name in (("device", self, "device"), ("dtype", self, "dtype"), ("model_path", self.model, "model_path")):
            if args.get(key):
                setattr(target, name, args[key])

    # -- onto this framework ---------------------------------------------------------------------------------------------------------
    def torch_dtype(self):
        import torch
        return {"auto": torch.bfloat16, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
                "fp32": torch.float32, "float32": torch.float32}[self.dtype]

    def to_engine_config(self, model_cfg: Any = None, device_memory_bytes: Optional[int] = None):
        """``serve.engine.YvEngineConfig``.  The number of cache blocks comes from the memory the cache may use -
        ``gpu_memory_utilization`` of the device (or ``memory_limit`` MB) minus the weights - and the bytes of one block."""
        from .engine import YvEngineConfig
        a = self.acceleration
        block = int(getattr(model_cfg, "kv_cache_block_size", 64) or 64)
        max_len = min(a.max_sequence_length, int(getattr(model_cfg, "max_position_embeddings", a.max_sequence_length) or a.max_sequence_length))
        blocks = 4096
        budget = self.memory_limit * (1 << 20) if self.memory_limit else (int(device_memory_bytes * a.gpu_memory_utilization) if device_memory_bytes else None)
        if budget and model_cfg is not None:
            per_tok = self.kv_bytes_per_token(model_cfg)
            n = getattr(model_cfg, "count_parameters", lambda: 0)()
            weights = int(n["total"] if isinstance(n, dict) else n) * 2 // max(a.tensor_parallel_size, 1)
            blocks = max(int((budget - weights) // max(per_tok * block, 1)), a.max_num_seqs)
        return YvEngineConfig(max_num_seqs=min(a.max_num_seqs, max(self.max_batch_size, 1)) if not a.use_vllm else a.max_num_seqs, num_blocks=blocks,
                              block_size=block, max_model_len=max_len, use_cuda_graphs=not a.enforce_eager)

    def kv_bytes_per_token(self, model_cfg: Any) -> int:
        """Bytes one token's keys and values take over all layers on one tensor-parallel rank, at 2 bytes an element (the
        compressed latent width when the model uses latent attention)."""
        layers = int(getattr(model_cfg, "n_layer", 0))
        lat = int(getattr(model_cfg, "kv_lora_rank", 0) or 0)
        if lat:
            width = lat + int(getattr(model_cfg, "qk_rope_head_dim", 0) or 0)
        else:
            kvh = int(getattr(model_cfg, "n_kv_head", getattr(model_cfg, "n_head", 1)))
            hd = int(getattr(model_cfg, "head_dim", 0) or (model_cfg.hidden_size // model_cfg.n_head))
            width = 2 * max(kvh // max(self.acceleration.tensor_parallel_size, 1), 1) * hd
        return layers * width * 2

    def to_sampling(self):
        """``models.generation.YvSamplingConfig`` for these generation and sampling switches."""
        from ..models.generation import YvSamplingConfig
        g, s = self.generation, self.sampling
        if s.beam_search or s.diverse_beam_search or g.num_beams > 1:
            strategy = "beam"
        elif s.contrastive_search:
            strategy = "contrastive"
        elif not g.do_sample or g.temperature == 0:
            strategy = "greedy"
        else:
            strategy = "top_k_top_p" if (s.nucleus_sampling or s.use_advanced_sampling) else "temperature"
        return YvSamplingConfig(strategy=strategy, temperature=max(g.temperature, 1e-5) if strategy != "greedy" else 1.0, top_k=g.top_k, top_p=g.top_p,
                                repetition_penalty=g.repetition_penalty, num_beams=max(g.num_beams, 1))


# ---- model specifications ------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxModelSpec:
    name: str
    hidden_size: int
    num_layers: int
    num_heads: int
    context_length: int
    moe_experts: int = 0
    moe_active: int = 0
    vocab_size: int = 151936
    intermediate_size: int = 0
    num_kv_heads: int = 0
    rope_theta: float = 10000.0
    max_position_embeddings: int = 0

    def __post_init__(self) -> None:
        if self.intermediate_size == 0:
            self.intermediate_size = self.hidden_size * 4 // 3 * 2
        if self.num_kv_heads == 0:
            self.num_kv_heads = self.num_heads
        if self.max_position_embeddings == 0:
            self.max_position_embeddings = self.context_length

    @classmethod
    def from_preset(cls, name: str, d: Dict[str, Any]) -> "PiscesLxModelSpec":
        ctx = int(d.get("max_position_embeddings", 0) or 0)
        return cls(name=name, hidden_size=int(d["hidden_size"]), num_layers=int(d["n_layer"]), num_heads=int(d["n_head"]), context_length=ctx,
                   moe_experts=int(d.get("moe_num_experts", 0) or 0), moe_active=int(d.get("moe_top_k", 0) or 0), vocab_size=int(d.get("vocab_size", 151936)),
                   intermediate_size=int(d.get("intermediate_size", 0) or 0), num_kv_heads=int(d.get("n_kv_head", 0) or 0),
                   rope_theta=float(d.get("rope_theta", 10000.0)), max_position_embeddings=ctx)


def _preset_dir() -> Path:
    return Path(__file__).resolve().parents[2] / "configs" / "model"


def _load_specs() -> Dict[str, PiscesLxModelSpec]:
    import yaml
    out: Dict[str, PiscesLxModelSpec] = {}
    d = _preset_dir()
    if not d.is_dir():
        return out
    for f in sorted(d.glob("*.yaml")):
        try:
            y = yaml.safe_load(f.read_text()) or {}
            if {"hidden_size", "n_layer", "n_head"} <= set(y):
                out[f.stem] = PiscesLxModelSpec.from_preset(f.stem, y)
        except (OSError, ValueError, KeyError, yaml.YAMLError):
            continue
    return out


MODEL_SPECS: Dict[str, PiscesLxModelSpec] = _load_specs()


@dataclass
class PiscesLxOPSSConfig:
    enable_mcp_plaza: bool = True
    enable_swarm_coordinator: bool = True
    enable_orchestrator: bool = True
    enable_mcp_bridge: bool = True
    mcp_max_workers: int = 10
    mcp_session_timeout: int = 3600
    swarm_max_agents: int = 20
    swarm_topology: str = "hierarchical"
    orchestrator_max_parallel: int = 5
    bridge_cache_ttl: int = 300
    bridge_retry_count: int = 3
    heartbeat_interval: float = 10.0
    heartbeat_timeout: float = 60.0


@dataclass
class PiscesLxRunConfig:
    run_id: Optional[str] = None
    run_dir: Optional[str] = None
    run_name: Optional[str] = None
    control_interval_s: float = 0.5
    max_concurrency: int = 8
    request_timeout_s: float = 120.0
    resource_interval_s: float = 5.0
    enable_resource_monitor: bool = True
    enable_heartbeat: bool = True
    enable_gpu_monitor: bool = True


@dataclass
class PiscesLxServiceConfig:
    model_size: str = "7B"
    model_spec: Optional[PiscesLxModelSpec] = None
    inference: PiscesLxInferenceConfig = field(default_factory=PiscesLxInferenceConfig)
    opss: PiscesLxOPSSConfig = field(default_factory=PiscesLxOPSSConfig)
    run: PiscesLxRunConfig = field(default_factory=PiscesLxRunConfig)
    host: str = "127.0.0.1"
    port: int = 8000
    api_key: Optional[str] = None
    cors_origins: List[str] = field(default_factory=lambda: ["*"])

    def __post_init__(self) -> None:
        if self.model_spec is None and self.model_size in MODEL_SPECS:
            self.model_spec = MODEL_SPECS[self.model_size]
        if not 0 < int(self.port) < 65536:
            raise ValueError(f"port {self.port} out of range")

    def to_dict(self, redact: bool = True) -> Dict[str, Any]:
        d = asdict(self)
        if redact and d.get("api_key"):
            d["api_key"] = "***"
        return d

    @classmethod
    def from_dict(cls, config_dict: Dict[str, Any]) -> "PiscesLxServiceConfig":
        return _from_dict(cls, config_dict)


class PiscesLxConfig:
    @staticmethod
    def get_model_spec(model_size: str) -> PiscesLxModelSpec:
        if model_size not in MODEL_SPECS:
            raise ValueError(f"Unknown model size: {model_size}. Available: {list(MODEL_SPECS.keys())}")
        return MODEL_SPECS[model_size]

    @staticmethod
    def list_available_models() -> List[str]:
        return list(MODEL_SPECS.keys())

    @staticmethod
    def default_service(model_size: str = "7B", **overrides: Any) -> PiscesLxServiceConfig:
        return PiscesLxServiceConfig(model_size=model_size, **overrides)
