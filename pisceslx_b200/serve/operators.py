"""Inference operators with the reference's operator ABI (``execute(inputs) -> PiscesLxOperatorResult``): sampling and
beam search (reference opss/infer/sampling.py), GPU check (opss/infer/check.py), selective-state-space layers
(opss/infer/mamba.py), native inference (opss/infer/native_ruchbah.py), and the tool registry of the agent layer
(opss/am/registry.py).  Each is a thin, working front of this package's own implementation."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, List, Optional

import torch

from ..models.generation import YvSampler, YvSamplingConfig
from ..utils.opsc import PiscesLxOperatorInterface


# ------------------------------------------------------------------------------------------------ sampling
@dataclass
class PiscesLxSamplingConfig:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    no_repeat_ngram_size: int = 0
    seed: Optional[int] = None

    def to_sampler(self) -> YvSampler:
        if self.temperature <= 0:
            strat = "greedy"
        elif self.top_k and self.top_p < 1.0:
            strat = "top_k_top_p"
        elif self.top_k:
            strat = "top_k"
        elif self.top_p < 1.0:
            strat = "top_p"
        else:
            strat = "top_k_top_p"
        return YvSampler(YvSamplingConfig(strategy=strat, temperature=max(self.temperature, 1e-6), top_k=self.top_k,
                                          top_p=self.top_p, min_p=self.min_p, repetition_penalty=self.repetition_penalty,
                                          no_repeat_ngram_size=self.no_repeat_ngram_size, seed=self.seed))


class PiscesLxSamplingOperator(PiscesLxOperatorInterface):
    """inputs: {"logits": [B, V], "generated": optional [B, S] ids (for the penalties)} -> {"tokens": [B]}."""
    name = "sampling"

    def __init__(self, config: Optional[PiscesLxSamplingConfig] = None):
        self.config = config or PiscesLxSamplingConfig()
        self.sampler = self.config.to_sampler()

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs.get("logits"), torch.Tensor) and inputs["logits"].dim() == 2

    def run(self, inputs: Dict[str, Any]) -> Dict[str, torch.Tensor]:
        return {"tokens": self.sampler.sample(inputs["logits"], inputs.get("generated"))}


class PiscesLxBeamSearchOperator(PiscesLxOperatorInterface):
    """inputs: {"model", "input_ids": [1, S], "num_beams", "max_new_tokens", "length_penalty"} -> {"sequence"}."""
    name = "beam_search"

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return "model" in inputs and isinstance(inputs.get("input_ids"), torch.Tensor)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, torch.Tensor]:
        from ..models.speculative import beam_search
        seq = beam_search(inputs["model"], inputs["input_ids"], int(inputs.get("num_beams", 4)),
                          int(inputs.get("max_new_tokens", 32)), float(inputs.get("length_penalty", 1.0)),
                          inputs.get("eos_token_id"))
        return {"sequence": seq}


# ------------------------------------------------------------------------------------------------ GPU check
@dataclass
class PiscesLxGPUMemoryInfo:
    index: int
    name: str
    total_gb: float
    free_gb: float
    compute_capability: str

    @property
    def used_gb(self) -> float:
        return self.total_gb - self.free_gb


class PiscesLxGPUCheckOperator(PiscesLxOperatorInterface):
    """Reports the visible GPUs and whether a model of ``required_gb`` fits on one of them (read-only queries).
    ``probe`` can be replaced for tests; the default asks the CUDA runtime."""
    name = "gpu_check"

    def __init__(self, probe: Optional[Callable[[], List[PiscesLxGPUMemoryInfo]]] = None):
        self.probe = probe or self._cuda_probe

    @staticmethod
    def _cuda_probe() -> List[PiscesLxGPUMemoryInfo]:
        out = []
        if torch.cuda.is_available():
            for i in range(torch.cuda.device_count()):
                free, total = torch.cuda.mem_get_info(i)
                p = torch.cuda.get_device_properties(i)
                out.append(PiscesLxGPUMemoryInfo(i, p.name, total / 2 ** 30, free / 2 ** 30, f"{p.major}.{p.minor}"))
        return out

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        need = float(inputs.get("required_gb", 0.0))
        gpus = self.probe()
        fits = [g.index for g in gpus if g.free_gb >= need]
        native = [g.index for g in gpus if g.compute_capability.startswith("10.")]
        return {"gpus": gpus, "count": len(gpus), "fits_on": fits, "sm_100_devices": native,
                "ok": bool(gpus) and bool(fits) and (not inputs.get("require_sm100") or bool(native))}


# ------------------------------------------------------------------------------------------------ SSM layers
class PiscesLxSSMType(str, Enum):
    MAMBA = "mamba"
    MAMBA2 = "mamba2"
    MAMBA3 = "mamba3"


@dataclass
class PiscesLxMambaConfig:
    hidden_size: int = 512
    d_state: int = 16
    expand: int = 2
    d_conv: int = 4
    ssm_type: PiscesLxSSMType = PiscesLxSSMType.MAMBA3


class PiscesLxMambaMixer(torch.nn.Module):
    """The selective-scan mixer of this package (``models.ssm.YvSelectiveSSM``) under the reference's name."""

    def __init__(self, cfg: PiscesLxMambaConfig):
        super().__init__()
        from ..models.ssm import YvSelectiveSSM
        self.inner = YvSelectiveSSM(cfg.hidden_size, state_dim=cfg.d_state, expansion_factor=cfg.expand,
                                    conv_kernel=cfg.d_conv)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.inner(x)


class PiscesLxMambaLayer(torch.nn.Module):
    """Pre-norm residual layer around the mixer."""

    def __init__(self, cfg: PiscesLxMambaConfig):
        super().__init__()
        from ..models.norms import YvRMSNorm
        self.norm, self.mixer = YvRMSNorm(cfg.hidden_size), PiscesLxMambaMixer(cfg)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.mixer(self.norm(x))


class PiscesLxMambaOperator(PiscesLxOperatorInterface):
    """inputs: {"hidden_states": [B, S, H]} -> {"hidden_states"} through ``n_layers`` SSM layers."""
    name = "mamba"

    def __init__(self, config: Optional[PiscesLxMambaConfig] = None, n_layers: int = 1):
        self.config = config or PiscesLxMambaConfig()
        self.layers = torch.nn.ModuleList([PiscesLxMambaLayer(self.config) for _ in range(n_layers)])

    def run(self, inputs: Dict[str, Any]) -> Dict[str, torch.Tensor]:
        h = inputs["hidden_states"]
        self.layers.to(h.device)
        for l in self.layers:
            h = l(h)
        return {"hidden_states": h}


class PiscesLxMamba2Operator(PiscesLxMambaOperator):
    name = "mamba2"

    def __init__(self, config: Optional[PiscesLxMambaConfig] = None, n_layers: int = 1):
        cfg = config or PiscesLxMambaConfig(ssm_type=PiscesLxSSMType.MAMBA2)
        super().__init__(cfg, n_layers)


# ------------------------------------------------------------------------------------------------ native inference
class PiscesLxNativeInferenceOperator(PiscesLxOperatorInterface):
    """inputs: {"prompt" | "input_ids", "max_new_tokens", "temperature", ...} -> {"text" | "output_ids", "stats"}.
    Built from a model instance, or from (model_size, checkpoint) through ``engine.loader``."""
    name = "native_inference"

    def __init__(self, model: Any = None, tokenizer: Any = None, model_size: str = "0.01B", ckpt: Optional[str] = None,
                 device: Optional[str] = None):
        if model is None:
            from ..engine.loader import load_model_for_inference
            model = load_model_for_inference(model_size, ckpt, device)
        self.model = model.eval()
        if tokenizer is None:
            from ..models.tokenizer import YvTokenizer
            vocab = int(getattr(getattr(self.model, "cfg", None), "vocab_size", 0) or 0)
            tokenizer = YvTokenizer.for_vocab(vocab) if vocab else YvTokenizer.instance()
        self.tok = tokenizer

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return "prompt" in inputs or "input_ids" in inputs

    @torch.no_grad()
    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        dev = next(self.model.parameters()).device
        ids = inputs.get("input_ids")
        if ids is None:
            ids = torch.tensor([self.tok.encode(inputs["prompt"])], dtype=torch.long)
        ids = ids.to(dev)
        t0 = time.perf_counter()
        out, stats = self.model.generate(ids, max_new_tokens=int(inputs.get("max_new_tokens", 32)),
                                         temperature=inputs.get("temperature"), top_k=inputs.get("top_k"),
                                         top_p=inputs.get("top_p"), eos_token_id=inputs.get("eos_token_id"))
        new = out[0, ids.shape[1]:].tolist()
        res: Dict[str, Any] = {"output_ids": new, "stats": {**stats, "seconds": time.perf_counter() - t0}}
        if "prompt" in inputs:
            res["text"] = self.tok.decode(new)
        return res


# ------------------------------------------------------------------------------------------------ tool registry (am)
class PiscesLxToolType(str, Enum):
    FUNCTION = "function"
    MCP = "mcp"
    BUILTIN = "builtin"


@dataclass
class PiscesLxToolInfo:
    name: str
    description: str = ""
    parameters: Dict[str, str] = field(default_factory=dict)
    tool_type: PiscesLxToolType = PiscesLxToolType.FUNCTION
    tags: List[str] = field(default_factory=list)
    calls: int = 0
    failures: int = 0


@dataclass
class PiscesLxToolResult:
    name: str
    success: bool
    output: Any = None
    error: Optional[str] = None
    seconds: float = 0.0


class PiscesLxToolRegistry:
    """Registry with call statistics and tag / text search; ``as_agent_registry`` gives the object the ReAct agent
    and the server routes use."""

    def __init__(self):
        self.infos: Dict[str, PiscesLxToolInfo] = {}
        self.fns: Dict[str, Callable[..., Any]] = {}

    def register(self, name: str, fn: Callable[..., Any], description: str = "", parameters: Optional[Dict[str, str]] = None,
                 tool_type: PiscesLxToolType = PiscesLxToolType.FUNCTION, tags: Optional[List[str]] = None) -> PiscesLxToolInfo:
        info = PiscesLxToolInfo(name, description, parameters or {}, tool_type, tags or [])
        self.infos[name], self.fns[name] = info, fn
        return info

    def unregister(self, name: str) -> bool:
        self.fns.pop(name, None)
        return self.infos.pop(name, None) is not None

    def execute(self, name: str, **kwargs: Any) -> PiscesLxToolResult:
        t0 = time.perf_counter()
        info = self.infos.get(name)
        if info is None:
            return PiscesLxToolResult(name, False, error=f"unknown tool {name!r}")
        info.calls += 1
        try:
            return PiscesLxToolResult(name, True, self.fns[name](**kwargs), None, time.perf_counter() - t0)
        except Exception as e:
            info.failures += 1
            return PiscesLxToolResult(name, False, None, f"{type(e).__name__}: {e}", time.perf_counter() - t0)

    def search(self, query: str = "", tag: Optional[str] = None) -> List[PiscesLxToolInfo]:
        q = query.lower()
        return [i for i in self.infos.values()
                if (not q or q in i.name.lower() or q in i.description.lower()) and (tag is None or tag in i.tags)]

    def as_agent_registry(self):
        from ..models.reasoning import YvToolRegistry
        reg = YvToolRegistry()
        for name, info in self.infos.items():
            reg.register(name, info.description, info.parameters)(self.fns[name])
        return reg
