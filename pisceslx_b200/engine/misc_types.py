"""Small configuration records, enumerations and error types of the training and run layers, each bound to the component that does
the work (reference opss/train/grpo.py ``PiscesLxAgenticRLConfig``, self_play.py ``PiscesLxSelfPlayConfig``, parallel_3d.py
``PiscesLxPipelineSchedule``, pref_align.py ``PiscesLxPreferenceAlignmentOperator``, profiler.py ``PiscesLxProfiler``,
subconscious_trainer.py:54-90, knowledge/builder.py, optim/offload.py ``PiscesLxTensorLifetime``, run/gpu_scheduler.py
``PiscesLxGPUAllocation``, run/recovery.py ``PiscesLxRecoveryState``, utils/vram_controller.py ``PiscesLxVRAMOptConfig``,
utils/host_memory.py, utils/muon.py, tools/train/run_reporter.py ``PiscesLxRunCancelled``, tools/train/core.py
``PiscesLxTrainingOperator``)."""
from __future__ import annotations

import time
from dataclasses import asdict, dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch
import torch.nn as nn

from ..utils.opsc import PiscesLxOperatorInterface
from .profiler import PiscesLxProfilingConfig, PiscesLxProfilingOperator
from .rl import PiscesLxGRPOConfig


# ---- errors ---------------------------------------------------------------------------------------------------------------------
class PiscesLxRunCancelled(Exception):
    """Raised between steps when the run's control file asks for a stop; carries the reason."""

    def __init__(self, reason: str = "cancelled"):
        self.reason = reason
        super().__init__(f"run cancelled: {reason}")


class PiscesLxHostMemoryBudgetError(MemoryError):
    """A stage would not fit, or a running step passed, the declared host-memory budget."""

    def __init__(self, needed_gb: float, budget_gb: float, stage: str = ""):
        self.needed_gb, self.budget_gb, self.stage = needed_gb, budget_gb, stage
        super().__init__(f"{stage or 'step'} needs {needed_gb:.2f} GB of host memory, the budget is {budget_gb:.2f} GB")


class PiscesLxMuonParameterError(ValueError):
    """A parameter was given to the orthogonalising optimizer group that it cannot handle (not a matrix, or an embedding / head)."""

    def __init__(self, name: str, shape: Sequence[int], why: str = "not a 2-D hidden weight"):
        self.name, self.shape = name, tuple(shape)
        super().__init__(f"parameter {name} {tuple(shape)} cannot go to the Muon group: {why}")


class YvHostTierError(RuntimeError):
    """The host tier (pinned staging of weights or cache blocks) could not serve a request."""


def check_muon_parameters(named_params: Sequence[Any], exclude: Sequence[str] = ("embed", "lm_head", "norm", "bias")) -> List[str]:
    """Names that may go to the Muon group; raises ``PiscesLxMuonParameterError`` for a matrix-group candidate that is not a matrix."""
    ok = []
    for n, p in named_params:
        if any(e in n for e in exclude):
            continue
        if p.dim() < 2:
            raise PiscesLxMuonParameterError(n, p.shape)
        ok.append(n)
    return ok


# ---- enumerations and records -------------------------------------------------------------------------------------------------
class PiscesLxPipelineSchedule(str, Enum):
    GPipe = "gpipe"
    ONE_F_ONE_B = "1f1b"
    INTERLEAVED = "interleaved"
    ZERO_BUBBLE = "zero_bubble"

    def bubble_fraction(self, stages: int, micro_batches: int, virtual_stages: int = 1) -> float:
        """Idle share of a pipeline step: (p - 1) / (m + p - 1) for GPipe and 1F1B, divided by the virtual stages when interleaved,
        and about a third of that with the backward split into input- and weight-gradient halves."""
        p, m = max(stages, 1), max(micro_batches, 1)
        base = (p - 1) / (m + p - 1)
        if self is PiscesLxPipelineSchedule.INTERLEAVED:
            return (p - 1) / (virtual_stages * m + p - 1)
        return base / 3.0 if self is PiscesLxPipelineSchedule.ZERO_BUBBLE else base

    def trainer_name(self) -> str:
        """The schedule ``engine.trainer.YvTrainerConfig.pipeline_schedule`` runs (interleaved and zero-bubble fall back to 1F1B)."""
        return "gpipe" if self is PiscesLxPipelineSchedule.GPipe else "1f1b"


class PiscesLxTrainingPhase(str, Enum):
    ROUTER_PRETRAIN = "router_pretrain"
    JOINT_RL = "joint_rl"
    SELF_PLAY = "self_play"


@dataclass
class PiscesLxSubconsciousTrainingConfig:
    phase: PiscesLxTrainingPhase = PiscesLxTrainingPhase.ROUTER_PRETRAIN
    router_learning_rate: float = 1e-5
    state_learning_rate: float = 3e-6
    film_learning_rate: float = 1e-6
    rl_learning_rate: float = 3e-6
    clip_epsilon: float = 0.2
    entropy_coef: float = 0.01
    value_coef: float = 0.5
    reward_normalize: bool = True
    kl_penalty_coef: float = 0.1
    aux_loss_coef: float = 0.01
    router_entropy_reg: float = 0.05
    max_grad_norm: float = 1.0
    use_ppo: bool = True
    ppo_epochs: int = 4
    ppo_minibatch_size: int = 256
    gamma: float = 0.99
    gae_lambda: float = 0.95

    def __post_init__(self) -> None:
        self.phase = PiscesLxTrainingPhase(getattr(self.phase, "value", self.phase))

    def learning_rate(self) -> float:
        return {PiscesLxTrainingPhase.ROUTER_PRETRAIN: self.router_learning_rate, PiscesLxTrainingPhase.JOINT_RL: self.rl_learning_rate,
                PiscesLxTrainingPhase.SELF_PLAY: self.rl_learning_rate}[self.phase]

    def param_groups(self, model: nn.Module) -> List[Dict[str, Any]]:
        """Router, state and FiLM parameters with their own rates (matched by name); the rest stays frozen in the router phase."""
        groups = {"router": ([], self.router_learning_rate), "state": ([], self.state_learning_rate), "film": ([], self.film_learning_rate)}
        rest: List[nn.Parameter] = []
        for n, p in model.named_parameters():
            if not p.requires_grad:
                continue
            key = next((k for k in groups if k in n.lower()), None)
            (groups[key][0] if key else rest).append(p)
        out = [{"params": ps, "lr": lr, "name": k} for k, (ps, lr) in groups.items() if ps]
        if rest and self.phase is not PiscesLxTrainingPhase.ROUTER_PRETRAIN:
            out.append({"params": rest, "lr": self.rl_learning_rate, "name": "rest"})
        return out

    def build_trainer(self, model: Any, router: nn.Module):
        from .knowledge import PiscesLxSubconsciousTrainer
        return PiscesLxSubconsciousTrainer(model, router, lr=self.learning_rate())


@dataclass
class PiscesLxAgenticRLConfig:
    name: str = "agentic_rl"
    agent_rollout_steps: int = 8
    max_tool_calls: int = 20
    tool_call_reward: float = 0.1
    task_completion_reward: float = 1.0
    efficiency_penalty: float = -0.01
    use_agentic_grpo: bool = False
    grpo_config: PiscesLxGRPOConfig = field(default_factory=PiscesLxGRPOConfig)

    def episode_reward(self, tool_calls_ok: int, steps: int, completed: bool, needed_steps: int = 0) -> float:
        """Reward of one episode: per successful tool call (capped at ``max_tool_calls``), completion, and a penalty per step beyond what
        the task needed."""
        extra = max(steps - needed_steps, 0)
        return min(tool_calls_ok, self.max_tool_calls) * self.tool_call_reward + (self.task_completion_reward if completed else 0.0) + extra * self.efficiency_penalty

    def build_trainer(self, model: Any, optimizer: torch.optim.Optimizer, env_factory: Callable[[], Any], **kw: Any):
        from .rl import PiscesLxAgenticRLTrainer
        return PiscesLxAgenticRLTrainer(model, optimizer, env_factory, group_size=self.grpo_config.group_size, max_turns=self.agent_rollout_steps, **kw)


@dataclass
class PiscesLxSelfPlayConfig:
    name: str = "self_play"
    num_rounds: int = 3
    num_samples: int = 4
    temperature: float = 0.8
    top_p: float = 0.9
    max_generation_length: int = 1024
    score_method: str = "self_critic"
    self_critic_prompt: str = "Rate the quality of the following response on a scale of 1 to 10:"
    grpo_group_size: int = 4
    grpo_temperature: float = 1.0
    grpo_clip_ratio: float = 0.2
    grpo_kl_coef: float = 0.1
    dpo_beta: float = 0.1
    max_prompt_length: int = 2048
    batch_size: int = 8
    learning_rate: float = 1e-6
    use_reward_model: bool = False
    reward_model_update_interval: int = 2
    diversity_penalty: float = 0.05
    use_mmr_diversity: bool = True
    mmr_lambda: float = 0.5

    def __post_init__(self) -> None:
        if self.score_method not in ("self_critic", "reward_model", "rule", "length_normalized_logprob"):
            raise ValueError(f"unknown score_method {self.score_method}")
        if not 0.0 <= self.mmr_lambda <= 1.0:
            raise ValueError("mmr_lambda must lie in [0, 1]")

    def select_diverse(self, scores: Sequence[float], similarity: Sequence[Sequence[float]], k: int) -> List[int]:
        """Maximal-marginal-relevance choice of ``k`` samples: score traded against the largest similarity to what is already chosen."""
        left, chosen = list(range(len(scores))), []
        while left and len(chosen) < k:
            def mmr(i: int) -> float:
                red = max((similarity[i][j] for j in chosen), default=0.0)
                return self.mmr_lambda * scores[i] - (1 - self.mmr_lambda) * red if self.use_mmr_diversity else scores[i]
            b = max(left, key=mmr)
            chosen.append(b)
            left.remove(b)
        return chosen

    def build_trainer(self, policy: nn.Module, optimizer: torch.optim.Optimizer, generate_fn: Callable, logprob_fn: Callable):
        from .alignment import PiscesLxSelfPlayTrainer
        return PiscesLxSelfPlayTrainer(policy, optimizer, generate_fn, logprob_fn, beta=self.dpo_beta)


@dataclass
class PiscesLxKnowledgeBuilderConfig:
    encoder_hidden: int = 640
    encoder_layers: int = 16
    encoder_experts: int = 4
    encoder_heads: int = 10
    knowledge_dim: int = 256
    knowledge_slots: int = 1 << 20
    chunk_size: int = 256
    chunk_overlap: int = 32
    contrastive_temperature: float = 0.07
    contrastive_epochs: int = 1
    n_list: int = 16
    pq_subvectors: int = 8

    def chunks(self, tokens: Sequence[int]) -> List[List[int]]:
        step = max(self.chunk_size - self.chunk_overlap, 1)
        return [list(tokens[i:i + self.chunk_size]) for i in range(0, max(len(tokens) - self.chunk_overlap, 1), step)]


class PiscesLxBuilder:
    """``PiscesLxBuilder(config, encode).build(texts)``: the knowledge store of ``engine.knowledge.PiscesLxKnowledgeBuilder`` from a
    configuration (``encode`` maps a list of texts to [n, knowledge_dim] vectors)."""

    def __init__(self, config: Optional[PiscesLxKnowledgeBuilderConfig] = None, encode: Optional[Callable[[List[str]], torch.Tensor]] = None):
        from .knowledge import PiscesLxKnowledgeBuilder
        self.config = config or PiscesLxKnowledgeBuilderConfig()
        if encode is None:
            raise ValueError("an encode function (texts -> vectors) is needed")
        self.builder = PiscesLxKnowledgeBuilder(encode, self.config.knowledge_dim, self.config.n_list, self.config.pq_subvectors)

    def build(self, texts: List[str]):
        self.builder.build(texts[: self.config.knowledge_slots])
        return self.builder


class PiscesLxKnowledgeBuildCli:
    @staticmethod
    def build_parser():
        import argparse
        p = argparse.ArgumentParser(prog="knowledge-build", description="Build the knowledge store from text files")
        p.add_argument("--input", required=True)
        p.add_argument("--output", required=True)
        p.add_argument("--knowledge-dim", dest="knowledge_dim", type=int, default=256)
        p.add_argument("--chunk-size", dest="chunk_size", type=int, default=256)
        p.add_argument("--n-list", dest="n_list", type=int, default=16)
        return p

    @classmethod
    def main(cls, argv: Optional[Sequence[str]] = None, encode: Optional[Callable[[List[str]], torch.Tensor]] = None) -> Dict[str, Any]:
        from pathlib import Path
        a = cls.build_parser().parse_args(list(argv) if argv is not None else None)
        src = Path(a.input)
        files = sorted(src.rglob("*.txt")) if src.is_dir() else [src]
        texts = [t for f in files for t in f.read_text(encoding="utf-8").split("\n\n") if t.strip()]
        cfg = PiscesLxKnowledgeBuilderConfig(knowledge_dim=a.knowledge_dim, chunk_size=a.chunk_size, n_list=min(a.n_list, max(len(texts), 1)))
        b = PiscesLxBuilder(cfg, encode).build(texts)
        Path(a.output).parent.mkdir(parents=True, exist_ok=True)
        torch.save({"config": asdict(cfg), "texts": texts, "state": {k: v for k, v in vars(b).items() if torch.is_tensor(v)}}, a.output)
        return {"texts": len(texts), "output": a.output}


@dataclass
class PiscesLxTensorLifetime:
    name: str
    create_step: int
    last_use_step: int
    size_bytes: int
    access_pattern: List[int] = field(default_factory=list)

    @property
    def lifetime(self) -> int:
        return self.last_use_step - self.create_step

    def next_use_after(self, step: int) -> Optional[int]:
        return next((s for s in sorted(self.access_pattern) if s > step), None)

    def idle_gap_at(self, step: int) -> int:
        """Steps until the next access (what an offload decision weighs against the transfer time); a tensor never used again: a large number."""
        n = self.next_use_after(step)
        return (n - step) if n is not None else 1 << 30

    def worth_offloading(self, step: int, bytes_per_step: float) -> bool:
        """True when the tensor can leave and come back within its idle gap at the given transfer budget per step."""
        return self.idle_gap_at(step) * bytes_per_step >= 2 * self.size_bytes


@dataclass
class PiscesLxGPUAllocation:
    task_id: str
    gpu_ids: List[int]
    allocated_at: str = field(default_factory=lambda: time.strftime("%Y-%m-%dT%H:%M:%S"))
    memory_required_mb: int = 0
    priority: str = "normal"

    def to_env(self) -> Dict[str, str]:
        return {"CUDA_VISIBLE_DEVICES": ",".join(str(g) for g in self.gpu_ids)}


@dataclass
class PiscesLxRecoveryState:
    restart_count: int = 0
    max_restarts: int = 3
    last_checkpoint: Optional[str] = None
    last_restart_at: Optional[str] = None
    recovery_enabled: bool = True
    recovery_history: List[Dict[str, Any]] = field(default_factory=list)

    def can_restart(self) -> bool:
        return self.recovery_enabled and self.restart_count < self.max_restarts

    def record_restart(self, reason: str, checkpoint: Optional[str] = None) -> bool:
        if not self.can_restart():
            return False
        self.restart_count += 1
        self.last_restart_at = time.strftime("%Y-%m-%dT%H:%M:%S")
        self.last_checkpoint = checkpoint or self.last_checkpoint
        self.recovery_history.append({"n": self.restart_count, "reason": reason, "checkpoint": self.last_checkpoint, "at": self.last_restart_at})
        return True

    def backoff_seconds(self, base: float = 5.0, cap: float = 300.0) -> float:
        return min(base * 2 ** max(self.restart_count - 1, 0), cap)


@dataclass
class PiscesLxVRAMOptConfig:
    use_flash_attention: bool = True
    use_mla: bool = True
    sdpa_prefer_flash: bool = True
    cache_quantization: bool = True
    use_mixed_precision_cache: bool = True
    kv_cache_block_size: int = 512
    use_partial_rope: bool = True
    use_gradient_checkpointing: bool = True
    adaptive_recomputation: bool = True
    selective_checkpointing: bool = True
    cpu_offload_optimizer: bool = False
    cpu_offload_weights: bool = False
    activation_quantization: bool = False
    enable_teraio: bool = False
    dynamic_expert_loading: bool = True
    max_experts_on_gpu: int = 4
    zero_stage: int = 3
    recommended_batch_size: int = 1
    recommended_grad_accum: int = 4
    recommended_seq_len: int = 2048

    @classmethod
    def for_device(cls, total_gb: float, model_gb: float) -> "PiscesLxVRAMOptConfig":
        """Settings by head-room: with weights + optimizer state (about 8 x the bf16 weights under Adam) well inside the device, nothing is
        offloaded and recomputation is selective; as the ratio tightens, sharding, then offloading, then activation quantisation come on."""
        need = 8.0 * model_gb
        room = total_gb / max(need, 1e-9)
        if room >= 1.5:
            return cls(cache_quantization=False, selective_checkpointing=True, adaptive_recomputation=False, zero_stage=1, dynamic_expert_loading=False,
                       max_experts_on_gpu=1 << 30, recommended_batch_size=8, recommended_grad_accum=1, recommended_seq_len=8192, kv_cache_block_size=64)
        if room >= 0.5:
            return cls(zero_stage=3, recommended_batch_size=2, recommended_grad_accum=4, recommended_seq_len=4096, kv_cache_block_size=64)
        return cls(zero_stage=3, cpu_offload_optimizer=True, enable_teraio=True, activation_quantization=True, recommended_batch_size=1, recommended_grad_accum=8)

    def apply(self, cfg: Any) -> Any:
        """Writes the fields the model configuration knows onto it."""
        for k in ("use_gradient_checkpointing", "kv_cache_block_size", "use_flash_attention", "use_mla"):
            if hasattr(cfg, k):
                setattr(cfg, k, getattr(self, k))
        return cfg


# ---- operators -------------------------------------------------------------------------------------------------------------------
class PiscesLxPreferenceAlignmentOperator(PiscesLxOperatorInterface):
    """One front for the preference methods: ``{"method": "dpo" | "ppo" | "kto" | "bco", ...}`` goes to the operator of that name with the
    remaining inputs."""

    name = "preference_alignment"
    METHODS = ("dpo", "ppo", "kto", "bco")

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return str(inputs.get("method", "")).lower() in self.METHODS and inputs.get("model") is not None

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        m = inputs["method"].lower()
        rest = {k: v for k, v in inputs.items() if k != "method"}
        if m == "dpo":
            from .stage_operators import PiscesLxDPOOperator
            return {"method": m, **PiscesLxDPOOperator().run(rest)}
        if m == "ppo":
            from .stage_operators import PiscesLxPPOStepOperator
            return {"method": m, **{k: v for k, v in PiscesLxPPOStepOperator().run(rest).items() if k != "ppo"}}
        from .rl import PiscesLxBCOOperator, PiscesLxKTOOperator
        cls = PiscesLxKTOOperator if m == "kto" else PiscesLxBCOOperator
        op = rest.get("operator") or cls(rest["model"], rest["optimizer"], rest.get("reference_model"), **(rest.get("kwargs") or {}))
        return {"method": m, "operator": op, **op.step(rest["prompts"], rest["completions"], rest["desirable"])}


class PiscesLxProfiler(PiscesLxProfilingOperator):
    """The step profiler under its short name (``engine.profiler.PiscesLxProfilingOperator``)."""


class PiscesLxTrainingOperator(PiscesLxOperatorInterface):
    """``tools/train``'s core operator: builds ``YvTrainer`` from a ``PiscesLxTrainingConfig`` and runs steps over batches."""

    name = "training_operator"

    def __init__(self, config: Any = None):
        from .train_config import PiscesLxTrainingConfig
        self.config = config if isinstance(config, PiscesLxTrainingConfig) else PiscesLxTrainingConfig.from_dict(config or {})
        self.trainer: Any = None

    def build(self, model: nn.Module, parallel: Any = None):
        from .trainer import YvTrainer
        problems = self.config.validate()
        if problems:
            raise ValueError("; ".join(problems))
        self.config.lora.apply(model)
        self.trainer = YvTrainer(model, self.config.to_trainer_config(), parallel=parallel)
        return self.trainer

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return (self.trainer is not None or isinstance(inputs.get("model"), nn.Module)) and inputs.get("batches") is not None

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        if self.trainer is None:
            self.build(inputs["model"], inputs.get("parallel"))
        hist = []
        for b in inputs["batches"]:
            if self.trainer.global_step >= self.config.max_steps:
                break
            hist.append(self.trainer.train_step(b))
        return {"steps": len(hist), "final_loss": hist[-1]["loss"] if hist else None, "history": hist, "trainer": self.trainer}
