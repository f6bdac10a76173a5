"""Training operators with the reference's operator ABI and names, built on this package's losses and trainers:
distillation (reference opss/train/distill.py), RLVR (rlvr.py), DAPO (dapo.py), on-policy distillation (opss/opd.py),
memory separation (memsep.py), the evolution pipeline (evolution_pipeline.py) and the advanced-training
coordinator (impl.py).  Models are anything callable as ``model(input_ids=...)`` returning ``.logits`` / ``["logits"]``;
generation and log-probabilities are injected as callables where a run needs them, so that the operators work with
the eager model, the serving engine or a test double alike."""
from __future__ import annotations

import copy
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..utils.opsc import PiscesLxOperatorInterface, PiscesLxOperatorResult, PiscesLxOperatorStatus
from . import alignment as A


def _logits(out: Any) -> torch.Tensor:
    return out["logits"] if isinstance(out, dict) else out.logits


# ------------------------------------------------------------------------------------------------ distillation
@dataclass
class PiscesLxDistillationConfig:
    temperature: float = 2.0
    alpha: float = 0.5                 # weight of the soft (teacher) term against the hard-label term
    hidden_weight: float = 0.0         # optional hidden-state matching
    lr: float = 1e-4
    max_steps: int = 100


class PiscesLxDistillationDataset(torch.utils.data.Dataset):
    def __init__(self, sequences: Sequence[torch.Tensor]):
        self.seqs = list(sequences)

    def __len__(self) -> int:
        return len(self.seqs)

    def __getitem__(self, i: int) -> Dict[str, torch.Tensor]:
        return {"input_ids": self.seqs[i], "labels": self.seqs[i]}


class PiscesLxDistillationOperator(PiscesLxOperatorInterface):
    """inputs: {"student", "teacher", "batches": iterable of [B, S] ids, "optimizer" (optional)} -> loss history."""
    name = "distillation"

    def __init__(self, config: Optional[PiscesLxDistillationConfig] = None):
        self.config = config or PiscesLxDistillationConfig()

    def step(self, student: nn.Module, teacher: nn.Module, ids: torch.Tensor, opt: torch.optim.Optimizer) -> Dict[str, float]:
        c = self.config
        with torch.no_grad():
            t_logits = _logits(teacher(input_ids=ids)).float()
        s_logits = _logits(student(input_ids=ids)).float()
        soft = A.distill_logits_loss(s_logits[:, :-1], t_logits[:, :-1], c.temperature)
        hard = F.cross_entropy(s_logits[:, :-1].reshape(-1, s_logits.shape[-1]), ids[:, 1:].reshape(-1))
        loss = c.alpha * soft + (1 - c.alpha) * hard
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return {"loss": float(loss.detach()), "soft": float(soft.detach()), "hard": float(hard.detach())}

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return all(k in inputs for k in ("student", "teacher", "batches"))

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        student, teacher = inputs["student"], inputs["teacher"].eval()
        opt = inputs.get("optimizer") or torch.optim.AdamW(student.parameters(), lr=self.config.lr)
        hist = []
        for i, ids in enumerate(inputs["batches"]):
            if i >= self.config.max_steps:
                break
            hist.append(self.step(student, teacher, ids, opt))
        return {"history": hist, "final_loss": hist[-1]["loss"] if hist else None}


# ------------------------------------------------------------------------------------------------ RLVR / DAPO
class PiscesLxRLVRVerifierType(str, Enum):
    EXACT = "exact"
    NUMERIC = "numeric"
    CUSTOM = "custom"


@dataclass
class PiscesLxRLVRConfig:
    verifier: PiscesLxRLVRVerifierType = PiscesLxRLVRVerifierType.EXACT
    group_size: int = 4
    clip_eps: float = 0.2
    clip_eps_high: Optional[float] = None      # set (> clip_eps) for the decoupled clipping of DAPO
    dynamic_sampling: bool = False             # drop groups whose rewards are all equal (DAPO)
    lr: float = 1e-5
    numeric_tol: float = 1e-6


class PiscesLxRLVRDataset(torch.utils.data.Dataset):
    """Rows: {"prompt": ids tensor, "answer": str}."""

    def __init__(self, rows: Sequence[Dict[str, Any]]):
        self.rows = list(rows)

    def __len__(self) -> int:
        return len(self.rows)

    def __getitem__(self, i: int) -> Dict[str, Any]:
        return self.rows[i]


class PiscesLxRLVRTrainer:
    """Group-relative policy optimisation against a verifiable reward.  ``sample_fn(policy, prompt_ids) ->
    (response_ids, text)`` draws one response; ``logprob_fn(policy, prompt_ids, response_ids) -> scalar`` scores it."""

    def __init__(self, policy: nn.Module, optimizer: torch.optim.Optimizer, sample_fn: Callable, logprob_fn: Callable,
                 config: Optional[PiscesLxRLVRConfig] = None, predicate: Optional[Callable[[str, str], bool]] = None):
        self.policy, self.opt, self.sample_fn, self.logprob_fn = policy, optimizer, sample_fn, logprob_fn
        self.cfg = config or PiscesLxRLVRConfig()
        kind = "numeric" if self.cfg.verifier == PiscesLxRLVRVerifierType.NUMERIC else "exact"
        self.verifier = A.PiscesLxRLVRVerifier(kind, self.cfg.numeric_tol, predicate)

    def step(self, rows: Sequence[Dict[str, Any]]) -> Dict[str, float]:
        G, cfg = self.cfg.group_size, self.cfg
        prompts, responses, rewards, old = [], [], [], []
        with torch.no_grad():
            for r in rows:
                for _ in range(G):
                    resp, text = self.sample_fn(self.policy, r["prompt"])
                    prompts.append(r["prompt"])
                    responses.append(resp)
                    rewards.append(self.verifier.reward(text, r["answer"]))
                    old.append(self.logprob_fn(self.policy, r["prompt"], resp))
        rew = torch.tensor(rewards)
        old_lp = torch.stack([o.detach().float().reshape(()) for o in old])
        keep = A.dapo_filter_groups(rew, G) if cfg.dynamic_sampling else torch.ones_like(rew, dtype=torch.bool)
        if not bool(keep.any()):
            return {"loss": 0.0, "mean_reward": float(rew.mean()), "kept_groups": 0}
        lp = torch.stack([self.logprob_fn(self.policy, p, r).float().reshape(()) for p, r in zip(prompts, responses)])
        if cfg.clip_eps_high is not None:
            loss = A.dapo_loss(lp[:, None], old_lp[:, None], rew, G, mask=keep[:, None], eps_low=cfg.clip_eps,
                               eps_high=cfg.clip_eps_high)
        else:
            adv = A.group_relative_advantages(rew, G)
            ratio = torch.exp(lp - old_lp)
            per = -torch.minimum(ratio * adv, ratio.clamp(1 - cfg.clip_eps, 1 + cfg.clip_eps) * adv)
            loss = (per * keep).sum() / keep.sum().clamp_min(1)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return {"loss": float(loss.detach()), "mean_reward": float(rew.mean()), "kept_groups": int(keep.sum()) // G}


class PiscesLxRLVROperator(PiscesLxOperatorInterface):
    """inputs: {"trainer": PiscesLxRLVRTrainer, "dataset": rows, "steps", "rows_per_step"} -> reward history."""
    name = "rlvr"

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return "trainer" in inputs and "dataset" in inputs

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        tr, ds = inputs["trainer"], inputs["dataset"]
        per, hist = int(inputs.get("rows_per_step", 2)), []
        for s in range(int(inputs.get("steps", 1))):
            rows = [ds[(s * per + i) % len(ds)] for i in range(per)]
            hist.append(tr.step(rows))
        return {"history": hist, "mean_reward": sum(h["mean_reward"] for h in hist) / max(len(hist), 1)}


class PiscesLxDAPO(PiscesLxRLVRTrainer):
    """DAPO = the RLVR trainer with decoupled clipping (higher upper clip) and dynamic sampling switched on."""

    def __init__(self, policy: nn.Module, optimizer: torch.optim.Optimizer, sample_fn: Callable, logprob_fn: Callable,
                 group_size: int = 4, eps_low: float = 0.2, eps_high: float = 0.28, **kw: Any):
        super().__init__(policy, optimizer, sample_fn, logprob_fn,
                         PiscesLxRLVRConfig(group_size=group_size, clip_eps=eps_low, clip_eps_high=eps_high,
                                            dynamic_sampling=True), **kw)


# ------------------------------------------------------------------------------------------------ on-policy distillation
@dataclass
class PiscesLxOPDConfig:
    lr: float = 1e-5
    max_new_tokens: int = 32
    reverse_kl: bool = True            # KL(student || teacher) on the student's own samples


class PiscesLxOPDTrainer:
    """On-policy distillation: the student generates, the teacher scores the student's tokens, and the student is
    pulled towards the teacher's distribution on the states the student actually visits."""

    def __init__(self, student: nn.Module, teacher: nn.Module, optimizer: torch.optim.Optimizer, generate_fn: Callable,
                 config: Optional[PiscesLxOPDConfig] = None):
        self.student, self.teacher, self.opt, self.generate_fn = student, teacher.eval(), optimizer, generate_fn
        self.cfg = config or PiscesLxOPDConfig()

    def step(self, prompts: Sequence[torch.Tensor]) -> Dict[str, float]:
        total, n = 0.0, 0
        self.opt.zero_grad(set_to_none=True)
        for p in prompts:
            with torch.no_grad():
                full = self.generate_fn(self.student, p, self.cfg.max_new_tokens)       # [1, S + n]
                t_lp = torch.log_softmax(_logits(self.teacher(input_ids=full)).float(), -1)
            s_lp = torch.log_softmax(_logits(self.student(input_ids=full)).float(), -1)
            lo = p.shape[-1] - 1
            s_gen, t_gen = s_lp[:, lo:-1], t_lp[:, lo:-1]
            if self.cfg.reverse_kl:
                kl = (s_gen.exp() * (s_gen - t_gen)).sum(-1).mean()
            else:
                kl = (t_gen.exp() * (t_gen - s_gen)).sum(-1).mean()
            (kl / len(prompts)).backward()
            total += float(kl.detach())
            n += 1
        self.opt.step()
        return {"kl": total / max(n, 1)}


PiscesLxOpd = PiscesLxOPDTrainer


# ------------------------------------------------------------------------------------------------ memory separation
class PiscesLxMemSepPhase(str, Enum):
    CORE_REASONING = "core_reasoning"                  # backbone trains, memory gate clamped to 0, router frozen
    MEMORY_ROUTER_TRAINING = "memory_router_training"  # backbone frozen, router + injection train, gate ramps up
    KNOWLEDGE_STORE_BUILD = "knowledge_store_build"    # offline: encode corpora, build the index


@dataclass
class PiscesLxMemSepTrainingConfig:
    gate_max: float = 1.0
    ramp_steps: int = 1000
    ramp_sharpness: float = 8.0
    memory_param_patterns: Tuple[str, ...] = ("subconscious", "knowledge", "memory", "film")
    memory_lr_scale: float = 1.0
    alignment_margin: float = 0.5
    consistency_weight: float = 0.01


class PiscesLxMemSepGateScheduler:
    """Gate value by phase: 0 in phase 1; a sigmoid ramp 0 -> gate_max over ``ramp_steps`` in phase 2; gate_max after."""

    def __init__(self, config: PiscesLxMemSepTrainingConfig):
        self.cfg, self.phase, self.step_in_phase = config, PiscesLxMemSepPhase.CORE_REASONING, 0

    def get_gate(self) -> float:
        import math
        if self.phase == PiscesLxMemSepPhase.CORE_REASONING:
            return 0.0
        if self.phase == PiscesLxMemSepPhase.MEMORY_ROUTER_TRAINING:
            x = self.step_in_phase / max(1, self.cfg.ramp_steps)
            s = lambda v: 1.0 / (1.0 + math.exp(-self.cfg.ramp_sharpness * (v - 0.5)))
            return self.cfg.gate_max * min(1.0, max(0.0, (s(x) - s(0.0)) / (s(1.0) - s(0.0))))
        return self.cfg.gate_max

    def advance_phase(self, phase: PiscesLxMemSepPhase) -> None:
        self.phase, self.step_in_phase = phase, 0

    def step(self) -> None:
        self.step_in_phase += 1


class PiscesLxMemSepParamManager:
    """Splits parameters into backbone and memory (by name patterns) and freezes the side a phase does not train."""

    def __init__(self, model: nn.Module, config: PiscesLxMemSepTrainingConfig):
        self.model, self.cfg = model, config
        self.memory, self.backbone = [], []
        for n, p in model.named_parameters():
            (self.memory if any(pat in n.lower() for pat in config.memory_param_patterns) else self.backbone).append((n, p))

    def set_phase(self, phase: PiscesLxMemSepPhase) -> None:
        train_backbone = phase == PiscesLxMemSepPhase.CORE_REASONING
        train_memory = phase == PiscesLxMemSepPhase.MEMORY_ROUTER_TRAINING
        for _, p in self.backbone:
            p.requires_grad_(train_backbone)
        for _, p in self.memory:
            p.requires_grad_(train_memory)

    def get_optimizer_param_groups(self, lr: float) -> List[Dict[str, Any]]:
        groups = []
        bb = [p for _, p in self.backbone if p.requires_grad]
        mm = [p for _, p in self.memory if p.requires_grad]
        if bb:
            groups.append({"params": bb, "lr": lr, "name": "backbone"})
        if mm:
            groups.append({"params": mm, "lr": lr * self.cfg.memory_lr_scale, "name": "memory"})
        return groups


class PiscesLxMemoryAlignmentLoss(nn.Module):
    """Router alignment: a hinge on the distances to the retrieved entries (retrieved knowledge should be within
    ``margin`` of the query) plus a consistency term that penalises the variance of the retrieved vectors across
    sequence positions."""

    def __init__(self, margin: float = 0.5, consistency_weight: float = 0.01):
        super().__init__()
        self.margin, self.consistency_weight = margin, consistency_weight

    def forward(self, knowledge_ctx: Optional[Dict[str, torch.Tensor]]) -> torch.Tensor:
        if not knowledge_ctx:
            return torch.zeros(())
        loss = torch.zeros((), device=next(iter(knowledge_ctx.values())).device)
        if "distances" in knowledge_ctx:
            loss = loss + F.relu(knowledge_ctx["distances"].float() - self.margin).mean()
        if "knowledge" in knowledge_ctx:
            k = knowledge_ctx["knowledge"].float()
            flat = k.reshape(-1, k.shape[-1])
            if flat.shape[0] > 1:
                loss = loss + self.consistency_weight * flat.var(dim=0).mean()
        return loss


class PiscesLxMemSepTrainer:
    """Drives the phases: freezes / unfreezes, pushes the scheduled gate into every module that has a
    ``memory_gate`` attribute (``set_gate`` if it has one), and adds the alignment loss."""

    def __init__(self, model: nn.Module, config: Optional[PiscesLxMemSepTrainingConfig] = None):
        self.model, self.cfg = model, config or PiscesLxMemSepTrainingConfig()
        self.sched = PiscesLxMemSepGateScheduler(self.cfg)
        self.params = PiscesLxMemSepParamManager(model, self.cfg)
        self.align = PiscesLxMemoryAlignmentLoss(self.cfg.alignment_margin, self.cfg.consistency_weight)
        self.start_phase(PiscesLxMemSepPhase.CORE_REASONING)

    def start_phase(self, phase: PiscesLxMemSepPhase) -> None:
        self.sched.advance_phase(phase)
        self.params.set_phase(phase)
        self._apply_gate()

    def _apply_gate(self) -> None:
        g = self.sched.get_gate()
        for m in self.model.modules():
            if hasattr(m, "set_gate"):
                m.set_gate(g)
            elif hasattr(m, "memory_gate") and not isinstance(getattr(m, "memory_gate"), nn.Parameter):
                m.memory_gate = g

    def pre_step(self) -> float:
        self._apply_gate()
        g = self.sched.get_gate()
        self.sched.step()
        return g

    def compute_memory_loss(self, knowledge_ctx: Optional[Dict[str, torch.Tensor]]) -> torch.Tensor:
        return self.align(knowledge_ctx) if self.sched.phase == PiscesLxMemSepPhase.MEMORY_ROUTER_TRAINING else torch.zeros(())

    def get_stats(self) -> Dict[str, Any]:
        return {"phase": self.sched.phase.value, "gate": self.sched.get_gate(), "step_in_phase": self.sched.step_in_phase,
                "trainable_backbone": sum(p.numel() for _, p in self.params.backbone if p.requires_grad),
                "trainable_memory": sum(p.numel() for _, p in self.params.memory if p.requires_grad)}


class PiscesLxMemsep:
    @staticmethod
    def create_memsep_trainer(model: nn.Module, **kw: Any) -> PiscesLxMemSepTrainer:
        return PiscesLxMemSepTrainer(model, PiscesLxMemSepTrainingConfig(**kw))


# ------------------------------------------------------------------------------------------------ evolution pipeline
class PiscesLxEvolutionStage(str, Enum):
    DISTILLATION = "distillation"
    GROWTH = "growth"
    SELF_EVOLUTION = "self_evolution"
    WEAK_TO_STRONG = "weak_to_strong"
    DONE = "done"


@dataclass
class PiscesLxGrowthStage:
    kind: str                        # "experts" | "expert_width" | "depth"
    value: Any                       # new expert count, new FFN width, or list of layer positions to duplicate
    train_steps: int = 0


@dataclass
class PiscesLxEvolutionConfig:
    stages: Tuple[PiscesLxEvolutionStage, ...] = (PiscesLxEvolutionStage.DISTILLATION, PiscesLxEvolutionStage.GROWTH)
    growth: Tuple[PiscesLxGrowthStage, ...] = ()
    distill: PiscesLxDistillationConfig = field(default_factory=PiscesLxDistillationConfig)
    lr: float = 1e-4


class PiscesLxEvolutionTracker:
    def __init__(self):
        self.t0, self.stage = time.time(), None
        self.metrics: Dict[str, List[Tuple[str, float]]] = {}
        self.stage_history: List[Tuple[str, float]] = []

    def set_stage(self, stage: PiscesLxEvolutionStage) -> None:
        self.stage = stage
        self.stage_history.append((stage.value, time.time() - self.t0))

    def log_step(self, name: str, value: float) -> None:
        self.metrics.setdefault(name, []).append((self.stage.value if self.stage else "", float(value)))

    def get_summary(self) -> Dict[str, Any]:
        return {"elapsed_s": time.time() - self.t0, "stages": [s for s, _ in self.stage_history],
                "last": {k: v[-1][1] for k, v in self.metrics.items()}, "n_logged": {k: len(v) for k, v in self.metrics.items()}}


class PiscesLxEvolutionPipeline(PiscesLxOperatorInterface):
    """Seed -> larger model: (1) distil a teacher into the seed, (2) grow it (experts, expert width, depth; each
    growth is function preserving) with training after every growth, (3) optional weak-to-strong polishing.
    inputs: {"model", "batches": callable -> iterable of [B, S] ids, "teacher" (for distillation),
    "train_step": callable(model, ids) -> loss (for the training after growth)}."""
    name = "evolution_pipeline"

    def __init__(self, config: Optional[PiscesLxEvolutionConfig] = None):
        self.config = config or PiscesLxEvolutionConfig()
        self.tracker = PiscesLxEvolutionTracker()

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return "model" in inputs and callable(inputs.get("batches"))

    def _grow(self, model: nn.Module, g: PiscesLxGrowthStage) -> None:
        if g.kind == "depth":
            A.grow_depth(model, list(g.value))
            return
        for blk in model.model.layers:
            mlp = getattr(blk, "mlp", None)
            if mlp is None or not hasattr(mlp, "experts_w13"):
                continue
            if g.kind == "experts":
                A.grow_experts(mlp, int(g.value))
            elif g.kind == "expert_width":
                A.grow_expert_width(mlp, int(g.value))
            else:
                raise ValueError(f"unknown growth kind {g.kind!r}")

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        model, batches = inputs["model"], inputs["batches"]
        for stage in self.config.stages:
            self.tracker.set_stage(stage)
            if stage == PiscesLxEvolutionStage.DISTILLATION:
                op = PiscesLxDistillationOperator(self.config.distill)
                res = op.run({"student": model, "teacher": inputs["teacher"], "batches": batches()})
                for h in res["history"]:
                    self.tracker.log_step("distill_loss", h["loss"])
            elif stage == PiscesLxEvolutionStage.GROWTH:
                for g in self.config.growth:
                    before = sum(p.numel() for p in model.parameters())
                    self._grow(model, g)
                    self.tracker.log_step("params", sum(p.numel() for p in model.parameters()))
                    self.tracker.log_step("params_added", sum(p.numel() for p in model.parameters()) - before)
                    step_fn = inputs.get("train_step")
                    if step_fn is not None and g.train_steps:
                        for i, ids in enumerate(batches()):
                            if i >= g.train_steps:
                                break
                            self.tracker.log_step("growth_loss", float(step_fn(model, ids)))
            elif stage == PiscesLxEvolutionStage.WEAK_TO_STRONG and "weak_labels" in inputs:
                for ids, weak in inputs["weak_labels"]():
                    logits = _logits(model(input_ids=ids)).float()
                    self.tracker.log_step("w2s_loss", float(A.weak_to_strong_loss(logits.reshape(-1, logits.shape[-1]), weak.reshape(-1))))
        self.tracker.set_stage(PiscesLxEvolutionStage.DONE)
        return self.tracker.get_summary()

    def get_progress(self) -> Dict[str, Any]:
        return self.tracker.get_summary()


# ------------------------------------------------------------------------------------------------ advanced training
@dataclass
class PiscesLxAdvancedTrainingConfig:
    mixed_precision: str = "bf16"
    grad_clip: float = 1.0
    grad_accumulation: int = 1
    weight_decay: float = 0.0
    label_smoothing: float = 0.0
    dropout: Optional[float] = None
    lr: float = 1e-4
    warmup_steps: int = 0
    total_steps: int = 1000
    schedule: str = "cosine"


class PiscesLxMixedPrecisionTrainingOperator(PiscesLxOperatorInterface):
    """inputs {"fn": callable, "device_type"} -> runs fn under autocast of the configured dtype (fp32 = no autocast)."""
    name = "mixed_precision"

    def __init__(self, config: PiscesLxAdvancedTrainingConfig):
        self.dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": None}[config.mixed_precision]

    def run(self, inputs: Dict[str, Any]) -> Any:
        if self.dtype is None:
            return inputs["fn"]()
        with torch.autocast(inputs.get("device_type", "cuda" if torch.cuda.is_available() else "cpu"), dtype=self.dtype):
            return inputs["fn"]()


class PiscesLxGradientOptimizationOperator(PiscesLxOperatorInterface):
    """inputs {"parameters"} -> clips the global gradient norm; reports the norm before clipping and non-finite grads."""
    name = "gradient_optimization"

    def __init__(self, config: PiscesLxAdvancedTrainingConfig):
        self.clip = config.grad_clip

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        ps = [p for p in inputs["parameters"] if p.grad is not None]
        bad = sum(int(not torch.isfinite(p.grad).all()) for p in ps)
        norm = torch.nn.utils.clip_grad_norm_(ps, self.clip if self.clip > 0 else float("inf"))
        return {"grad_norm": float(norm), "non_finite_tensors": bad, "clipped": self.clip > 0 and float(norm) > self.clip}


class PiscesLxRegularizationOperator(PiscesLxOperatorInterface):
    """inputs {"logits", "labels"} -> cross entropy with the configured label smoothing; {"model"} -> sets dropout."""
    name = "regularization"

    def __init__(self, config: PiscesLxAdvancedTrainingConfig):
        self.cfg = config

    def run(self, inputs: Dict[str, Any]) -> Any:
        if "model" in inputs and self.cfg.dropout is not None:
            n = 0
            for m in inputs["model"].modules():
                if isinstance(m, nn.Dropout):
                    m.p = self.cfg.dropout
                    n += 1
            return {"dropout_modules": n}
        lg = inputs["logits"].float()
        return F.cross_entropy(lg.reshape(-1, lg.shape[-1]), inputs["labels"].reshape(-1), label_smoothing=self.cfg.label_smoothing)


class PiscesLxLearningRateSchedulerOperator(PiscesLxOperatorInterface):
    """inputs {"optimizer", "step"} -> sets and returns the learning rate of the configured schedule."""
    name = "lr_scheduler"

    def __init__(self, config: PiscesLxAdvancedTrainingConfig):
        self.cfg = config

    def lr_at(self, step: int) -> float:
        import math
        c = self.cfg
        if c.warmup_steps and step < c.warmup_steps:
            return c.lr * (step + 1) / c.warmup_steps
        t = min(1.0, (step - c.warmup_steps) / max(1, c.total_steps - c.warmup_steps))
        if c.schedule == "cosine":
            return c.lr * 0.5 * (1 + math.cos(math.pi * t))
        if c.schedule == "linear":
            return c.lr * (1 - t)
        return c.lr

    def run(self, inputs: Dict[str, Any]) -> float:
        lr = self.lr_at(int(inputs["step"]))
        for g in inputs["optimizer"].param_groups:
            g["lr"] = lr * g.get("lr_scale", 1.0)
        return lr


class PiscesLxDistributedTrainingOperator(PiscesLxOperatorInterface):
    """inputs {"tp", "ep", "pp"} -> initialises the mesh (``parallel.state.init_parallel``) and returns its sizes."""
    name = "distributed_training"

    def run(self, inputs: Dict[str, Any]) -> Dict[str, int]:
        from ..parallel.state import init_parallel
        st = init_parallel(tp=int(inputs.get("tp", 1)), ep=int(inputs.get("ep", 1)), pp=int(inputs.get("pp", 1)),
                           backend=inputs.get("backend"), device=inputs.get("device"))
        return {"world": st.world_size, "tp": st.tp_size, "ep": st.ep_size, "pp": st.pp_size, "dp": st.dp_size}


class PiscesLxAdvancedTrainingCoordinator:
    """One optimisation step composed from the operators above: schedule -> (accumulated) forward/backward under the
    precision policy -> gradient clipping -> optimizer step."""

    def __init__(self, model: nn.Module, optimizer: torch.optim.Optimizer, config: Optional[PiscesLxAdvancedTrainingConfig] = None):
        self.model, self.opt, self.cfg = model, optimizer, config or PiscesLxAdvancedTrainingConfig()
        self.amp = PiscesLxMixedPrecisionTrainingOperator(self.cfg)
        self.grad = PiscesLxGradientOptimizationOperator(self.cfg)
        self.reg = PiscesLxRegularizationOperator(self.cfg)
        self.sched = PiscesLxLearningRateSchedulerOperator(self.cfg)
        self.step_idx = 0

    def train_step(self, micro_batches: Sequence[Dict[str, torch.Tensor]], device_type: str = "cpu") -> Dict[str, float]:
        lr = self.sched.run({"optimizer": self.opt, "step": self.step_idx})
        self.opt.zero_grad(set_to_none=True)
        total = 0.0
        for mb in micro_batches:
            def fwd():
                logits = _logits(self.model(input_ids=mb["input_ids"]))
                return self.reg.run({"logits": logits[:, :-1], "labels": mb["labels"][:, 1:]})
            loss = self.amp.run({"fn": fwd, "device_type": device_type}) / len(micro_batches)
            loss.backward()
            total += float(loss.detach())
        g = self.grad.run({"parameters": list(self.model.parameters())})
        self.opt.step()
        self.step_idx += 1
        return {"loss": total, "lr": lr, **g}
