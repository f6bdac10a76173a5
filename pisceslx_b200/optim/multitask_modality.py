"""Two training aids for models with several objectives or several modalities (reference
opss/train/multitask_uncertainty.py:114-791, opss/train/modality_scheduler.py:111-765).

**Task-uncertainty weighting.**  L = sum_i ( L_i / (2 sigma_i^2) + log sigma_i ) with one learned log sigma per task
(classification-type tasks use 1 / sigma^2 without the half, following the derivation for a softmax likelihood).  The
operator owns the parameters (an ``nn.Module``: add ``operator.parameters()`` to the optimizer, with their own
learning-rate multiple), supports a warm-up during which the tasks are simply averaged, clamping, freezing, initial
values from observed loss scales, and reports the weights.  The combined loss uses the SUM of the weighted losses - the
regulariser sums over tasks, so a mean over tasks on the data term (the reference's default, multitask_uncertainty.py:
466-469) would make the balance depend on the number of tasks.

**Per-modality learning-rate schedules.**  Parameters are assigned to a modality by name (vision, audio, fusion, text,
other); each modality follows its own cosine schedule with warm restarts (period T_0 growing by T_mult, floor eta_min)
as a multiple of its group's base rate.  The schedule is a closed-form function of the step, groups are created once by
``setup`` (one optimizer group per modality that has parameters), and a joint linear warm-up can precede the cycles.
The reference builds one ``CosineAnnealingWarmRestarts`` per modality on the WHOLE optimizer, so each scheduler
overwrites every group's rate and only the last one created takes effect (modality_scheduler.py:449-455, 626-637)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..utils.opsc import PiscesLxOperatorInterface


# ---------------------------------------------------------------------------------------------------------------- multi-task
class PiscesLxTaskType(str, Enum):
    REGRESSION = "regression"
    CLASSIFICATION = "classification"
    RANKING = "ranking"
    GENERATION = "generation"
    MULTIMODAL = "multimodal"


@dataclass
class PiscesLxMultiTaskConfig:
    num_tasks: int = 1
    initial_uncertainty: float = 1.0
    learnable_uncertainty: bool = True
    uncertainty_lr: float = 1.0                 # multiple of the model's learning rate for the sigma parameters
    clamp_uncertainty: bool = False
    uncertainty_min: float = 0.01
    uncertainty_max: float = 10.0
    separate_uncertainty: bool = True           # one sigma per task (False: one shared sigma)
    uncertainty_init_strategy: str = "uniform"  # "uniform" | "empirical" (sigma_i^2 = first observed L_i)
    warmup_steps: int = 0
    task_names: List[str] = field(default_factory=list)
    task_types: List[Any] = field(default_factory=list)

    def __post_init__(self) -> None:
        if self.num_tasks < 1:
            raise ValueError("num_tasks must be at least 1")
        if len(self.task_names) != self.num_tasks:
            self.task_names = [f"task_{i}" for i in range(self.num_tasks)]
        if len(self.task_types) != self.num_tasks:
            self.task_types = [PiscesLxTaskType.REGRESSION] * self.num_tasks
        self.task_types = [PiscesLxTaskType(getattr(t, "value", t)) for t in self.task_types]
        if self.uncertainty_init_strategy not in ("uniform", "empirical"):
            raise ValueError(f"unknown uncertainty_init_strategy {self.uncertainty_init_strategy!r}")


class PiscesLxMultiTaskOperator(nn.Module, PiscesLxOperatorInterface):
    name = "multitask_uncertainty"

    def __init__(self, config: Optional[PiscesLxMultiTaskConfig] = None):
        nn.Module.__init__(self)
        self.config = c = config or PiscesLxMultiTaskConfig()
        n = c.num_tasks if c.separate_uncertainty else 1
        self.log_uncertainty = nn.Parameter(torch.full((n,), math.log(c.initial_uncertainty)), requires_grad=c.learnable_uncertainty)
        halves = [0.5 if t in (PiscesLxTaskType.REGRESSION, PiscesLxTaskType.RANKING) else 1.0 for t in c.task_types]
        self.register_buffer("data_coefficient", torch.tensor(halves))
        self.steps = 0
        self._initialised = c.uncertainty_init_strategy == "uniform"
        self._last: Dict[str, torch.Tensor] = {}

    def _sigma_log(self) -> torch.Tensor:
        c = self.config
        s = self.log_uncertainty if c.separate_uncertainty else self.log_uncertainty.expand(c.num_tasks)
        if c.clamp_uncertainty:
            s = s.clamp(math.log(c.uncertainty_min), math.log(c.uncertainty_max))
        return s

    def _compute_uncertainty_weighted_loss(self, task_losses: Sequence[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(total, weighted data terms [n], regulariser)."""
        L = torch.stack([l.float().reshape(()) for l in task_losses])
        s = self._sigma_log().float()
        weighted = self.data_coefficient.to(L.device) * L * torch.exp(-2.0 * s)
        reg = s.sum()
        return weighted.sum() + reg, weighted, reg

    def compute_loss(self, task_losses: Sequence[torch.Tensor]) -> torch.Tensor:
        c = self.config
        if len(task_losses) != c.num_tasks:
            raise ValueError(f"expected {c.num_tasks} task losses, got {len(task_losses)}")
        self.steps += 1
        if not self._initialised:
            with torch.no_grad():
                first = torch.stack([l.detach().float().reshape(()) for l in task_losses]).clamp_min(1e-8)
                init = 0.5 * torch.log(first)                               # sigma^2 = L makes every weighted term 1/2 or 1
                self.log_uncertainty.copy_(init if c.separate_uncertainty else init.mean().reshape(1))
            self._initialised = True
        if self.steps <= c.warmup_steps:
            total = torch.stack([l.float().reshape(()) for l in task_losses]).mean()
            self._last = {"total": total.detach(), "weighted": torch.stack([l.detach().float().reshape(()) for l in task_losses]) / c.num_tasks,
                          "regulariser": total.new_zeros(())}
            return total
        total, weighted, reg = self._compute_uncertainty_weighted_loss(task_losses)
        self._last = {"total": total.detach(), "weighted": weighted.detach(), "regulariser": reg.detach()}
        return total

    forward = compute_loss

    def get_uncertainties(self) -> List[float]:
        return torch.exp(self._sigma_log().detach()).tolist()

    _get_uncertainties = get_uncertainties

    def get_task_weights(self) -> Dict[str, float]:
        w = (self.data_coefficient.cpu() * torch.exp(-2.0 * self._sigma_log().detach().cpu())).tolist()
        return dict(zip(self.config.task_names, w))

    def get_uncertainty_parameters(self) -> nn.Parameter:
        return self.log_uncertainty

    def param_group(self, model_lr: float) -> Dict[str, Any]:
        """The optimizer group of the sigma parameters: no weight decay, ``uncertainty_lr`` x the model's rate."""
        return {"params": [self.log_uncertainty], "lr": model_lr * self.config.uncertainty_lr, "weight_decay": 0.0}

    def freeze_uncertainty(self) -> None:
        self.log_uncertainty.requires_grad_(False)

    def unfreeze_uncertainty(self) -> None:
        self.log_uncertainty.requires_grad_(True)

    def get_statistics(self) -> Dict[str, Any]:
        return {"steps": self.steps, "uncertainties": dict(zip(self.config.task_names, self.get_uncertainties())),
                "weights": self.get_task_weights(), "last_total": float(self._last["total"]) if self._last else None,
                "in_warmup": self.steps <= self.config.warmup_steps}

    def reset(self) -> None:
        with torch.no_grad():
            self.log_uncertainty.fill_(math.log(self.config.initial_uncertainty))
        self.steps, self._last = 0, {}
        self._initialised = self.config.uncertainty_init_strategy == "uniform"

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs.get("task_losses"), (list, tuple)) and len(inputs["task_losses"]) == self.config.num_tasks

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        total = self.compute_loss(inputs["task_losses"])
        return {"loss": total, "weighted_losses": self._last["weighted"], "uncertainties": self.get_uncertainties()}


class PiscesLxMultiTaskFacade:
    def __init__(self, num_tasks: int = 2, task_names: Optional[List[str]] = None, **kw: Any):
        self.operator = PiscesLxMultiTaskOperator(PiscesLxMultiTaskConfig(num_tasks=num_tasks, task_names=task_names or [], **kw))

    def compute_loss(self, task_losses: Sequence[torch.Tensor]) -> torch.Tensor:
        return self.operator.compute_loss(task_losses)

    def get_uncertainties(self) -> List[float]:
        return self.operator.get_uncertainties()

    def parameters(self) -> Iterable[nn.Parameter]:
        return self.operator.parameters()


class PiscesLxTaskUncertaintyWeighting:
    """Stateless-looking helper: ``compute(task_losses)`` creates the operator on first use (sized by the number of
    losses) and returns the combined loss."""

    def __init__(self, config: Optional[PiscesLxMultiTaskConfig] = None):
        self.config, self.operator = config, None

    def compute(self, task_losses: Sequence[torch.Tensor], model: Optional[nn.Module] = None) -> torch.Tensor:
        if self.operator is None:
            c = self.config or PiscesLxMultiTaskConfig(num_tasks=len(task_losses))
            self.operator = PiscesLxMultiTaskOperator(c).to(task_losses[0].device)
        return self.operator.compute_loss(task_losses)


# ---------------------------------------------------------------------------------------------------------------- modalities
class PiscesLxModalityType(str, Enum):
    VISION = "vision"
    AUDIO = "audio"
    FUSION = "fusion"
    TEXT = "text"
    OTHER = "other"


_PATTERNS = ((PiscesLxModalityType.FUSION, ("fusion", "multimodal", "cross_attn", "cross_modal", "modal_fusion")),
             (PiscesLxModalityType.VISION, ("vision", "visual", "image", "vit", "video", "patch_embed", "siglip")),
             (PiscesLxModalityType.AUDIO, ("audio", "speech", "wav2vec", "whisper", "hubert", "mel")),
             (PiscesLxModalityType.TEXT, ("text", "language", "lm_head", "embed", "layers.", "decoder", "encoder")))


@dataclass
class PiscesLxModalitySchedulerConfig:
    base_lr: float = 1.0                         # multiple applied to every group's own rate
    vision_t0: int = 10
    vision_t_mult: float = 2.0
    vision_eta_min: float = 1e-7
    audio_t0: int = 15
    audio_t_mult: float = 2.0
    audio_eta_min: float = 5e-8
    fusion_t0: int = 5
    fusion_t_mult: float = 1.0
    fusion_eta_min: float = 2e-7
    text_t0: int = 8
    text_t_mult: float = 1.0
    text_eta_min: float = 1e-7
    other_t0: int = 8
    other_t_mult: float = 1.0
    other_eta_min: float = 1e-7
    warmup_steps: int = 0
    warmup_lr: float = 0.0                       # the joint warm-up starts from this fraction of a group's rate
    lr_multipliers: Dict[str, float] = field(default_factory=dict)      # e.g. {"vision": 0.1}: a slower vision tower

    def cycle(self, modality: PiscesLxModalityType) -> Tuple[int, float, float]:
        m = modality.value
        return int(getattr(self, f"{m}_t0")), float(getattr(self, f"{m}_t_mult")), float(getattr(self, f"{m}_eta_min"))


class PiscesLxModalitySchedulerOperator(PiscesLxOperatorInterface):
    name = "modality_scheduler"

    def __init__(self, config: Optional[PiscesLxModalitySchedulerConfig] = None):
        self.config = config or PiscesLxModalitySchedulerConfig()
        self.optimizer: Optional[torch.optim.Optimizer] = None
        self._groups: List[Tuple[PiscesLxModalityType, float]] = []           # per optimizer group: modality, base rate
        self.last_step = 0

    @staticmethod
    def _detect_modality(param_name: str) -> PiscesLxModalityType:
        n = param_name.lower()
        for modality, pats in _PATTERNS:
            if any(p in n for p in pats):
                return modality
        return PiscesLxModalityType.OTHER

    def _organize_parameters_by_modality(self, model: nn.Module) -> Dict[PiscesLxModalityType, List[nn.Parameter]]:
        out: Dict[PiscesLxModalityType, List[nn.Parameter]] = {m: [] for m in PiscesLxModalityType}
        for name, p in model.named_parameters():
            if p.requires_grad:
                out[self._detect_modality(name)].append(p)
        return out

    def build_param_groups(self, model: nn.Module, lr: float, **group_kw: Any) -> List[Dict[str, Any]]:
        """One optimizer group per modality that has parameters, tagged with ``modality`` and its rate."""
        groups = []
        for m, ps in self._organize_parameters_by_modality(model).items():
            if ps:
                groups.append({"params": ps, "lr": lr * self.config.lr_multipliers.get(m.value, 1.0), "modality": m.value, **group_kw})
        return groups

    def setup(self, optimizer: torch.optim.Optimizer, model: Optional[nn.Module] = None) -> Dict[str, int]:
        """Attach to an optimizer whose groups carry a ``modality`` tag (``build_param_groups``); untagged groups are
        classified by the majority modality of their parameters when a model is given, otherwise they are ``other``."""
        self.optimizer = optimizer
        names = {id(p): n for n, p in model.named_parameters()} if model is not None else {}
        self._groups = []
        for g in optimizer.param_groups:
            tag = g.get("modality")
            if tag is None:
                votes: Dict[PiscesLxModalityType, int] = {}
                for p in g["params"]:
                    m = self._detect_modality(names.get(id(p), ""))
                    votes[m] = votes.get(m, 0) + p.numel()
                tag = max(votes, key=votes.get).value if votes else "other"
                g["modality"] = tag
            self._groups.append((PiscesLxModalityType(tag), float(g["lr"])))
        self._apply(self.last_step)
        counts: Dict[str, int] = {}
        for m, _ in self._groups:
            counts[m.value] = counts.get(m.value, 0) + 1
        return counts

    @staticmethod
    def _cosine_restart(t: int, t0: int, t_mult: float) -> float:
        """Position in [0, 1) inside the current cycle of step t."""
        t0 = max(t0, 1)
        if abs(t_mult - 1.0) < 1e-12:
            return (t % t0) / t0
        k = int(math.floor(math.log(1 + t * (t_mult - 1) / t0, t_mult) + 1e-9))
        start = lambda kk: t0 * (t_mult ** kk - 1) / (t_mult - 1)
        while start(k + 1) <= t:
            k += 1
        while start(k) > t:
            k -= 1
        return (t - start(k)) / (t0 * t_mult ** k)

    def factor_at(self, modality: PiscesLxModalityType, step: int, base: float = 1.0) -> float:
        """The learning rate of a group of base rate ``base`` at ``step``."""
        c = self.config
        peak = base * c.base_lr
        if c.warmup_steps > 0 and step < c.warmup_steps:
            lo = peak * c.warmup_lr
            return lo + (peak - lo) * (step + 1) / c.warmup_steps
        t0, mult, eta = c.cycle(modality)
        pos = self._cosine_restart(step - c.warmup_steps, t0, mult)
        return eta + (peak - eta) * 0.5 * (1 + math.cos(math.pi * pos))

    def _apply(self, step: int) -> None:
        if self.optimizer is None:
            return
        for g, (m, base) in zip(self.optimizer.param_groups, self._groups):
            g["lr"] = self.factor_at(m, step, base)

    def step(self, epoch: Optional[int] = None) -> None:
        self.last_step = self.last_step + 1 if epoch is None else int(epoch)
        self._apply(self.last_step)

    def get_lr(self) -> Dict[str, float]:
        out: Dict[str, float] = {}
        if self.optimizer is not None:
            for g, (m, _) in zip(self.optimizer.param_groups, self._groups):
                out.setdefault(m.value, g["lr"])
        return out

    def state_dict(self) -> Dict[str, Any]:
        return {"last_step": self.last_step, "groups": [(m.value, b) for m, b in self._groups]}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.last_step = int(sd.get("last_step", 0))
        if sd.get("groups") and len(sd["groups"]) == len(self._groups):
            self._groups = [(PiscesLxModalityType(m), float(b)) for m, b in sd["groups"]]
        self._apply(self.last_step)

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return inputs.get("action", "step") in ("setup", "step", "get_lr")

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        a = inputs.get("action", "step")
        if a == "setup":
            return {"groups": self.setup(inputs["optimizer"], inputs.get("model"))}
        if a == "step":
            self.step(inputs.get("epoch"))
        return {"lr": self.get_lr(), "step": self.last_step}


class PiscesLxModalitySchedulerFacade:
    """``f = PiscesLxModalitySchedulerFacade(vision_t0=10, ...)``; ``opt = AdamW(f.param_groups(model, lr))``;
    ``f.setup(opt)``; then ``f.step()`` once per epoch or step."""

    def __init__(self, config: Optional[PiscesLxModalitySchedulerConfig] = None, **overrides: Any):
        self.operator = PiscesLxModalitySchedulerOperator(config or PiscesLxModalitySchedulerConfig(**overrides))

    def param_groups(self, model: nn.Module, lr: float, **kw: Any) -> List[Dict[str, Any]]:
        return self.operator.build_param_groups(model, lr, **kw)

    def setup(self, optimizer: torch.optim.Optimizer, model: Optional[nn.Module] = None) -> Dict[str, int]:
        return self.operator.setup(optimizer, model)

    def step(self, epoch: Optional[int] = None) -> None:
        self.operator.step(epoch)

    def get_lr(self) -> Dict[str, float]:
        return self.operator.get_lr()
