"""Learning-rate schedules with warm-up: cosine, linear, polynomial, inverse square root, step, exponential,
constant (reference opss/train/lr_scheduler.py: ``PiscesLxLRSchedulerOperator`` and the warm-up wrappers).
A schedule is a pure function of the step, so resuming only needs the step counter."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional


@dataclass
class YvLRSchedulerConfig:
    scheduler_type: str = "cosine"      # cosine | linear | polynomial | inverse_sqrt | step | exponential | constant
    base_lr: float = 1e-3
    warmup_steps: int = 0
    total_steps: int = 1000
    min_lr_ratio: float = 0.1
    power: float = 1.0                  # polynomial
    step_size: int = 1000               # step
    gamma: float = 0.1                  # step / exponential


def lr_at(cfg: YvLRSchedulerConfig, step: int) -> float:
    """Learning rate after ``step`` optimizer steps have been taken (step 0 = first update)."""
    base, lo = cfg.base_lr, cfg.base_lr * cfg.min_lr_ratio
    if cfg.warmup_steps > 0 and step < cfg.warmup_steps:
        return base * (step + 1) / cfg.warmup_steps
    t = step - cfg.warmup_steps
    span = max(cfg.total_steps - cfg.warmup_steps, 1)
    frac = min(max(t / span, 0.0), 1.0)
    kind = cfg.scheduler_type
    if kind == "cosine":
        return lo + 0.5 * (base - lo) * (1 + math.cos(math.pi * frac))
    if kind == "linear":
        return lo + (base - lo) * (1 - frac)
    if kind == "polynomial":
        return lo + (base - lo) * (1 - frac) ** cfg.power
    if kind == "inverse_sqrt":
        w = max(cfg.warmup_steps, 1)
        return max(lo, base * math.sqrt(w / max(step + 1, w)))
    if kind == "step":
        return max(lo, base * cfg.gamma ** (t // max(cfg.step_size, 1)))
    if kind == "exponential":
        return max(lo, base * cfg.gamma ** (t / span))
    return base


class YvLRScheduler:
    """Drives the ``lr`` of every param group, keeping each group's ratio to the base LR."""

    def __init__(self, optimizer, cfg: YvLRSchedulerConfig):
        self.optimizer, self.cfg = optimizer, cfg
        self.ratios: List[float] = [g["lr"] / cfg.base_lr if cfg.base_lr > 0 else 1.0 for g in optimizer.param_groups]
        self.last_step = 0
        self._set(0)

    def _set(self, step: int) -> None:
        lr = lr_at(self.cfg, step)
        for g, r in zip(self.optimizer.param_groups, self.ratios):
            g["lr"] = lr * r

    def step(self) -> float:
        self.last_step += 1
        self._set(self.last_step)
        return self.get_last_lr()[0]

    def get_last_lr(self) -> List[float]:
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self) -> Dict[str, Any]:
        return {"last_step": self.last_step, "ratios": list(self.ratios), "cfg": dict(self.cfg.__dict__)}

    def load_state_dict(self, sd: Dict[str, Any], reset_lr: bool = False) -> None:
        if reset_lr:
            self.last_step = 0
        else:
            self.last_step = int(sd.get("last_step", 0))
        self._set(self.last_step)



# ---------------------------------------------------------------------------------------------------------------------------
# The operator family (reference opss/train/lr_scheduler.py:80-560): scheduler types incl. cosine with restarts and the
# warm-up shapes, gradient-accumulation awareness, history, state, named subclasses and a factory.
# ---------------------------------------------------------------------------------------------------------------------------
from enum import Enum
from typing import Callable

from ..utils.opsc import PiscesLxOperatorInterface


class PiscesLxSchedulerType(str, Enum):
    LINEAR = "linear"
    COSINE = "cosine"
    COSINE_WITH_RESTARTS = "cosine_with_restarts"
    POLYNOMIAL = "polynomial"
    INVERSE_SQUARE = "inverse_square"
    STEP = "step"
    EXPONENTIAL = "exponential"
    WARMUP_DECAY = "warmup_decay"
    CONSTANT = "constant"
    WSD = "wsd"                        # warm-up, stable plateau, short decay at the end


@dataclass
class PiscesLxLRSchedulerConfig:
    type: str = "cosine"
    initial_lr: float = 1e-4           # what inverse-square and warm-up-decay start from after the warm-up
    min_lr: float = 1e-6
    max_lr: float = 1e-3
    warmup_steps: int = 1000
    warmup_ratio: Optional[float] = None
    warmup_type: str = "linear"        # linear | cubic | exponential
    warmup_start_ratio: float = 0.01   # the warm-up starts at this fraction of max_lr
    total_steps: Optional[int] = None
    decay_steps: Optional[int] = None
    decay_ratio: float = 0.1
    decay_gamma: float = 0.1
    power: float = 1.0
    cycle_first_step: int = 1000
    cycle_min_lr: float = 1e-6
    cycle_scaling_factor: float = 1.0  # each cycle is this many times as long as the one before
    cycle_peak_decay: float = 1.0      # each cycle peaks at this fraction of the previous peak
    stable_ratio: float = 0.8          # wsd: share of the post-warm-up steps spent on the plateau
    gradient_accumulation_steps: int = 1
    apply_at_step: int = 0
    last_step: int = -1

    def __post_init__(self) -> None:
        self.type = PiscesLxSchedulerType(getattr(self.type, "value", self.type)).value
        if self.warmup_ratio is not None and self.total_steps is not None:
            self.warmup_steps = int(self.warmup_ratio * self.total_steps)
        if self.warmup_type not in ("linear", "cubic", "exponential"):
            raise ValueError(f"unknown warmup_type {self.warmup_type!r}")
        if self.min_lr > self.max_lr:
            raise ValueError("min_lr must not exceed max_lr")


class PiscesLxLRSchedulerOperator(PiscesLxOperatorInterface):
    """The learning rate as a pure function of the optimizer step (``get_lr_at_step``), plus the stateful side: ``step()``
    advances by one MICRO step and moves the optimizer's groups once per ``gradient_accumulation_steps``, a history of
    the values set, and a state dictionary.  Param groups keep their ratio to the first group's rate.

    Cosine with restarts is computed in closed form from the step (cycle k has length first x scaling^k), so seeking to
    any step - a resume - gives the same value as stepping there; the reference advances mutable cycle counters inside
    the formula and therefore cannot be evaluated at an earlier step again (lr_scheduler.py:375-386)."""

    name = "lr_scheduler"

    def __init__(self, config: Optional[PiscesLxLRSchedulerConfig] = None, optimizer: Any = None):
        self.config = config or PiscesLxLRSchedulerConfig()
        self.optimizer = optimizer
        self.micro_step = 0
        self.current_step = max(self.config.last_step + 1, 0)
        self._history: List[float] = []
        self._ratios: List[float] = []
        if optimizer is not None:
            base = optimizer.param_groups[0]["lr"] or 1.0
            self._ratios = [g["lr"] / base for g in optimizer.param_groups]
            self._apply(self.current_step)

    # -- the function of the step ------------------------------------------------------------------------------------------------
    def _get_warmup_function(self) -> Callable[[float], float]:
        kind = self.config.warmup_type
        if kind == "cubic":
            return lambda x: x ** 3
        if kind == "exponential":
            return lambda x: (1 - math.exp(-4 * x)) / (1 - math.exp(-4))      # fast start, reaches 1 at x = 1
        return lambda x: x

    def _compute_warmup_lr(self, step: int) -> float:
        c = self.config
        start = c.max_lr * c.warmup_start_ratio
        return start + (c.max_lr - start) * self._get_warmup_function()(min(1.0, (step + 1) / c.warmup_steps))

    def _get_total_decay_steps(self) -> int:
        c = self.config
        if c.total_steps is not None:
            return max(1, c.total_steps - c.warmup_steps)
        return max(1, c.decay_steps or 10000)

    def _cycle_of(self, t: int) -> tuple:
        """(cycle index, position inside it, its length) of decay step t."""
        c = self.config
        first, f = max(c.cycle_first_step, 1), c.cycle_scaling_factor
        if abs(f - 1.0) < 1e-12:
            k = t // first
            return k, t - k * first, first
        # lengths first * f^k: the start of cycle k is first * (f^k - 1) / (f - 1)
        k = int(math.floor(math.log(1 + t * (f - 1) / first, f) + 1e-9))
        start = lambda kk: first * (f ** kk - 1) / (f - 1)
        while start(k + 1) <= t:
            k += 1
        while start(k) > t:
            k -= 1
        return k, t - start(k), first * f ** k

    def _compute_decay_lr(self, t: int) -> float:
        c = self.config
        T = self._get_total_decay_steps()
        p = min(1.0, t / T)
        kind = c.type
        if kind == "linear":
            return c.max_lr - (c.max_lr - c.min_lr) * p
        if kind == "cosine":
            return c.min_lr + (c.max_lr - c.min_lr) * 0.5 * (1 + math.cos(math.pi * p))
        if kind == "cosine_with_restarts":
            k, pos, length = self._cycle_of(t)
            peak = max(c.cycle_min_lr, c.max_lr * c.cycle_peak_decay ** k)
            return c.cycle_min_lr + (peak - c.cycle_min_lr) * 0.5 * (1 + math.cos(math.pi * pos / length))
        if kind == "polynomial":
            return c.min_lr + (c.max_lr - c.min_lr) * (1 - p) ** c.power
        if kind == "inverse_square":
            w = max(c.warmup_steps, 1)
            return max(c.min_lr, c.max_lr * math.sqrt(w / (w + t)))
        if kind == "step":
            return max(c.min_lr, c.max_lr * c.decay_ratio ** (t // max(c.decay_steps or 10000, 1)))
        if kind == "exponential":
            return max(c.min_lr, c.max_lr * math.exp(-c.decay_gamma * t / max(c.decay_steps or 10000, 1)))
        if kind == "warmup_decay":
            return max(c.min_lr, c.max_lr * (1 - p) ** c.power)
        if kind == "wsd":
            stable = int(T * c.stable_ratio)
            if t < stable:
                return c.max_lr
            q = min(1.0, (t - stable) / max(T - stable, 1))
            return c.min_lr + (c.max_lr - c.min_lr) * 0.5 * (1 + math.cos(math.pi * q))
        return c.max_lr

    def get_lr_at_step(self, step: int) -> float:
        c = self.config
        if step < c.apply_at_step:
            return c.max_lr * c.warmup_start_ratio if c.warmup_steps > 0 else c.max_lr
        s = step - c.apply_at_step
        if c.warmup_steps > 0 and s < c.warmup_steps:
            return self._compute_warmup_lr(s)
        return self._compute_decay_lr(s - c.warmup_steps)

    _compute_lr = get_lr_at_step

    # -- the stateful side --------------------------------------------------------------------------------------------------------
    def _apply(self, step: int) -> float:
        lr = self.get_lr_at_step(step)
        if self.optimizer is not None:
            for g, r in zip(self.optimizer.param_groups, self._ratios):
                g["lr"] = lr * r
        self._history.append(lr)
        return lr

    def step(self) -> float:
        """One micro step; the rate moves when an accumulation window completes."""
        self.micro_step += 1
        if self.micro_step % max(self.config.gradient_accumulation_steps, 1) == 0:
            self.current_step += 1
            return self._apply(self.current_step)
        return self._history[-1] if self._history else self.get_lr_at_step(self.current_step)

    def get_last_lr(self) -> List[float]:
        if self.optimizer is not None:
            return [g["lr"] for g in self.optimizer.param_groups]
        return [self._history[-1] if self._history else self.get_lr_at_step(self.current_step)]

    def get_lr_history(self) -> List[float]:
        return list(self._history)

    def reset(self) -> None:
        self.micro_step, self.current_step = 0, 0
        self._history.clear()
        if self.optimizer is not None:
            self._apply(0)

    def state_dict(self) -> Dict[str, Any]:
        return {"current_step": self.current_step, "micro_step": self.micro_step, "ratios": list(self._ratios),
                "config": dict(self.config.__dict__)}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.current_step, self.micro_step = int(sd.get("current_step", 0)), int(sd.get("micro_step", 0))
        if self.optimizer is not None:
            self._apply(self.current_step)

    # -- operator front -----------------------------------------------------------------------------------------------------------
    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return inputs.get("action", "step") in ("step", "get_lr", "history", "reset")

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        a = inputs.get("action", "step")
        if a == "step":
            return {"lr": self.step(), "step": self.current_step}
        if a == "get_lr":
            return {"lr": self.get_lr_at_step(int(inputs.get("step", self.current_step)))}
        if a == "reset":
            self.reset()
            return {"step": 0}
        return {"history": self.get_lr_history()}


class PiscesLxCosineWarmupScheduler(PiscesLxLRSchedulerOperator):
    def __init__(self, max_lr: float = 1e-3, min_lr: float = 1e-6, warmup_steps: int = 1000, total_steps: Optional[int] = None,
                 optimizer: Any = None, **kw: Any):
        super().__init__(PiscesLxLRSchedulerConfig(type="cosine", max_lr=max_lr, min_lr=min_lr, warmup_steps=warmup_steps,
                                                   total_steps=total_steps, **kw), optimizer)


class PiscesLxLinearWarmupScheduler(PiscesLxLRSchedulerOperator):
    def __init__(self, max_lr: float = 1e-3, min_lr: float = 1e-6, warmup_steps: int = 1000, total_steps: Optional[int] = None,
                 optimizer: Any = None, **kw: Any):
        super().__init__(PiscesLxLRSchedulerConfig(type="linear", max_lr=max_lr, min_lr=min_lr, warmup_steps=warmup_steps,
                                                   total_steps=total_steps, **kw), optimizer)


class PiscesLxInverseSquareRootScheduler(PiscesLxLRSchedulerOperator):
    def __init__(self, max_lr: float = 1e-3, min_lr: float = 1e-6, warmup_steps: int = 4000, optimizer: Any = None, **kw: Any):
        super().__init__(PiscesLxLRSchedulerConfig(type="inverse_square", max_lr=max_lr, min_lr=min_lr, warmup_steps=warmup_steps, **kw),
                         optimizer)


class PiscesLxLrScheduler:
    """Factory: ``create_scheduler("cosine", optimizer, max_lr=..., ...)``."""

    _NAMED = {"cosine": PiscesLxCosineWarmupScheduler, "linear": PiscesLxLinearWarmupScheduler,
              "inverse_square": PiscesLxInverseSquareRootScheduler, "inverse_sqrt": PiscesLxInverseSquareRootScheduler}

    @classmethod
    def create_scheduler(cls, scheduler_type: str = "cosine", optimizer: Any = None, **kw: Any) -> PiscesLxLRSchedulerOperator:
        t = getattr(scheduler_type, "value", scheduler_type)
        if t in cls._NAMED:
            return cls._NAMED[t](optimizer=optimizer, **kw)
        return PiscesLxLRSchedulerOperator(PiscesLxLRSchedulerConfig(type=t, **kw), optimizer)
