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


PiscesLxLRSchedulerOperator = YvLRScheduler
