"""Optimizers and schedules: Muon/AdamW hybrid, fused AdamW, Ink (quantised-moment) optimizer, LR schedules."""
from __future__ import annotations

from typing import Any, Optional

import torch

from .adamw import PiscesLxFusedAdamW, YvFusedAdamW
from .lr import PiscesLxLRSchedulerOperator, YvLRScheduler, YvLRSchedulerConfig, lr_at
from .muon import YvMuon, newton_schulz_batched
from .galore import PiscesLxGaLoreConfig, PiscesLxGaLoreOperator, PiscesLxGaLoreOptimizerAdapter
from .root import PiscesLxROOTConfig, PiscesLxROOTOperator, PiscesLxROOTOptimizer, PiscesLxROOTScheduler

PiscesLxMuon = YvMuon


def build_optimizer(model: torch.nn.Module, name: str = "muon", lr: float = 2e-4, weight_decay: float = 0.1,
                    state_dtype: Optional[torch.dtype] = None, cfg: Any = None, **kw: Any) -> torch.optim.Optimizer:
    """``name``: muon | adamw | fused_adamw | ink | root | sgd  (reference trainer choices, tools/train/core.py:1656-1791)."""
    name = name.lower()
    if name == "muon":
        return YvMuon(model.named_parameters(), lr=lr, weight_decay=weight_decay, state_dtype=state_dtype,
                      cfg=cfg if cfg is not None else getattr(model, "cfg", None), **kw)
    decay = [p for n, p in model.named_parameters() if p.requires_grad and p.dim() >= 2]
    no_decay = [p for n, p in model.named_parameters() if p.requires_grad and p.dim() < 2]
    groups = [dict(params=decay, weight_decay=weight_decay), dict(params=no_decay, weight_decay=0.0)]
    groups = [g for g in groups if g["params"]]
    if name in ("adamw", "fused_adamw"):
        return YvFusedAdamW(groups, lr=lr, state_dtype=state_dtype, **kw)
    if name == "ink":
        from .ink import YvInkOptimizer
        return YvInkOptimizer(groups, lr=lr, **kw)
    if name == "root":
        return PiscesLxROOTOptimizer(groups, lr=lr, **kw)
    if name == "sgd":
        return torch.optim.SGD(groups, lr=lr, momentum=kw.get("momentum", 0.9))
    raise ValueError(f"unknown optimizer {name!r}")
