"""Seeding of every random generator a run uses (reference utils/seed.py: ``PiscesLxDeterminism``)."""
from __future__ import annotations

import random

import torch


class PiscesLxDeterminism:
    @staticmethod
    def seed_everything(seed: int, deterministic: bool = False) -> None:
        random.seed(seed)
        try:
            import numpy as np
            np.random.seed(seed % (2 ** 32))
        except Exception:
            pass
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)
        if deterministic:
            torch.use_deterministic_algorithms(True, warn_only=True)


def worker_seed(base_seed: int, rank: int, worker: int = 0) -> int:
    """Distinct, reproducible seed for data-loader worker ``worker`` of rank ``rank``."""
    return (base_seed * 1000003 + rank * 9176 + worker * 31) % (2 ** 31 - 1)
