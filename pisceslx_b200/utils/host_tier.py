"""Host / device capability tiers and numerical guards (reference model/host_tier.py ``YvHostTierResolver.enforce``
:106-185; model/utils/safety.py ``YvNumericalGuard``; utils/vram_controller.py; utils/dtype_safe.py)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch


@dataclass
class YvHostTier:
    name: str
    bf16: bool
    tcgen05: bool
    fp8: bool
    memory_gb: float


class YvHostTierResolver:
    """Classifies the device and rejects configurations it cannot run.  The sm_100a kernels of this framework need
    compute capability 10.x; everything else is the CPU tier (fp32 reference path)."""

    @staticmethod
    def resolve(device: Optional[torch.device] = None, props: Any = None) -> YvHostTier:
        if props is None:
            if device is None or device.type != "cuda" or not torch.cuda.is_available():
                return YvHostTier("cpu", False, False, False, 0.0)
            props = torch.cuda.get_device_properties(device)
        major = getattr(props, "major", 0)
        mem = getattr(props, "total_memory", 0) / 2 ** 30
        if major >= 10:
            return YvHostTier("blackwell", True, True, True, mem)
        if major >= 8:
            return YvHostTier("ampere_hopper", True, False, major >= 9, mem)
        return YvHostTier("legacy", False, False, False, mem)

    @classmethod
    def enforce(cls, cfg: Any, device: Optional[torch.device] = None, props: Any = None) -> YvHostTier:
        tier = cls.resolve(device, props)
        dtype = str(getattr(cfg, "torch_dtype", getattr(cfg, "dtype", "bfloat16")))
        if "bf" in dtype and not tier.bf16 and tier.name != "cpu":
            raise RuntimeError(f"bf16 was requested but the {tier.name} tier has no bf16 tensor cores")
        if tier.name not in ("cpu", "blackwell"):
            raise RuntimeError(f"the CUDA kernels of this framework are built for sm_100a only; found tier {tier.name}")
        return tier


class YvNumericalGuard:
    @staticmethod
    def straight_through_gate(s: torch.Tensor) -> torch.Tensor:
        """Value 1, gradient of sigmoid(s) / sigmoid(s): lets a gate open without changing the forward value."""
        g = torch.sigmoid(s)
        return g / g.detach()

    @staticmethod
    def safe_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        x = x.float()
        x = x - x.amax(dim, keepdim=True).clamp_min(-1e30)
        return torch.nan_to_num(torch.softmax(x, dim), nan=0.0)

    @staticmethod
    def clamp_finite(x: torch.Tensor, limit: float = 6e4) -> torch.Tensor:
        return torch.nan_to_num(x, nan=0.0, posinf=limit, neginf=-limit).clamp(-limit, limit)

    @staticmethod
    def check(name: str, x: torch.Tensor) -> None:
        if not torch.isfinite(x).all():
            raise FloatingPointError(f"non-finite values in {name}")


class PiscesLxVramController:
    """Keeps a running estimate of free device memory and proposes the micro-batch size that fits."""

    def __init__(self, device: Optional[torch.device] = None, reserve_gb: float = 4.0, reader=None):
        self.device, self.reserve = device, reserve_gb * 2 ** 30
        self.reader = reader or (lambda: torch.cuda.mem_get_info(self.device))

    def free_bytes(self) -> int:
        free, _total = self.reader()
        return max(0, int(free - self.reserve))

    def fit_micro_batch(self, bytes_per_sample: int, max_micro: int) -> int:
        return max(1, min(max_micro, self.free_bytes() // max(bytes_per_sample, 1)))
