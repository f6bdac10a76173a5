"""Numerical, shape and device guards plus the functional rotary front (reference model/utils/safety.py:29-133
``YvEPS`` / ``YvNumericalGuard`` / ``YvShapeGuard`` / ``YvDeviceGuard``, model/utils/device.py:42 ``YvDeviceResolver``,
model/utils/rope.py:268 ``YvRope``).  Cheap checks that fail with the tensor shapes in the message instead of a
kernel-side error; none of them is on a timed path."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple, Union

import torch

from ..ops import reference as ref


class YvEPS:
    """Smallest safe denominators per dtype (an fp32 epsilon underflows in half precision)."""
    FP32 = 1e-8
    BF16 = 1e-3
    FP16 = 1e-4
    FP8 = 1e-2


class YvNumericalGuard:
    @staticmethod
    def get_eps(dtype: torch.dtype) -> float:
        return {torch.float32: YvEPS.FP32, torch.float64: 1e-12, torch.bfloat16: YvEPS.BF16,
                torch.float16: YvEPS.FP16}.get(dtype, YvEPS.FP8 if "float8" in str(dtype) else YvEPS.FP32)

    @staticmethod
    def safe_div(num: torch.Tensor, den: torch.Tensor, eps: Optional[float] = None) -> torch.Tensor:
        """num / den with |den| kept away from zero (sign preserved)."""
        e = YvNumericalGuard.get_eps(den.dtype) if eps is None else eps
        return num / torch.where(den >= 0, den.clamp_min(e), den.clamp_max(-e))

    @staticmethod
    def safe_log(x: torch.Tensor, eps: Optional[float] = None) -> torch.Tensor:
        return torch.log(x.clamp_min(YvNumericalGuard.get_eps(x.dtype) if eps is None else eps))

    @staticmethod
    def safe_clamp(x: torch.Tensor, low: float, high: Union[float, torch.Tensor]) -> torch.Tensor:
        return torch.minimum(x.clamp_min(low), torch.as_tensor(high, dtype=x.dtype, device=x.device))

    @staticmethod
    def nan_to_num(x: torch.Tensor, nan: float = 0.0, posinf: Optional[float] = None, neginf: Optional[float] = None) -> torch.Tensor:
        return torch.nan_to_num(x, nan=nan, posinf=posinf, neginf=neginf)

    @staticmethod
    def straight_through_gate(scalar: torch.Tensor) -> torch.Tensor:
        """Forward value 1 or 0 (hard decision at 0.5), gradient of the soft scalar."""
        hard = (scalar > 0.5).to(scalar.dtype)
        return hard + (scalar - scalar.detach())          # the bracket is exactly zero: the value stays exactly 0 or 1


class YvShapeGuard:
    @staticmethod
    def check_matmul(a: torch.Tensor, b: torch.Tensor, msg: str = "") -> None:
        if a.shape[-1] != b.shape[-2 if b.dim() > 1 else 0]:
            raise ValueError(f"matmul shape mismatch {tuple(a.shape)} @ {tuple(b.shape)} {msg}".strip())

    @staticmethod
    def check_cat(tensors: Sequence[torch.Tensor], dim: int, msg: str = "") -> None:
        if not tensors:
            raise ValueError(f"cat of an empty list {msg}".strip())
        base = list(tensors[0].shape)
        d = dim % len(base)
        for t in tensors[1:]:
            s = list(t.shape)
            if len(s) != len(base) or any(x != y for i, (x, y) in enumerate(zip(s, base)) if i != d):
                raise ValueError(f"cat shape mismatch along dim {dim}: {[tuple(x.shape) for x in tensors]} {msg}".strip())

    @staticmethod
    def check_broadcast(a: torch.Tensor, b: torch.Tensor, msg: str = "") -> Tuple[int, ...]:
        try:
            return tuple(torch.broadcast_shapes(a.shape, b.shape))
        except RuntimeError:
            raise ValueError(f"shapes {tuple(a.shape)} and {tuple(b.shape)} do not broadcast {msg}".strip()) from None


class YvDeviceGuard:
    @staticmethod
    def align(*tensors: Optional[torch.Tensor], device: Optional[torch.device] = None,
              dtype: Optional[torch.dtype] = None) -> List[Optional[torch.Tensor]]:
        """Move every given tensor to the device / dtype of the first one (or to the ones named)."""
        first = next((t for t in tensors if t is not None), None)
        if first is None:
            return list(tensors)
        device, dtype = device or first.device, dtype or first.dtype
        return [None if t is None else t.to(device=device, dtype=dtype if t.is_floating_point() else None) for t in tensors]

    @staticmethod
    def assert_same_device(*tensors: Optional[torch.Tensor], msg: str = "") -> None:
        devs = {str(t.device) for t in tensors if t is not None}
        if len(devs) > 1:
            raise ValueError(f"tensors live on different devices {sorted(devs)} {msg}".strip())

    @staticmethod
    def assert_same_dtype(*tensors: Optional[torch.Tensor], msg: str = "") -> None:
        dts = {str(t.dtype) for t in tensors if t is not None}
        if len(dts) > 1:
            raise ValueError(f"tensors have different dtypes {sorted(dts)} {msg}".strip())


class YvDeviceResolver:
    """``auto`` / ``cuda`` / ``cuda:N`` / ``cpu`` -> a device that exists here, and the dtype the model runs in on it."""

    @staticmethod
    def resolve(spec: Optional[str] = "auto") -> torch.device:
        spec = (spec or "auto").lower()
        if spec == "auto":
            return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        dev = torch.device(spec)
        if dev.type == "cuda":
            if not torch.cuda.is_available():
                raise RuntimeError(f"device {spec!r} was requested but no CUDA device is visible")
            if dev.index is not None and dev.index >= torch.cuda.device_count():
                raise RuntimeError(f"device {spec!r} does not exist ({torch.cuda.device_count()} visible)")
        return dev

    @staticmethod
    def compute_dtype(device: torch.device) -> torch.dtype:
        return torch.bfloat16 if device.type == "cuda" else torch.float32


class YvRope:
    """Functional rotary helpers over the shared tables (same arithmetic as the kernels' oracle)."""

    @staticmethod
    def precompute_freqs_cis(dim: int, end: int, theta: float = 1e4, scale: float = 1.0,
                             device: Optional[torch.device] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        return ref.rope_tables(end, dim, theta, scale, device=device)

    @staticmethod
    def apply_rotary_emb(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                         positions: Optional[torch.Tensor] = None, rot_dim: Optional[int] = None):
        """q [T, hq, d], k [T, hk, d] rotated at ``positions`` (default 0..T-1)."""
        T, d = q.shape[0], q.shape[-1]
        pos = torch.arange(T, device=q.device) if positions is None else positions
        rd = rot_dim or d
        return ref.apply_rope(q, cos, sin, pos, rd), ref.apply_rope(k, cos, sin, pos, rd)
