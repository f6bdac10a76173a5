"""Normalisation layers, FiLM modulation and rotary position embeddings.

Reference parity: ``YvRMSNorm`` (model/core/norms.py:178), ``YvLayerNorm``, ``YvFiLMModulation.apply``
(norms.py:135-175: ``h*(1+scale)+shift``, a dict without both keys raises ``ValueError``),
``YvRotaryEmbedding`` / ``YvUnifiedRotaryEmbedding`` (norms.py:317-664: plain, linear-scaled,
dynamic-NTK and YaRN tables; rotate-half layout; partial rotation of the first ``rot_dim`` dims).
On GPU the norm and the rotation run the kernels in ``ops/csrc/elementwise.cu``.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F_
from ..ops import reference as ref


class YvFiLMModulation:
    """Feature-wise linear modulation contract shared by every block."""

    @staticmethod
    def validate(film_params: Optional[Dict[str, torch.Tensor]]) -> None:
        if film_params is None:
            return
        if not isinstance(film_params, dict) or "scale" not in film_params or "shift" not in film_params:
            raise ValueError("film_params must be a dict with both 'scale' and 'shift'")

    @staticmethod
    def apply(h: torch.Tensor, film_params: Optional[Dict[str, torch.Tensor]]) -> torch.Tensor:
        """``None`` is the identity; otherwise ``h * (1 + scale) + shift`` with broadcasting over the sequence."""
        if film_params is None:
            return h
        YvFiLMModulation.validate(film_params)
        return F_.film(h, film_params["scale"], film_params["shift"])


class YvRMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                film_params: Optional[Dict[str, torch.Tensor]] = None):
        """Without ``residual`` returns the normalised tensor; with it returns ``(normed, x + residual)``."""
        fs = fb = None
        if film_params is not None:
            YvFiLMModulation.validate(film_params)
            fs, fb = film_params["scale"], film_params["shift"]
        y, res = F_.rms_norm(x, self.weight, self.eps, residual, fs, fb)
        return y if residual is None else (y, res)


class YvLayerNorm(nn.LayerNorm):
    """LayerNorm used by the vision / audio encoders (library op: not on the text hot path)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        return super().forward(x.float()).to(x.dtype)


class YvRotaryEmbedding(nn.Module):
    """cos/sin tables for rotate-half RoPE with optional linear / dynamic-NTK / YaRN scaling."""

    def __init__(self, rot_dim: int, max_position: int = 8192, theta: float = 1e4, scaling_type: str = "none",
                 scaling_factor: float = 1.0, original_max_position: Optional[int] = None):
        super().__init__()
        self.rot_dim, self.theta = rot_dim, theta
        self.scaling_type, self.scaling_factor = scaling_type, scaling_factor
        self.original_max = original_max_position or max_position
        self.max_position = 0
        self.register_buffer("cos", torch.empty(0), persistent=False)
        self.register_buffer("sin", torch.empty(0), persistent=False)
        self._build(max_position, torch.device("cpu"))

    def _build(self, max_position: int, device: torch.device) -> None:
        theta = self.theta
        if self.scaling_type == "yarn" and self.scaling_factor > 1:
            cos, sin = ref.yarn_tables(max_position, self.rot_dim, theta, self.scaling_factor, self.original_max,
                                       device=device)
        else:
            lin = 1.0
            if self.scaling_type == "linear":
                lin = self.scaling_factor
            elif self.scaling_type == "dynamic_ntk" and max_position > self.original_max:
                s = max_position / self.original_max
                theta = theta * (self.scaling_factor * s - (self.scaling_factor - 1)) ** (
                    self.rot_dim / max(self.rot_dim - 2, 1))
            cos, sin = ref.rope_tables(max_position, self.rot_dim, theta, lin, device=device)
        self.cos, self.sin = cos, sin
        self.max_position = max_position

    def tables(self, needed: int, device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
        if needed > self.max_position or self.cos.device != device:
            self._build(max(needed, self.max_position), device)
        return self.cos, self.sin

    def forward(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Rotate x [T, heads, d] (oracle path; the fused GPU path rotates inside ``rope_attention``)."""
        cos, sin = self.tables(int(positions.max().item()) + 1, x.device)
        return ref.apply_rope(x, cos, sin, positions, self.rot_dim)


class YvSpatioTemporalRoPE3D(nn.Module):
    """3-D (time, height, width) rotary embedding for video tokens (reference multimodal/vision.py:96-303):
    the head dimension is split into three sections rotated by the t / h / w coordinate of each token."""

    def __init__(self, head_dim: int, theta: float = 1e4, sections: Optional[Tuple[int, int, int]] = None):
        super().__init__()
        if sections is None:
            dt = (head_dim // 4) // 2 * 2
            dh = ((head_dim - dt) // 2) // 2 * 2
            sections = (dt, dh, head_dim - dt - dh)
        assert sum(sections) <= head_dim and all(s % 2 == 0 for s in sections)
        self.sections, self.theta, self.head_dim = tuple(sections), theta, head_dim

    @staticmethod
    def grid_positions(frames: int, height: int, width: int, device=None) -> torch.Tensor:
        t, h, w = torch.meshgrid(torch.arange(frames), torch.arange(height), torch.arange(width), indexing="ij")
        return torch.stack([t, h, w], -1).reshape(-1, 3).to(device=device, dtype=torch.int32)

    def forward(self, q: torch.Tensor, k: torch.Tensor, pos_thw: torch.Tensor):
        """q [T, hq, d], k [T, hk, d] -> rotated copies."""
        if q.is_cuda and q.dtype == torch.bfloat16:
            from ..ops import kernels
            q2, k2 = q.contiguous().clone(), k.contiguous().clone()
            kernels().rope3d(q2, k2, pos_thw.int().contiguous(), q.shape[1], k.shape[1], self.head_dim,
                             self.sections[0], self.sections[1], self.sections[2], self.theta, False)
            return q2, k2
        return (ref.apply_rope3d(q, pos_thw, self.sections, self.theta),
                ref.apply_rope3d(k, pos_thw, self.sections, self.theta))
