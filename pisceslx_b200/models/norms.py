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
        w = self.weight.float() if self.weight is not None else None
        b = self.bias.float() if self.bias is not None else None
        return torch.nn.functional.layer_norm(x.float(), self.normalized_shape, w, b, self.eps).to(x.dtype)


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


class YvUnifiedRotaryEmbedding(nn.Module):
    """One rotary embedding that folds every position-scaling mechanism into a single per-frequency multiplier
    (reference model/core/norms.py:466-664): base frequencies ``base^(-2i/d)``, optional mixed-radix factors
    (MrRoPE, ``1 + 0.1 * (i+1)/half`` in ``pro`` mode), dynamic-NTK growth of the base once the sequence passes
    ``original_max_position_embeddings`` (``base * ratio^(d/(d-2))``), a linear position divisor, and - with
    ``use_dynamic`` - learned scalars that temper the NTK factor.  Unlike the reference, which recomputes cos / sin
    on every call, tables are cached per (length, device) and rebuilt only when a longer sequence arrives or the
    learned scalars changed (training).  ``forward(x, seq_len)`` returns ``(cos, sin)`` of shape ``[seq_len, dim]`` in
    the rotate-half layout; ``apply(q, k, positions)`` rotates ``[T, heads, d]`` tensors."""

    def __init__(self, dim: int, max_position_embeddings: int = 10485760, base: float = 10000.0, scale: float = 32.0,
                 original_max_position_embeddings: int = 4096, device: Optional[torch.device] = None,
                 use_mr_rope: bool = False, mr_rope_mode: str = "pro", use_dynamic: bool = False,
                 enable_learned_scaling: bool = True, linear_scale: float = 1.0):
        super().__init__()
        self.dim, self.base, self.scale = dim, float(base), float(scale)
        self.max_position_embeddings = max_position_embeddings
        self.original_max_position_embeddings = original_max_position_embeddings
        self.use_mr_rope, self.mr_rope_mode = use_mr_rope, mr_rope_mode
        self.use_dynamic, self.linear_scale = use_dynamic, float(linear_scale)
        half = dim // 2
        radices = torch.ones(half)
        if use_mr_rope and mr_rope_mode == "pro":
            radices = 1.0 + 0.1 * torch.arange(1, half + 1, dtype=torch.float32) / half
        self.register_buffer("mr_radices", radices.to(device) if device is not None else radices, persistent=False)
        self.learned = use_dynamic and enable_learned_scaling
        if self.learned:
            self.learned_scale = nn.Parameter(torch.tensor(1.0))
            self.ntk_scale_factor = nn.Parameter(torch.tensor(1.0))
        self.max_seq_len_seen = 0
        self._cache: Dict[Tuple[int, str], Tuple[torch.Tensor, torch.Tensor]] = {}

    def ntk_factor(self, seq_len: int) -> float:
        """Multiplier of the rotary base for a sequence of ``seq_len`` tokens (1 inside the trained range)."""
        if seq_len <= self.original_max_position_embeddings:
            return 1.0
        ratio = min(seq_len / self.original_max_position_embeddings, self.scale)
        f = ratio ** (self.dim / max(self.dim - 2, 1))
        if self.learned:
            gate = float(torch.sigmoid(self.learned_scale.detach()) * 2.0 * torch.sigmoid(self.ntk_scale_factor.detach()) * 2.0
                         / (4.0 * torch.sigmoid(torch.tensor(1.0)) ** 2))
            f = 1.0 + (f - 1.0) * gate                       # gate == 1 at initialisation
        return f

    def inv_freq(self, seq_len: int, device: torch.device) -> torch.Tensor:
        base = self.base * self.ntk_factor(seq_len)
        i = torch.arange(0, self.dim, 2, device=device, dtype=torch.float32)
        return self.mr_radices.to(device) / (base ** (i / self.dim)) / self.linear_scale

    def forward(self, x: torch.Tensor, seq_len: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        seq_len = int(seq_len if seq_len is not None else x.shape[-2])
        self.max_seq_len_seen = max(self.max_seq_len_seen, seq_len)
        key = (seq_len, str(x.device))
        if key not in self._cache or (self.learned and self.training):
            t = torch.arange(seq_len, device=x.device, dtype=torch.float32)
            ang = torch.outer(t, self.inv_freq(seq_len, x.device))
            emb = torch.cat([ang, ang], dim=-1)
            self._cache = {key: (emb.cos(), emb.sin())}      # one live table: the longest / latest length
        cos, sin = self._cache[key]
        return cos.to(x.dtype), sin.to(x.dtype)

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        n = int(positions.max().item()) + 1
        cos, sin = self.forward(q, n)
        half = self.dim // 2
        return (ref.apply_rope(q, cos[:, :half].float(), sin[:, :half].float(), positions, self.dim),
                ref.apply_rope(k, cos[:, :half].float(), sin[:, :half].float(), positions, self.dim))


class YvDynamicYaRNRotaryEmbedding(YvUnifiedRotaryEmbedding):
    """YaRN with a context-dependent factor (reference model/core/norms.py:666-698): the unified embedding with
    the dynamic learned scalars switched on, the YaRN attention temperature ``0.1 * ln(s) + 1`` exposed as
    ``attention_scale(seq_len)``, and per-frequency blending between interpolated and extrapolated frequencies over
    the YaRN ramp (low frequencies are interpolated by ``s``, high frequencies are left alone)."""

    def __init__(self, dim: int, max_position_embeddings: int = 10485760, base: float = 10000.0, scale: float = 32.0,
                 original_max_position_embeddings: int = 4096, beta_fast: float = 32.0, beta_slow: float = 1.0,
                 device: Optional[torch.device] = None):
        super().__init__(dim, max_position_embeddings, base, scale, original_max_position_embeddings, device,
                         use_dynamic=True)
        self.beta_fast, self.beta_slow = beta_fast, beta_slow

    def context_scale(self, seq_len: int) -> float:
        return max(1.0, min(seq_len / self.original_max_position_embeddings, self.scale))

    def attention_scale(self, seq_len: int) -> float:
        s = self.context_scale(seq_len)
        return 0.1 * math.log(s) + 1.0 if s > 1 else 1.0

    def inv_freq(self, seq_len: int, device: torch.device) -> torch.Tensor:
        s = self.context_scale(seq_len)
        i = torch.arange(0, self.dim, 2, device=device, dtype=torch.float32)
        extrap = 1.0 / (self.base ** (i / self.dim))
        if s <= 1.0:
            return extrap * self.mr_radices.to(device)
        interp = extrap / s

        def corr(n_rot: float) -> float:                    # dimension whose wavelength makes n_rot turns in the trained range
            return self.dim * math.log(self.original_max_position_embeddings / (n_rot * 2 * math.pi)) / (2 * math.log(self.base))

        lo, hi = max(math.floor(corr(self.beta_fast)), 0), min(math.ceil(corr(self.beta_slow)), self.dim // 2 - 1)
        ramp = ((torch.arange(self.dim // 2, device=device, dtype=torch.float32) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
        return (interp * ramp + extrap * (1 - ramp)) * self.mr_radices.to(device)
