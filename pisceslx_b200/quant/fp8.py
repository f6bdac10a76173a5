"""Block-scaled fp8."""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F_

E4M3_MAX = 448.0
E5M2_MAX = 57344.0


def _fp8_dtype(fmt: str):
    return torch.float8_e4m3fn if fmt == "e4m3" else torch.float8_e5m2


def quantize_fp8_blockwise(x: torch.Tensor, block: Tuple[int, int] = (1, 128), fmt: str = "e4m3",
                           pow2_scales: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [R, C] -> (q fp8 [R, C], scales fp32 [ceil(R/br), ceil(C/bc)]) with ``x ~= q * scale`` per block.
    ``block`` = (1, 128) for activations (one scale per row per 128 columns), (128, 128) for weights."""
    R, C = x.shape
    br, bc = block
    Rp, Cp = (R + br - 1) // br * br, (C + bc - 1) // bc * bc
    xp = torch.zeros(Rp, Cp, dtype=torch.float32, device=x.device)
    xp[:R, :C] = x.float()
    blocks = xp.view(Rp // br, br, Cp // bc, bc)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    fmax = E4M3_MAX if fmt == "e4m3" else E5M2_MAX
    scale = amax / fmax
    if pow2_scales:                                           # ue8m0-style: scale is a power of two
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = (blocks / scale[:, None, :, None]).clamp(-fmax, fmax).to(_fp8_dtype(fmt))
    return q.view(Rp, Cp)[:R, :C].contiguous(), scale


def dequantize_fp8_blockwise(q: torch.Tensor, scale: torch.Tensor, block: Tuple[int, int] = (1, 128)) -> torch.Tensor:
    R, C = q.shape
    br, bc = block
    s = scale.repeat_interleave(br, 0)[:R].repeat_interleave(bc, 1)[:, :C]
    return q.float() * s


def fp8_gemm_reference(a_q, a_s, b_q, b_s) -> torch.Tensor:
    """y = (a_q * a_s) @ (b_q * b_s).T in fp32: the oracle of every fp8 matrix product."""
    return dequantize_fp8_blockwise(a_q, a_s, (1, 128)) @ dequantize_fp8_blockwise(b_q, b_s, (128, 128)).t()


class _FP8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, fmt_bwd):
        x2 = x.reshape(-1, x.shape[-1])
        xq, xs = quantize_fp8_blockwise(x2, (1, 128), "e4m3")
        wq, ws = quantize_fp8_blockwise(w, (128, 128), "e4m3")
        xd = dequantize_fp8_blockwise(xq, xs, (1, 128)).to(x.dtype)
        wd = dequantize_fp8_blockwise(wq, ws, (128, 128)).to(w.dtype)
        ctx.save_for_backward(xd, wd)
        ctx.fmt_bwd, ctx.shape = fmt_bwd, x.shape
        return F_.linear(xd, wd).view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        xd, wd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        gq, gs = quantize_fp8_blockwise(dy2, (1, 128), ctx.fmt_bwd)          # gradients in E5M2 (wider range)
        gd = dequantize_fp8_blockwise(gq, gs, (1, 128)).to(dy.dtype)
        dx = F_.linear(gd, wd.t().contiguous()).view(ctx.shape)
        dw = F_.linear(gd.t().contiguous(), xd.t().contiguous())
        return dx, dw.to(wd.dtype), None


class YvFP8Linear(nn.Module):
    """Linear layer whose forward operands are E4M3 with 1x128 / 128x128 block scales and whose backward
    gradients are E5M2 with 1x128 block scales; master weights stay in the parameter dtype."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype).normal_(std=0.02))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype)) if bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = _FP8LinearFn.apply(x, self.weight, "e5m2")
        return y if self.bias is None else y + self.bias


class PiscesLxFP8QuantizationEngine:
    """PTQ entry for fp8 weights: per-tensor, per-channel or block scales; delayed scaling keeps an amax history
    (reference opss/quantize/engine.py:808-1103)."""

    def __init__(self, fmt: str = "e4m3", granularity: str = "block", history: int = 16):
        self.fmt, self.granularity, self.history = fmt, granularity, history
        self.amax_history = {}

    def quantize_weight(self, name: str, w: torch.Tensor):
        if self.granularity == "block":
            return quantize_fp8_blockwise(w, (128, 128), self.fmt)
        fmax = E4M3_MAX if self.fmt == "e4m3" else E5M2_MAX
        if self.granularity == "channel":
            amax = w.float().abs().amax(1, keepdim=True).clamp_min(1e-12)
        else:
            hist = self.amax_history.setdefault(name, [])
            hist.append(float(w.float().abs().max()))
            del hist[:-self.history]
            amax = torch.tensor(max(hist), device=w.device).clamp_min(1e-12)
        scale = amax / fmax
        return (w.float() / scale).clamp(-fmax, fmax).to(_fp8_dtype(self.fmt)), scale
