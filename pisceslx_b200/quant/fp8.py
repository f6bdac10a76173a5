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


class YvFP8DelayedScaling:
    """Per-tensor delayed scaling (the recipe of the reference's fp8 operator, opss/train/fp8.py:381-399: amax history,
    scale = fp8_max / max(history) / 2^margin).  The scale used at step t comes from the amax values of earlier steps,
    so quantisation needs no extra pass over the tensor and no host synchronisation: the quantise kernel folds the
    current tensor's amax into a device scalar that ``update()`` rolls into the history."""

    def __init__(self, device: torch.device, history: int = 16, margin: int = 0, fmax: float = E4M3_MAX):
        self.history, self.margin, self.fmax = history, margin, fmax
        self.amax_hist = torch.zeros(history, dtype=torch.float32, device=device)
        self.amax_now = torch.zeros(1, dtype=torch.float32, device=device)
        self.scale = torch.ones(1, dtype=torch.float32, device=device)       # multiplies x before the cast
        self.scale_inv = torch.ones(1, dtype=torch.float32, device=device)   # dequantisation factor
        self.steps = 0

    def update(self) -> None:
        """Roll the amax recorded by the last quantisation into the history and derive the next scale (all on the
        device, no synchronisation)."""
        self.amax_hist = torch.roll(self.amax_hist, 1)
        self.amax_hist[0] = self.amax_now[0]
        self.amax_now.zero_()
        amax = self.amax_hist.max().clamp_min(1e-12)
        self.scale = (self.fmax / amax / (2.0 ** self.margin)).reshape(1)
        self.scale_inv = (1.0 / self.scale).reshape(1)
        self.steps += 1


def fp8_quantize_delayed(x: torch.Tensor, meta: YvFP8DelayedScaling) -> torch.Tensor:
    """bf16 CUDA tensor -> e4m3 with ``meta.scale``; records the tensor's amax in ``meta.amax_now``."""
    from ..ops import kernels
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    kernels().fp8_quantize(x.contiguous(), meta.scale, q, meta.amax_now)
    return q


class _FP8GemmLinearFn(torch.autograd.Function):
    """Forward on the fp8 tensor cores (tcgen05 ``kind::f8f6f4``, e4m3 x e4m3, fp32 accumulation, the product of the
    two dequantisation factors applied in the epilogue); backward in bf16 from the saved bf16 operands."""

    @staticmethod
    def forward(ctx, x, w, mx, mw):
        from ..ops import kernels, status_word
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        if mx.steps == 0:                      # first call: no history yet, take the scale from this tensor
            for t, m in ((x2, mx), (w, mw)):
                m.amax_now.copy_(t.detach().abs().max().float().reshape(1))
                m.update()
        xq, wq = fp8_quantize_delayed(x2, mx), fp8_quantize_delayed(w.contiguous(), mw)
        y = torch.empty(x2.shape[0], w.shape[0], dtype=torch.bfloat16, device=x.device)
        kernels().gemm_fp8(xq, wq, y, mx.scale_inv * mw.scale_inv, 0, status_word(x.device))
        mx.update()
        mw.update()
        ctx.save_for_backward(x2, w)
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        dx = F_.gemm(dy2, w, b_mn=True).view(ctx.shape)
        dw = F_.gemm(dy2, x2, a_mn=True, b_mn=True)
        return dx, dw, None, None


class YvFP8GemmLinear(nn.Module):
    """Linear layer whose forward runs the e4m3 GEMM kernel with delayed per-tensor scaling (CUDA, bf16 parameters;
    in/out features multiples of 16)."""

    def __init__(self, in_features: int, out_features: int, device=None, history: int = 16):
        super().__init__()
        device = torch.device(device or "cuda")
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=torch.bfloat16, device=device).normal_(std=0.02))
        self.meta_x = YvFP8DelayedScaling(device, history)
        self.meta_w = YvFP8DelayedScaling(device, history)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _FP8GemmLinearFn.apply(x.to(torch.bfloat16), self.weight, self.meta_x, self.meta_w)


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
