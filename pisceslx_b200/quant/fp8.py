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


# ------------------------------------------------------------------------------------------------------------------
# MX block scaling: e4m3 elements, one power-of-two (e8m0) scale per 32 elements of the reduction dimension.  The
# tensor cores apply the scales themselves (tcgen05 ``kind::mxf8f6f4.block_scale``), so the GEMM needs no fp32
# rescaling pass and no amax history.
# ------------------------------------------------------------------------------------------------------------------
MX_BLOCK = 32


def quantize_mx_reference(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [R, K] (K % 32 == 0) -> (q e4m3 [R, K], exponent bytes uint8 [R, K / 32]); the block's scale
    ``2 ** (byte - 127)`` is the smallest power of two that brings the block's largest magnitude to at most 448
    (byte 127 for an all-zero block), so nothing saturates.  Plain PyTorch on any device: the oracle of the quantise
    kernel."""
    R, K = x.shape
    b = x.float().view(R, K // MX_BLOCK, MX_BLOCK)
    amax = b.abs().amax(-1)
    mant, ex = torch.frexp(amax)                            # amax = mant * 2^ex, 0.5 <= mant < 1; 448 = 0.875 * 2^9
    e = (ex - 9 + (mant > 0.875).to(ex.dtype)).float()
    e = torch.where(amax > 0, e, torch.zeros_like(e)).clamp(-127, 126)
    q = (b * torch.exp2(-e)[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(R, K), (e + 127).to(torch.uint8)


def dequantize_mx(q: torch.Tensor, exp_bytes: torch.Tensor) -> torch.Tensor:
    """fp32 values of an MX tensor (q [R, K], exponent bytes [R, K / 32])."""
    R, K = q.shape
    s = torch.exp2(exp_bytes.float() - 127.0)
    return (q.float().view(R, K // MX_BLOCK, MX_BLOCK) * s[..., None]).view(R, K)


def mx_scales_to_chunks(exp_bytes: torch.Tensor) -> torch.Tensor:
    """[R, K / 32] exponent bytes -> the layout the GEMM kernel copies into tensor memory:
    ``[ceil(R / 128), K / 128, 512]``, where byte ``(r % 32) * 16 + (r // 32) * 4 + j`` of a chunk holds row ``r`` of
    the 128-row tile and 32-element block ``j`` of the 128-element K chunk (missing rows get 127 = 1.0)."""
    R, KB = exp_bytes.shape
    assert KB % 4 == 0, "K must be a multiple of 128"
    tiles = (R + 127) // 128
    full = torch.full((tiles * 128, KB), 127, dtype=torch.uint8, device=exp_bytes.device)
    full[:R] = exp_bytes
    v = full.view(tiles, 4, 32, KB // 4, 4)                 # tile, r // 32, r % 32, chunk, j
    return v.permute(0, 3, 2, 1, 4).contiguous().view(tiles, KB // 4, 512)


def mx_chunks_to_scales(chunks: torch.Tensor, rows: int) -> torch.Tensor:
    """Inverse of ``mx_scales_to_chunks``."""
    tiles, kc, _ = chunks.shape
    v = chunks.view(tiles, kc, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(tiles * 128, kc * 4)
    return v[:rows]


def quantize_mx(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [R, K] (K % 128 == 0) -> (q e4m3 [R, K], scale chunks uint8 [ceil(R/128), K/128, 512]).  CUDA: one kernel;
    elsewhere the reference above."""
    R, K = x.shape
    if not x.is_cuda:
        q, e = quantize_mx_reference(x)
        return q, mx_scales_to_chunks(e)
    from ..ops import kernels
    q = torch.empty(R, K, dtype=torch.float8_e4m3fn, device=x.device)
    tiles = (R + 127) // 128
    alloc = torch.empty if R % 128 == 0 else (lambda *a, **k: torch.full(*a, 127, **k))
    sf = alloc((tiles, K // 128, 512), dtype=torch.uint8, device=x.device)
    kernels().mx_quantize(x.to(torch.bfloat16).contiguous(), q, sf)
    return q, sf


def gemm_mx(a_q: torch.Tensor, a_sf: torch.Tensor, b_q: torch.Tensor, b_sf: torch.Tensor,
            tile_expert: Optional[torch.Tensor] = None, num_m_tiles: Optional[torch.Tensor] = None,
            bn: int = 0) -> torch.Tensor:
    """bf16 ``A @ B.T`` of two MX tensors on the block-scaled tensor-core path.  With ``tile_expert`` the 128-row tile
    ``i`` of ``a_q`` multiplies ``b_q[tile_expert[i]]`` (``b_q`` [E, N, K]): the routed experts' grouped product."""
    from ..ops import kernels, status_word
    N = b_q.shape[-2]
    c = torch.empty(a_q.shape[0], N, dtype=torch.bfloat16, device=a_q.device)
    kernels().gemm_mxfp8(a_q, a_sf, b_q, b_sf, c, tile_expert, num_m_tiles, bn, status_word(a_q.device))
    return c


class _MXLinearFn(torch.autograd.Function):
    """Forward: both operands quantised per 32-element block and multiplied on the block-scaled tensor cores.
    Backward in bf16 from the saved bf16 operands (reference opss/train/fp8.py:381-399 keeps its backward in the
    compute dtype as well)."""

    @staticmethod
    def forward(ctx, x, w, cache):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        xq, xs = quantize_mx(x2)
        key = (w.data_ptr(), w._version)
        if cache.get("key") != key:                       # the weight is re-quantised only after it changed
            cache["key"], cache["q"] = key, quantize_mx(w.detach().contiguous())
        wq, ws = cache["q"]
        y = gemm_mx(xq, xs, wq, ws)
        ctx.save_for_backward(x2, w)
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        dx = F_.gemm(dy2, w, b_mn=True).view(ctx.shape)
        dw = F_.gemm(dy2, x2, a_mn=True, b_mn=True)
        return dx, dw, None


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
    """Linear layer whose forward runs on the fp8 tensor cores (CUDA, bf16 parameters).

    ``scaling="mx"`` (default when the shapes allow: in_features a multiple of 128, out_features of 128): e4m3 with
    one power-of-two scale per 32 elements, applied by the tensor cores.  ``scaling="delayed"``: per-tensor scales
    from an amax history, applied in the GEMM epilogue (in/out features multiples of 16)."""

    def __init__(self, in_features: int, out_features: int, device=None, history: int = 16, scaling: str = "auto"):
        super().__init__()
        device = torch.device(device or "cuda")
        if scaling == "auto":
            scaling = "mx" if in_features % 128 == 0 and out_features % 128 == 0 else "delayed"
        assert scaling in ("mx", "delayed")
        self.scaling = scaling
        self._mx_cache: dict = {}
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=torch.bfloat16, device=device).normal_(std=0.02))
        self.meta_x = YvFP8DelayedScaling(device, history)
        self.meta_w = YvFP8DelayedScaling(device, history)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.scaling == "mx":
            return _MXLinearFn.apply(x.to(torch.bfloat16), self.weight, self._mx_cache)
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
