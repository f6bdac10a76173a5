"""FP4 (E2M1) block quantisation with stochastic rounding and fp32 master weights (reference opss/optim/fp4.py,
opss/quantization/quartet.py)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

# representable magnitudes of E2M1
_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


class PiscesLxFP4Quantizer:
    def __init__(self, block_size: int = 16, stochastic: bool = True, seed: Optional[int] = None):
        self.block, self.stochastic = block_size, stochastic
        self.gen = torch.Generator().manual_seed(seed) if seed is not None else None

    def quantize(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns (values on the fp4 grid times nothing, scales): x ~= q * scale per block of ``block_size``."""
        shape = x.shape
        flat = x.float().flatten()
        pad = (-flat.numel()) % self.block
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        b = flat.view(-1, self.block)
        scale = b.abs().amax(1, keepdim=True).clamp_min(1e-12) / 6.0
        y = b / scale
        grid = _E2M1.to(y.device)
        mag = y.abs().clamp(max=6.0)
        hi_idx = torch.searchsorted(grid, mag.contiguous()).clamp(max=grid.numel() - 1)
        lo_idx = (hi_idx - 1).clamp(min=0)
        lo, hi = grid[lo_idx], grid[hi_idx]
        span = (hi - lo).clamp_min(1e-12)
        frac = ((mag - lo) / span).clamp(0, 1)
        if self.stochastic:
            u = torch.rand(frac.shape, generator=self.gen).to(frac.device) if self.gen is not None else torch.rand_like(frac)
            pick_hi = u < frac
        else:
            pick_hi = frac >= 0.5
        q = torch.where(pick_hi, hi, lo) * torch.sign(y)
        q = q.flatten()[: x.numel()].view(shape)
        return q, scale.squeeze(1)

    def dequantize(self, q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        flat = q.float().flatten()
        pad = (-flat.numel()) % self.block
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        return (flat.view(-1, self.block) * scale.unsqueeze(1)).flatten()[: q.numel()].view(q.shape)

    def fake_quant(self, x: torch.Tensor) -> torch.Tensor:
        q, s = self.quantize(x)
        return self.dequantize(q, s).to(x.dtype)


class _FP4STE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, quantizer):
        return quantizer.fake_quant(w)

    @staticmethod
    def backward(ctx, g):
        return g, None


class PiscesLxFP4Linear(nn.Module):
    """Linear layer with fp4 fake-quantised weights in the forward pass and a straight-through gradient to the
    fp32 master weight."""

    def __init__(self, in_features: int, out_features: int, block_size: int = 16, stochastic: bool = True):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features).normal_(std=0.02))
        self.quantizer = PiscesLxFP4Quantizer(block_size, stochastic)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(x, _FP4STE.apply(self.weight, self.quantizer).to(x.dtype))


PiscesLxQuartetLinear = PiscesLxFP4Linear
