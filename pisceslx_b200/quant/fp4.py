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



# ----------------------------------------------------------------------------------------------------------------------
# Quartet: weights STORED in fp4 (reference opss/quantization/quartet.py:36-166)
# ----------------------------------------------------------------------------------------------------------------------
def pack_fp4(q: torch.Tensor) -> torch.Tensor:
    """Values on the E2M1 grid -> 4-bit codes (sign bit + 3-bit magnitude index), two per byte."""
    grid = _E2M1.to(q.device)
    idx = torch.searchsorted(grid, q.abs().float().flatten().contiguous()).clamp(max=7)
    code = (idx | ((q.flatten() < 0).long() << 3)).to(torch.uint8)
    if code.numel() % 2:
        code = torch.cat([code, code.new_zeros(1)])
    return code[0::2] | (code[1::2] << 4)


def unpack_fp4(packed: torch.Tensor, numel: int) -> torch.Tensor:
    code = torch.stack([packed & 0xF, packed >> 4], 1).flatten()[:numel].long()
    mag = _E2M1.to(packed.device)[code & 7]
    return torch.where((code & 8) > 0, -mag, mag)


class PiscesLxQuartetLinear(nn.Module):
    """Linear layer whose weight lives as packed E2M1 codes (half a byte per element) plus one fp32 scale per block.
    The forward dequantises into the compute dtype; ``apply_update`` adds a step to the dequantised weight and
    re-quantises with stochastic rounding, which is what keeps training unbiased at 4 bits.  A straight-through
    ``weight_shadow`` parameter carries the gradient (it holds no information of its own: it is overwritten from the
    codes before every forward)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, block_size: int = 16,
                 init: Optional[torch.Tensor] = None, seed: Optional[int] = None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.quantizer = PiscesLxFP4Quantizer(block_size, stochastic=True, seed=seed)
        w = init if init is not None else torch.empty(out_features, in_features).normal_(std=0.02)
        self.weight_shadow = nn.Parameter(torch.zeros(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.register_buffer("weight_fp4", torch.zeros((w.numel() + 1) // 2, dtype=torch.uint8))
        self.register_buffer("scale", torch.zeros((w.numel() + block_size - 1) // block_size))
        self.store(w)

    @torch.no_grad()
    def store(self, w: torch.Tensor) -> None:
        q, s = self.quantizer.quantize(w.detach().float().cpu())
        self.weight_fp4.copy_(pack_fp4(q).to(self.weight_fp4.device))
        self.scale.copy_(s.to(self.scale.device))

    def dequantized(self) -> torch.Tensor:
        q = unpack_fp4(self.weight_fp4, self.in_features * self.out_features).view(self.out_features, self.in_features)
        return self.quantizer.dequantize(q, self.scale)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            self.weight_shadow.copy_(self.dequantized())
        return torch.nn.functional.linear(x, self.weight_shadow.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))

    @torch.no_grad()
    def apply_update(self, delta: torch.Tensor) -> None:
        """weight <- stochastic_round_fp4(weight + delta)."""
        self.store(self.dequantized() + delta.to(self.scale.device).float())

    def storage_bytes(self) -> int:
        return self.weight_fp4.numel() + self.scale.numel() * 4


class PiscesLxQuartetTrainer:
    """Converts every ``nn.Linear`` of a model to fp4 storage and applies SGD-style steps through stochastic
    re-quantisation (reference quartet.py:124-160)."""

    def __init__(self, model: nn.Module, block_size: int = 16, skip: Tuple[str, ...] = ("lm_head",)):
        self.model, self.block = model, block_size
        self.converted = 0
        self._bytes_before = sum(p.numel() * p.element_size() for p in model.parameters())
        self._convert(model, skip)

    def _convert(self, mod: nn.Module, skip: Tuple[str, ...], prefix: str = "") -> None:
        for name, child in list(mod.named_children()):
            full = f"{prefix}{name}"
            if isinstance(child, nn.Linear) and not any(s in full for s in skip):
                q = PiscesLxQuartetLinear(child.in_features, child.out_features, child.bias is not None, self.block,
                                          init=child.weight.data)
                if child.bias is not None:
                    q.bias.data.copy_(child.bias.data)
                setattr(mod, name, q)
                self.converted += 1
            else:
                self._convert(child, skip, full + ".")

    @torch.no_grad()
    def step(self, lr: float) -> None:
        for m in self.model.modules():
            if isinstance(m, PiscesLxQuartetLinear) and m.weight_shadow.grad is not None:
                m.apply_update(-lr * m.weight_shadow.grad)
                m.weight_shadow.grad = None

    def get_compression_ratio(self) -> float:
        now = 0
        for m in self.model.modules():
            if isinstance(m, PiscesLxQuartetLinear):
                now += m.storage_bytes() + (m.bias.numel() * 4 if m.bias is not None else 0)
        seen = {id(p) for m in self.model.modules() if isinstance(m, PiscesLxQuartetLinear) for p in m.parameters()}
        now += sum(p.numel() * p.element_size() for p in self.model.parameters() if id(p) not in seen)
        return self._bytes_before / max(now, 1)


class PiscesLxQuartetQuantizer(PiscesLxFP4Quantizer):
    """Name used by the reference for the functional form (quartet.py:163)."""
