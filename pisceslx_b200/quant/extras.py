"""Further quantisers of the reference's compression toolbox.

``PiscesLxHyperQuant``: vector quantisation on the E8 lattice after a randomised Hadamard rotation (reference
opss/quantize/hyperquant.py: rotation + lattice codebook); ``PiscesLxTWLAQuantizer``: ternary weights with a low-rank
additive correction (opss/quantize/twla.py); ``PiscesLxSTARKVQuantizer``: KV-cache quantisation with salient tokens
kept at full precision (opss/quantize/star_kv.py)."""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch


def hadamard(n: int, device=None, dtype=torch.float32) -> torch.Tensor:
    """Sylvester Hadamard matrix of order n (a power of two), scaled to be orthonormal."""
    assert n & (n - 1) == 0 and n > 0
    H = torch.ones(1, 1, device=device, dtype=dtype)
    while H.shape[0] < n:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    return H / math.sqrt(n)


def _nearest_d8(x: torch.Tensor) -> torch.Tensor:
    """Nearest point of D8 (integer vectors with an even coordinate sum) to each row of x [..., 8]."""
    r = torch.round(x)
    odd = (r.sum(-1).long() % 2) != 0
    # where the sum is odd, re-round the coordinate with the largest rounding error the other way
    err = x - r
    idx = err.abs().argmax(-1, keepdim=True)
    step = torch.where(torch.gather(err, -1, idx) >= 0, 1.0, -1.0).to(x.dtype)
    fix = torch.zeros_like(r).scatter_(-1, idx, step)
    return torch.where(odd[..., None], r + fix, r)


def nearest_e8(x: torch.Tensor) -> torch.Tensor:
    """Nearest point of the E8 lattice = D8 union (D8 + 1/2): the closer of the two coset candidates."""
    a = _nearest_d8(x)
    b = _nearest_d8(x - 0.5) + 0.5
    da, db = (x - a).pow(2).sum(-1, keepdim=True), (x - b).pow(2).sum(-1, keepdim=True)
    return torch.where(da <= db, a, b)


class PiscesLxHyperQuant:
    """Weights are rotated by a sign-randomised Hadamard transform (spreads outliers), scaled per group of 8 columns
    blocks, and snapped to E8 lattice points; ``scale`` sets the bits per weight (finer lattice = more bits)."""

    def __init__(self, bits: float = 4.0, seed: int = 0):
        self.bits, self.seed = bits, seed

    def quantize(self, w: torch.Tensor) -> Dict[str, torch.Tensor]:
        O, I = w.shape
        n = 1 << (I - 1).bit_length()
        g = torch.Generator(device="cpu").manual_seed(self.seed)
        signs = (torch.randint(0, 2, (n,), generator=g) * 2 - 1).to(w.device, torch.float32)
        wp = torch.zeros(O, n, device=w.device)
        wp[:, :I] = w.float()
        rot = (wp * signs) @ hadamard(n, w.device)
        # per-row scale: the lattice covers about +-2**(bits-1) per coordinate
        s = rot.abs().amax(-1, keepdim=True).clamp_min(1e-8) / (2 ** (self.bits - 1))
        pts = nearest_e8((rot / s).reshape(O, n // 8, 8)).reshape(O, n)
        lim = 2 ** (self.bits - 1)
        pts = pts.clamp(-lim, lim)
        return {"points": (pts * 2).to(torch.int8), "scale": s, "signs": signs, "in_features": torch.tensor(I)}

    @staticmethod
    def dequantize(q: Dict[str, torch.Tensor], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        pts = q["points"].float() / 2
        n = pts.shape[1]
        w = ((pts * q["scale"]) @ hadamard(n, pts.device).t()) * q["signs"]
        return w[:, : int(q["in_features"])].to(dtype)


class PiscesLxTWLAQuantizer:
    """Ternary weights {-a, 0, +a} per output row plus a rank-``rank`` correction fitted to the residual by SVD."""

    def __init__(self, rank: int = 8, threshold: float = 0.7):
        self.rank, self.threshold = rank, threshold

    def quantize(self, w: torch.Tensor) -> Dict[str, torch.Tensor]:
        wf = w.float()
        delta = self.threshold * wf.abs().mean(-1, keepdim=True)
        t = torch.where(wf > delta, 1.0, torch.where(wf < -delta, -1.0, 0.0))
        alpha = (wf.abs() * t.abs()).sum(-1, keepdim=True) / t.abs().sum(-1, keepdim=True).clamp_min(1)
        resid = wf - alpha * t
        r = min(self.rank, min(wf.shape))
        U, S, Vh = torch.linalg.svd(resid, full_matrices=False)
        return {"ternary": t.to(torch.int8), "alpha": alpha, "A": U[:, :r] * S[:r], "B": Vh[:r]}

    @staticmethod
    def dequantize(q: Dict[str, torch.Tensor], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return (q["alpha"] * q["ternary"].float() + q["A"] @ q["B"]).to(dtype)


class YvQuantizationConfig:
    """quantization_type: int8 | int4 | fp8 | fp16 | bf16 (reference model/utils/quantization.py:100-290);
    per_channel scales along the output dimension; symmetric or with a zero point."""

    def __init__(self, quantization_type: str = "int8", per_channel: bool = True, symmetric: bool = True,
                 skip_modules: Tuple[str, ...] = ("lm_head", "embed", "router", "norm")):
        if quantization_type not in ("int8", "int4", "fp8", "fp16", "bf16"):
            raise ValueError(f"unsupported quantization type {quantization_type!r}")
        self.quantization_type, self.per_channel, self.symmetric = quantization_type, per_channel, symmetric
        self.skip_modules = tuple(skip_modules)


class _YvQuantizedLinear(torch.nn.Module):
    """Weight-only quantised linear: integer (or fp8) weights + scale (+ zero point), dequantised per call."""

    def __init__(self, q_weight, scale, zero_point, bias, kind: str):
        super().__init__()
        self.register_buffer("q_weight", q_weight)
        self.register_buffer("scale", scale)
        self.register_buffer("zero_point", zero_point if zero_point is not None else torch.zeros(()))
        self.bias, self.kind = bias, kind

    def weight(self, dtype: torch.dtype) -> torch.Tensor:
        return ((self.q_weight.float() - self.zero_point) * self.scale).to(dtype)

    def forward(self, x):
        return torch.nn.functional.linear(x, self.weight(x.dtype), None if self.bias is None else self.bias.to(x.dtype))


class YvQuantizer:
    """Tensor / module / model level weight quantisation (reference ``YvQuantizer`` :292-485)."""

    def __init__(self, config: Optional[YvQuantizationConfig] = None):
        self.config = config or YvQuantizationConfig()
        self.records: Dict[str, Dict[str, torch.Tensor]] = {}

    def quantize_tensor(self, w: torch.Tensor) -> Dict[str, torch.Tensor]:
        c, t = self.config, self.config.quantization_type
        x = w.float()
        if t in ("fp16", "bf16"):
            return {"q": x.to(torch.float16 if t == "fp16" else torch.bfloat16), "scale": torch.ones(()), "zero": torch.zeros(())}
        dim = tuple(range(1, x.dim())) if c.per_channel and x.dim() > 1 else None
        if t == "fp8":
            amax = x.abs().amax(dim, keepdim=True) if dim else x.abs().max()
            s = amax.clamp_min(1e-12) / 448.0
            return {"q": (x / s).to(torch.float8_e4m3fn), "scale": s, "zero": torch.zeros(())}
        bits = 8 if t == "int8" else 4
        if c.symmetric:
            qmax = 2 ** (bits - 1) - 1
            amax = x.abs().amax(dim, keepdim=True) if dim else x.abs().max()
            s = amax.clamp_min(1e-12) / qmax
            return {"q": torch.round(x / s).clamp(-qmax - 1, qmax).to(torch.int8), "scale": s, "zero": torch.zeros(())}
        lo = x.amin(dim, keepdim=True) if dim else x.min()
        hi = x.amax(dim, keepdim=True) if dim else x.max()
        s = ((hi - lo) / (2 ** bits - 1)).clamp_min(1e-12)
        z = torch.round(-lo / s)
        return {"q": (torch.round(x / s) + z).clamp(0, 2 ** bits - 1).to(torch.uint8), "scale": s, "zero": z}

    @staticmethod
    def dequantize_tensor(r: Dict[str, torch.Tensor], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return ((r["q"].float() - r["zero"]) * r["scale"]).to(dtype)

    def quantize_linear(self, lin: torch.nn.Linear) -> _YvQuantizedLinear:
        r = self.quantize_tensor(lin.weight.data)
        return _YvQuantizedLinear(r["q"], r["scale"], r["zero"], lin.bias, self.config.quantization_type)

    def quantize_model(self, model: torch.nn.Module) -> int:
        """Replaces every ``nn.Linear`` not matched by ``skip_modules`` in place; returns how many were replaced."""
        n = 0
        for name, mod in list(model.named_modules()):
            for cname, child in list(mod.named_children()):
                full = f"{name}.{cname}" if name else cname
                if isinstance(child, torch.nn.Linear) and not any(s in full for s in self.config.skip_modules):
                    q = self.quantize_linear(child)
                    setattr(mod, cname, q)
                    self.records[full] = {"q": q.q_weight, "scale": q.scale, "zero": q.zero_point}
                    n += 1
        return n

    def get_state_dict(self) -> Dict[str, torch.Tensor]:
        return {f"{k}.{f}": v for k, r in self.records.items() for f, v in r.items()}


class PiscesLxSTARKVQuantizer:
    """KV-cache quantisation that keeps the ``keep`` most attended tokens (by accumulated attention mass) in full
    precision and stores the rest as per-token int``bits`` with a scale and a zero point."""

    def __init__(self, bits: int = 4, keep: int = 32):
        self.bits, self.keep = bits, keep

    def quantize(self, kv: torch.Tensor, attn_mass: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        """kv [T, H, D]; attn_mass [T]."""
        T = kv.shape[0]
        if attn_mass is None:
            attn_mass = kv.float().norm(dim=(-1, -2))
        k = min(self.keep, T)
        salient = torch.topk(attn_mass, k).indices.sort().values
        x = kv.float()
        lo, hi = x.amin((-1, -2), keepdim=True), x.amax((-1, -2), keepdim=True)
        qmax = 2 ** self.bits - 1
        scale = ((hi - lo) / qmax).clamp_min(1e-8)
        q = torch.round((x - lo) / scale).clamp(0, qmax).to(torch.uint8)
        return {"q": q, "scale": scale, "zero": lo, "salient_idx": salient, "salient": kv[salient].clone()}

    @staticmethod
    def dequantize(c: Dict[str, torch.Tensor], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        x = (c["q"].float() * c["scale"] + c["zero"]).to(dtype)
        x[c["salient_idx"]] = c["salient"].to(dtype)
        return x
