"""Post-training quantisation methods (reference opss/quantize/methods.py): GPTQ (Hessian-guided column-wise
rounding with error compensation), AWQ (activation-aware per-channel scaling before rounding), SmoothQuant
(migrating activation outliers into the weights), block-wise INT4, KV-cache quantisation (per-token int8 / fp8)."""
from __future__ import annotations

from typing import Any, Dict, Iterable, Optional, Tuple

import torch


def _quant_sym(w: torch.Tensor, bits: int, dim: int = -1) -> Tuple[torch.Tensor, torch.Tensor]:
    qmax = 2 ** (bits - 1) - 1
    scale = w.abs().amax(dim, keepdim=True).clamp_min(1e-12) / qmax
    return torch.round(w / scale).clamp(-qmax - 1, qmax), scale


class PiscesLxBlockWiseINT4Quantizer:
    def __init__(self, group_size: int = 128, bits: int = 4):
        self.group, self.bits = group_size, bits

    def quantize(self, w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        out, inp = w.shape
        g = self.group
        pad = (-inp) % g
        wf = torch.nn.functional.pad(w.float(), (0, pad)).view(out, -1, g)
        q, s = _quant_sym(wf, self.bits)
        return q.to(torch.int8), s.squeeze(-1)

    def dequantize(self, q: torch.Tensor, s: torch.Tensor, in_features: int) -> torch.Tensor:
        return (q.float() * s.unsqueeze(-1)).flatten(1)[:, :in_features]

    def fake_quant(self, w: torch.Tensor) -> torch.Tensor:
        q, s = self.quantize(w)
        return self.dequantize(q, s, w.shape[1]).to(w.dtype)


class PiscesLxGPTQQuantizer:
    """One linear layer at a time: H = 2 X^T X from calibration activations, columns quantised in order with the
    rounding error pushed onto the not-yet-quantised columns through the inverse Hessian."""

    def __init__(self, bits: int = 4, group_size: int = 128, damp: float = 0.01):
        self.bits, self.group, self.damp = bits, group_size, damp

    def quantize(self, w: torch.Tensor, calib_x: torch.Tensor) -> torch.Tensor:
        W = w.float().clone()
        X = calib_x.float().reshape(-1, W.shape[1])
        H = 2.0 * X.t() @ X / max(X.shape[0], 1)
        dead = torch.diag(H) == 0
        H[dead, dead] = 1.0
        W[:, dead] = 0.0
        H += self.damp * torch.diag(H).mean() * torch.eye(H.shape[0], device=H.device)
        Hinv = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True)
        Q = torch.zeros_like(W)
        qmax = 2 ** (self.bits - 1) - 1
        scale = None
        for i in range(W.shape[1]):
            if i % self.group == 0:
                blk = W[:, i:i + self.group]
                scale = blk.abs().amax(1, keepdim=True).clamp_min(1e-12) / qmax
            col = W[:, i:i + 1]
            q = torch.round(col / scale).clamp(-qmax - 1, qmax) * scale
            Q[:, i:i + 1] = q
            err = (col - q) / Hinv[i, i]
            if i + 1 < W.shape[1]:
                W[:, i + 1:] -= err @ Hinv[i:i + 1, i + 1:]
        return Q.to(w.dtype)


class PiscesLxAWQQuantizer:
    """Search a per-input-channel scale s = mean|x|^alpha that minimises the output error after rounding W * s."""

    def __init__(self, bits: int = 4, group_size: int = 128, grid: int = 10):
        self.bits, self.grid = bits, grid
        self.base = PiscesLxBlockWiseINT4Quantizer(group_size, bits)

    def quantize(self, w: torch.Tensor, calib_x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        X = calib_x.float().reshape(-1, w.shape[1])
        act = X.abs().mean(0).clamp_min(1e-8)
        ref = X @ w.float().t()
        best, best_err, best_s = None, float("inf"), None
        for i in range(self.grid + 1):
            alpha = i / self.grid
            s = act.pow(alpha)
            s = s / (s.max() * s.min()).sqrt().clamp_min(1e-8)
            wq = self.base.fake_quant(w.float() * s) / s
            err = float(((X @ wq.t()) - ref).pow(2).mean())
            if err < best_err:
                best, best_err, best_s = wq, err, s
        return best.to(w.dtype), best_s


class PiscesLxSmoothQuantizer:
    """s_j = max|x_j|^alpha / max|w_j|^(1-alpha); activations are divided and weights multiplied by s."""

    def __init__(self, alpha: float = 0.5):
        self.alpha = alpha

    def scales(self, w: torch.Tensor, calib_x: torch.Tensor) -> torch.Tensor:
        ax = calib_x.float().reshape(-1, w.shape[1]).abs().amax(0).clamp_min(1e-5)
        aw = w.float().abs().amax(0).clamp_min(1e-5)
        return (ax.pow(self.alpha) / aw.pow(1 - self.alpha)).clamp_min(1e-5)

    def apply(self, w: torch.Tensor, calib_x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        s = self.scales(w, calib_x)
        return (w.float() * s).to(w.dtype), s


class PiscesLxKVCacheQuantizer:
    """Per-token symmetric int8 (or fp8) quantisation of cache rows [tokens, heads*dim]."""

    def __init__(self, mode: str = "int8"):
        self.mode = mode

    def quantize(self, kv: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.mode == "fp8":
            s = kv.float().abs().amax(-1, keepdim=True).clamp_min(1e-12) / 448.0
            return (kv.float() / s).to(torch.float8_e4m3fn), s
        q, s = _quant_sym(kv.float(), 8)
        return q.to(torch.int8), s

    def dequantize(self, q: torch.Tensor, s: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return (q.float() * s).to(dtype)


def quantize_model_weights(model: torch.nn.Module, method: str = "int4", group_size: int = 128,
                           skip: Iterable[str] = ("embed", "lm_head", "norm", "router")) -> Dict[str, float]:
    """In-place fake quantisation of every 2-D / 3-D weight; returns the relative error per tensor."""
    qz = PiscesLxBlockWiseINT4Quantizer(group_size, 4 if method == "int4" else 8)
    report: Dict[str, float] = {}
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() < 2 or any(k in n for k in skip):
                continue
            w2 = p.data.reshape(-1, p.shape[-1])
            wq = qz.fake_quant(w2)
            report[n] = float((wq.float() - w2.float()).norm() / w2.float().norm().clamp_min(1e-12))
            p.data.copy_(wq.view_as(p))
    return report
