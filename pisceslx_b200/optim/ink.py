"""Ink optimizer: Adam with block-quantised moments, optional top-k gradient sparsification, low-rank (GaLore)
projection of 2-D gradients and block-cyclic partial updates.

Follows the reference's ``PiscesLxInkOptimizer`` (opss/optim/ink/optimizer.py:84-638): int8 first moment / int4-range
second moment stored per block of ``block_size`` values with an fp32 scale (``ink/quantizer.py``), top-k sparse
gradients with error feedback (``ink/sparse.py``), GaLore projection refreshed every ``galore_update_interval`` steps
(``opss/optim/galore.py``), and one cyclic block of parameters updated per step (:344-349).
"""
from __future__ import annotations

import math
from typing import Any, Dict, Iterable, Optional, Tuple

import torch


class PiscesLxInkBlockQuantizer:
    """Symmetric per-block quantisation to ``bits`` (values stored in int8)."""

    def __init__(self, bits: int = 8, block_size: int = 256):
        self.bits, self.block = bits, block_size
        self.qmax = 2 ** (bits - 1) - 1

    def quantize(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Size, int]:
        flat = x.detach().float().flatten()
        n = flat.numel()
        pad = (-n) % self.block
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        blocks = flat.view(-1, self.block)
        scale = blocks.abs().amax(1, keepdim=True).clamp_min(1e-12) / self.qmax
        q = torch.round(blocks / scale).clamp(-self.qmax, self.qmax).to(torch.int8)
        return q, scale.squeeze(1), x.shape, n

    def dequantize(self, q: torch.Tensor, scale: torch.Tensor, shape: torch.Size, n: int) -> torch.Tensor:
        return (q.float() * scale.unsqueeze(1)).flatten()[:n].view(shape)


class PiscesLxInkSparseSelector:
    """Keep the ``ratio`` largest-magnitude gradient entries; the rest accumulates as error feedback."""

    def __init__(self, ratio: float = 0.01):
        self.ratio = ratio
        self.residual: Dict[int, torch.Tensor] = {}

    def select(self, p: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
        if self.ratio >= 1.0:
            return g
        r = self.residual.get(id(p))
        g = g + r if r is not None else g
        k = max(1, int(g.numel() * self.ratio))
        thr = torch.topk(g.abs().flatten(), k).values[-1]
        mask = g.abs() >= thr
        self.residual[id(p)] = g * (~mask)
        return g * mask


class PiscesLxGaLoreProjector:
    def __init__(self, rank: int = 128, update_interval: int = 200, scale: float = 1.0):
        self.rank, self.interval, self.scale = rank, update_interval, scale
        self.P: Optional[torch.Tensor] = None
        self.left = True

    def project(self, g: torch.Tensor, step: int) -> torch.Tensor:
        if self.P is None or step % self.interval == 0:
            U, _, Vh = torch.linalg.svd(g.float(), full_matrices=False)
            self.left = g.shape[0] <= g.shape[1]
            self.P = (U[:, : self.rank] if self.left else Vh[: self.rank].t()).to(g.dtype)
        return self.P.t() @ g if self.left else g @ self.P

    def project_back(self, u: torch.Tensor) -> torch.Tensor:
        return (self.P @ u if self.left else u @ self.P.t()) * self.scale


class YvInkOptimizer(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, momentum_bits: int = 8, variance_bits: int = 8, block_size: int = 256,
                 sparse_ratio: float = 1.0, galore_rank: int = 0, galore_update_interval: int = 200,
                 cyclic_blocks: int = 1):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.qm = PiscesLxInkBlockQuantizer(momentum_bits, block_size)
        self.qv = PiscesLxInkBlockQuantizer(variance_bits, block_size)
        self.sparse = PiscesLxInkSparseSelector(sparse_ratio)
        self.galore_rank, self.galore_interval = galore_rank, galore_update_interval
        self.cyclic_blocks = max(1, cyclic_blocks)
        self._step = 0

    def state_bytes(self) -> int:
        n = 0
        for st in self.state.values():
            for v in st.values():
                if torch.is_tensor(v):
                    n += v.numel() * v.element_size()
        return n

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._step += 1
        idx = 0
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                idx += 1
                if p.grad is None:
                    continue
                if self.cyclic_blocks > 1 and (idx % self.cyclic_blocks) != (self._step % self.cyclic_blocks):
                    continue                                   # this parameter's block is not scheduled this step
                g = self.sparse.select(p, p.grad.float())
                st = self.state[p]
                proj = None
                if self.galore_rank and p.dim() == 2 and min(p.shape) > self.galore_rank:
                    proj = st.get("galore")
                    if proj is None:
                        proj = st["galore"] = PiscesLxGaLoreProjector(self.galore_rank, self.galore_interval)
                    g = proj.project(g, self._step)
                if "m_q" not in st:
                    st["t"] = 0
                    z = torch.zeros_like(g)
                    st["m_q"], st["m_s"], st["shape"], st["n"] = self.qm.quantize(z)
                    st["v_q"], st["v_s"], _, _ = self.qv.quantize(z)
                st["t"] += 1
                m = self.qm.dequantize(st["m_q"], st["m_s"], st["shape"], st["n"])
                v = self.qv.dequantize(st["v_q"], st["v_s"], st["shape"], st["n"]).pow(2)      # sqrt(v) is what is stored
                m = b1 * m + (1 - b1) * g
                v = b2 * v + (1 - b2) * g * g
                st["m_q"], st["m_s"], _, _ = self.qm.quantize(m)
                st["v_q"], st["v_s"], _, _ = self.qv.quantize(v.sqrt())
                mh = m / (1 - b1 ** st["t"])
                vh = v / (1 - b2 ** st["t"])
                upd = mh / (vh.sqrt() + group["eps"])
                if proj is not None:
                    upd = proj.project_back(upd)
                p.data.add_((-group["lr"] * (upd + group["weight_decay"] * p.data.float())).to(p.dtype))
        return loss


PiscesLxInkOptimizer = YvInkOptimizer
