"""Block-level building blocks beside the main transformer block (reference model/core/blocks.py: ``YvLoRA`` /
``YvDoRA`` adapters, LayerScale, ``YvMixtureOfDepths``, ``YvAdaptiveComputationTime``, ``YvParallelBlock``,
``YvDeepNormBlock``, ``YvCrossAttentionBlock``, ``YvGeGLU``; norms ``YvLayerNorm`` / ``YvDeepNorm`` /
``YvParallelResidualNorm`` from model/core/norms.py:699-801)."""
from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as F_
from .attention_variants import causal_mask, masked_attention
from .norms import YvRMSNorm


class YvLoRA(nn.Module):
    """y = x W^T + (alpha / r) * (x A^T) B^T on a frozen base weight."""

    def __init__(self, base_weight: torch.Tensor, rank: int = 8, alpha: float = 16.0, dropout: float = 0.0):
        super().__init__()
        out_f, in_f = base_weight.shape
        self.weight = nn.Parameter(base_weight.detach().clone(), requires_grad=False)
        self.lora_a = nn.Parameter(torch.empty(rank, in_f).normal_(std=1.0 / rank))
        self.lora_b = nn.Parameter(torch.zeros(out_f, rank))
        self.scaling, self.dropout = alpha / rank, nn.Dropout(dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F_.linear(x, self.weight) + self.scaling * F_.linear(F_.linear(self.dropout(x), self.lora_a.to(x.dtype)),
                                                                  self.lora_b.to(x.dtype))

    def merged_weight(self) -> torch.Tensor:
        return self.weight + self.scaling * (self.lora_b @ self.lora_a).to(self.weight.dtype)


class YvDoRA(YvLoRA):
    """Weight-decomposed adaptation: direction = (W + BA) normalised per output row, magnitude learned."""

    def __init__(self, base_weight: torch.Tensor, rank: int = 8, alpha: float = 16.0):
        super().__init__(base_weight, rank, alpha)
        self.magnitude = nn.Parameter(base_weight.detach().float().norm(dim=1))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.merged_weight().float()
        w = w * (self.magnitude / w.norm(dim=1).clamp_min(1e-8))[:, None]
        return F_.linear(x, w.to(x.dtype))


class YvLayerScale(nn.Module):
    def __init__(self, hidden: int, init: float = 1e-4):
        super().__init__()
        self.gamma = nn.Parameter(torch.full((hidden,), init))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x * self.gamma.to(x.dtype)


class YvGeGLU(nn.Module):
    def __init__(self, hidden: int, inner: int):
        super().__init__()
        self.w13 = nn.Parameter(torch.empty(2 * inner, hidden).normal_(std=0.02))
        self.w2 = nn.Parameter(torch.empty(hidden, inner).normal_(std=0.02))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        g, u = F_.linear(x, self.w13).chunk(2, -1)
        return F_.linear(F.gelu(g) * u, self.w2)


class YvMixtureOfDepths(nn.Module):
    """Token-level routing around a block: the ``capacity`` fraction of tokens with the highest router score go
    through ``block``; the rest skip it.  The router weight multiplies the block's update so that it gets gradient."""

    def __init__(self, hidden: int, capacity: float = 0.5):
        super().__init__()
        self.router = nn.Parameter(torch.zeros(1, hidden))
        self.capacity = capacity

    def forward(self, x: torch.Tensor, block: Callable[[torch.Tensor], torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        B, S, H = x.shape
        score = F_.linear(x, self.router.to(x.dtype)).squeeze(-1).float()           # [B, S]
        k = max(1, int(math.ceil(self.capacity * S)))
        idx = score.topk(k, dim=1).indices.sort(1).values
        sel = torch.gather(x, 1, idx[..., None].expand(B, k, H))
        upd = block(sel) - sel
        w = torch.sigmoid(torch.gather(score, 1, idx))[..., None].to(x.dtype)
        out = x.scatter_add(1, idx[..., None].expand(B, k, H), w * upd)
        return out, idx


class YvAdaptiveComputationTime(nn.Module):
    """Halting over repeated applications of ``block``: per-token halting probabilities accumulate until 1 - eps;
    the output is the halting-weighted mixture of the intermediate states; ``ponder`` is the cost term."""

    def __init__(self, hidden: int, max_steps: int = 4, eps: float = 0.01):
        super().__init__()
        self.halt = nn.Parameter(torch.zeros(1, hidden))
        self.halt_bias = nn.Parameter(torch.ones(1))
        self.max_steps, self.eps = max_steps, eps

    def forward(self, x: torch.Tensor, block: Callable[[torch.Tensor], torch.Tensor]):
        acc = torch.zeros(x.shape[:-1], device=x.device)
        out = torch.zeros_like(x)
        ponder = torch.zeros_like(acc)
        state = x
        for step in range(self.max_steps):
            state = block(state)
            p = torch.sigmoid(F_.linear(state, self.halt.to(x.dtype)).squeeze(-1).float() + self.halt_bias)
            running = acc < 1 - self.eps
            last = step == self.max_steps - 1
            use = torch.where(running, torch.where((acc + p > 1 - self.eps) | last, 1 - acc, p), torch.zeros_like(p))
            out = out + use[..., None].to(x.dtype) * state
            acc = acc + use
            ponder = ponder + running.float()
            if not bool((acc < 1 - self.eps).any()):
                break
        return out, ponder.mean()


class YvLayerNorm(nn.LayerNorm):
    pass


class YvDeepNorm(nn.Module):
    """DeepNorm residual: LayerNorm(alpha * x + f(x)) with alpha = (2L)^(1/4)."""

    def __init__(self, hidden: int, n_layers: int):
        super().__init__()
        self.alpha = (2 * n_layers) ** 0.25
        self.beta = (8 * n_layers) ** -0.25                  # init gain of the sub-layer weights
        self.norm = nn.LayerNorm(hidden)

    def forward(self, x: torch.Tensor, fx: torch.Tensor) -> torch.Tensor:
        return self.norm(self.alpha * x + fx)


class YvParallelResidualNorm(nn.Module):
    """One shared pre-norm feeding attention and MLP in parallel: x + attn(n(x)) + mlp(n(x))."""

    def __init__(self, hidden: int, eps: float = 1e-6):
        super().__init__()
        self.norm = YvRMSNorm(hidden, eps)

    def forward(self, x, attn: Callable, mlp: Callable) -> torch.Tensor:
        n = self.norm(x)
        return x + attn(n) + mlp(n)


class YvParallelBlock(nn.Module):
    def __init__(self, hidden: int, attn: nn.Module, mlp: nn.Module):
        super().__init__()
        self.res, self.attn, self.mlp = YvParallelResidualNorm(hidden), attn, mlp

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.res(x, self.attn, self.mlp)


class YvDeepNormBlock(nn.Module):
    def __init__(self, hidden: int, n_layers: int, attn: nn.Module, mlp: nn.Module):
        super().__init__()
        self.n1, self.n2, self.attn, self.mlp = YvDeepNorm(hidden, n_layers), YvDeepNorm(hidden, n_layers), attn, mlp

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.n1(x, self.attn(x))
        return self.n2(x, self.mlp(x))


class YvCrossAttentionBlock(nn.Module):
    """Pre-norm cross attention from ``x`` to a memory (encoder states, modal tokens) + feed-forward."""

    def __init__(self, hidden: int, n_head: int, mlp: Optional[nn.Module] = None):
        super().__init__()
        self.h, self.d = n_head, hidden // n_head
        self.nq, self.nkv, self.nm = YvRMSNorm(hidden), YvRMSNorm(hidden), YvRMSNorm(hidden)
        self.q = nn.Parameter(torch.empty(hidden, hidden).normal_(std=0.02))
        self.kv = nn.Parameter(torch.empty(2 * hidden, hidden).normal_(std=0.02))
        self.o = nn.Parameter(torch.empty(hidden, hidden).normal_(std=0.02))
        self.mlp = mlp or YvGeGLU(hidden, 2 * hidden)

    def forward(self, x: torch.Tensor, memory: torch.Tensor, memory_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, S, H = x.shape
        T = memory.shape[1]
        q = F_.linear(self.nq(x), self.q).view(B, S, self.h, self.d).transpose(1, 2)
        k, v = F_.linear(self.nkv(memory), self.kv).chunk(2, -1)
        k, v = k.view(B, T, self.h, self.d).transpose(1, 2), v.view(B, T, self.h, self.d).transpose(1, 2)
        m = memory_mask[:, None, None, :].bool() if memory_mask is not None else None
        a = masked_attention(q, k, v, m).transpose(1, 2).reshape(B, S, H)
        x = x + F_.linear(a, self.o)
        return x + self.mlp(self.nm(x))
