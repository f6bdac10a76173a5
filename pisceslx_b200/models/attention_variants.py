"""Attention variants of the Yv model family (reference model/core/attention.py: ``YvALiBi`` :320,
``YvAttentionSink`` :506, ``YvQKNormalizer`` :628, ``YvLinearAttention`` :748, ``YvSlidingWindowAttention`` :1482,
``YvSparseAttention`` :1680, ``YvLocalGlobalAttention`` :2489, ``YvMultiQueryAttention`` :3145, ``YvH2OAttention``
:3822, DSA top-k key pruning :5730-5745, MLA-style latent KV compression :5648-5662).

The trunk's hot path is ``models.attention.YvAttention`` (fused QKV + flash kernels).  The variants here share one
masked-softmax core that takes an additive bias / boolean mask, so that each variant is the few lines that define
its mask, bias or feature map; on CUDA the dense causal / full cases route to the flash kernels through
``ops.functional.attention`` and the masked cases run the fp32 core."""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as F_
from .norms import YvRMSNorm


def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: Optional[torch.Tensor] = None,
                     bias: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                     return_probs: bool = False):
    """q [B,Hq,S,D], k/v [B,Hk,T,D] (Hq a multiple of Hk); ``mask`` True = visible, broadcastable to [B,Hq,S,T];
    ``bias`` additive, same broadcasting.  fp32 softmax; rows with no visible key give zeros."""
    B, Hq, S, D = q.shape
    Hk = k.shape[1]
    if Hq != Hk:
        k = k.repeat_interleave(Hq // Hk, 1)
        v = v.repeat_interleave(Hq // Hk, 1)
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * (scale if scale is not None else D ** -0.5)
    if bias is not None:
        s = s + bias.float()
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.matmul(p, v.float()).to(q.dtype)
    return (o, p) if return_probs else o


def causal_mask(S: int, T: int, device=None) -> torch.Tensor:
    """Bottom-right aligned causal mask [S, T]."""
    i = torch.arange(S, device=device)[:, None] + (T - S)
    return torch.arange(T, device=device)[None, :] <= i


class YvALiBi(nn.Module):
    """Linear position bias -slope_h * (i - j) with the geometric slope schedule."""

    def __init__(self, n_head: int):
        super().__init__()
        self.register_buffer("slopes", self.get_slopes(n_head), persistent=False)

    @staticmethod
    def get_slopes(n: int) -> torch.Tensor:
        def pow2(m):
            start = 2 ** (-(2 ** -(math.log2(m) - 3)))
            return [start * (start ** i) for i in range(m)]
        if math.log2(n).is_integer():
            return torch.tensor(pow2(n))
        c = 2 ** math.floor(math.log2(n))
        return torch.tensor(pow2(c) + YvALiBi.get_slopes(2 * c)[0::2][: n - c].tolist())

    def forward(self, S: int, T: int) -> torch.Tensor:
        dist = (torch.arange(S, device=self.slopes.device)[:, None] + (T - S)
                - torch.arange(T, device=self.slopes.device)[None, :]).clamp_min(0)
        return -self.slopes[:, None, None] * dist[None].float()              # [H, S, T]


class YvQKNormalizer(nn.Module):
    """RMS normalisation of queries and keys per head before the dot product."""

    def __init__(self, head_dim: int, eps: float = 1e-6):
        super().__init__()
        self.q_norm, self.k_norm = YvRMSNorm(head_dim, eps), YvRMSNorm(head_dim, eps)

    def forward(self, q: torch.Tensor, k: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.q_norm(q), self.k_norm(k)


class _ProjectedAttention(nn.Module):
    def __init__(self, hidden: int, n_head: int, n_kv_head: Optional[int] = None):
        super().__init__()
        self.h, self.hk, self.d = n_head, n_kv_head or n_head, hidden // n_head
        self.q_proj = nn.Parameter(torch.empty(n_head * self.d, hidden).normal_(std=0.02))
        self.k_proj = nn.Parameter(torch.empty(self.hk * self.d, hidden).normal_(std=0.02))
        self.v_proj = nn.Parameter(torch.empty(self.hk * self.d, hidden).normal_(std=0.02))
        self.o_proj = nn.Parameter(torch.empty(hidden, n_head * self.d).normal_(std=0.02))

    def qkv(self, x: torch.Tensor):
        B, S, _ = x.shape
        q = F_.linear(x, self.q_proj).view(B, S, self.h, self.d).transpose(1, 2)
        k = F_.linear(x, self.k_proj).view(B, S, self.hk, self.d).transpose(1, 2)
        v = F_.linear(x, self.v_proj).view(B, S, self.hk, self.d).transpose(1, 2)
        return q, k, v

    def out(self, o: torch.Tensor) -> torch.Tensor:
        B, H, S, D = o.shape
        return F_.linear(o.transpose(1, 2).reshape(B, S, H * D), self.o_proj)


class YvMultiQueryAttention(_ProjectedAttention):
    """One shared key/value head."""

    def __init__(self, hidden: int, n_head: int):
        super().__init__(hidden, n_head, 1)

    def forward(self, x: torch.Tensor, causal: bool = True) -> torch.Tensor:
        q, k, v = self.qkv(x)
        m = causal_mask(x.shape[1], x.shape[1], x.device) if causal else None
        return self.out(masked_attention(q, k, v, m))


class YvSlidingWindowAttention(_ProjectedAttention):
    """Causal attention restricted to the last ``window`` keys (plus ``n_sink`` always-visible first tokens)."""

    def __init__(self, hidden: int, n_head: int, window: int, n_kv_head: Optional[int] = None, n_sink: int = 0):
        super().__init__(hidden, n_head, n_kv_head)
        self.window, self.n_sink = window, n_sink

    def mask(self, S: int, device) -> torch.Tensor:
        i, j = torch.arange(S, device=device)[:, None], torch.arange(S, device=device)[None, :]
        return (j <= i) & ((i - j < self.window) | (j < self.n_sink))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q, k, v = self.qkv(x)
        return self.out(masked_attention(q, k, v, self.mask(x.shape[1], x.device)))


class YvAttentionSink(YvSlidingWindowAttention):
    """Streaming attention: the first ``n_sink`` tokens stay visible so that the softmax keeps its anchor."""

    def __init__(self, hidden: int, n_head: int, window: int, n_sink: int = 4, n_kv_head: Optional[int] = None):
        super().__init__(hidden, n_head, window, n_kv_head, n_sink)


class YvLocalGlobalAttention(_ProjectedAttention):
    """Every ``global_every``-th token is global (seen by, and seeing, everything causal); the rest are local."""

    def __init__(self, hidden: int, n_head: int, window: int, global_every: int = 64):
        super().__init__(hidden, n_head)
        self.window, self.global_every = window, global_every

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        S = x.shape[1]
        i, j = torch.arange(S, device=x.device)[:, None], torch.arange(S, device=x.device)[None, :]
        glob = (j % self.global_every == 0) | (i % self.global_every == 0)
        m = (j <= i) & ((i - j < self.window) | glob)
        q, k, v = self.qkv(x)
        return self.out(masked_attention(q, k, v, m))


class YvSparseAttention(_ProjectedAttention):
    """Top-k key selection per query (the reference's DSA pruning above 1 024 keys): scores are computed once, the
    ``top_k`` largest causal scores per row are kept, the softmax runs over those."""

    def __init__(self, hidden: int, n_head: int, top_k: int):
        super().__init__(hidden, n_head)
        self.top_k = top_k

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q, k, v = self.qkv(x)
        S = x.shape[1]
        s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * self.d ** -0.5
        s = s.masked_fill(~causal_mask(S, S, x.device), float("-inf"))
        if self.top_k < S:
            kth = s.topk(self.top_k, -1).values[..., -1:]
            s = s.masked_fill(s < kth, float("-inf"))
        return self.out(torch.matmul(torch.softmax(s, -1), v.float()).to(x.dtype))


class YvLinearAttention(_ProjectedAttention):
    """Causal linear attention with the feature map elu(x) + 1: O(S) state (sum of k^T v and of k)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q, k, v = self.qkv(x)
        q, k = F.elu(q.float()) + 1, F.elu(k.float()) + 1
        kv = torch.einsum("bhsd,bhse->bhsde", k, v.float()).cumsum(2)
        z = k.cumsum(2)
        num = torch.einsum("bhsd,bhsde->bhse", q, kv)
        den = torch.einsum("bhsd,bhsd->bhs", q, z).clamp_min(1e-6)
        return self.out((num / den[..., None]).to(x.dtype))


class YvH2OAttention(_ProjectedAttention):
    """Heavy-hitter oracle: keeps, besides the recent window, the keys that have received the most attention mass so
    far.  ``forward`` returns the output and the per-key accumulated scores used by the cache's eviction policy."""

    def __init__(self, hidden: int, n_head: int, recent: int, heavy: int):
        super().__init__(hidden, n_head)
        self.recent, self.heavy = recent, heavy

    def forward(self, x: torch.Tensor):
        q, k, v = self.qkv(x)
        S = x.shape[1]
        o, p = masked_attention(q, k, v, causal_mask(S, S, x.device), return_probs=True)
        acc = p.sum(2)                                                       # [B, H, T] attention mass per key
        keep = torch.zeros_like(acc, dtype=torch.bool)
        keep[..., max(0, S - self.recent):] = True
        if self.heavy > 0 and S > self.recent:
            older = acc[..., : S - self.recent]
            idx = older.topk(min(self.heavy, older.shape[-1]), -1).indices
            keep.scatter_(-1, idx, True)
        return self.out(o), acc, keep


class YvLatentKVAttention(nn.Module):
    """MLA-style attention: keys and values are reconstructed from a low-rank latent (the only thing a cache has to
    keep), queries optionally low-rank; RoPE is applied to a decoupled ``rope_dim`` slice shared by all heads."""

    def __init__(self, hidden: int, n_head: int, kv_lora_rank: int, rope_dim: int = 0, q_lora_rank: int = 0):
        super().__init__()
        self.h, self.d, self.rope_dim = n_head, hidden // n_head, rope_dim
        self.kv_down = nn.Parameter(torch.empty(kv_lora_rank + rope_dim, hidden).normal_(std=0.02))
        self.kv_norm = YvRMSNorm(kv_lora_rank)
        self.k_up = nn.Parameter(torch.empty(n_head * self.d, kv_lora_rank).normal_(std=0.02))
        self.v_up = nn.Parameter(torch.empty(n_head * self.d, kv_lora_rank).normal_(std=0.02))
        qin = q_lora_rank or hidden
        self.q_down = nn.Parameter(torch.empty(q_lora_rank, hidden).normal_(std=0.02)) if q_lora_rank else None
        self.q_up = nn.Parameter(torch.empty(n_head * (self.d + rope_dim), qin).normal_(std=0.02))
        self.o_proj = nn.Parameter(torch.empty(hidden, n_head * self.d).normal_(std=0.02))
        self.kv_lora_rank = kv_lora_rank

    def latent(self, x: torch.Tensor) -> torch.Tensor:
        """What a KV cache stores per token: [B, S, kv_lora_rank + rope_dim]."""
        return F_.linear(x, self.kv_down)

    def forward(self, x: torch.Tensor, rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
        B, S, _ = x.shape
        lat = self.latent(x)
        c, k_rope = lat[..., : self.kv_lora_rank], lat[..., self.kv_lora_rank:]
        c = self.kv_norm(c)
        k = F_.linear(c, self.k_up).view(B, S, self.h, self.d)
        v = F_.linear(c, self.v_up).view(B, S, self.h, self.d)
        qh = F_.linear(x, self.q_down) if self.q_down is not None else x
        q = F_.linear(qh, self.q_up).view(B, S, self.h, self.d + self.rope_dim)
        q_nope, q_rope = q[..., : self.d], q[..., self.d:]
        if self.rope_dim:
            if rope is not None:
                cos, sin = rope
                rot = lambda t: torch.cat([t[..., : self.rope_dim // 2] * cos - t[..., self.rope_dim // 2:] * sin,
                                           t[..., self.rope_dim // 2:] * cos + t[..., : self.rope_dim // 2] * sin], -1)
                q_rope, k_rope = rot(q_rope), rot(k_rope[:, :, None, :])[:, :, 0]
            k = torch.cat([k, k_rope[:, :, None, :].expand(B, S, self.h, self.rope_dim)], -1)
            q_nope = torch.cat([q_nope, q_rope], -1)
        o = masked_attention(q_nope.transpose(1, 2), k.transpose(1, 2),
                             F.pad(v, (0, k.shape[-1] - v.shape[-1])).transpose(1, 2),
                             causal_mask(S, S, x.device), scale=(self.d + self.rope_dim) ** -0.5)
        return F_.linear(o.transpose(1, 2)[..., : self.d].reshape(B, S, self.h * self.d), self.o_proj)
