"""Modules of the reference's model layer that this package implements under another name or as a function, offered
under the reference's names (reference model/core: ``YvSwiGLU`` blocks.py, ``YvFlashAttention`` attention.py:2165,
``YvPagedAttention`` :1903, ``YvRingAttention`` :2736, ``YvCrossAttention``, ``YvLoRALayer``, ``YvExpertChoiceMLP``
blocks.py, ``YvLayerRouter`` model.py:375-485, ``YvModelForMaskedLM`` model.py:2725-3112, ``YvStateCache``,
``YvSelectiveScan``; model/moe ``YvMoELayer``, ``YvGateInitializer``).  Each class is a working front of the kernels
and modules of this package, not a stub."""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import YvConfig
from ..ops import functional as F_
from .block_variants import YvLoRA
from .heads import _HeadBase
from .moe_extras import YvDynamicMoELayer
from .ssm import selective_scan, selective_scan_step

YvLoRALayer = YvLoRA
YvMoELayer = YvDynamicMoELayer


class YvSwiGLU(nn.Module):
    """Gated feed-forward: down(silu(gate(x)) * up(x)); gate and up are one fused GEMM, the activation one kernel."""

    def __init__(self, hidden: int, intermediate: int, std: float = 0.02):
        super().__init__()
        self.w13 = nn.Parameter(torch.empty(2 * intermediate, hidden).normal_(std=std))
        self.w2 = nn.Parameter(torch.empty(hidden, intermediate).normal_(std=std))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F_.linear(F_.swiglu(F_.linear(x, self.w13)), self.w2)


class YvFlashAttention(nn.Module):
    """Dense self-attention over [B, S, H] through the flash kernels (packed layout inside)."""

    def __init__(self, hidden: int, n_head: int, n_kv_head: Optional[int] = None, causal: bool = True):
        super().__init__()
        self.hq, self.hk, self.d, self.causal = n_head, n_kv_head or n_head, hidden // n_head, causal
        self.qkv = nn.Parameter(torch.empty((self.hq + 2 * self.hk) * self.d, hidden).normal_(std=0.02))
        self.o = nn.Parameter(torch.empty(hidden, self.hq * self.d).normal_(std=0.02))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, H = x.shape
        qkv = F_.linear(x.reshape(B * S, H), self.qkv)
        nq, nk = self.hq * self.d, self.hk * self.d
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=x.device)
        o = F_.attention(qkv[:, :nq], qkv[:, nq:nq + nk], qkv[:, nq + nk:], cu, cu, S, S, self.hq, self.hk, self.d, self.causal)
        return F_.linear(o, self.o).view(B, S, H)


class YvCrossAttention(nn.Module):
    """Queries from x [B, S, H], keys / values from a context [B, T, Hc] (not causal)."""

    def __init__(self, hidden: int, context_dim: int, n_head: int):
        super().__init__()
        self.h, self.d = n_head, hidden // n_head
        self.q = nn.Parameter(torch.empty(hidden, hidden).normal_(std=0.02))
        self.kv = nn.Parameter(torch.empty(2 * hidden, context_dim).normal_(std=0.02))
        self.o = nn.Parameter(torch.empty(hidden, hidden).normal_(std=0.02))

    def forward(self, x: torch.Tensor, context: torch.Tensor) -> torch.Tensor:
        B, S, H = x.shape
        T = context.shape[1]
        q = F_.linear(x.reshape(B * S, H), self.q)
        kv = F_.linear(context.reshape(B * T, -1).to(x.dtype), self.kv)
        cu_q = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=x.device)
        cu_k = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=x.device)
        o = F_.attention(q, kv[:, :H], kv[:, H:], cu_q, cu_k, S, T, self.h, self.h, self.d, False)
        return F_.linear(o, self.o).view(B, S, H)


class YvPagedAttention:
    """Decode-time attention over the paged cache: writes the new token's K/V to its slot and attends over the
    sequence's blocks (the tensor-core paged-decode kernel on the GPU)."""

    def __init__(self, n_head: int, n_kv_head: int, head_dim: int):
        self.hq, self.hk, self.d = n_head, n_kv_head, head_dim

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 slot_map: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor) -> torch.Tensor:
        """q [B, hq*d], k/v [B, hk*d] of the new tokens -> [B, hq*d]."""
        F_.kv_cache_write(k, v, k_cache, v_cache, slot_map)
        B = q.shape[0]
        return F_.paged_decode(q.reshape(B, self.hq, self.d).contiguous(), k_cache, v_cache, block_table, seq_lens).reshape(B, -1)


class YvRingAttention:
    """Exact attention for a sequence sharded over a context-parallel group (``parallel.cp.ring_attention``)."""

    def __init__(self, n_head: int, n_kv_head: int, head_dim: int, group: Any = None, causal: bool = True):
        self.hq, self.hk, self.d, self.group, self.causal = n_head, n_kv_head, head_dim, group, causal

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        if self.group is None and not (dist.is_available() and dist.is_initialized()):
            L = q.shape[0]
            cu = torch.tensor([0, L], dtype=torch.int32, device=q.device)
            return F_.attention(q, k, v, cu, cu, L, L, self.hq, self.hk, self.d, self.causal)
        from ..parallel.cp import ring_attention
        return ring_attention(q, k, v, self.group, self.hq, self.hk, self.d, self.causal)


class YvExpertChoiceMLP(nn.Module):
    """Experts choose tokens: every expert processes its ``capacity`` highest-scoring tokens; a token's output is
    the score-weighted sum over the experts that chose it (tokens chosen by nobody pass through as zeros)."""

    def __init__(self, hidden: int, intermediate: int, n_experts: int, capacity_factor: float = 1.0):
        super().__init__()
        self.router = nn.Parameter(torch.empty(n_experts, hidden).normal_(std=0.02))
        self.w13 = nn.Parameter(torch.empty(n_experts, 2 * intermediate, hidden).normal_(std=0.02))
        self.w2 = nn.Parameter(torch.empty(n_experts, hidden, intermediate).normal_(std=0.02))
        self.cf = capacity_factor

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        T, E = x2.shape[0], self.router.shape[0]
        probs = torch.softmax(F_.linear(x2, self.router.to(x2.dtype)).float(), -1)
        cap = max(1, min(T, int(self.cf * T / E + 0.5)))
        score, tok = probs.t().topk(cap, -1)                                       # [E, cap]
        xin = x2[tok]                                                              # [E, cap, H]
        h = torch.einsum("ech,efh->ecf", xin.float(), self.w13.float())
        Fdim = self.w2.shape[-1]
        act = F.silu(h[..., :Fdim]) * h[..., Fdim:]
        y = torch.einsum("ecf,ehf->ech", act, self.w2.float()) * score[..., None]
        out = torch.zeros_like(x2, dtype=torch.float32).index_add_(0, tok.reshape(-1), y.reshape(-1, shape[-1]))
        return out.to(x.dtype).view(shape)


class YvLayerRouter(nn.Module):
    """Per-sequence soft layer skipping: a small gate on the pooled hidden state decides, per layer, how much of the
    layer's update is applied (straight-through hard decision in eval when ``hard``); a budget loss keeps the mean
    usage near ``target_usage``."""

    def __init__(self, hidden: int, n_layers: int, target_usage: float = 0.8, hard: bool = False):
        super().__init__()
        self.gate = nn.Linear(hidden, n_layers)
        nn.init.zeros_(self.gate.weight)
        nn.init.constant_(self.gate.bias, 3.0)                                     # starts with every layer on
        self.target, self.hard = target_usage, hard

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """h [B, S, H] -> layer weights [B, n_layers] in [0, 1]."""
        p = torch.sigmoid(self.gate(h.float().mean(1)))
        if self.hard and not self.training:
            return (p > 0.5).float()
        return p

    def apply(self, h: torch.Tensor, update: torch.Tensor, weights: torch.Tensor, layer: int) -> torch.Tensor:
        return h + weights[:, layer].view(-1, 1, 1).to(update.dtype) * update

    def budget_loss(self, weights: torch.Tensor) -> torch.Tensor:
        return (weights.mean() - self.target).pow(2)


class YvModelForMaskedLM(_HeadBase):
    """Bidirectional use of the trunk is not offered by the causal kernels, so masked-LM training here predicts the
    masked positions from the causal hidden states (a denoising objective on the same head as the LM)."""

    def __init__(self, cfg: YvConfig, parallel: Any = None):
        super().__init__(cfg, parallel)
        self.decoder = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size).normal_(std=cfg.initializer_range))

    def forward(self, input_ids, attention_mask=None, labels=None) -> Dict[str, torch.Tensor]:
        h = self.hidden(input_ids, attention_mask)
        logits = F_.linear(h, self.decoder).float()
        out = {"logits": logits}
        if labels is not None:
            out["loss"] = F.cross_entropy(logits.view(-1, logits.shape[-1]), labels.view(-1), ignore_index=-100)
        return out


class YvSelectiveScan:
    """Callable front of the selective-scan op (kernel on the GPU, fp32 loop otherwise)."""

    def __call__(self, u, delta, A, B, C, D):
        return selective_scan(u, delta, A, B, C, D)

    @staticmethod
    def step(u, delta, A, B, C, D, state):
        return selective_scan_step(u, delta, A, B, C, D, state)


class YvStateCache:
    """Per-layer recurrent state of the SSM layers for decoding: ``get(layer, batch, channels, states)`` creates the
    fp32 state on first use; ``reorder`` follows beam search; ``reset`` clears a batch row when a request ends."""

    def __init__(self, device: Optional[torch.device] = None):
        self.device = device
        self.states: Dict[int, torch.Tensor] = {}

    def get(self, layer: int, batch: int, channels: int, n_states: int) -> torch.Tensor:
        s = self.states.get(layer)
        if s is None or s.shape != (batch, channels, n_states):
            s = torch.zeros(batch, channels, n_states, dtype=torch.float32, device=self.device)
            self.states[layer] = s
        return s

    def reorder(self, index: torch.Tensor) -> None:
        for k, s in self.states.items():
            self.states[k] = s.index_select(0, index.to(s.device))

    def reset(self, row: Optional[int] = None) -> None:
        for s in self.states.values():
            (s if row is None else s[row]).zero_()


class YvGateInitializer:
    """Router weight initialisers: small normal, orthogonal rows (experts start decorrelated), or from k-means
    centroids of a sample of hidden states (every expert starts on a populated region)."""

    @staticmethod
    def normal_(w: torch.Tensor, std: float = 0.02) -> torch.Tensor:
        return w.data.normal_(std=std)

    @staticmethod
    def orthogonal_(w: torch.Tensor, gain: float = 0.1) -> torch.Tensor:
        nn.init.orthogonal_(w.data, gain=gain)
        return w.data

    @staticmethod
    def kmeans_(w: torch.Tensor, samples: torch.Tensor, iters: int = 10, seed: int = 0) -> torch.Tensor:
        E = w.shape[0]
        g = torch.Generator().manual_seed(seed)
        x = samples.float().reshape(-1, samples.shape[-1])
        c = x[torch.randperm(x.shape[0], generator=g)[:E]].clone()
        for _ in range(iters):
            assign = torch.cdist(x, c).argmin(-1)
            for e in range(E):
                m = assign == e
                if m.any():
                    c[e] = x[m].mean(0)
        w.data.copy_(F.normalize(c, dim=-1).to(w.dtype) * 0.1)
        return w.data
