"""Block-sparse, hierarchical and hybrid attention variants (reference model/core/attention.py:
``YvCirculantAttention`` :1198, ``YvDynamicH2OAttention`` :3320, ``YvHISAAttention`` :4268, ``YvMixtureBlockAttention``
:4771, ``YvHydraHeadAttention`` :5819, ``YvLatentCondensedAttention`` :6010, ``YvAttentionMaskFactory`` :6165;
``YvEGMLA`` core/eg_mla.py:43; ``YvTokenSparseAttention`` core/token_sparse_attn.py:57; ``YvMemoryCrossAttention``
core/memory_attention.py:30).

Every block-selecting variant is written as "score block representatives, build a boolean [S, T] visibility mask,
run the shared masked-softmax core": the selection rule is the variant, the attention arithmetic is common."""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as F_
from .attention_variants import _ProjectedAttention, causal_mask, masked_attention


class YvAttentionMaskFactory:
    """Boolean visibility masks [S, T] (True = visible), bottom-right aligned when T > S."""

    @staticmethod
    def causal(S: int, T: Optional[int] = None, device=None) -> torch.Tensor:
        return causal_mask(S, T or S, device)

    @staticmethod
    def sliding_window(S: int, window: int, T: Optional[int] = None, n_sink: int = 0, device=None) -> torch.Tensor:
        T = T or S
        i = torch.arange(S, device=device)[:, None] + (T - S)
        j = torch.arange(T, device=device)[None, :]
        return (j <= i) & ((i - j < window) | (j < n_sink))

    @staticmethod
    def prefix_lm(S: int, prefix: int, device=None) -> torch.Tensor:
        m = causal_mask(S, S, device)
        m[:, :prefix] = True
        return m

    @staticmethod
    def block_diagonal(seq_ids: torch.Tensor, causal: bool = True) -> torch.Tensor:
        """Packed sequences: token i sees token j only inside the same sequence id. seq_ids [S]."""
        m = seq_ids[:, None] == seq_ids[None, :]
        return m & causal_mask(len(seq_ids), len(seq_ids), seq_ids.device) if causal else m

    @staticmethod
    def padding(lengths: torch.Tensor, T: int) -> torch.Tensor:
        """[B, 1, 1, T] key-padding mask from per-sample lengths."""
        return (torch.arange(T, device=lengths.device)[None, :] < lengths[:, None])[:, None, None, :]

    @staticmethod
    def dilated(S: int, window: int, dilation: int, device=None) -> torch.Tensor:
        i = torch.arange(S, device=device)[:, None]
        j = torch.arange(S, device=device)[None, :]
        return (j <= i) & ((i - j) % dilation == 0) & ((i - j) < window * dilation)


def _block_means(k: torch.Tensor, bs: int) -> torch.Tensor:
    """k [B,H,T,D] -> per-block mean keys [B,H,ceil(T/bs),D] (the last block averages its real tokens)."""
    B, H, T, D = k.shape
    nb = (T + bs - 1) // bs
    pad = nb * bs - T
    kp = F.pad(k.float(), (0, 0, 0, pad)).view(B, H, nb, bs, D).sum(3)
    cnt = torch.full((nb,), float(bs), device=k.device)
    if pad:
        cnt[-1] = bs - pad
    return kp / cnt[None, None, :, None]


def _expand_block_mask(sel: torch.Tensor, bs: int, S: int, T: int) -> torch.Tensor:
    """sel [B,H,S,nb] bool -> [B,H,S,T] token mask."""
    return sel.repeat_interleave(bs, -1)[..., :T]


class YvMixtureBlockAttention(_ProjectedAttention):
    """MoBA: each query attends to its own block (causally) plus the ``top_k`` earlier blocks whose mean key scores
    highest against it."""

    def __init__(self, hidden: int, n_head: int, block_size: int = 64, top_k: int = 3, n_kv_head: Optional[int] = None):
        super().__init__(hidden, n_head, n_kv_head)
        self.bs, self.top_k = block_size, top_k

    def select(self, q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
        B, H, S, D = q.shape
        T = k.shape[2]
        if k.shape[1] != H:
            k = k.repeat_interleave(H // k.shape[1], 1)
        rep = _block_means(k, self.bs)                                        # [B,H,nb,D]
        nb = rep.shape[2]
        sc = torch.matmul(q.float(), rep.transpose(-1, -2))                   # [B,H,S,nb]
        qblk = (torch.arange(S, device=q.device) + (T - S)) // self.bs
        blk = torch.arange(nb, device=q.device)
        earlier = blk[None, :] < qblk[:, None]                                # strictly earlier blocks only
        sc = sc.masked_fill(~earlier, float("-inf"))
        kk = min(self.top_k, nb)
        idx = sc.topk(kk, -1).indices
        sel = torch.zeros(B, H, S, nb, dtype=torch.bool, device=q.device).scatter_(-1, idx, True) & earlier
        sel |= (blk[None, :] == qblk[:, None])
        return sel

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q, k, v = self.qkv(x)
        S = T = x.shape[1]
        mask = _expand_block_mask(self.select(q, k), self.bs, S, T) & causal_mask(S, T, x.device)
        return self.out(masked_attention(q, k, v, mask=mask))


class YvTokenSparseAttention(_ProjectedAttention):
    """Block selection by cumulative score mass: blocks are ranked by the softmax of representative scores and the
    smallest prefix reaching ``target`` of the mass is kept (at most ``max_blocks``); the query's own block always."""

    def __init__(self, hidden: int, n_head: int, block_size: int = 64, target: float = 0.8, max_blocks: int = 8,
                 select_rank: int = 0):
        super().__init__(hidden, n_head)
        self.bs, self.target, self.max_blocks = block_size, target, max_blocks
        self.rank = select_rank or self.d

    def select(self, q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
        B, H, S, D = q.shape
        T = k.shape[2]
        r = self.rank
        rep = _block_means(k[..., :r], self.bs)
        nb = rep.shape[2]
        sc = torch.matmul(q[..., :r].float(), rep.transpose(-1, -2)) * r ** -0.5
        qblk = (torch.arange(S, device=q.device) + (T - S)) // self.bs
        blk = torch.arange(nb, device=q.device)
        # Only STRICTLY EARLIER blocks are ranked: the mean key of the query's own block contains tokens after the
        # query, and letting it into the softmax would make the choice of earlier blocks (hence the output of this
        # token) depend on the future.  The own block is kept unconditionally and attended under the causal mask.
        earlier = blk[None, :] < qblk[:, None]
        p = torch.nan_to_num(torch.softmax(sc.masked_fill(~earlier, float("-inf")), -1), nan=0.0)
        ps, order = p.sort(-1, descending=True)
        before = ps.cumsum(-1) - ps                                           # mass accumulated before each block
        keep_sorted = (before < self.target) & (torch.arange(nb, device=q.device) < self.max_blocks)
        sel = torch.zeros_like(p, dtype=torch.bool).scatter_(-1, order, keep_sorted) & earlier
        sel |= (blk[None, :] == qblk[:, None])
        return sel

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q, k, v = self.qkv(x)
        S = T = x.shape[1]
        mask = _expand_block_mask(self.select(q, k), self.bs, S, T) & causal_mask(S, T, x.device)
        return self.out(masked_attention(q, k, v, mask=mask))


class YvHISAAttention(_ProjectedAttention):
    """Three-level selection: super-blocks (``sb`` blocks each) are ranked first, then blocks inside the chosen
    super-blocks, then tokens inside the chosen blocks attend exactly: O(N sqrt N) scored pairs."""

    def __init__(self, hidden: int, n_head: int, block_size: int = 32, super_size: int = 4, top_super: int = 2,
                 top_blocks: int = 4):
        super().__init__(hidden, n_head)
        self.bs, self.sb, self.top_super, self.top_blocks = block_size, super_size, top_super, top_blocks

    def select(self, q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
        B, H, S, D = q.shape
        T = k.shape[2]
        rep = _block_means(k, self.bs)                                        # [B,H,nb,D]
        nb = rep.shape[2]
        srep = _block_means(rep, self.sb)                                     # [B,H,ns,D]
        ns = srep.shape[2]
        qblk = (torch.arange(S, device=q.device) + (T - S)) // self.bs
        blk = torch.arange(nb, device=q.device)
        sblk = torch.arange(ns, device=q.device)
        # Ranking uses representatives made of PAST tokens only: super-blocks strictly before the query's own, and
        # blocks strictly before its own block.  The own super-block and the own block are always kept (the causal
        # mask handles the tokens inside), so a later token can never change what an earlier one selects.
        s_earlier = sblk[None, :] < (qblk // self.sb)[:, None]
        ssc = torch.matmul(q.float(), srep.transpose(-1, -2)).masked_fill(~s_earlier, float("-inf"))
        sidx = ssc.topk(min(self.top_super, ns), -1).indices
        ssel = torch.zeros(B, H, S, ns, dtype=torch.bool, device=q.device).scatter_(-1, sidx, True) & s_earlier
        ssel |= (sblk[None, :] == (qblk // self.sb)[:, None])
        b_earlier = (blk[None, :] < qblk[:, None]) & ssel.repeat_interleave(self.sb, -1)[..., :nb]
        bsc = torch.matmul(q.float(), rep.transpose(-1, -2)).masked_fill(~b_earlier, float("-inf"))
        bidx = bsc.topk(min(self.top_blocks, nb), -1).indices
        bsel = torch.zeros(B, H, S, nb, dtype=torch.bool, device=q.device).scatter_(-1, bidx, True) & b_earlier
        bsel |= (blk[None, :] == qblk[:, None])
        return bsel

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q, k, v = self.qkv(x)
        S = T = x.shape[1]
        mask = _expand_block_mask(self.select(q, k), self.bs, S, T) & causal_mask(S, T, x.device)
        return self.out(masked_attention(q, k, v, mask=mask))


class YvCirculantAttention(nn.Module):
    """Token mixing by a learned, input-conditioned circular convolution evaluated with FFTs (O(N log N)): per head,
    the softmax over positions of a pooled query-key product gives the first column of a circulant mixing matrix,
    which multiplies the values in the frequency domain.  ``causal`` zero-pads to 2N so that the convolution does not
    wrap around (with a FIXED kernel, output t reads values at positions <= t only).  The kernel itself is pooled over
    the whole sequence, so the layer is an encoder-style mixer and NOT autoregressive: it is not offered as a block of
    the causal language model."""

    def __init__(self, hidden: int, n_head: int, causal: bool = True):
        super().__init__()
        self.h, self.d, self.causal = n_head, hidden // n_head, causal
        self.qk = nn.Parameter(torch.empty(2 * hidden, hidden).normal_(std=0.02))
        self.v = nn.Parameter(torch.empty(hidden, hidden).normal_(std=0.02))
        self.o = nn.Parameter(torch.empty(hidden, hidden).normal_(std=0.02))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, H = x.shape
        q, k = F_.linear(x, self.qk).view(B, S, 2, self.h, self.d).unbind(2)
        v = F_.linear(x, self.v).view(B, S, self.h, self.d).float()
        # first column of the circulant: c[t] = softmax_t( <mean_s q_s, k_t> ) taken at lag t
        c = torch.softmax(torch.einsum("bhd,bthd->bth", q.float().mean(1), k.float()) * self.d ** -0.5, 1)   # [B,S,h]
        n = 2 * S if self.causal else S
        y = torch.fft.irfft(torch.fft.rfft(c, n=n, dim=1)[..., None] * torch.fft.rfft(v, n=n, dim=1), n=n, dim=1)[:, :S]
        return F_.linear(y.reshape(B, S, H).to(x.dtype), self.o)


class YvHydraHeadAttention(_ProjectedAttention):
    """Head-level hybrid: the first ``n_linear`` heads run causal linear attention with an ELU+1 feature map (O(N)),
    the rest run softmax attention; outputs are concatenated head-wise before the output projection."""

    def __init__(self, hidden: int, n_head: int, la_ratio: float = 0.5):
        super().__init__(hidden, n_head)
        self.n_linear = int(round(n_head * la_ratio))

    @staticmethod
    def linear_causal(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        fq, fk = F.elu(q.float()) + 1, F.elu(k.float()) + 1
        kv = torch.einsum("bhtd,bhte->bhtde", fk, v.float()).cumsum(2)
        z = fk.cumsum(2)
        num = torch.einsum("bhtd,bhtde->bhte", fq, kv)
        den = torch.einsum("bhtd,bhtd->bht", fq, z).clamp_min(1e-6)
        return (num / den[..., None]).to(q.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q, k, v = self.qkv(x)
        n, S = self.n_linear, x.shape[1]
        parts = []
        if n:
            parts.append(self.linear_causal(q[:, :n], k[:, :n], v[:, :n]))
        if n < self.h:
            parts.append(masked_attention(q[:, n:], k[:, n:], v[:, n:], mask=causal_mask(S, S, x.device)))
        return self.out(torch.cat(parts, 1))


class YvLatentCondensedAttention(_ProjectedAttention):
    """Keys and values older than ``keep_recent`` are condensed ``ratio``:1 along the sequence by a learned weighted
    pooling; queries attend to [condensed past ; recent tokens]."""

    def __init__(self, hidden: int, n_head: int, ratio: int = 4, keep_recent: int = 64):
        super().__init__(hidden, n_head)
        self.ratio, self.keep = ratio, keep_recent
        self.pool = nn.Parameter(torch.zeros(n_head, ratio))

    def condense(self, t: torch.Tensor) -> torch.Tensor:
        B, H, T, D = t.shape
        n = T // self.ratio
        w = torch.softmax(self.pool.float(), -1)                              # [H, ratio]
        return torch.einsum("bhnrd,hr->bhnd", t[:, :, : n * self.ratio].float().view(B, H, n, self.ratio, D), w).to(t.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q, k, v = self.qkv(x)
        S = x.shape[1]
        old = max(0, S - self.keep) // self.ratio * self.ratio
        if old == 0:
            return self.out(masked_attention(q, k, v, mask=causal_mask(S, S, x.device)))
        kc, vc = self.condense(k[:, :, :old]), self.condense(v[:, :, :old])
        n = kc.shape[2]
        i = torch.arange(S, device=x.device)[:, None]
        # a condensed slot is visible once its last source token is in the past; recent tokens causally
        m_old = (torch.arange(n, device=x.device)[None, :] + 1) * self.ratio - 1 <= i
        j = torch.arange(old, S, device=x.device)[None, :]
        m = torch.cat([m_old, j <= i], 1)
        # queries inside the condensed region still need their own neighbourhood: give them exact causal attention
        exact = masked_attention(q[:, :, :old], k[:, :, :old], v[:, :, :old], mask=causal_mask(old, old, x.device))
        mixed = masked_attention(q[:, :, old:], torch.cat([kc, k[:, :, old:]], 2), torch.cat([vc, v[:, :, old:]], 2),
                                 mask=m[old:])
        return self.out(torch.cat([exact, mixed], 2))


class YvDynamicH2OAttention(_ProjectedAttention):
    """Heavy-hitter cache with three tiers chosen from accumulated attention mass: the ``recent`` window is kept
    exactly, the ``heavy`` highest-mass older tokens are kept exactly, and the remainder is archived as one mean
    key/value per ``archive_block`` tokens.  ``budget_ratio`` scales ``heavy`` with sequence length."""

    def __init__(self, hidden: int, n_head: int, recent: int = 64, heavy: int = 64, archive_block: int = 16,
                 budget_ratio: float = 0.0):
        super().__init__(hidden, n_head)
        self.recent, self.heavy, self.ab, self.ratio = recent, heavy, archive_block, budget_ratio

    def compress(self, k: torch.Tensor, v: torch.Tensor, mass: torch.Tensor) -> Dict[str, torch.Tensor]:
        """k, v [H, T, D]; mass [H, T] -> tiers per head."""
        H, T, D = k.shape
        heavy = max(self.heavy, int(self.ratio * T))
        old = max(0, T - self.recent)
        n_h = min(heavy, old)
        out = {"recent_k": k[:, old:], "recent_v": v[:, old:]}
        if old == 0:
            return out
        idx = mass[:, :old].topk(n_h, -1).indices.sort(-1).values if n_h else mass.new_zeros(H, 0, dtype=torch.long)
        out["heavy_idx"] = idx
        out["heavy_k"] = torch.gather(k, 1, idx[..., None].expand(-1, -1, D))
        out["heavy_v"] = torch.gather(v, 1, idx[..., None].expand(-1, -1, D))
        rest = torch.ones(H, old, dtype=torch.bool, device=k.device).scatter_(1, idx, False)
        nb = (old + self.ab - 1) // self.ab
        pad = nb * self.ab - old
        w = F.pad(rest.float(), (0, pad)).view(H, nb, self.ab)
        kk = F.pad(k[:, :old].float(), (0, 0, 0, pad)).view(H, nb, self.ab, D)
        vv = F.pad(v[:, :old].float(), (0, 0, 0, pad)).view(H, nb, self.ab, D)
        cnt = w.sum(-1).clamp_min(1)
        out["archive_k"] = ((kk * w[..., None]).sum(2) / cnt[..., None]).to(k.dtype)
        out["archive_v"] = ((vv * w[..., None]).sum(2) / cnt[..., None]).to(v.dtype)
        out["archive_count"] = w.sum(-1)
        return out

    def decode_step(self, q: torch.Tensor, tiers: Dict[str, torch.Tensor]) -> torch.Tensor:
        """q [H, 1, D] against the tiers; an archived slot of n tokens is weighted by log n (it stands for n keys)."""
        ks, vs, bias = [tiers["recent_k"]], [tiers["recent_v"]], [torch.zeros(q.shape[0], tiers["recent_k"].shape[1], device=q.device)]
        if "heavy_k" in tiers:
            ks += [tiers["heavy_k"], tiers["archive_k"]]
            vs += [tiers["heavy_v"], tiers["archive_v"]]
            bias += [torch.zeros(q.shape[0], tiers["heavy_k"].shape[1], device=q.device),
                     torch.log(tiers["archive_count"].clamp_min(1e-9))]
        K, V, Bz = torch.cat(ks, 1), torch.cat(vs, 1), torch.cat(bias, 1)
        s = torch.einsum("hqd,htd->hqt", q.float(), K.float()) * q.shape[-1] ** -0.5 + Bz[:, None, :]
        return torch.einsum("hqt,htd->hqd", torch.softmax(s, -1), V.float()).to(q.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Training / prefill: exact causal attention (the tiers only bound the decode-time cache)."""
        q, k, v = self.qkv(x)
        S = x.shape[1]
        return self.out(masked_attention(q, k, v, mask=causal_mask(S, S, x.device)))


class YvEGMLA(nn.Module):
    """Embedding-gated latent attention: keys and values are reconstructed from a rank-``kv_lora_rank`` latent (the
    only thing cached); a sigmoid gate computed from the token embedding scales the latent per channel before the
    up-projections.  Returns (output, latent) so that a cache stores ``latent`` alone."""

    def __init__(self, hidden: int, n_head: int, kv_lora_rank: int, q_lora_rank: int = 0):
        super().__init__()
        self.h, self.d, self.r = n_head, hidden // n_head, kv_lora_rank
        w = lambda o, i: nn.Parameter(torch.empty(o, i).normal_(std=0.02))
        # one fused down-projection gives the latent and its gate
        self.kv_down_gate = w(2 * kv_lora_rank, hidden)
        self.kv_up = w(2 * hidden, kv_lora_rank)
        if q_lora_rank:
            self.q_down, self.q_up = w(q_lora_rank, hidden), w(hidden, q_lora_rank)
        else:
            self.q_down, self.q_up = None, w(hidden, hidden)
        self.o = w(hidden, hidden)

    def latent(self, x: torch.Tensor) -> torch.Tensor:
        c, g = F_.linear(x, self.kv_down_gate).chunk(2, -1)
        return c * torch.sigmoid(g.float()).to(c.dtype)

    def forward(self, x: torch.Tensor, past_latent: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        B, S, H = x.shape
        lat = self.latent(x)
        if past_latent is not None:
            lat = torch.cat([past_latent, lat], 1)
        T = lat.shape[1]
        k, v = F_.linear(lat, self.kv_up).view(B, T, 2, self.h, self.d).unbind(2)
        qh = F_.linear(x, self.q_down) if self.q_down is not None else x
        q = F_.linear(qh, self.q_up).view(B, S, self.h, self.d)
        o = masked_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), mask=causal_mask(S, T, x.device))
        return F_.linear(o.transpose(1, 2).reshape(B, S, H), self.o), lat

    def cache_reduction(self) -> float:
        return 1.0 - self.r / (2.0 * self.h * self.d)


class YvMemoryCrossAttention(nn.Module):
    """Cross attention from the token stream to an external memory bank [B, M, Hm] with a learned fusion gate
    (reference YvMemoryFusionGate): out = x + sigmoid(W[x ; read]) * read."""

    def __init__(self, hidden: int, mem_dim: int, n_head: int = 8):
        super().__init__()
        self.h, self.d = n_head, hidden // n_head
        w = lambda o, i: nn.Parameter(torch.empty(o, i).normal_(std=0.02))
        self.q, self.kv, self.o, self.gate = w(hidden, hidden), w(2 * hidden, mem_dim), w(hidden, hidden), w(hidden, 2 * hidden)

    def forward(self, x: torch.Tensor, memory: torch.Tensor, memory_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, S, H = x.shape
        M = memory.shape[1]
        q = F_.linear(x, self.q).view(B, S, self.h, self.d).transpose(1, 2)
        k, v = F_.linear(memory.to(x.dtype), self.kv).view(B, M, 2, self.h, self.d).unbind(2)
        mask = memory_mask[:, None, None, :] if memory_mask is not None else None
        r = masked_attention(q, k.transpose(1, 2), v.transpose(1, 2), mask=mask)
        r = F_.linear(r.transpose(1, 2).reshape(B, S, H), self.o)
        g = torch.sigmoid(F_.linear(torch.cat([x, r], -1), self.gate).float()).to(x.dtype)
        return x + g * r
