"""Fused projections and latent-space decoding for the gated low-rank attention (reference
opss/infer/fused_mla.py:43-250, ``PiscesLxFusedMLAProjector``).

``YvAttention`` with ``use_mla`` keeps its projections as separate tensors (the checkpoint layout) and concatenates
them at every call.  For serving, ``PiscesLxFusedMLAProjector.from_attention`` builds the fused weights once:

  * one GEMM ``x -> [latent | gate | q]`` (a low-rank query pair is merged into a single matrix);
  * one GEMM ``latent -> [k | v | k_rope]``.

It goes further than the reference's fusion of GEMMs: ``decode_absorbed`` attends in the LATENT space.  Because
k_h = W_k[h] c and v_h = W_v[h] c for the cached latent c, the key projection can be absorbed into the query
(q_h . k_h = (W_k[h]^T q_h) . c) and the value projection applied after the weighted sum
(sum_s p_s v_{h,s} = W_v[h] sum_s p_s c_s), so a decode step reads ``kv_lora_rank`` (+ ``rope_dim``) numbers per cached
token instead of ``2 x n_kv_head x head_dim`` and never materialises keys or values.  With the decoupled rotary slice
the score has a second term q_rope . rot(k_rope), where k_rope is one vector per token shared by the heads; the cache
stores it already rotated.  The bytes read per cached token shrink by 2 hk d / (r + rope), which is what bounds decode
on HBM."""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F_
from ..ops import reference as ref


class PiscesLxFusedMLAProjector(nn.Module):
    def __init__(self, hidden_size: int, n_head: int, n_kv_head: int, head_dim: int, kv_lora_rank: int,
                 mla_rope_dim: int = 0, dtype: torch.dtype = torch.float32, device: Any = None):
        super().__init__()
        assert n_head % n_kv_head == 0
        self.hidden_size, self.n_head, self.n_kv_head, self.head_dim = hidden_size, n_head, n_kv_head, head_dim
        self.kv_lora_rank, self.mla_rope_dim = kv_lora_rank, min(int(mla_rope_dim), head_dim)
        r, nq, nk = kv_lora_rank, n_head * head_dim, n_kv_head * head_dim
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device).normal_(std=0.02))
        self.in_fused = mk(2 * r + nq, hidden_size)                      # rows: latent | gate | q
        self.kv_decompress_fused = mk(2 * nk + self.mla_rope_dim, r)     # rows: k | v | k_rope
        self.scale = 1.0 / math.sqrt(head_dim)

    @property
    def enhanced(self) -> bool:
        return self.mla_rope_dim > 0

    # -- construction from the separate tensors ----------------------------------------------------------------------------
    @classmethod
    def from_attention(cls, att: nn.Module) -> "PiscesLxFusedMLAProjector":
        """From a ``YvAttention`` built with ``use_mla`` (its ``kv_compress``, ``embedding_gate``, ``k_decompress``,
        ``v_decompress``, ``q_proj`` or ``q_compress`` + ``q_decompress``, and ``rope_decompress`` when enhanced)."""
        if not getattr(att, "use_mla", False):
            raise ValueError("the attention module was not built with use_mla")
        q = att.q_proj if att.q_proj is not None else att.q_decompress.float() @ att.q_compress.float()
        rope = att.rope_decompress if getattr(att, "enhanced", False) else None
        return cls.from_separate(att.kv_compress, att.embedding_gate, att.k_decompress, att.v_decompress, q, rope,
                                 att.hq, att.hk, att.d)

    @classmethod
    def from_separate(cls, kv_compress: torch.Tensor, embedding_gate: torch.Tensor, k_decompress: torch.Tensor,
                      v_decompress: torch.Tensor, q_weight: torch.Tensor, rope_decompress: Optional[torch.Tensor],
                      n_head: int, n_kv_head: int, head_dim: int) -> "PiscesLxFusedMLAProjector":
        w = lambda t: (t.weight if isinstance(t, nn.Linear) else t).detach()
        kvc, eg, kd, vd, qw = w(kv_compress), w(embedding_gate), w(k_decompress), w(v_decompress), w(q_weight)
        rd = w(rope_decompress) if rope_decompress is not None else None
        p = cls(kvc.shape[1], n_head, n_kv_head, head_dim, kvc.shape[0], rd.shape[0] if rd is not None else 0, kvc.dtype, kvc.device)
        with torch.no_grad():
            p.in_fused.copy_(torch.cat([kvc, eg, qw.to(kvc.dtype)], 0))
            p.kv_decompress_fused.copy_(torch.cat([kd, vd] + ([rd] if rd is not None else []), 0))
        return p

    # -- projections -------------------------------------------------------------------------------------------------------
    def compress(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """x [T, H] -> (q [T, hq, d], latent [T, r]) with one GEMM."""
        r = self.kv_lora_rank
        y = F_.linear(x, self.in_fused)
        latent = y[:, :r] * torch.sigmoid(y[:, r:2 * r].float()).to(y.dtype)
        return y[:, 2 * r:].reshape(-1, self.n_head, self.head_dim), latent

    def decompress_kv(self, latent: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
        """latent [T, r] -> (k [T, hk, d], v [T, hk, d], k_rope [T, rope] or None) with one GEMM; with the rotary slice
        k already carries it in its first ``rope`` dims (not yet rotated)."""
        nk, T = self.n_kv_head * self.head_dim, latent.shape[0]
        y = F_.linear(latent.contiguous(), self.kv_decompress_fused)
        k, v = y[:, :nk].reshape(T, self.n_kv_head, self.head_dim), y[:, nk:2 * nk].reshape(T, self.n_kv_head, self.head_dim)
        if not self.enhanced:
            return k, v, None
        k_rope = y[:, 2 * nk:]
        k = torch.cat([k_rope.unsqueeze(1).expand(T, self.n_kv_head, self.mla_rope_dim), k[:, :, self.mla_rope_dim:]], 2)
        return k, v, k_rope

    def qkv(self, x: torch.Tensor) -> torch.Tensor:
        """The packed ``[q | k | v]`` that ``YvAttention`` computes from its separate tensors (two GEMMs)."""
        q, latent = self.compress(x)
        k, v, _ = self.decompress_kv(latent)
        T = x.shape[0]
        return torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1)

    # -- latent cache --------------------------------------------------------------------------------------------------------
    def cache_entry(self, latent: torch.Tensor, positions: torch.Tensor, cos: Optional[torch.Tensor] = None,
                    sin: Optional[torch.Tensor] = None) -> torch.Tensor:
        """What the latent cache stores per token: ``[latent | rotated k_rope]`` ([T, r + rope])."""
        if not self.enhanced:
            return latent
        nk = self.n_kv_head * self.head_dim
        k_rope = F_.linear(latent.contiguous(), self.kv_decompress_fused[2 * nk:])
        k_rope = ref.apply_rope(k_rope.unsqueeze(1), cos, sin, positions, self.mla_rope_dim).squeeze(1)
        return torch.cat([latent, k_rope.to(latent.dtype)], -1)

    def bytes_per_token(self, element_size: int = 2) -> Dict[str, int]:
        full = 2 * self.n_kv_head * self.head_dim * element_size
        lat = (self.kv_lora_rank + self.mla_rope_dim) * element_size
        return {"keys_values": full, "latent": lat, "ratio": full / lat}

    # -- decode in the latent space ---------------------------------------------------------------------------------------------
    def absorbed_weights(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(W_k [hk, d, r], W_v [hk, d, r]) views of the fused decompression weight."""
        nk = self.n_kv_head * self.head_dim
        w = self.kv_decompress_fused
        return w[:nk].view(self.n_kv_head, self.head_dim, -1), w[nk:2 * nk].view(self.n_kv_head, self.head_dim, -1)

    def decode_absorbed(self, q: torch.Tensor, cache: torch.Tensor, lengths: Optional[torch.Tensor] = None,
                        q_positions: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                        sin: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One decode step for a batch.  q [B, hq, d] (not rotated), cache [B, S, r (+ rope)] as built by
        ``cache_entry`` (the entry of the current token included), lengths [B] valid cache entries per sample.
        Returns the attention output [B, hq, d] before the output projection."""
        B, hq, d = q.shape
        r, rope, g = self.kv_lora_rank, self.mla_rope_dim, self.n_head // self.n_kv_head
        Wk, Wv = self.absorbed_weights()
        qf = q.float()
        latent = cache[..., :r].float()                                            # [B, S, r]
        if self.enhanced:
            qf = ref.apply_rope(qf.reshape(B, hq, d), cos, sin, q_positions, rope)
            q_rope, q_nope = qf[..., :rope], qf[..., rope:]
            Wk_n = Wk[:, rope:, :].float()                                         # the rotary dims of k come from k_rope
            q_abs = torch.einsum("bkgd,kdr->bkgr", q_nope.view(B, self.n_kv_head, g, d - rope), Wk_n).reshape(B, hq, r)
            scores = torch.einsum("bhr,bsr->bhs", q_abs, latent) + torch.einsum("bhd,bsd->bhs", q_rope, cache[..., r:].float())
        else:
            q_abs = torch.einsum("bkgd,kdr->bkgr", qf.view(B, self.n_kv_head, g, d), Wk.float()).reshape(B, hq, r)
            scores = torch.einsum("bhr,bsr->bhs", q_abs, latent)
        scores = scores * self.scale
        if lengths is not None:
            S = cache.shape[1]
            scores = scores.masked_fill(torch.arange(S, device=q.device)[None, None, :] >= lengths.view(B, 1, 1), float("-inf"))
        p = torch.softmax(scores, -1)
        ctx = torch.einsum("bhs,bsr->bhr", p, latent)                              # attend over latents
        out = torch.einsum("bkgr,kdr->bkgd", ctx.view(B, self.n_kv_head, g, r), Wv.float()).reshape(B, hq, d)
        return out.to(q.dtype)
