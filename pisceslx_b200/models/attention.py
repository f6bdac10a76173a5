"""Grouped-query attention with rotary embeddings over packed sequences.

``YvAttention`` covers what the reference's ``YvAttention`` does on its GQA path
(model/core/attention.py:5186-5816): q/k/v/o projections, optional QK RMS-norm, full or partial RoPE,
causal softmax attention, paged-KV prefill and decode — with one fused QKV projection feeding the
sm_100a flash-attention kernel instead of SDPA with a materialised mask (model/core/model.py:2171-2178).
Tensor parallelism shards heads: the QKV GEMM consumes the all-gathered sequence-parallel input and the
output GEMM ends in a reduce-scatter (``parallel.tp``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch
import torch.nn as nn

from ..config import YvConfig
from ..ops import functional as F_
from .norms import YvRMSNorm, YvRotaryEmbedding


@dataclass
class AttnContext:
    """Per-forward description of the packed batch shared by all layers."""
    positions: Optional[torch.Tensor]            # int32 [T]
    cu_seqlens: torch.Tensor                     # int32 [B+1]
    max_len: int
    cos: Optional[torch.Tensor] = None
    sin: Optional[torch.Tensor] = None
    causal: bool = True
    # paged-KV inference
    cache: Any = None                            # models.cache.YvPagedKVCache
    slot_map: Optional[torch.Tensor] = None      # int32 [T] flat cache slot per token (-1 = do not store)
    block_table: Optional[torch.Tensor] = None   # int32 [B, max_blocks]
    seq_lens: Optional[torch.Tensor] = None      # int32 [B] lengths after this step
    decode: bool = False
    extras: Dict[str, Any] = field(default_factory=dict)


class YvAttention(nn.Module):
    def __init__(self, cfg: YvConfig, layer_idx: int = 0, tp_size: int = 1, tp_group=None):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.tp_size, self.tp_group = tp_size, tp_group
        assert cfg.n_head % tp_size == 0 and cfg.n_kv_head % tp_size == 0
        self.hq, self.hk, self.d = cfg.n_head // tp_size, cfg.n_kv_head // tp_size, cfg.head_dim
        self.rot_dim = cfg.partial_rope_dim if cfg.use_partial_rope else cfg.head_dim
        self.scale = 1.0 / math.sqrt(self.d)
        H = cfg.hidden_size
        self.qkv_proj = nn.Parameter(torch.empty((self.hq + 2 * self.hk) * self.d, H))
        self.o_proj = nn.Parameter(torch.empty(H, self.hq * self.d))
        std = cfg.initializer_range
        nn.init.normal_(self.qkv_proj, std=std)
        nn.init.normal_(self.o_proj, std=std / math.sqrt(2 * cfg.n_layer) if cfg.use_scaled_init else std)
        self.q_norm = YvRMSNorm(self.d, cfg.layer_norm_eps) if cfg.use_qk_norm else None
        self.k_norm = YvRMSNorm(self.d, cfg.layer_norm_eps) if cfg.use_qk_norm else None

    # -- projections (tensor-parallel aware) ----------------------------------------------------------
    def _qkv(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            from ..parallel import tp
            return tp.allgather_linear(x, self.qkv_proj, self.tp_group)
        return F_.linear(x, self.qkv_proj)

    def _out(self, o: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            from ..parallel import tp
            return tp.linear_reduce_scatter(o, self.o_proj, self.tp_group)
        return F_.linear(o, self.o_proj)

    def _qk_norm(self, qkv: torch.Tensor) -> torch.Tensor:
        T = qkv.shape[0]
        nq, nk = self.hq * self.d, self.hk * self.d
        q = self.q_norm(qkv[:, :nq].reshape(T * self.hq, self.d)).reshape(T, nq)
        k = self.k_norm(qkv[:, nq:nq + nk].reshape(T * self.hk, self.d)).reshape(T, nk)
        return torch.cat([q, k, qkv[:, nq + nk:]], dim=1)

    def forward(self, x: torch.Tensor, ctx: AttnContext) -> torch.Tensor:
        """x [T, H] (packed tokens; sequence-sharded when tensor parallel) -> [T, H]."""
        qkv = self._qkv(x)
        if self.q_norm is not None:
            qkv = self._qk_norm(qkv)
        nq, nk = self.hq * self.d, self.hk * self.d
        if ctx.decode:
            o = self._decode(qkv, ctx)
        else:
            o = F_.rope_attention(qkv, ctx.cos, ctx.sin, ctx.positions, ctx.cu_seqlens, ctx.max_len, self.hq,
                                  self.hk, self.d, self.rot_dim, ctx.causal, self.scale)
            if ctx.cache is not None and ctx.slot_map is not None:
                kc, vc = ctx.cache.layer(self.layer_idx)
                if qkv.is_cuda:
                    # the fused path rotated k in place inside the projection buffer
                    k_rot, v_new = qkv[:, nq:nq + nk], qkv[:, nq + nk:]
                else:
                    from ..ops import reference as ref
                    k_rot = qkv[:, nq:nq + nk]
                    if ctx.cos is not None:
                        k_rot = ref.apply_rope(k_rot.reshape(-1, self.hk, self.d), ctx.cos, ctx.sin, ctx.positions,
                                               self.rot_dim).reshape(-1, nk)
                    v_new = qkv[:, nq + nk:]
                F_.kv_cache_write(k_rot.detach(), v_new.detach(), kc, vc, ctx.slot_map)
        return self._out(o)

    def _decode(self, qkv: torch.Tensor, ctx: AttnContext) -> torch.Tensor:
        B = qkv.shape[0]
        nq, nk = self.hq * self.d, self.hk * self.d
        q, k, v = qkv[:, :nq], qkv[:, nq:nq + nk], qkv[:, nq + nk:]
        if ctx.cos is not None:
            if qkv.is_cuda:
                from ..ops import kernels
                kernels().rope(q, k, ctx.cos, ctx.sin, ctx.positions, self.hq, self.hk, self.d, self.rot_dim, False)
            else:
                from ..ops import reference as ref
                q = ref.apply_rope(q.reshape(B, self.hq, self.d), ctx.cos, ctx.sin, ctx.positions,
                                   self.rot_dim).reshape(B, nq)
                k = ref.apply_rope(k.reshape(B, self.hk, self.d), ctx.cos, ctx.sin, ctx.positions,
                                   self.rot_dim).reshape(B, nk)
        kc, vc = ctx.cache.layer(self.layer_idx)
        F_.kv_cache_write(k, v, kc, vc, ctx.slot_map)
        o = F_.paged_decode(q.reshape(B, self.hq, self.d).contiguous(), kc, vc, ctx.block_table, ctx.seq_lens,
                            self.scale)
        return o.reshape(B, nq)

    # -- checkpoint key mapping ----------------------------------------------------------------------------
    def export_state(self, prefix: str, out: Dict[str, torch.Tensor]) -> None:
        nq, nk = self.hq * self.d, self.hk * self.d
        w = self.qkv_proj.detach()
        out[prefix + "q_proj.weight"] = w[:nq].clone()
        out[prefix + "k_proj.weight"] = w[nq:nq + nk].clone()
        out[prefix + "v_proj.weight"] = w[nq + nk:].clone()
        out[prefix + "o_proj.weight"] = self.o_proj.detach().clone()
        if self.q_norm is not None:
            out[prefix + "q_norm.weight"] = self.q_norm.weight.detach().clone()
            out[prefix + "k_norm.weight"] = self.k_norm.weight.detach().clone()

    def import_state(self, prefix: str, sd: Dict[str, torch.Tensor]) -> None:
        with torch.no_grad():
            w = torch.cat([sd[prefix + "q_proj.weight"], sd[prefix + "k_proj.weight"], sd[prefix + "v_proj.weight"]], 0)
            self.qkv_proj.copy_(w.to(self.qkv_proj.dtype))
            self.o_proj.copy_(sd[prefix + "o_proj.weight"].to(self.o_proj.dtype))
            if self.q_norm is not None and prefix + "q_norm.weight" in sd:
                self.q_norm.weight.copy_(sd[prefix + "q_norm.weight"])
                self.k_norm.weight.copy_(sd[prefix + "k_norm.weight"])
