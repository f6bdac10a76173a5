"""Grouped-query attention with rotary embeddings over packed sequences.

``YvAttention`` covers what the reference's ``YvAttention`` does on its GQA path
(model/core/attention.py:5186-5816): q/k/v/o projections, optional QK RMS-norm, full or partial RoPE,
causal softmax attention, paged-KV prefill and decode — with one fused QKV projection feeding the
sm_100a flash-attention kernel instead of SDPA with a materialised mask (model/core/model.py:2171-2178).
Configuration options that follow the reference's main attention:
  * ``use_mla``: keys and values come from a low-rank latent, ``latent = (x W_c) * sigmoid(x W_g)`` (KV compression
    with the sigmoid embedding gate, attention.py:5648-5662), ``k, v = latent W_k, latent W_v``; queries optionally
    through a low-rank pair (``mla_q_lora_rank``); with ``use_enhanced_mla`` the last ``mla_rope_dim`` dims of every
    key head are one shared rotary slice decompressed from the latent (``rope_decompress``, :5683-5706).  The
    parameters keep the reference's names (``kv_compress, embedding_gate, k_decompress, v_decompress,
    rope_decompress, q_proj``), and ``latent_for_cache`` is what an MLA cache stores per token.
  * ``learnable_attention_scale``: a learned log-scale folded into the queries (:5589-5605).
  * ``attention_output_gate``: a per-head sigmoid gate on the attention output (:5786-5790).
The projections of all variants end in the same packed ``[T, (hq + 2 hk) d]`` buffer, so the flash-attention and
paged-decode kernels serve every option.
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
    # context parallelism: this rank holds one chunk of every sequence; K/V are gathered over cp_group
    cp_group: Any = None
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
        std = cfg.initializer_range
        self.use_mla = bool(getattr(cfg, "use_mla", False))
        self.o_proj = nn.Parameter(torch.empty(H, self.hq * self.d))
        if self.use_mla:
            assert tp_size == 1, "the latent-KV path is not tensor-parallel"
            r = cfg.kv_lora_rank
            self.kv_lora_rank = r
            self.kv_compress = nn.Parameter(torch.empty(r, H))
            self.embedding_gate = nn.Parameter(torch.empty(r, H))
            self.k_decompress = nn.Parameter(torch.empty(self.hk * self.d, r))
            self.v_decompress = nn.Parameter(torch.empty(self.hk * self.d, r))
            qr = cfg.mla_q_lora_rank
            if qr:
                self.q_compress = nn.Parameter(torch.empty(qr, H))
                self.q_decompress = nn.Parameter(torch.empty(self.hq * self.d, qr))
                self.q_proj = None
            else:
                self.q_proj = nn.Parameter(torch.empty(self.hq * self.d, H))
            self.enhanced = bool(getattr(cfg, "use_enhanced_mla", False))
            if self.enhanced:
                self.mla_rope_dim = min(cfg.mla_rope_dim, self.d)
                self.rope_decompress = nn.Parameter(torch.empty(self.mla_rope_dim, r))
                self.rot_dim = self.mla_rope_dim          # only the shared slice is rotated
            for w in (getattr(self, n, None) for n in ("kv_compress", "embedding_gate", "k_decompress", "v_decompress",
                                                       "q_proj", "q_compress", "q_decompress", "rope_decompress")):
                if w is not None:
                    nn.init.normal_(w, std=std)
            self.qkv_proj = None
        else:
            self.qkv_proj = nn.Parameter(torch.empty((self.hq + 2 * self.hk) * self.d, H))
            nn.init.normal_(self.qkv_proj, std=std)
        self.log_scale = nn.Parameter(torch.zeros(())) if getattr(cfg, "learnable_attention_scale", False) else None
        self.out_gate = None
        if getattr(cfg, "attention_output_gate", False):
            self.out_gate = nn.Parameter(torch.zeros(self.hq, H))     # zero logits: every head starts at gate 1/2 ...
            self.out_gate_bias = nn.Parameter(torch.full((self.hq,), 4.0))   # ... plus 4: effectively open
        self.latent_for_cache: Optional[torch.Tensor] = None
        nn.init.normal_(self.o_proj, std=std / math.sqrt(2 * cfg.n_layer) if cfg.use_scaled_init else std)
        self.q_norm = YvRMSNorm(self.d, cfg.layer_norm_eps) if cfg.use_qk_norm else None
        self.k_norm = YvRMSNorm(self.d, cfg.layer_norm_eps) if cfg.use_qk_norm else None

    # -- projections (tensor-parallel aware) ----------------------------------------------------------
    def _qkv_mla(self, x: torch.Tensor) -> torch.Tensor:
        """Packed ``[q | k | v]`` from the gated low-rank latent."""
        r = self.kv_lora_rank
        lg = F_.linear(x, torch.cat([self.kv_compress, self.embedding_gate], 0))        # one GEMM for latent + gate
        latent = lg[:, :r] * torch.sigmoid(lg[:, r:].float()).to(lg.dtype)
        self.latent_for_cache = latent.detach()
        kv = F_.linear(latent.contiguous(), torch.cat([self.k_decompress, self.v_decompress], 0))
        nk = self.hk * self.d
        k, v = kv[:, :nk], kv[:, nk:]
        if self.q_proj is not None:
            q = F_.linear(x, self.q_proj)
        else:
            q = F_.linear(F_.linear(x, self.q_compress), self.q_decompress)
        if self.enhanced:
            # decoupled RoPE: the last mla_rope_dim dims of every key head are ONE slice decompressed from the latent
            # (shared by the heads); the rotary kernel then rotates exactly that slice of q and k.  The slice sits at
            # the end of the head in the reference; the kernel rotates the first rot_dim dims, so it is placed first
            # here, which is the same attention up to a fixed permutation of each head's dims.
            T = x.shape[0]
            k_pe = F_.linear(latent.contiguous(), self.rope_decompress)                 # [T, rope_dim]
            k = torch.cat([k_pe.unsqueeze(1).expand(T, self.hk, self.mla_rope_dim),
                           k.reshape(T, self.hk, self.d)[:, :, self.mla_rope_dim:]], dim=2).reshape(T, nk)
        return torch.cat([q, k, v], dim=1).contiguous()

    def _qkv(self, x: torch.Tensor) -> torch.Tensor:
        if self.use_mla:
            return self._qkv_mla(x)
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
        if self.log_scale is not None:
            qkv = torch.cat([qkv[:, :nq] * torch.exp(self.log_scale).to(qkv.dtype), qkv[:, nq:]], dim=1)
        if self.out_gate is not None:
            o = self._decode(qkv, ctx) if ctx.decode else self._attend(qkv, ctx)
            g = torch.sigmoid(torch.nn.functional.linear(x.float(), self.out_gate.float(), self.out_gate_bias.float()))
            if self.tp_size > 1 and g.shape[0] != o.shape[0]:
                raise RuntimeError("attention_output_gate needs the un-sharded sequence (tensor parallel size 1)")
            o = (o.reshape(-1, self.hq, self.d) * g.to(o.dtype).unsqueeze(-1)).reshape(-1, nq)
            return self._out(o)
        o = self._decode(qkv, ctx) if ctx.decode else self._attend(qkv, ctx)
        return self._out(o)

    def _attend(self, qkv: torch.Tensor, ctx: AttnContext) -> torch.Tensor:
        """Prefill / training attention over the packed projection, writing the paged cache when one is attached."""
        nq, nk = self.hq * self.d, self.hk * self.d
        if ctx.cp_group is not None:
            return self._attend_context_parallel(qkv, ctx)
        o = F_.rope_attention(qkv, ctx.cos, ctx.sin, ctx.positions, ctx.cu_seqlens, ctx.max_len, self.hq, self.hk,
                              self.d, self.rot_dim, ctx.causal, self.scale)
        if ctx.cache is not None and ctx.slot_map is not None:
            kc, vc = ctx.cache.layer(self.layer_idx)
            k_rot, v_new = qkv[:, nq:nq + nk], qkv[:, nq + nk:]
            if not qkv.is_cuda and ctx.cos is not None:
                from ..ops import reference as ref
                k_rot = ref.apply_rope(k_rot.reshape(-1, self.hk, self.d), ctx.cos, ctx.sin, ctx.positions,
                                       self.rot_dim).reshape(-1, nk)
            F_.kv_cache_write(k_rot.detach(), v_new.detach(), kc, vc, ctx.slot_map)
        return o

    def _attend_context_parallel(self, qkv: torch.Tensor, ctx: AttnContext) -> torch.Tensor:
        """Training attention when every sequence is split over the ranks of ``ctx.cp_group`` (contiguous chunks):
        rotate q / k at their GLOBAL positions, all-gather K / V of each sequence (differentiable: the backward is a
        reduce-scatter) and attend the local queries up to their causal horizon (``parallel.cp``)."""
        from ..ops import reference as ref
        from ..parallel import cp
        T = qkv.shape[0]
        nq, nk = self.hq * self.d, self.hk * self.d
        q, k, v = qkv[:, :nq], qkv[:, nq:nq + nk], qkv[:, nq + nk:]
        if ctx.cos is not None:
            q = ref.apply_rope(q.reshape(T, self.hq, self.d), ctx.cos, ctx.sin, ctx.positions, self.rot_dim).reshape(T, nq)
            k = ref.apply_rope(k.reshape(T, self.hk, self.d), ctx.cos, ctx.sin, ctx.positions, self.rot_dim).reshape(T, nk)
        cu = ctx.cu_seqlens.tolist()
        outs = []
        ring = getattr(self.cfg, "context_parallel_mode", "allgather") == "ring"
        for b in range(len(cu) - 1):
            sl = slice(cu[b], cu[b + 1])
            if ring:
                # blocks of K / V travel round the ranks in both passes: no rank ever holds the whole sequence's keys
                outs.append(cp.ring_attention_train(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(),
                                                    ctx.cp_group, self.hq, self.hk, self.d, causal=ctx.causal,
                                                    scale=self.scale))
                continue
            outs.append(cp.allgather_attention(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), ctx.cp_group,
                                               self.hq, self.hk, self.d, causal=ctx.causal, scale=self.scale))
        return torch.cat(outs, 0).to(qkv.dtype)

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
    _MLA_NAMES = ("kv_compress", "embedding_gate", "k_decompress", "v_decompress", "rope_decompress", "q_proj",
                  "q_compress", "q_decompress")

    def _export_extras(self, prefix: str, out: Dict[str, torch.Tensor]) -> None:
        if self.log_scale is not None:
            out[prefix + "log_scale"] = self.log_scale.detach().clone()
        if self.out_gate is not None:
            out[prefix + "out_gate.weight"] = self.out_gate.detach().clone()
            out[prefix + "out_gate.bias"] = self.out_gate_bias.detach().clone()

    def export_state(self, prefix: str, out: Dict[str, torch.Tensor]) -> None:
        nq, nk = self.hq * self.d, self.hk * self.d
        self._export_extras(prefix, out)
        if self.use_mla:
            for n in self._MLA_NAMES:
                w = getattr(self, n, None)
                if w is not None:
                    out[prefix + n + ".weight"] = w.detach().clone()
            out[prefix + "o_proj.weight"] = self.o_proj.detach().clone()
            if self.q_norm is not None:
                out[prefix + "q_norm.weight"] = self.q_norm.weight.detach().clone()
                out[prefix + "k_norm.weight"] = self.k_norm.weight.detach().clone()
            return
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
            if self.log_scale is not None and prefix + "log_scale" in sd:
                self.log_scale.copy_(sd[prefix + "log_scale"])
            if self.out_gate is not None and prefix + "out_gate.weight" in sd:
                self.out_gate.copy_(sd[prefix + "out_gate.weight"])
                self.out_gate_bias.copy_(sd[prefix + "out_gate.bias"])
            if self.use_mla:
                for n in self._MLA_NAMES:
                    w = getattr(self, n, None)
                    if w is not None:
                        w.copy_(sd[prefix + n + ".weight"].to(w.dtype))
                self.o_proj.copy_(sd[prefix + "o_proj.weight"].to(self.o_proj.dtype))
                if self.q_norm is not None and prefix + "q_norm.weight" in sd:
                    self.q_norm.weight.copy_(sd[prefix + "q_norm.weight"])
                    self.k_norm.weight.copy_(sd[prefix + "k_norm.weight"])
                return
            w = torch.cat([sd[prefix + "q_proj.weight"], sd[prefix + "k_proj.weight"], sd[prefix + "v_proj.weight"]], 0)
            self.qkv_proj.copy_(w.to(self.qkv_proj.dtype))
            self.o_proj.copy_(sd[prefix + "o_proj.weight"].to(self.o_proj.dtype))
            if self.q_norm is not None and prefix + "q_norm.weight" in sd:
                self.q_norm.weight.copy_(sd[prefix + "q_norm.weight"])
                self.k_norm.weight.copy_(sd[prefix + "k_norm.weight"])
