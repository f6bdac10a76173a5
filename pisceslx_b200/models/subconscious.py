"""Subconscious systems: FiLM parameter sources that modulate the residual stream at block entry.

Three sources share one small interface (``begin(h, batch)``, ``film_params(layer_idx, hidden)``, ``end()``):

``YvSubconsciousSystem``   the mechanism in the reference code (model/core/subconscious.py:32-166 and
                           dual_injector.py:33-58): a knowledge router summarises the sequence-pooled hidden state at
                           layer 0, a state ``tanh(W[h_mean; k; s])`` evolves, and a per-layer FiLM generator emits
                           ``{"scale", "shift"}`` of shape [B, 1, H].
``YvPQKnowledgeField``     the product-quantised knowledge field the reference documents (README.md:70-78,
                           configs/model/7B.yaml:455-464) but does not implement: 16 codebooks x 131 072 entries x 128
                           dims; a 2-layer navigation MLP emits 16 groups of codebook logits per token, the arg-max
                           entries are gathered (row-sharded over GPUs: the gather reads the owners' memory), summed
                           and projected to per-token FiLM scale / shift on every ``pq_film_interval``-th layer.
``YvSubconsciousBlockField`` the 628-block field (``models.block_field``; reference model/core/block_field.py:63-541): low-rank read of a
                           resident block, bounded ``gamma = g_max * tanh`` and ``beta``, applied to the embeddings.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch
import torch.nn as nn

from ..config import YvConfig
from ..ops import functional as F_
from ..ops import kernels, reference as ref


class YvKnowledgeRouter(nn.Module):
    def __init__(self, hidden: int, kdim: int):
        super().__init__()
        self.proj = nn.Linear(hidden, kdim)
        self.value = nn.Linear(kdim, kdim)

    def forward(self, pooled: torch.Tensor) -> torch.Tensor:
        return self.value(torch.tanh(self.proj(pooled.float())))


class YvSubconsciousState(nn.Module):
    def __init__(self, hidden: int, kdim: int, sdim: int):
        super().__init__()
        self.evolve = nn.Linear(hidden + kdim + sdim, sdim)
        self.sdim = sdim

    def forward(self, pooled: torch.Tensor, k: torch.Tensor, s: Optional[torch.Tensor]) -> torch.Tensor:
        if s is None:
            s = pooled.new_zeros(pooled.shape[0], self.sdim, dtype=torch.float32)
        return torch.tanh(self.evolve(torch.cat([pooled.float(), k, s], -1)))


class YvFiLMGenerator(nn.Module):
    def __init__(self, sdim: int, hidden: int):
        super().__init__()
        self.gamma = nn.Linear(sdim, hidden)
        self.beta = nn.Linear(sdim, hidden)
        nn.init.zeros_(self.gamma.weight); nn.init.zeros_(self.gamma.bias)
        nn.init.zeros_(self.beta.weight); nn.init.zeros_(self.beta.bias)

    def forward(self, s: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {"scale": self.gamma(s).unsqueeze(1), "shift": self.beta(s).unsqueeze(1)}


class YvSubconsciousSystem(nn.Module):
    def __init__(self, cfg: YvConfig):
        super().__init__()
        H, kd, sd = cfg.hidden_size, cfg.subconscious_knowledge_dim, cfg.subconscious_state_dim
        self.router = YvKnowledgeRouter(H, kd)
        self.state_evolver = YvSubconsciousState(H, kd, sd)
        self.film_generators = nn.ModuleList([YvFiLMGenerator(sd, H) for _ in range(cfg.n_layer)])
        self.float()
        self._state: Optional[torch.Tensor] = None
        self._batch = 1

    def begin(self, h: torch.Tensor, batch: int) -> None:
        self._state, self._batch = None, batch

    def film_params(self, layer_idx: int, hidden: torch.Tensor) -> Optional[Dict[str, torch.Tensor]]:
        B = self._batch
        if layer_idx == 0 or self._state is None:
            pooled = hidden.view(B, -1, hidden.shape[-1]).float().mean(1)
            k = self.router(pooled)
            self._state = self.state_evolver(pooled, k, self._state)
        f = self.film_generators[layer_idx](self._state)
        return {"scale": f["scale"].to(hidden.dtype), "shift": f["shift"].to(hidden.dtype)}

    def end(self) -> None:
        self._state = None                     # the state lives for one forward (reference model.py:2410)


class YvDualInjector(nn.Module):
    """Holds the Subconscious system and hands FiLM parameters to the trunk (reference dual_injector.py)."""

    def __init__(self, cfg: YvConfig):
        super().__init__()
        self.subconscious = YvSubconsciousSystem(cfg)

    def inject(self, layer_idx: int, hidden: torch.Tensor) -> Optional[Dict[str, torch.Tensor]]:
        return self.subconscious.film_params(layer_idx, hidden)


# --------------------------------------------------------------------------------------------------
class _PQGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, idx, field):
        ctx.field = field
        ctx.save_for_backward(idx)
        ctx.table_shape = table.shape
        if field.shard_buf is not None:
            from ..parallel import fused as fz
            return fz.pq_gather_sum_sharded(field.shard_buf, idx, field.C, field.rows_per_rank, field.D)
        out = torch.empty(idx.shape[0], table.shape[2], dtype=torch.bfloat16, device=table.device)
        from ..ops import status_word
        kernels().pq_gather_sum(table, idx, out, status_word(table.device))
        return out

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        return _PQGather.table_grad(ctx.field, dout, idx, ctx.table_shape), None, None

    @staticmethod
    def table_grad(field, dout, idx, table_shape):
        """Gradient of the (local shard of the) table from the gradient of the summed entries."""
        C, N, D = table_shape
        if field.shard_buf is not None:
            # each rank keeps the gradient rows of its own shard: ids outside the shard are dropped locally and
            # the token gradients of all ranks are exchanged first
            import torch.distributed as dist
            g = [torch.empty_like(dout) for _ in range(field.world)]
            i = [torch.empty_like(idx) for _ in range(field.world)]
            dist.all_gather(g, dout.contiguous(), group=field.group)
            dist.all_gather(i, idx.contiguous(), group=field.group)
            dout, idx = torch.cat(g), torch.cat(i)
            lo = field.rank * field.rows_per_rank
            idx = torch.where((idx >= lo) & (idx < lo + field.rows_per_rank), idx - lo, torch.full_like(idx, -1))
        dt = torch.zeros(C, N, D, dtype=torch.float32, device=dout.device)
        kernels().pq_scatter_grad(dout.contiguous(), idx.contiguous(), dt)
        return dt.to(torch.bfloat16)


class _PQFilmFused(torch.autograd.Function):
    """``h * (1 + s) + b`` with ``(s | b) = (sum of the tokens' field entries) @ film_proj^T`` as ONE kernel (peer loads of
    the entries, tensor-core projection, modulation of the h tile in shared memory).  Backward with the saved summed
    entries ``e`` [T, 128]: the projection is recomputed, the table gradient scatters ``de`` like the plain lookup."""

    @staticmethod
    def forward(ctx, h, table, w, idx, field):
        from ..ops import status_word
        T, H = h.shape
        out = torch.empty_like(h)
        e = torch.empty(T, field.D, dtype=torch.bfloat16, device=h.device) if torch.is_grad_enabled() or h.requires_grad \
            else None
        kernels().pq_film(field.table_ptrs(), idx, w, h, out, e, field.C, field.rows_per_rank, status_word(h.device))
        ctx.field, ctx.table_shape = field, table.shape
        if e is not None:
            ctx.save_for_backward(h, w, idx, e)
        return out

    @staticmethod
    def backward(ctx, dout):
        h, w, idx, e = ctx.saved_tensors
        field = ctx.field
        H = h.shape[1]
        dout = dout.contiguous()
        s = F_.gemm(e, w[:H])                                               # [T, H] scale, recomputed
        dh = dout * (1 + s)
        ds = dout * h
        de = F_.gemm(ds, w[:H], b_mn=True) + F_.gemm(dout, w[H:], b_mn=True)  # [T, 128]
        dw = torch.cat([F_.gemm(ds, e, a_mn=True, b_mn=True), F_.gemm(dout, e, a_mn=True, b_mn=True)])
        dtable = _PQGather.table_grad(field, de, idx, ctx.table_shape)
        return dh, dtable, dw, None, None


class YvPQKnowledgeField(nn.Module):
    def __init__(self, cfg: YvConfig, group: Any = None):
        super().__init__()
        self.cfg = cfg
        self.C, self.N, self.D = cfg.pq_num_codebooks, cfg.pq_codebook_size, cfg.pq_entry_dim
        H = cfg.hidden_size
        self.interval = max(1, cfg.pq_film_interval)
        self.group = group
        self.world, self.rank = 1, 0
        if group is not None:
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.N % self.world == 0
        self.rows_per_rank = self.N // self.world
        # navigation head: hidden -> nav_hidden -> C * n_logits; logits index a coarse cell of each codebook
        self.nav_cells = min(self.N, 1024)
        self.nav1 = nn.Parameter(torch.empty(cfg.pq_nav_hidden, H).normal_(std=cfg.initializer_range))
        self.nav2 = nn.Parameter(torch.empty(self.C * self.nav_cells, cfg.pq_nav_hidden).normal_(std=cfg.initializer_range))
        self.codebook = nn.Parameter(torch.empty(self.C, self.rows_per_rank, self.D).normal_(std=cfg.pq_init_std))
        self.film_proj = nn.Parameter(torch.zeros(2 * H, self.D))
        self.shard_buf = None
        self._film_cache: Optional[Dict[str, torch.Tensor]] = None
        self._batch = 1

    def materialise_shards(self) -> None:
        """Move the local codebook shard into symmetric memory so that peers can gather from it."""
        if self.world == 1 or not self.codebook.is_cuda:
            return
        from ..parallel import fused as fz
        heap = fz.heap_for(self.group)
        buf = heap.get("pq_codebook", self.codebook.numel() * 2)
        t = buf.tensor(torch.bfloat16, self.codebook.numel()).view_as(self.codebook)
        t.copy_(self.codebook.data)
        self.codebook.data = t
        self.shard_buf = buf
        heap.barrier()

    def navigate(self, hidden: torch.Tensor) -> torch.Tensor:
        """hidden [T, H] -> entry ids [T, C] (arg-max cell of each codebook, spread over the codebook by a fixed
        stride so that all entries are reachable from the coarse logits plus the token position hash)."""
        n = torch.nn.functional.gelu(F_.linear(hidden, self.nav1))
        logits = F_.linear(n, self.nav2)
        T = logits.shape[0]
        if logits.is_cuda:
            cell = torch.empty(T, self.C, dtype=torch.int32, device=logits.device)
            kernels().argmax_rows(logits.contiguous(), cell, self.C)
        else:
            cell = logits.view(T, self.C, self.nav_cells).argmax(-1).int()
        stride = self.N // self.nav_cells
        fine = (torch.arange(T, device=hidden.device, dtype=torch.int32) % stride).unsqueeze(1)
        return (cell * stride + fine).int()

    def table_ptrs(self) -> torch.Tensor:
        """Device pointers of every rank's shard (own rank included), as the kernels take them."""
        if self.shard_buf is not None:
            return self.shard_buf.ptrs
        ptr = self.codebook.data_ptr()
        if getattr(self, "_ptrs", None) is None or int(self._ptrs[0]) != ptr:
            self._ptrs = torch.tensor([ptr], dtype=torch.int64)
        return self._ptrs

    @property
    def fused_ok(self) -> bool:
        """The one-kernel path covers the shapes the field is specified with: 128-dim entries, at most 16 codebooks."""
        return (self.D == 128 and self.C <= 16 and self.cfg.hidden_size % 64 == 0 and self.codebook.is_cuda
                and self.codebook.dtype == torch.bfloat16 and self.film_proj.dtype == torch.bfloat16)

    def wants(self, layer_idx: int) -> bool:
        return layer_idx % self.interval == 0

    def apply_fused(self, hidden: torch.Tensor) -> torch.Tensor:
        """The modulated residual stream [T, H] (CUDA, bf16, entry dimension 128): navigation, then one kernel for
        gather + sum + projection + ``h * (1 + scale) + shift``."""
        idx = self.navigate(hidden.detach())
        return _PQFilmFused.apply(hidden.contiguous(), self.codebook, self.film_proj, idx.contiguous(), self)

    def lookup(self, idx: torch.Tensor) -> torch.Tensor:
        if idx.is_cuda:
            return _PQGather.apply(self.codebook, idx.contiguous(), self)
        return ref.pq_gather_sum(self.codebook, idx)

    def begin(self, h: torch.Tensor, batch: int) -> None:
        self._film_cache, self._batch = None, batch

    def film_params(self, layer_idx: int, hidden: torch.Tensor) -> Optional[Dict[str, torch.Tensor]]:
        if layer_idx % self.interval != 0:
            return None
        idx = self.navigate(hidden.detach())
        e = self.lookup(idx)                                            # [T, D]
        f = F_.linear(e, self.film_proj)                                 # [T, 2H]
        H = hidden.shape[-1]
        B = self._batch
        return {"scale": f[:, :H].reshape(B, -1, H), "shift": f[:, H:].reshape(B, -1, H)}

    def end(self) -> None:
        self._film_cache = None


# The block field (blocks, resident pool, trace addresser) lives in ``models.block_field``; the names stay importable
# from here.
from .block_field import (YvAddressingStatistics, YvKnowledgeBlockModule, YvResidentBlockPool,  # noqa: E402,F401
                          YvResonantTraceAddresser, YvSubconsciousBlockField)
