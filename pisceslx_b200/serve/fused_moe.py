"""Fused MoE dispatch for serving (reference opss/infer/fused_moe.py:32-150): route a flat batch of tokens through the selected
experts and combine the outputs.

Two paths.  Experts that are uniform SwiGLU blocks (``models.moe.YvSwiGLUExpert``) are stacked once into [E, 2F, H] / [E, H, F]
and run through ``ops.moe.moe_experts`` - on a GPU that is the grouped tensor-core kernel (permute, two grouped GEMMs with the
activation fused between them, weighted un-permute), with no host read at all.  Any other ``nn.ModuleList`` goes through the
sort-based path: one stable argsort, one bincount, ONE host read of the per-expert counts (the reference reads the active ids
and the offsets separately, fused_moe.py:95-96), contiguous chunks per active expert, one ``index_add_`` back."""
from __future__ import annotations

from typing import Any, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from ..models.moe import YvSwiGLUExpert
from ..ops import moe as moe_ops


class PiscesLxFusedMoEDispatch(nn.Module):
    def __init__(self, num_experts: int, top_k: int):
        super().__init__()
        self.num_experts, self.top_k = num_experts, top_k
        self._stack: Optional[Tuple[int, torch.Tensor, torch.Tensor]] = None

    def _stacked(self, experts: nn.ModuleList) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        """Stacked weights of uniform SwiGLU experts, cached while the module list and its weights' versions stay the same."""
        if not len(experts) or not all(type(e) is YvSwiGLUExpert and e.tp_size == 1 for e in experts):
            return None
        if len({(tuple(e.w13.shape), tuple(e.w2.shape)) for e in experts}) != 1:
            return None
        key = hash((id(experts),) + tuple(e.w13._version + e.w2._version for e in experts))
        if self._stack is None or self._stack[0] != key:
            self._stack = (key, torch.stack([e.w13 for e in experts]), torch.stack([e.w2 for e in experts]))
        return self._stack[1], self._stack[2]

    def forward(self, x_flat: torch.Tensor, routing_weights: torch.Tensor, expert_indices: torch.Tensor, experts: nn.ModuleList,
                collect_stats: bool = False) -> Union[torch.Tensor, Tuple[torch.Tensor, List[torch.Tensor]]]:
        T, H = x_flat.shape
        k = expert_indices.shape[-1] if expert_indices.dim() > 1 else 1
        idx, w = expert_indices.reshape(T, k) if expert_indices.numel() == T * k else None, routing_weights.reshape(-1, k)
        if idx is None or w.shape[0] != T:
            raise ValueError(f"fused dispatch: {expert_indices.numel()} assignments cannot come from {T} tokens with {k} experts each")
        st = None if (collect_stats or torch.is_grad_enabled() and any(p.requires_grad for p in experts.parameters())) else self._stacked(experts)
        if st is not None:
            return moe_ops.moe_experts(x_flat, st[0], st[1], w.to(torch.float32), idx).to(x_flat.dtype)
        flat = idx.reshape(-1)
        token = torch.arange(T, device=x_flat.device).repeat_interleave(k)
        perm = torch.argsort(flat, stable=True)
        s_tok, s_w = token[perm], w.reshape(-1)[perm]
        counts = torch.bincount(flat, minlength=self.num_experts).tolist()               # the one host read
        xs = x_flat[s_tok]
        out = torch.zeros(T * k, H, device=x_flat.device, dtype=x_flat.dtype)
        stats: List[torch.Tensor] = []
        start = 0
        for e, n in enumerate(counts):
            if n:
                y = experts[e](xs[start:start + n])
                out[start:start + n] = y
                if collect_stats:
                    stats.append(y.mean(0))
                start += n
        res = torch.zeros_like(x_flat).index_add_(0, s_tok, s_w.unsqueeze(1).to(out.dtype) * out)
        return (res, stats) if collect_stats else res


class PiscesLxFusedMoe:
    @staticmethod
    def fused_moe_dispatch(x_flat: torch.Tensor, routing_weights: torch.Tensor, expert_indices: torch.Tensor, experts: nn.ModuleList, num_experts: int,
                           top_k: int) -> torch.Tensor:
        return PiscesLxFusedMoEDispatch(num_experts, top_k)(x_flat, routing_weights, expert_indices, experts)

    @staticmethod
    def reference_dispatch(x_flat: torch.Tensor, routing_weights: torch.Tensor, expert_indices: torch.Tensor, experts: nn.ModuleList) -> torch.Tensor:
        """The per-expert mask loop the fused paths replace (for checking them)."""
        out = torch.zeros_like(x_flat)
        for e, ex in enumerate(experts):
            m = expert_indices == e
            rows = m.any(-1)
            if rows.any():
                out[rows] += (routing_weights * m)[rows].sum(-1, keepdim=True).to(out.dtype) * ex(x_flat[rows])
        return out
