"""Tensor parallelism with a sequence-parallel residual stream.

The residual stream is sharded along tokens (``[T / tp, H]`` per rank); a column-parallel projection
consumes the all-gathered tokens, a row-parallel projection ends in a reduce-scatter.  Two implementations
of each pair:

  * NCCL (baseline mode): ``all_gather_into_tensor`` / ``reduce_scatter_tensor`` around the local GEMM;
  * fused (``parallel.fused``): one sm_100a kernel per pair that moves peer tiles over NVLink while the
    tensor cores work on the tiles that have already arrived.

The reference has no working tensor parallelism: its helper slices ``nn.Linear`` weights by names that do
not occur in the Yv model and inserts no collective (opss/train/parallel_3d.py:352-366), and
``PiscesLxTensorParallelOperator`` (utils/opsc/distributed.py:742-863) is never called by the model.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist

from ..ops import functional as F_


def _size(group: Any) -> int:
    return dist.get_world_size(group) if group is not None else 1


def _rank(group: Any) -> int:
    return dist.get_rank(group) if group is not None else 0


def all_gather_rows(x: torch.Tensor, group: Any) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    out = torch.empty(n * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def reduce_scatter_rows(x: torch.Tensor, group: Any) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    assert x.shape[0] % n == 0, "token count must divide by the tensor-parallel size"
    out = torch.empty(x.shape[0] // n, *x.shape[1:], dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
    else:                                                    # Gloo has no reduce_scatter: all-reduce then slice
        y = x.contiguous().clone()
        dist.all_reduce(y, group=group)
        r = _rank(group)
        out.copy_(y[r * out.shape[0]:(r + 1) * out.shape[0]])
    return out


class _ScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n, r = _size(group), _rank(group)
        rows = x.shape[0] // n
        return x[r * rows:(r + 1) * rows].contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather_rows(g, ctx.group), None


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        # every tensor-parallel rank computes the same loss from the gathered tokens, so the incoming
        # gradients are identical across ranks: keep the local rows
        n, r = _size(ctx.group), _rank(ctx.group)
        rows = g.shape[0] // n
        return g[r * rows:(r + 1) * rows].contiguous(), None


def scatter_sequence(x: torch.Tensor, group: Any) -> torch.Tensor:
    """[T, H] replicated -> [T / tp, H] local rows (backward: all-gather)."""
    return _ScatterSeq.apply(x, group)


def gather_sequence(x: torch.Tensor, group: Any) -> torch.Tensor:
    """[T / tp, H] -> [T, H] (backward: local slice)."""
    return _GatherSeq.apply(x, group)


class _AllGatherLinear(torch.autograd.Function):
    """y [T, N_local] = all_gather(x_shard) @ w_local.T"""

    @staticmethod
    def forward(ctx, x, w, group, fused):
        ctx.group, ctx.fused = group, fused
        if fused and x.is_cuda:
            from . import fused_tp as fz
            xg, y = fz.allgather_gemm(x, w, group)
        else:
            xg = all_gather_rows(x, group)
            y = F_.linear(xg, w) if not x.is_cuda else F_.gemm(xg.contiguous(), w)
        ctx.save_for_backward(x, w)          # the gathered input is rebuilt in backward (memory over traffic)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        group = ctx.group
        dy = dy.contiguous()
        if x.is_cuda:
            if ctx.fused:
                from . import fused_tp as fz
                dx = fz.gemm_reduce_scatter(dy, w, group, b_mn=True)          # (dy @ w) reduce-scattered
            else:
                dx = reduce_scatter_rows(F_.gemm(dy, w, b_mn=True), group)
            xg = all_gather_rows(x, group)
            dw = F_.gemm(dy, xg, a_mn=True, b_mn=True)
        else:
            dx = reduce_scatter_rows(dy @ w.to(dy.dtype), group)
            xg = all_gather_rows(x, group)
            dw = dy.t() @ xg
        return dx, dw.to(w.dtype), None, None


class _LinearReduceScatter(torch.autograd.Function):
    """y_shard [T / tp, N] = reduce_scatter(x @ w_local.T)"""

    @staticmethod
    def forward(ctx, x, w, group, fused):
        ctx.group, ctx.fused = group, fused
        ctx.save_for_backward(x, w)
        if x.is_cuda:
            if fused:
                from . import fused_tp as fz
                return fz.gemm_reduce_scatter(x.contiguous(), w, group, b_mn=False)
            return reduce_scatter_rows(F_.gemm(x.contiguous(), w), group)
        return reduce_scatter_rows(x @ w.to(x.dtype).t(), group)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        if x.is_cuda:
            if ctx.fused:
                from . import fused_tp as fz
                dyg, dx = fz.allgather_gemm(dy.contiguous(), w, ctx.group, b_mn=True)   # all_gather(dy) @ w
            else:
                dyg = all_gather_rows(dy.contiguous(), ctx.group)
                dx = F_.gemm(dyg, w, b_mn=True)
            dw = F_.gemm(dyg, x.contiguous(), a_mn=True, b_mn=True)
        else:
            dyg = all_gather_rows(dy.contiguous(), ctx.group)
            dx = dyg @ w.to(dyg.dtype)
            dw = dyg.t() @ x
        return dx, dw.to(w.dtype), None, None


def _fused_enabled(x: torch.Tensor) -> bool:
    if not x.is_cuda:
        return False
    from .state import get_state
    from . import fused as fz
    return fz.enabled()


def allgather_linear(x_shard: torch.Tensor, w_local: torch.Tensor, group: Any, fused: Optional[bool] = None):
    """Column-parallel projection on a sequence-sharded input: [T/tp, K] x [N/tp, K] -> [T, N/tp]."""
    fused = _fused_enabled(x_shard) if fused is None else fused
    return _AllGatherLinear.apply(x_shard, w_local, group, fused)


def linear_reduce_scatter(x: torch.Tensor, w_local: torch.Tensor, group: Any, fused: Optional[bool] = None):
    """Row-parallel projection ending sequence-sharded: [T, K/tp] x [N, K/tp] -> [T/tp, N]."""
    fused = _fused_enabled(x) if fused is None else fused
    return _LinearReduceScatter.apply(x, w_local, group, fused)
