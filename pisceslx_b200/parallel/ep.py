"""Expert parallelism: every rank of the EP group owns ``E / ep`` consecutive experts; tokens travel to the
owner of each selected expert and the results travel back.

Layout trick shared by both implementations: the sender sorts its assignments by global expert id and pads
every expert segment to a multiple of 128 rows (``ops.moe.permute_tokens``).  A destination therefore
receives, from every source, whole 128-row tiles that each belong to one local expert - the grouped tcgen05
GEMM runs directly on the receive buffer with a tile -> expert table and no second permutation.

  * NCCL mode (baseline): ``all_to_all_single`` with per-destination row counts (one small device->host read
    per layer for the split sizes), grouped GEMMs, ``all_to_all_single`` back, weighted combine.
  * fused mode (``parallel.fused``): the permutation kernel stores rows straight into the owner's receive
    buffer over NVLink and the combine kernel loads result rows from the owner's memory; no host read.

The reference's expert-parallel operator splits tokens equally and ignores routing, and is never called
(utils/opsc/distributed.py:1059-1158); its MoE layers loop over all experts locally (model/moe/layer.py:929-936).
"""
from __future__ import annotations

from typing import Any, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import kernels, reference as ref, status_word
from ..ops import moe as moe_ops

_BF16 = torch.bfloat16


# --------------------------------------------------------------------------------------------------
# differentiable all-to-all with explicit row splits
# --------------------------------------------------------------------------------------------------
class _AllToAllRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send_rows, recv_rows, group):
        ctx.group, ctx.send_rows, ctx.recv_rows = group, send_rows, recv_rows
        out = torch.empty(sum(recv_rows), *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_rows, input_split_sizes=send_rows,
                               group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty(sum(ctx.send_rows), *g.shape[1:], dtype=g.dtype, device=g.device)
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send_rows,
                               input_split_sizes=ctx.recv_rows, group=ctx.group)
        return out, None, None, None


def all_to_all_rows(x: torch.Tensor, send_rows: List[int], recv_rows: List[int], group: Any) -> torch.Tensor:
    return _AllToAllRows.apply(x, send_rows, recv_rows, group)


# --------------------------------------------------------------------------------------------------
# differentiable pieces of the routed-expert computation (GPU)
# --------------------------------------------------------------------------------------------------
class _PermuteFn(torch.autograd.Function):
    """x [T,H] -> expert-sorted padded rows xp [max_rows, H] (+ plan tensors, non-differentiable)."""

    @staticmethod
    def forward(ctx, x, idx, counts, num_experts, deterministic):
        xp, plan = moe_ops.permute_tokens(x.contiguous(), idx, counts, num_experts, deterministic)
        ctx.save_for_backward(plan.row_map)
        ctx.k, ctx.shape = idx.shape[1], x.shape
        ctx.mark_non_differentiable(plan.seg_offsets, plan.tile_expert, plan.num_m_tiles, plan.row_map)
        return xp, plan.seg_offsets, plan.tile_expert, plan.num_m_tiles, plan.row_map

    @staticmethod
    def backward(ctx, dxp, *_):
        (row_map,) = ctx.saved_tensors
        dx = torch.empty(ctx.shape, dtype=_BF16, device=dxp.device)
        kernels().moe_unpermute_sum(dxp.contiguous(), row_map, dx, ctx.k)
        return dx, None, None, None, None


class _CombineFn(torch.autograd.Function):
    """out[t] = sum_j w[t,j] * y[row_map[t,j]]"""

    @staticmethod
    def forward(ctx, y, row_map, weights, zero_seg, zero_counts):
        T, k = row_map.shape
        out = torch.empty(T, y.shape[1], dtype=_BF16, device=y.device)
        w = weights.float().contiguous()
        kernels().moe_combine(y.contiguous(), row_map, w, None, out)
        ctx.save_for_backward(y, row_map, w, zero_seg, zero_counts)
        ctx.w_dtype = weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        y, row_map, w, zero_seg, zero_counts = ctx.saved_tensors
        T, k = row_map.shape
        dy = torch.zeros_like(y) if zero_seg is None else torch.empty_like(y)
        dw = torch.empty(T, k, dtype=torch.float32, device=y.device)
        kernels().moe_combine_bwd(dout.contiguous(), y, row_map, w, dy, dw)
        if zero_seg is not None:
            kernels().moe_zero_pad(dy, zero_seg, zero_counts)
        return dy, None, dw.to(ctx.w_dtype), None, None


class _GroupedFFNFn(torch.autograd.Function):
    """SwiGLU experts on tile-aligned rows.  ``blocks`` lists (row0, rows, seg_offsets, tile_expert, num_tiles)
    for every contiguous block whose segments are expert-sorted (one block per source rank)."""

    @staticmethod
    def forward(ctx, xr, w13, w2, blocks):
        K = kernels()
        st = status_word(xr.device)
        F = w13.shape[1] // 2
        rows = xr.shape[0]
        y1 = torch.empty(rows, 2 * F, dtype=_BF16, device=xr.device)
        for (r0, n, seg, te, nt) in blocks:
            if n:
                K.gemm_grouped_m(xr[r0:r0 + n], w13, y1[r0:r0 + n], te, nt, False, 0, st)
        act = torch.empty(rows, F, dtype=_BF16, device=xr.device)
        K.swiglu_fwd(y1, act)
        y2 = torch.empty(rows, w2.shape[1], dtype=_BF16, device=xr.device)
        for (r0, n, seg, te, nt) in blocks:
            if n:
                K.gemm_grouped_m(act[r0:r0 + n], w2, y2[r0:r0 + n], te, nt, False, 0, st)
        ctx.save_for_backward(xr, y1, act, w13, w2)
        ctx.blocks = blocks
        return y2

    @staticmethod
    def backward(ctx, dy2):
        K = kernels()
        xr, y1, act, w13, w2 = ctx.saved_tensors
        st = status_word(xr.device)
        dy2 = dy2.contiguous()
        F = w13.shape[1] // 2
        rows = xr.shape[0]
        dact = torch.empty(rows, F, dtype=_BF16, device=xr.device)
        dw2 = torch.zeros_like(w2)
        dw13 = torch.zeros_like(w13)
        for (r0, n, seg, te, nt) in ctx.blocks:
            if n:
                K.gemm_grouped_m(dy2[r0:r0 + n], w2, dact[r0:r0 + n], te, nt, True, 0, st)
                K.gemm_grouped_k(dy2[r0:r0 + n], act[r0:r0 + n], dw2, seg, True, 0, st)
        dy1 = torch.empty_like(y1)
        K.swiglu_bwd(y1, dact, dy1)
        dxr = torch.empty_like(xr)
        for (r0, n, seg, te, nt) in ctx.blocks:
            if n:
                K.gemm_grouped_m(dy1[r0:r0 + n], w13, dxr[r0:r0 + n], te, nt, True, 0, st)
                K.gemm_grouped_k(dy1[r0:r0 + n], xr[r0:r0 + n], dw13, seg, True, 0, st)
        return dxr, dw13, dw2, None


# --------------------------------------------------------------------------------------------------
# expert-parallel routed experts
# --------------------------------------------------------------------------------------------------
def _exchange_counts(per_expert: torch.Tensor, ep: int, group: Any) -> torch.Tensor:
    """per_expert [E] (rows this rank sends to every global expert) -> [ep, E_local] rows received from every
    source for each local expert."""
    e_local = per_expert.numel() // ep
    send = per_expert.view(ep, e_local).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def _moe_experts_ep_reference(x, w13, w2, weights, idx, num_experts, group):
    """Pure-PyTorch expert parallelism (CPU / Gloo): same data movement, dense math."""
    ep = dist.get_world_size(group)
    T, k = idx.shape
    flat_e = idx.flatten().long()
    order = torch.argsort(flat_e, stable=True)
    tok = torch.div(order, k, rounding_mode="floor")
    xs = x[tok]
    counts = torch.bincount(flat_e, minlength=num_experts)
    recv_counts = _exchange_counts(counts, ep, group)
    send_rows = counts.view(ep, -1).sum(1).tolist()
    recv_rows = recv_counts.sum(1).tolist()
    xr = all_to_all_rows(xs, send_rows, recv_rows, group)
    outs, o = [], 0
    rc = recv_counts.tolist()
    for src in range(ep):
        for e in range(len(rc[src])):
            c = rc[src][e]
            if c:
                seg = xr[o:o + c]
                outs.append(ref.swiglu(seg @ w13[e].to(seg.dtype).t()) @ w2[e].to(seg.dtype).t())
                o += c
    yr = torch.cat(outs, 0) if outs else xr.new_zeros(0, x.shape[1])
    y = all_to_all_rows(yr, recv_rows, send_rows, group)
    wsorted = weights.flatten()[order].to(y.dtype).unsqueeze(-1)
    out = torch.zeros_like(x).index_add(0, tok, y * wsorted)
    return out


def moe_experts_ep(x: torch.Tensor, w13_local: torch.Tensor, w2_local: torch.Tensor, weights: torch.Tensor,
                   idx: torch.Tensor, num_experts: int, group: Any, fused: bool = True,
                   deterministic: bool = False, counts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Routed experts with the experts sharded over ``group``; same result as ``ops.moe.moe_experts`` on the
    unsharded weights.  x [T,H] local tokens; idx holds global expert ids."""
    if not x.is_cuda:
        return _moe_experts_ep_reference(x, w13_local, w2_local, weights, idx, num_experts, group)
    if fused:
        from . import fused as fz
        if fz.enabled():
            return fz.moe_experts_ep_fused(x, w13_local, w2_local, weights, idx, num_experts, group, deterministic,
                                           counts)
    ep = dist.get_world_size(group)
    e_local = num_experts // ep
    dev = x.device
    idx = idx.int()
    if counts is None:
        counts = torch.bincount(idx.flatten().long(), minlength=num_experts)
    counts = counts.int()
    xp, seg, _te, _nt, row_map = _PermuteFn.apply(x.to(_BF16), idx, counts, num_experts, deterministic)
    padded = (seg[1:] - seg[:-1]).contiguous()                          # padded rows per global expert
    recv_counts = _exchange_counts(padded, ep, group)                   # [ep(src), e_local]
    host = torch.cat([padded.view(ep, e_local).sum(1), recv_counts.flatten()]).cpu().tolist()   # one D2H read
    send_rows = [int(v) for v in host[:ep]]
    rc = [[int(v) for v in host[ep + s * e_local: ep + (s + 1) * e_local]] for s in range(ep)]
    recv_rows = [sum(r) for r in rc]
    total_send = sum(send_rows)
    xr = all_to_all_rows(xp[:total_send], send_rows, recv_rows, group)
    blocks = []
    r0 = 0
    ar = torch.arange(e_local, device=dev, dtype=torch.int32)
    for s in range(ep):
        n = recv_rows[s]
        if n:
            cnt = recv_counts[s]
            seg_s = torch.zeros(e_local + 1, dtype=torch.int32, device=dev)
            seg_s[1:] = torch.cumsum(cnt, 0)
            te = torch.repeat_interleave(ar, (cnt // 128).long(), output_size=n // 128).int()
            nt = torch.full((1,), n // 128, dtype=torch.int32, device=dev)
            blocks.append((r0, n, seg_s, te, nt))
        r0 += n
    y2r = _GroupedFFNFn.apply(xr, w13_local, w2_local, tuple(blocks))
    y2 = all_to_all_rows(y2r, recv_rows, send_rows, group)
    return _CombineFn.apply(y2, row_map, weights, seg, counts)
