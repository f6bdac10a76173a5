"""Context parallelism: the sequence is sharded over the ranks of a group and attention stays exact.

Two schemes:

``ring_attention``       K/V blocks travel round the ring; every step attends the local queries to the block in hand
                         and merges with the running result through the log-sum-exp (online softmax), so the output
                         equals full softmax attention.  The reference's distributed ring sums ``exp(s - chunk_max)``
                         without rescaling by a running maximum and applies the causal mask only on ring step 0
                         (model/core/attention.py:2961-2980) - not reproduced.  The next block is fetched while the
                         current one is computed: NCCL ``isend/irecv`` on the NCCL stream, or a pull copy from the
                         owner's published K/V in symmetric memory on a side stream (the remote block is brought into
                         local memory once and every CTA reads it from there).
``allgather_attention``  differentiable variant for training: K/V are all-gathered (backward: reduce-scatter of their
                         gradients) and every rank attends its query chunk to the keys up to its causal horizon.  With
                         ``zigzag`` every rank owns chunk r and chunk 2W-1-r, which balances causal work.
"""
from __future__ import annotations

import math
from typing import Any, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import functional as F_
from ..ops import kernels, reference as ref, status_word


def merge_partials(o1: torch.Tensor, lse1: torch.Tensor, o2: torch.Tensor, lse2: torch.Tensor):
    """Combine two attention partials over disjoint key sets.  o [T, h, d] fp32, lse [T, h] natural log."""
    lse = torch.logaddexp(lse1, lse2)
    w1 = torch.exp(lse1 - lse).unsqueeze(-1)
    w2 = torch.exp(lse2 - lse).unsqueeze(-1)
    w1 = torch.nan_to_num(w1, nan=0.0)
    w2 = torch.nan_to_num(w2, nan=0.0)
    return o1 * w1 + o2 * w2, lse


def _attend_block(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, hq: int, hk: int, d: int, causal: bool,
                  scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """One sequence: q [Lq, hq*d], k/v [Lk, hk*d] -> (o [Lq, hq, d] fp32, lse [Lq, hq])."""
    Lq, Lk = q.shape[0], k.shape[0]
    if q.is_cuda:
        K = kernels()
        o = torch.empty(Lq, hq * d, dtype=torch.bfloat16, device=q.device)
        lse = torch.empty(hq, Lq, dtype=torch.float32, device=q.device)
        cq = torch.tensor([0, Lq], dtype=torch.int32, device=q.device)
        ck = torch.tensor([0, Lk], dtype=torch.int32, device=q.device)
        K.attn_fwd(q.contiguous(), k.contiguous(), v.contiguous(), o, lse, cq, ck, Lq, Lk, hq, hk, d, causal, scale,
                   status_word(q.device))
        return o.view(Lq, hq, d).float(), lse.t().contiguous()
    qq = q.float().view(Lq, hq, d).transpose(0, 1)
    kk = k.float().view(Lk, hk, d).transpose(0, 1).repeat_interleave(hq // hk, 0)
    vv = v.float().view(Lk, hk, d).transpose(0, 1).repeat_interleave(hq // hk, 0)
    s = qq @ kk.transpose(1, 2) * scale
    if causal:
        i = torch.arange(Lq).unsqueeze(1)
        j = torch.arange(Lk).unsqueeze(0)
        s = s.masked_fill(j > i + (Lk - Lq), float("-inf"))
    lse = torch.logsumexp(s, -1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    return (p @ vv).transpose(0, 1).contiguous(), lse.t().contiguous()


@torch.no_grad()
def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group: Any, hq: int, hk: int, d: int,
                   causal: bool = True, scale: Optional[float] = None, fused: Optional[bool] = None) -> torch.Tensor:
    """Exact attention for a sequence sharded contiguously over ``group``: rank r holds tokens
    [r*L, (r+1)*L).  q [L, hq*d], k/v [L, hk*d] local shards -> local output [L, hq*d]."""
    W, r = dist.get_world_size(group), dist.get_rank(group)
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    L = q.shape[0]
    use_fused = fused
    if use_fused is None:
        from . import fused as fz
        use_fused = q.is_cuda and fz.enabled()
    pub = None
    if use_fused:
        from . import fused as fz
        heap = fz.heap_for(group)
        nbytes = k.numel() * 2
        pub = heap.get("cp_kv_pub", 2 * nbytes)
        heap.barrier()
        t = pub.tensor(torch.bfloat16, 2 * k.numel())
        t[: k.numel()].copy_(k.reshape(-1))
        t[k.numel():].copy_(v.reshape(-1))
        heap.barrier()
    o_acc = lse_acc = None
    cur_k, cur_v = k.contiguous(), v.contiguous()
    side = torch.cuda.Stream() if (use_fused and q.is_cuda) else None
    for step in range(W):
        src = (r - step) % W                         # owner of the block in hand
        nxt = None
        if step + 1 < W:
            nsrc = (r - step - 1) % W
            if use_fused:
                nk, nv = torch.empty_like(k), torch.empty_like(v)
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    kernels().peer_copy(nk.data_ptr(), pub.peer_ptrs[nsrc], k.numel() * 2)
                    kernels().peer_copy(nv.data_ptr(), pub.peer_ptrs[nsrc] + k.numel() * 2, k.numel() * 2)
                nxt = (nk, nv, None)
            else:
                nk, nv = torch.empty_like(k), torch.empty_like(v)
                reqs = dist.batch_isend_irecv([
                    dist.P2POp(dist.isend, cur_k, dist.get_global_rank(group, (r + 1) % W), group),
                    dist.P2POp(dist.isend, cur_v, dist.get_global_rank(group, (r + 1) % W), group),
                    dist.P2POp(dist.irecv, nk, dist.get_global_rank(group, (r - 1) % W), group),
                    dist.P2POp(dist.irecv, nv, dist.get_global_rank(group, (r - 1) % W), group)])
                nxt = (nk, nv, reqs)
        if not causal or src <= r:
            o_b, lse_b = _attend_block(q, cur_k, cur_v, hq, hk, d, causal and src == r, scale)
            if o_acc is None:
                o_acc, lse_acc = o_b, lse_b
            else:
                o_acc, lse_acc = merge_partials(o_acc, lse_acc, o_b, lse_b)
        if nxt is not None:
            if nxt[2] is not None:
                for rq in nxt[2]:
                    rq.wait()
            elif side is not None:
                torch.cuda.current_stream().wait_stream(side)
            cur_k, cur_v = nxt[0], nxt[1]
    return o_acc.reshape(L, hq * d).to(q.dtype)


# --------------------------------------------------------------------------------------------------
# differentiable ring attention
# --------------------------------------------------------------------------------------------------
def _ring_exchange(tensors: List[torch.Tensor], group: Any, r: int, W: int) -> Tuple[List[torch.Tensor], list]:
    """Post the sends of ``tensors`` to rank r+1 and the receives of their successors from rank r-1."""
    recv = [torch.empty_like(t) for t in tensors]
    nxt, prv = dist.get_global_rank(group, (r + 1) % W), dist.get_global_rank(group, (r - 1) % W)
    ops = [dist.P2POp(dist.isend, t, nxt, group) for t in tensors] + [dist.P2POp(dist.irecv, t, prv, group) for t in recv]
    return recv, dist.batch_isend_irecv(ops)


def _merge_into(o_acc: torch.Tensor, lse_acc: torch.Tensor, o_b: torch.Tensor, lse_b: torch.Tensor):
    """Running result (fp32 [L, hq, d], [L, hq]) <- merged with one block's partial.  On the GPU one kernel does the
    log-sum-exp, the two weights and the weighted sum in place."""
    if o_acc.is_cuda:
        kernels().attn_merge(o_acc, lse_acc, o_b.contiguous(), lse_b.contiguous())
        return o_acc, lse_acc
    return merge_partials(o_acc, lse_acc, o_b, lse_b)


def _block_backward(do, q, k, v, o, lse, hq, hk, d, causal, scale):
    """Gradients of ONE key/value block given the GLOBAL output and log-sum-exp of the local queries:
    p = exp(s - lse), dv = p^T do, ds = p * (do v^T - rowsum(do * o)), dq = ds k, dk = ds^T q."""
    L, Lk = q.shape[0], k.shape[0]
    if q.is_cuda:
        K = kernels()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty(hq, L, dtype=torch.float32, device=q.device)
        cq = torch.tensor([0, L], dtype=torch.int32, device=q.device)
        ck = torch.tensor([0, Lk], dtype=torch.int32, device=q.device)
        K.attn_bwd(do, q, k, v, o, lse, dq, dk, dv, delta, cq, ck, L, Lk, hq, hk, d, causal, scale, status_word(q.device))
        return dq.float(), dk.float(), dv.float()
    g = hq // hk
    qq = q.float().view(L, hq, d).transpose(0, 1)
    kk = k.float().view(Lk, hk, d).transpose(0, 1).repeat_interleave(g, 0)
    vv = v.float().view(Lk, hk, d).transpose(0, 1).repeat_interleave(g, 0)
    dd = do.float().view(L, hq, d).transpose(0, 1)
    oo = o.float().view(L, hq, d).transpose(0, 1)
    s_ = qq @ kk.transpose(1, 2) * scale
    if causal:
        i = torch.arange(L).unsqueeze(1)
        j = torch.arange(Lk).unsqueeze(0)
        s_ = s_.masked_fill(j > i + (Lk - L), float("-inf"))
    p_ = torch.nan_to_num(torch.exp(s_ - lse.unsqueeze(-1)), nan=0.0)             # lse [hq, L]
    dv = (p_.transpose(1, 2) @ dd).view(hk, g, Lk, d).sum(1)
    ds = p_ * (dd @ vv.transpose(1, 2) - (dd * oo).sum(-1, keepdim=True)) * scale
    dq = ds @ kk
    dk = (ds.transpose(1, 2) @ qq).view(hk, g, Lk, d).sum(1)
    return (dq.transpose(0, 1).reshape(L, hq * d), dk.transpose(0, 1).reshape(Lk, hk * d),
            dv.transpose(0, 1).reshape(Lk, hk * d))


class _RingAttention(torch.autograd.Function):
    """Exact causal / full attention over a sequence sharded contiguously over ``group`` with O(L) key/value memory
    per rank in BOTH directions.  Forward: K/V blocks travel round the ring, partials are merged through the
    log-sum-exp; only q, the local k/v, the bf16 output and the log-sum-exp are kept.  Backward: the blocks travel
    again together with their dK/dV accumulators; every rank adds the contribution of its queries to the block in
    hand (recomputing p from the saved global log-sum-exp), and after W hops each accumulator is back at its owner."""

    @staticmethod
    def forward(ctx, q, k, v, group, hq, hk, d, causal, scale):
        W, r = dist.get_world_size(group), dist.get_rank(group)
        L = q.shape[0]
        q, cur_k, cur_v = q.contiguous(), k.contiguous(), v.contiguous()
        o_acc = lse_acc = None
        for step in range(W):
            src = (r - step) % W
            nxt = _ring_exchange([cur_k, cur_v], group, r, W) if step + 1 < W else None
            if not causal or src <= r:
                o_b, lse_b = _attend_block(q, cur_k, cur_v, hq, hk, d, causal and src == r, scale)
                if o_acc is None:
                    o_acc, lse_acc = o_b.contiguous(), lse_b.contiguous()
                else:
                    o_acc, lse_acc = _merge_into(o_acc, lse_acc, o_b, lse_b)
            if nxt is not None:
                for rq in nxt[1]:
                    rq.wait()
                cur_k, cur_v = nxt[0]
        o = o_acc.reshape(L, hq * d).to(q.dtype)
        ctx.save_for_backward(q, k.contiguous(), v.contiguous(), o, lse_acc.t().contiguous())       # lse as [hq, L]
        ctx.cfg = (group, hq, hk, d, causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        group, hq, hk, d, causal, scale = ctx.cfg
        W, r = dist.get_world_size(group), dist.get_rank(group)
        do = do.contiguous().to(q.dtype)
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        cur = [k, v, torch.zeros(k.shape, dtype=torch.float32, device=k.device),
               torch.zeros(v.shape, dtype=torch.float32, device=v.device)]
        for step in range(W):
            src = (r - step) % W
            if not causal or src <= r:
                dq_b, dk_b, dv_b = _block_backward(do, q, cur[0], cur[1], o, lse, hq, hk, d, causal and src == r, scale)
                dq += dq_b
                cur[2] = cur[2] + dk_b
                cur[3] = cur[3] + dv_b
            # every hop moves the block and its gradient accumulators on; the last hop brings them home
            send = cur if step + 1 < W else cur[2:]
            recv, reqs = _ring_exchange([t.contiguous() for t in send], group, r, W)
            for rq in reqs:
                rq.wait()
            cur = recv if step + 1 < W else [None, None] + recv
        return dq.to(q.dtype), cur[2].to(k.dtype), cur[3].to(v.dtype), None, None, None, None, None, None


def ring_attention_train(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group: Any, hq: int, hk: int, d: int,
                         causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    """Differentiable ring attention: q [L, hq*d], k/v [L, hk*d] are this rank's contiguous chunk of one sequence."""
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    return _RingAttention.apply(q, k, v, group, hq, hk, d, causal, scale)


class _AllGatherKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        W = dist.get_world_size(group)
        out = torch.empty(W * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        W, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        n = g.shape[0] // W
        g = g.contiguous()
        if g.is_cuda:
            out = torch.empty(n, *g.shape[1:], dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out, g, group=ctx.group)
        else:
            g = g.clone()
            dist.all_reduce(g, group=ctx.group)
            out = g[r * n:(r + 1) * n].contiguous()
        return out, None


def allgather_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group: Any, hq: int, hk: int, d: int,
                        causal: bool = True, scale: Optional[float] = None, zigzag: bool = False) -> torch.Tensor:
    """Differentiable context-parallel attention for one sequence.  Contiguous layout: rank r holds chunk r.
    Zig-zag layout: rank r holds chunks (r, 2W-1-r) stacked, each of length L/2."""
    W, r = dist.get_world_size(group), dist.get_rank(group)
    kg, vg = _AllGatherKV.apply(k, group), _AllGatherKV.apply(v, group)
    L = q.shape[0]

    def attend(qc: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, is_causal: bool) -> torch.Tensor:
        cq = torch.tensor([0, qc.shape[0]], dtype=torch.int32, device=q.device)
        ck = torch.tensor([0, kc.shape[0]], dtype=torch.int32, device=q.device)
        return F_.attention(qc, kc, vc, cq, ck, qc.shape[0], kc.shape[0], hq, hk, d, causal=is_causal, scale=scale)

    if not zigzag:
        horizon = (r + 1) * L if causal else W * L
        return attend(q, kg[:horizon], vg[:horizon], causal)
    half = L // 2
    # gathered order is [r0: (c0, c_{2W-1})], [r1: (c1, c_{2W-2})], ... ; rebuild the sequence order
    idx = []
    for c in range(2 * W):
        owner = c if c < W else 2 * W - 1 - c
        slot = 0 if c < W else 1
        idx.append(torch.arange(owner * L + slot * half, owner * L + (slot + 1) * half, device=q.device))
    order = torch.cat(idx)
    ks, vs = kg[order], vg[order]
    outs = []
    for slot, c in enumerate((r, 2 * W - 1 - r)):
        horizon = (c + 1) * half if causal else 2 * W * half
        outs.append(attend(q[slot * half:(slot + 1) * half], ks[:horizon], vs[:horizon], causal))
    return torch.cat(outs, 0)
