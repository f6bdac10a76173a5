"""Mixture-of-experts operators: routing (gate kernel), and the routed expert computation
(permute -> grouped GEMM -> SwiGLU -> grouped GEMM -> weighted combine) as one autograd function that
never synchronises with the host: the expert-sorted row buffer is sized by its upper bound
``T*k + E*127`` and the grouped GEMM reads the real tile count from device memory.

Replaces the reference's Python expert loop (model/moe/layer.py:915-936) and its "fused" dispatch with a
``.cpu().tolist()`` sync (opss/infer/fused_moe.py:54-123).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import kernels, reference as ref, status_word

_BF16 = torch.bfloat16


def _k():
    return kernels()


# --------------------------------------------------------------------------------------------------
# routing
# --------------------------------------------------------------------------------------------------
class _GateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, k, bias_in_combine, renorm_mode):
        T, E = logits.shape
        lf = logits.float().contiguous()
        w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
        idx = torch.empty(T, k, dtype=torch.int32, device=logits.device)
        probs = torch.empty(T, E, dtype=torch.float32, device=logits.device)
        counts = torch.zeros(E, dtype=torch.int32, device=logits.device)
        _k().gate_topk(lf, bias, w, idx, probs, counts, bias_in_combine, renorm_mode)
        ctx.save_for_backward(probs, idx, w)
        ctx.renorm_mode = renorm_mode
        ctx.in_dtype = logits.dtype
        ctx.mark_non_differentiable(idx, counts, probs)
        return w, idx, counts, probs

    @staticmethod
    def backward(ctx, dw, _didx, _dcounts, _dprobs):
        probs, idx, w = ctx.saved_tensors
        dlogits = torch.empty_like(probs)
        _k().gate_topk_bwd(dw.float().contiguous(), probs, idx, w, dlogits, ctx.renorm_mode)
        return dlogits.to(ctx.in_dtype), None, None, None, None


def gate_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], k: int, bias_in_combine: bool = True,
              renorm_mode: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """logits [T,E] -> (weights [T,k] fp32, idx [T,k], counts [E], probs [T,E]).

    ``bias`` (aux-loss-free balancing) is added before the softmax when ``bias_in_combine`` (reference
    behaviour, model/moe/gate.py:378) or only to the selection key otherwise (DeepSeek-V3 style).
    ``renorm_mode`` 0 divides the selected probabilities by their sum; 1 applies a softmax over them
    (reference, gate.py:1221)."""
    if logits.is_cuda:
        b = bias.float().contiguous() if bias is not None else None
        return _GateFn.apply(logits, b, k, bias_in_combine, renorm_mode)
    w, idx, probs, counts = ref.gate_topk(logits, bias, k, bias_in_combine, renorm_mode)
    return w, idx, counts, probs


# --------------------------------------------------------------------------------------------------
# dispatch plan
# --------------------------------------------------------------------------------------------------
class DispatchPlan:
    """Device-side description of one expert-sorted, 128-row-padded token layout."""
    __slots__ = ("seg_offsets", "tile_expert", "num_m_tiles", "row_map", "counts", "max_rows", "k")

    def __init__(self, seg_offsets, tile_expert, num_m_tiles, row_map, counts, max_rows, k):
        self.seg_offsets, self.tile_expert, self.num_m_tiles = seg_offsets, tile_expert, num_m_tiles
        self.row_map, self.counts, self.max_rows, self.k = row_map, counts, max_rows, k


def padded_rows_bound(num_assignments: int, num_experts: int) -> int:
    """Upper bound of the padded row count: every expert wastes at most 127 rows."""
    return ((num_assignments + num_experts * 127 + 127) // 128) * 128


def permute_tokens(x: torch.Tensor, idx: torch.Tensor, counts: torch.Tensor, num_experts: int,
                   deterministic: bool = False, zero_pad: bool = True) -> Tuple[torch.Tensor, DispatchPlan]:
    """Scatter token rows into expert-sorted order.  Returns (xp [max_rows, H], plan).  The pad rows of every expert
    segment are zeroed unless ``zero_pad`` is off: the weight-gradient GEMMs sum over whole segments, so training
    needs zeros there; inference never reads what the pad rows produce."""
    T, H = x.shape
    k = idx.shape[1]
    dev = x.device
    max_rows = padded_rows_bound(T * k, num_experts)
    K = _k()
    seg = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(max_rows // 128, dtype=torch.int32, device=dev)
    num_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    cursor = torch.empty(num_experts, dtype=torch.int32, device=dev)
    K.moe_plan(counts, seg, tile_expert, num_tiles, cursor)
    xp = torch.empty(max_rows, H, dtype=_BF16, device=dev)
    row_map = torch.empty(T, k, dtype=torch.int32, device=dev)
    if deterministic:
        # assignment order inside an expert follows token order (what a stable sort by expert would give): one CTA per
        # expert counts its assignments in order
        K.moe_rank(idx.contiguous(), seg, row_map)
        K.moe_permute(x, idx, None, row_map, xp)
    else:
        K.moe_permute(x, idx, cursor, row_map, xp)
    if zero_pad:
        K.moe_zero_pad(xp, seg, counts)
    return xp, DispatchPlan(seg, tile_expert, num_tiles, row_map, counts, max_rows, k)


class _MoEExpertsFn(torch.autograd.Function):
    """Keeps only the token rows ``x`` and the up-projection output ``y1`` for backward (per micro-batch of 8192
    tokens x top-6 at hidden 4096 / FFN 1408: 0.07 + 0.28 GB instead of 1.3 GB with the permuted rows, the activation
    and the expert outputs).  Backward rebuilds what it needs:
      * the permuted rows from ``x`` and the saved row map (one gather);
      * the activation from ``y1`` inside the SwiGLU-backward kernel;
      * the combine-weight gradient without the expert outputs: with ``dA' = dout[token] @ W2[e]`` (the UNWEIGHTED
        activation gradient), ``d weight = <SwiGLU(y1), dA'>`` per row, and the weight is applied afterwards
        (``dy1 = w * dSwiGLU(y1, dA')``, ``dW2 = dout^T (w * act)``).  That is also exact for assignments whose weight
        is zero (dropped by the capacity rule)."""

    @staticmethod
    def forward(ctx, x, w13, w2, weights, idx, counts, deterministic, training=True, fp8=None):
        K = _k()
        st = status_word(x.device)
        T, H = x.shape
        E, twoF, _ = w13.shape
        F = twoF // 2
        x = x.contiguous()
        mx = fp8 == "mx" and H % 128 == 0 and twoF % 128 == 0 and F % 128 == 0
        xp, plan = permute_tokens(x, idx, counts, E, deterministic, zero_pad=training or mx)
        y1 = torch.empty(plan.max_rows, twoF, dtype=_BF16, device=x.device)
        act = torch.empty(plan.max_rows, F, dtype=_BF16, device=x.device)
        y2 = torch.empty(plan.max_rows, H, dtype=_BF16, device=x.device)
        if mx:
            # forward products on the block-scaled fp8 tensor cores: rows quantised per 32 elements on the fly, the
            # expert weights once per optimizer step; backward stays in bf16 from the saved bf16 tensors
            from ..quant import fp8 as q8
            xq, xs = q8.quantize_mx(xp)
            del xp
            wq, ws = _mx_weight(w13)
            K.gemm_mxfp8(xq, xs, wq, ws, y1, plan.tile_expert, plan.num_m_tiles, 0, st)
            del xq, xs
            K.swiglu_fwd(y1, act)
            aq, as_ = q8.quantize_mx(act)
            wq, ws = _mx_weight(w2)
            K.gemm_mxfp8(aq, as_, wq, ws, y2, plan.tile_expert, plan.num_m_tiles, 0, st)
            del aq, as_
        else:
            K.gemm_grouped_m(xp, w13, y1, plan.tile_expert, plan.num_m_tiles, False, 0, st)
            del xp
            K.swiglu_fwd(y1, act)
            K.gemm_grouped_m(act, w2, y2, plan.tile_expert, plan.num_m_tiles, False, 0, st)
        del act
        out = torch.empty(T, H, dtype=_BF16, device=x.device)
        wts = weights.float().contiguous()
        K.moe_combine(y2, plan.row_map, wts, None, out)
        ctx.save_for_backward(x, y1, w13, w2, wts, idx, plan.row_map, plan.seg_offsets, plan.tile_expert,
                              plan.num_m_tiles, plan.counts)
        ctx.dims = (T, H, E, F, plan.max_rows, idx.shape[1])
        ctx.w_dtype = weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        K = _k()
        x, y1, w13, w2, wts, idx, row_map, seg, tile_expert, num_tiles, counts = ctx.saved_tensors
        T, H, E, F, max_rows, k = ctx.dims
        st = status_word(dout.device)
        dev = dout.device
        dout = dout.contiguous()
        # combine weight of every expert row (0 on pad rows)
        row_w = torch.zeros(max_rows, dtype=torch.float32, device=dev)
        row_w.index_put_((row_map.flatten().long(),), wts.flatten())
        # unweighted output gradient in expert-row order
        dy2 = torch.empty(max_rows, H, dtype=_BF16, device=dev)
        K.moe_permute(dout, idx, None, row_map, dy2)
        K.moe_zero_pad(dy2, seg, counts)
        # down projection (unweighted activation gradient), then the activation with the weights applied
        dact = torch.empty(max_rows, F, dtype=_BF16, device=dev)
        K.gemm_grouped_m(dy2, w2, dact, tile_expert, num_tiles, True, 0, st)          # dy2 [rows,H] x w2[e] [H,F]
        dy1 = torch.empty_like(y1)
        act_w = torch.empty(max_rows, F, dtype=_BF16, device=dev)
        rowdot = torch.empty(max_rows, dtype=torch.float32, device=dev)
        K.swiglu_bwd_rows(y1, dact, row_w, dy1, act_w, rowdot)
        del dact
        dw2 = torch.empty_like(w2)
        K.gemm_grouped_k(dy2, act_w, dw2, seg, False, 0, st)                          # [H, rows_e] x [rows_e, F]
        del dy2, act_w
        dwts = rowdot[row_map.flatten().long()].view(T, k)
        # up projection
        dxp = torch.empty(max_rows, H, dtype=_BF16, device=dev)
        K.gemm_grouped_m(dy1, w13, dxp, tile_expert, num_tiles, True, 0, st)          # dy1 [rows,2F] x w13[e] [2F,H]
        xp = torch.empty(max_rows, H, dtype=_BF16, device=dev)
        K.moe_permute(x, idx, None, row_map, xp)
        K.moe_zero_pad(xp, seg, counts)
        dw13 = torch.empty_like(w13)
        K.gemm_grouped_k(dy1, xp, dw13, seg, False, 0, st)
        del xp, dy1
        dx = torch.empty(T, H, dtype=_BF16, device=dev)
        K.moe_unpermute_sum(dxp, row_map, dx, k)
        return dx, dw13, dw2, dwts.to(ctx.w_dtype), None, None, None, None, None


_MX_WEIGHTS: dict = {}


def _mx_weight(w: torch.Tensor):
    """Block-scaled copy of a stacked expert weight [E, N, K] (quantised again only after the tensor changed)."""
    from ..quant import fp8 as q8
    key = (w.data_ptr(), w._version, tuple(w.shape))
    hit = _MX_WEIGHTS.get(w.data_ptr())
    if hit is None or hit[0] != key:
        E, N, Kd = w.shape
        q, sf = q8.quantize_mx(w.detach().reshape(E * N, Kd))
        hit = (key, q.view(E, N, Kd), sf)
        _MX_WEIGHTS[w.data_ptr()] = hit
    return hit[1], hit[2]


def moe_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, weights: torch.Tensor, idx: torch.Tensor,
                counts: Optional[torch.Tensor] = None, deterministic: bool = False,
                fp8: Optional[str] = None) -> torch.Tensor:
    """Routed experts: out[t] = sum_j weights[t,j] * SwiGLU_FFN_{idx[t,j]}(x[t]).

    x [T,H]; w13 [E, 2F, H] (gate rows then up rows); w2 [E, H, F]; weights/idx [T,k]; counts [E] int32
    (the histogram the gate kernel produced; recomputed when omitted).  ``fp8="mx"`` runs the two forward products
    with e4m3 operands and one power-of-two scale per 32 elements (CUDA; H, F multiples of 128)."""
    if not x.is_cuda:
        return ref.moe_experts(x, w13, w2, weights, idx)
    E = w13.shape[0]
    if counts is None:
        counts = torch.bincount(idx.flatten().long(), minlength=E).int()
    # without autograd (inference) nothing reads what the pad rows of the expert segments produce: skip zeroing them
    return _MoEExpertsFn.apply(x.to(_BF16), w13, w2, weights, idx.int(), counts.int(), deterministic,
                               torch.is_grad_enabled(), fp8)


def capacity_mask(weights: torch.Tensor, idx: torch.Tensor, probs: torch.Tensor, counts: torch.Tensor,
                  capacity: int) -> torch.Tensor:
    """Capacity rule on the GPU: inside every expert keep the ``capacity`` assignments with the highest routing
    probability (ties by token order), zero the others and renormalise each token's weights.  No autograd: the
    result replaces the gate's weights in the forward value, gradients flow through the kept weights' own graph in
    the caller."""
    keep = torch.empty(idx.shape, dtype=torch.uint8, device=idx.device)
    out = torch.empty(idx.shape, dtype=torch.float32, device=idx.device)
    _k().moe_capacity_mask(weights.detach().float().contiguous(), idx.int().contiguous(), probs.detach().float().contiguous(),
                           counts.int().contiguous(), keep, out, int(capacity))
    return out, keep


def update_gate_bias(bias: torch.Tensor, counts: torch.Tensor, rate: float, clamp: float = 2.0) -> None:
    """Aux-loss-free balancing: bias += rate * (1/E - usage), clamped (reference gate.py:1059-1094)."""
    if bias.is_cuda:
        _k().gate_bias_update(bias, counts.int(), rate, clamp)
        return
    usage = counts.float() / counts.sum().clamp_min(1).float()
    bias.add_(rate * (1.0 / bias.numel() - usage)).clamp_(-clamp, clamp)
