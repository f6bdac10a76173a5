"""Differentiable operator API used by the models.

CUDA tensors run the sm_100a kernels through ``torch.autograd.Function`` wrappers that allocate their
outputs with the caching allocator and never synchronise with the host; CPU tensors run
``ops.reference``.  Shapes follow the "tokens first" convention: activations are 2-D ``[T, features]``
with sequences packed along ``T`` and described by ``cu_seqlens``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import kernels, reference as ref, status_word

_BF16 = torch.bfloat16
_NORM_BWD_BLOCKS = 148 * 4


def _k():
    return kernels()


def _st(t: torch.Tensor) -> torch.Tensor:
    return status_word(t.device)


def _as2d(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1, x.shape[-1])


# --------------------------------------------------------------------------------------------------
# linear
# --------------------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = _BF16, accumulate: bool = False,
         bn: int = 0) -> torch.Tensor:
    """Raw tcgen05 GEMM: C[M,N] = A * B with the storage layouts described in ``csrc/yv_ops.h``."""
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    _k().gemm(a, b, out, a_mn, b_mn, accumulate, bn, _st(a))
    return out


_SPLITK_OFFSETS: dict = {}
_SPLITK_WS: dict = {}


def _splitk_plan(M: int, N: int, K: int) -> int:
    """Number of K slices for a skinny product (0 = do not split).  With at most 128 rows the N tiles alone cover
    a fraction of the 148 SMs and the weight matrix streams at a fraction of HBM bandwidth; slicing K multiplies
    the CTAs that pull weight bytes.  The choice depends on (N, K) only, so a row's result does not depend on how
    many other rows share the launch."""
    if M > 128 or K % 64 != 0 or N % 4 != 0:
        return 0
    tiles_n = (N + 255) // 256
    if tiles_n >= 74:
        return 0
    # the kernel is persistent with one CTA per SM and a static round-robin over work items: tiles_n * slices must not
    # exceed 148, or a second, nearly empty wave doubles the time
    want = min(16, 148 // tiles_n)
    slices = max(1, min(want, K // 256))
    return slices if slices > 1 else 0


def gemm_skinny(x2: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """y = x2 @ w.T through the split-K path, or None when the shape does not call for it."""
    M, K = x2.shape
    N = w.shape[0]
    slices = _splitk_plan(M, N, K)
    if slices == 0 or w.stride(1) != 1 or x2.stride(1) != 1:
        return None
    dev = x2.device
    key = (dev.index, K, slices)
    offs = _SPLITK_OFFSETS.get(key)
    if offs is None:
        per = -(-(K // 64) // slices) * 64
        offs = torch.tensor([min(K, i * per) for i in range(slices + 1)], dtype=torch.int32, device=dev)
        _SPLITK_OFFSETS[key] = offs
    need = slices * 128 * N
    ws = _SPLITK_WS.get(dev.index)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 16 * 128 * 8192), dtype=torch.float32, device=dev)
        _SPLITK_WS[dev.index] = ws
    out = torch.empty(M, N, dtype=_BF16, device=dev)
    _k().gemm_splitk(x2, w, ws, offs, bias, out, _st(x2))
    return out


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, out_fp32):
        x2 = _as2d(x)
        if not x2.is_contiguous() and x2.stride(1) != 1:
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        if not out_fp32 and x2.shape[0] <= 128:
            ys = gemm_skinny(x2, w)
            if ys is not None:
                return ys.view(*x.shape[:-1], w.shape[0])
        y = gemm(x2, w, out_dtype=torch.float32 if out_fp32 else _BF16)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _as2d(dy)
        if dy2.dtype != _BF16:
            dy2 = dy2.to(_BF16)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view(ctx.x_shape)           # [M,N] x [N,K]
        if ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True)                # [N,M] x [M,K]
        return dx, dw, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_fp32: bool = False) -> torch.Tensor:
    """y = x @ w.T (+ bias); w is [out, in]."""
    if x.is_cuda:
        if x.dtype != _BF16:
            x = x.to(_BF16)
        y = _LinearFn.apply(x, w if w.dtype == _BF16 else w.to(_BF16), out_fp32)
    else:
        y = torch.nn.functional.linear(x, w.to(x.dtype))
        if out_fp32:
            y = y.float()
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y


# --------------------------------------------------------------------------------------------------
# RMSNorm (+ residual add, + FiLM epilogue)
# --------------------------------------------------------------------------------------------------
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, eps, film_scale, film_shift):
        shape = x.shape
        x2 = _as2d(x).contiguous()
        rows, cols = x2.shape
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        res_out = None
        r2 = None
        if residual is not None:
            r2 = _as2d(residual).contiguous()
            res_out = torch.empty_like(x2)
        film_rows = 1
        fs = fb = None
        if film_scale is not None:
            fs = _as2d(film_scale).contiguous()
            fb = _as2d(film_shift).contiguous()
            assert rows % fs.shape[0] == 0, "FiLM groups must divide the rows"
            film_rows = rows // fs.shape[0]
        _k().rmsnorm_fwd(x2, r2, w, fs, fb, film_rows, y, res_out, rstd, eps)
        normed_in = res_out if res_out is not None else x2
        ctx.save_for_backward(normed_in, w, rstd, fs, fb)
        ctx.has_res = residual is not None
        ctx.film_rows = film_rows
        ctx.shape = shape
        if res_out is not None:
            return y.view(shape), res_out.view(shape)
        return y.view(shape), None

    @staticmethod
    def backward(ctx, dy, dres):
        xin, w, rstd, fs, fb = ctx.saved_tensors
        dy2 = _as2d(dy).contiguous()
        rows, cols = xin.shape
        dfs = dfb = None
        if fs is not None:
            # y = n * (1 + s) + b  ->  dn = dy * (1 + s), ds = sum_rows dy * n, db = sum_rows dy
            G = fs.shape[0]
            xf = xin.float() * rstd.unsqueeze(1) * w.float()
            dyf = dy2.float().view(G, ctx.film_rows, cols)
            dfs = (dyf * xf.view(G, ctx.film_rows, cols)).sum(1).to(fs.dtype)
            dfb = dyf.sum(1).to(fs.dtype)
            dy2 = (dyf * (1.0 + fs.float()).unsqueeze(1)).view(rows, cols).to(_BF16)
        dx = torch.empty_like(xin)
        dwp = torch.empty(min(rows, _NORM_BWD_BLOCKS), cols, dtype=torch.float32, device=xin.device)
        dw = torch.empty(cols, dtype=torch.float32, device=xin.device)
        dres2 = _as2d(dres).contiguous() if dres is not None else None
        _k().rmsnorm_bwd(dy2, xin, w, rstd, dres2, dx, dwp, dw, False)
        dx = dx.view(ctx.shape)
        return dx, (dx if ctx.has_res else None), dw.to(w.dtype), None, dfs, dfb


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None,
             film_scale: Optional[torch.Tensor] = None, film_shift: Optional[torch.Tensor] = None):
    """Returns ``(y, new_residual)``: y = rmsnorm(x + residual) * w [then FiLM]; new_residual = x + residual
    (``None`` when no residual is given)."""
    if x.is_cuda:
        return _RMSNormFn.apply(x, residual, w, eps, film_scale, film_shift)
    s = x if residual is None else x + residual
    y = ref.rms_norm(s, w, eps)
    if film_scale is not None:
        g = film_scale.shape[0] if film_scale.dim() == 2 else None
        y2 = y.reshape(film_scale.reshape(-1, y.shape[-1]).shape[0], -1, y.shape[-1])
        y = ref.film(y2, film_scale.reshape(-1, 1, y.shape[-1]), film_shift.reshape(-1, 1, y.shape[-1])).reshape(y.shape)
    return y, (s if residual is not None else None)


class _FiLMFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, shift):
        x2 = _as2d(x).contiguous()
        s2, b2 = _as2d(scale).contiguous(), _as2d(shift).contiguous()
        rows = x2.shape[0]
        assert rows % s2.shape[0] == 0
        y = torch.empty_like(x2)
        _k().film(x2, s2, b2, y, rows // s2.shape[0])
        ctx.save_for_backward(x2, s2)
        ctx.shapes = (x.shape, scale.shape, shift.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, s2 = ctx.saved_tensors
        G, cols = s2.shape
        dyf = _as2d(dy).float().view(G, -1, cols)
        dx = (dyf * (1.0 + s2.float()).unsqueeze(1)).to(dy.dtype).view(ctx.shapes[0])
        ds = (dyf * x2.float().view(G, -1, cols)).sum(1).to(s2.dtype).view(ctx.shapes[1])
        db = dyf.sum(1).to(s2.dtype).view(ctx.shapes[2])
        return dx, ds, db


def film(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    """x*(1+scale)+shift; scale/shift are ``[B,1,H]`` (per sample) or ``[B,S,H]`` (per token) for x ``[B,S,H]``."""
    if x.is_cuda and x.dtype == _BF16:
        return _FiLMFn.apply(x, scale.to(_BF16), shift.to(_BF16))
    return ref.film(x, scale.to(x.dtype), shift.to(x.dtype))


# --------------------------------------------------------------------------------------------------
# SwiGLU
# --------------------------------------------------------------------------------------------------
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        g2 = _as2d(gate_up).contiguous()
        f = g2.shape[1] // 2
        out = torch.empty(g2.shape[0], f, dtype=_BF16, device=g2.device)
        _k().swiglu_fwd(g2, out)
        ctx.save_for_backward(g2)
        ctx.shape = gate_up.shape
        return out.view(*gate_up.shape[:-1], f)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        din = torch.empty_like(g2)
        _k().swiglu_bwd(g2, _as2d(dout).contiguous(), din)
        return din.view(ctx.shape)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x[..., :F]) * x[..., F:]"""
    if gate_up.is_cuda and gate_up.dtype == _BF16:
        return _SwiGLUFn.apply(gate_up)
    return ref.swiglu(gate_up)


# --------------------------------------------------------------------------------------------------
# RoPE + flash attention on a fused QKV buffer
# --------------------------------------------------------------------------------------------------
class _RopeAttentionFn(torch.autograd.Function):
    """qkv [T, (hq+2hk)*d] -> o [T, hq*d].  RoPE is applied in place to the q and k columns of the buffer
    (after the call the buffer holds the rotated q/k, which is what a KV cache stores)."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, positions, cu_q, max_len, hq, hk, d, rot_dim, causal, scale):
        T = qkv.shape[0]
        q = qkv[:, : hq * d]
        k = qkv[:, hq * d: (hq + hk) * d]
        v = qkv[:, (hq + hk) * d:]
        K = _k()
        if cos is not None:
            K.rope(q, k, cos, sin, positions, hq, hk, d, rot_dim, False)
        o = torch.empty(T, hq * d, dtype=_BF16, device=qkv.device)
        lse = torch.empty(hq, T, dtype=torch.float32, device=qkv.device)
        K.attn_fwd(q, k, v, o, lse, cu_q, None, max_len, max_len, hq, hk, d, causal, scale, _st(qkv))
        ctx.save_for_backward(qkv, o, lse, cos, sin, positions, cu_q)
        ctx.cfg = (max_len, hq, hk, d, rot_dim, causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, cos, sin, positions, cu_q = ctx.saved_tensors
        max_len, hq, hk, d, rot_dim, causal, scale = ctx.cfg
        T = qkv.shape[0]
        q = qkv[:, : hq * d]
        k = qkv[:, hq * d: (hq + hk) * d]
        v = qkv[:, (hq + hk) * d:]
        dqkv = torch.empty_like(qkv)
        dq = dqkv[:, : hq * d]
        dk = dqkv[:, hq * d: (hq + hk) * d]
        dv = dqkv[:, (hq + hk) * d:]
        delta = torch.empty(hq, T, dtype=torch.float32, device=qkv.device)
        K = _k()
        K.attn_bwd(do.contiguous(), q, k, v, o, lse, dq, dk, dv, delta, cu_q, None, max_len, max_len, hq, hk, d,
                   causal, scale, _st(qkv))
        if cos is not None:
            K.rope(dq, dk, cos, sin, positions, hq, hk, d, rot_dim, True)
        return (dqkv,) + (None,) * 11


def rope_attention(qkv: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                   positions: Optional[torch.Tensor], cu_seqlens: torch.Tensor, max_len: int, hq: int, hk: int,
                   d: int, rot_dim: int, causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    """Self-attention over packed sequences from a fused projection ``qkv [T, (hq+2hk)*d]``."""
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if qkv.is_cuda:
        return _RopeAttentionFn.apply(qkv, cos, sin, positions, cu_seqlens, max_len, hq, hk, d, rot_dim, causal,
                                      scale)
    T = qkv.shape[0]
    q = qkv[:, : hq * d].reshape(T, hq, d)
    k = qkv[:, hq * d: (hq + hk) * d].reshape(T, hk, d)
    v = qkv[:, (hq + hk) * d:].reshape(T, hk, d)
    if cos is not None:
        q = ref.apply_rope(q, cos, sin, positions, rot_dim)
        k = ref.apply_rope(k, cos, sin, positions, rot_dim)
    return ref.attention_varlen(q, k, v, cu_seqlens, None, causal, scale).reshape(T, hq * d)


class _AttentionFn(torch.autograd.Function):
    """Separate q [Tq, hq*d], k/v [Tk, hk*d] (cross attention, no RoPE)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, hq, hk, d, causal, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o = torch.empty_like(q)
        lse = torch.empty(hq, q.shape[0], dtype=torch.float32, device=q.device)
        _k().attn_fwd(q, k, v, o, lse, cu_q, cu_k, max_q, max_k, hq, hk, d, causal, scale, _st(q))
        ctx.save_for_backward(q, k, v, o, lse, cu_q, cu_k)
        ctx.cfg = (max_q, max_k, hq, hk, d, causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, cu_q, cu_k = ctx.saved_tensors
        max_q, max_k, hq, hk, d, causal, scale = ctx.cfg
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty(hq, q.shape[0], dtype=torch.float32, device=q.device)
        _k().attn_bwd(do.contiguous(), q, k, v, o, lse, dq, dk, dv, delta, cu_q, cu_k, max_q, max_k, hq, hk, d, causal,
                      scale, _st(q))
        return (dq, dk, dv) + (None,) * 9


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q: torch.Tensor,
              cu_k: Optional[torch.Tensor], max_q: int, max_k: int, hq: int, hk: int, d: int,
              causal: bool = False, scale: Optional[float] = None) -> torch.Tensor:
    """Packed attention with separate query / key sequences: q [Tq, hq*d], k/v [Tk, hk*d] -> [Tq, hq*d]."""
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if q.is_cuda:
        return _AttentionFn.apply(q.to(_BF16), k.to(_BF16), v.to(_BF16), cu_q, cu_k, max_q, max_k, hq, hk, d,
                                  causal, scale)
    o = ref.attention_varlen(q.reshape(-1, hq, d), k.reshape(-1, hk, d), v.reshape(-1, hk, d), cu_q, cu_k, causal,
                             scale)
    return o.reshape(-1, hq * d)


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                 seq_lens: torch.Tensor, scale: Optional[float] = None, splits: int = 0) -> torch.Tensor:
    """One decode step over the paged cache: q [B,hq,d] -> [B,hq,d] (no autograd)."""
    B, hq, d = q.shape
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if not q.is_cuda:
        return ref.paged_decode(q, k_cache, v_cache, block_table, seq_lens, scale)
    if splits <= 0:
        ctas = B * k_cache.shape[2]
        # one CTA per SM is resident: aim at four or more waves of CTAs so that the last, partial wave is a small
        # share of the run, without cutting a sequence into pieces shorter than two 128-key tiles
        splits = max(1, min(32, -(-(4 * 148) // max(ctas, 1))))
        splits = min(splits, max(1, block_table.shape[1] // 4))
    o = torch.empty_like(q)
    po = torch.empty(B, hq, splits, d, dtype=torch.float32, device=q.device)
    pml = torch.empty(B, hq, splits, 2, dtype=torch.float32, device=q.device)
    _k().paged_decode(q.contiguous(), k_cache, v_cache, block_table, seq_lens, o, po, pml, splits, scale, _st(q))
    return o


def kv_cache_write(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   slot_map: torch.Tensor) -> None:
    """Append rows k/v [T, hk*d] to the paged caches at flat slots ``slot_map`` (int32, -1 = skip)."""
    if k.is_cuda:
        _k().kv_cache_write(k, v, k_cache, v_cache, slot_map, _st(k))
        return
    row = k.shape[1]
    kc, vc = k_cache.view(-1, row), v_cache.view(-1, row)
    keep = slot_map >= 0
    kc[slot_map[keep].long()] = k[keep]
    vc[slot_map[keep].long()] = v[keep]
