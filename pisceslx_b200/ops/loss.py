"""Fused LM-head + cross-entropy: logits are produced chunk by chunk ([chunk, V] fp32), turned into
per-token losses and logit gradients by one kernel, and immediately contracted into dH and dW, so the
[T, V] logits tensor never exists (the reference materialises it, model/core/model.py:2440,2505).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import kernels, reference as ref, status_word

_BF16 = torch.bfloat16


class _LinearCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, labels, ignore_index, scale, chunk):
        K = kernels()
        st = status_word(h.device)
        T, H = h.shape
        V = w.shape[0]
        dev = h.device
        h = h.contiguous()
        need_dh = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        loss_rows = torch.empty(T, dtype=torch.float32, device=dev)
        dh = torch.empty_like(h) if need_dh else None
        n_chunks = (T + chunk - 1) // chunk
        dw32 = None
        dw = None
        if need_dw:
            if n_chunks > 1:
                dw32 = torch.zeros(V, H, dtype=torch.float32, device=dev)
            else:
                dw = torch.empty(V, H, dtype=_BF16, device=dev)
        logits = torch.empty(min(chunk, T), V, dtype=torch.float32, device=dev)
        dlogits = torch.empty(min(chunk, T), V, dtype=_BF16, device=dev) if (need_dh or need_dw) else None
        for c in range(n_chunks):
            r0, r1 = c * chunk, min(T, (c + 1) * chunk)
            n = r1 - r0
            lg = logits[:n]
            K.gemm(h[r0:r1], w, lg, False, False, False, 0, st)
            dl = dlogits[:n] if dlogits is not None else None
            K.ce_fwd_bwd(lg, labels[r0:r1], loss_rows[r0:r1], dl, ignore_index, scale)
            if need_dh:
                K.gemm(dl, w, dh[r0:r1], False, True, False, 0, st)                 # [n,V] x [V,H]
            if need_dw:
                if dw32 is not None:
                    K.gemm(dl, h[r0:r1], dw32, True, True, True, 0, st)             # [V,n] x [n,H], accumulate
                else:
                    K.gemm(dl, h[r0:r1], dw, True, True, False, 0, st)
        if dw32 is not None:
            dw = dw32.to(_BF16)
            del dw32
        ctx.save_for_backward(dh, dw)
        return loss_rows.sum() * scale

    @staticmethod
    def backward(ctx, gout):
        dh, dw = ctx.saved_tensors
        K = kernels()
        g = gout.reshape(1).float().contiguous()
        if dh is not None:
            K.scale_(dh, g, 1.0)
        if dw is not None:
            K.scale_(dw, g, 1.0)
        return dh, dw, None, None, None, None


def linear_cross_entropy(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                         num_valid: Optional[int] = None, chunk: int = 2048) -> torch.Tensor:
    """Mean next-token loss of ``softmax(h @ w.T)`` against ``labels`` (already shifted by the caller).

    h [T,H], w [V,H], labels [T] int64.  ``num_valid`` is the number of labels != ignore_index; pass it
    from the host-side batch to avoid a device synchronisation (it is counted on the device otherwise)."""
    if num_valid is None:
        num_valid = int((labels != ignore_index).sum().item())
    scale = 1.0 / max(num_valid, 1)
    if h.is_cuda:
        return _LinearCEFn.apply(h.to(_BF16), w, labels.contiguous(), ignore_index, scale, chunk)
    loss, _ = ref.linear_cross_entropy(h, w, labels, ignore_index)
    return loss * scale
