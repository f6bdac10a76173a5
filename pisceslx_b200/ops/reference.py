"""Plain PyTorch statements of every op (the oracle the CUDA kernels are tested against, and the code
path CPU tensors take).  Everything here is differentiable by autograd and dtype-agnostic; tests call
it in fp32.

Reference-parity notes: RMSNorm math follows model/core/norms.py:1003-1007 of the reference; FiLM is
``h*(1+scale)+shift`` (norms.py:171); the gate is softmax -> top-k -> renormalise
(model/moe/gate.py:1211-1240); AdamW applies decay to the pre-update parameter
(opss/kernels/fused_adamw.py:89); Muon's Newton-Schulz uses the reference's coefficient schedule
(utils/muon.py:258-271).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------------------
# normalisation / FiLM / activations
# --------------------------------------------------------------------------------------------------
def film(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    return x * (1.0 + scale) + shift


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return y.to(x.dtype)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    f = gate_up.shape[-1] // 2
    return F.silu(gate_up[..., :f]) * gate_up[..., f:]


# --------------------------------------------------------------------------------------------------
# rotary embeddings (rotate-half layout)
# --------------------------------------------------------------------------------------------------
def rope_tables(max_pos: int, rot_dim: int, theta: float = 1e4, scaling: float = 1.0,
                device: Optional[torch.device] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables fp32 [max_pos, rot_dim/2]; ``scaling`` divides positions (linear RoPE scaling)."""
    half = rot_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / rot_dim))
    pos = torch.arange(max_pos, dtype=torch.float64) / scaling
    ang = torch.outer(pos, inv)
    return ang.cos().float().to(device), ang.sin().float().to(device)


def yarn_tables(max_pos: int, rot_dim: int, theta: float, factor: float, original_max: int,
                beta_fast: float = 32.0, beta_slow: float = 1.0,
                device: Optional[torch.device] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """YaRN: interpolate low frequencies by ``factor``, keep high ones, blend in between."""
    half = rot_dim // 2
    idx = torch.arange(0, half, dtype=torch.float64)
    inv = 1.0 / (theta ** (idx * 2.0 / rot_dim))

    def corr(n_rot: float) -> float:
        return rot_dim * math.log(original_max / (n_rot * 2 * math.pi)) / (2 * math.log(theta))

    lo, hi = max(math.floor(corr(beta_fast)), 0), min(math.ceil(corr(beta_slow)), half - 1)
    ramp = ((idx - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
    inv = inv / factor * ramp + inv * (1 - ramp)
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), inv)
    m = 0.1 * math.log(factor) + 1.0 if factor > 1 else 1.0
    return (ang.cos() * m).float().to(device), (ang.sin() * m).float().to(device)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor,
               rot_dim: int) -> torch.Tensor:
    """x: [T, heads, d]; rotates the first ``rot_dim`` dims of every head."""
    half = rot_dim // 2
    c = cos[positions.long()].unsqueeze(1).to(torch.float32)
    s = sin[positions.long()].unsqueeze(1).to(torch.float32)
    xf = x.float()
    a, b, rest = xf[..., :half], xf[..., half:rot_dim], xf[..., rot_dim:]
    out = torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)
    return out.to(x.dtype)


def apply_rope3d(x: torch.Tensor, pos_thw: torch.Tensor, sections: Sequence[int], theta: float = 1e4) -> torch.Tensor:
    """x: [T, heads, d]; the head dim is split into (t, h, w) sections, each rotated by its own position."""
    xf = x.float()
    outs, off = [], 0
    for s_i, dsec in enumerate(sections):
        half = dsec // 2
        inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32, device=x.device) * 2.0 / dsec))
        ang = pos_thw[:, s_i].float().unsqueeze(-1) * inv
        c, s = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
        a, b = xf[..., off:off + half], xf[..., off + half:off + dsec]
        outs += [a * c - b * s, b * c + a * s]
        off += dsec
    outs.append(xf[..., off:])
    return torch.cat(outs, -1).to(x.dtype)


# --------------------------------------------------------------------------------------------------
# MoE
# --------------------------------------------------------------------------------------------------
def gate_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], k: int, bias_in_combine: bool = True,
              renorm_mode: int = 0):
    """Returns (weights [T,k] fp32, idx [T,k] int64, probs [T,E], counts [E])."""
    lf = logits.float()
    sel = lf + bias.float() if bias is not None else lf
    probs = torch.softmax(sel if bias_in_combine else lf, dim=-1)
    # ties resolve to the lower expert id, like the kernel: sort by (-value, index)
    idx = torch.topk(sel, k, dim=-1, sorted=True).indices
    top = probs.gather(-1, idx)
    if renorm_mode == 1:
        w = torch.softmax(top, dim=-1)
    else:
        w = top / top.sum(-1, keepdim=True).clamp_min(1e-20)
    counts = torch.bincount(idx.flatten(), minlength=logits.shape[-1])
    return w, idx, probs, counts


def apply_capacity(weights: torch.Tensor, idx: torch.Tensor, probs: torch.Tensor, capacity: int) -> torch.Tensor:
    """Drop the lowest-scoring assignments of every expert above ``capacity`` by zeroing their weight and
    renormalising the row (reference model/moe/gate.py:1223-1241)."""
    E = probs.shape[-1]
    T, k = idx.shape
    score = probs.gather(-1, idx)                        # [T,k]
    allowed = torch.ones_like(idx, dtype=torch.bool)
    flat_e = idx.flatten()
    flat_s = score.flatten()
    for e in range(E):
        sel = (flat_e == e).nonzero(as_tuple=True)[0]
        if sel.numel() > capacity:
            drop = sel[torch.topk(flat_s[sel], sel.numel() - capacity, largest=False).indices]
            allowed.view(-1)[drop] = False
    w = weights * allowed.to(weights.dtype)
    tot = w.sum(-1, keepdim=True)
    return torch.where(tot > 0, w / tot.clamp_min(1e-20), torch.zeros_like(w))


def moe_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, weights: torch.Tensor,
                idx: torch.Tensor) -> torch.Tensor:
    """Dense per-expert loop.  x [T,H]; w13 [E,2F,H]; w2 [E,H,F]; weights/idx [T,k]."""
    E = w13.shape[0]
    out = torch.zeros_like(x, dtype=torch.float32)
    for e in range(E):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = swiglu(x[tok].float() @ w13[e].float().t()) @ w2[e].float().t()
        out.index_add_(0, tok, h * weights[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)


# --------------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------------
def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q: torch.Tensor,
                     cu_k: Optional[torch.Tensor], causal: bool, scale: float) -> torch.Tensor:
    """q [Tq, hq, d], k/v [Tk, hk, d] packed; exact softmax attention per sequence (bottom-right causal)."""
    cu_k = cu_q if cu_k is None else cu_k
    hq, hk = q.shape[1], k.shape[1]
    outs: List[torch.Tensor] = []
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for b in range(len(cq) - 1):
        qq = q[cq[b]:cq[b + 1]].float().transpose(0, 1)
        kk = k[ck[b]:ck[b + 1]].float().transpose(0, 1).repeat_interleave(hq // hk, 0)
        vv = v[ck[b]:ck[b + 1]].float().transpose(0, 1).repeat_interleave(hq // hk, 0)
        s = qq @ kk.transpose(1, 2) * scale
        lq, lk = qq.shape[1], kk.shape[1]
        if causal:
            i = torch.arange(lq, device=q.device).unsqueeze(1)
            j = torch.arange(lk, device=q.device).unsqueeze(0)
            s = s.masked_fill(j > i + (lk - lq), float("-inf"))
        p = torch.softmax(s, -1)
        p = torch.nan_to_num(p, nan=0.0)
        outs.append((p @ vv).transpose(0, 1))
    return torch.cat(outs, 0).to(q.dtype)


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                 seq_lens: torch.Tensor, scale: float) -> torch.Tensor:
    """q [B,hq,d]; caches [blocks, block, hk, d]; returns [B,hq,d]."""
    B, hq, d = q.shape
    hk = k_cache.shape[2]
    outs = []
    for b in range(B):
        L = int(seq_lens[b])
        ks = k_cache[block_table[b].long()].reshape(-1, hk, d)[:L].float().repeat_interleave(hq // hk, 1)
        vs = v_cache[block_table[b].long()].reshape(-1, hk, d)[:L].float().repeat_interleave(hq // hk, 1)
        s = torch.einsum("hd,lhd->hl", q[b].float(), ks) * scale
        outs.append(torch.einsum("hl,lhd->hd", torch.softmax(s, -1), vs))
    return torch.stack(outs).to(q.dtype)


# --------------------------------------------------------------------------------------------------
# loss
# --------------------------------------------------------------------------------------------------
def linear_cross_entropy(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100):
    """Sum of token losses and the number of counted tokens; h [T,H], w [V,H], labels [T]."""
    logits = h.float() @ w.float().t()
    loss = F.cross_entropy(logits, labels, ignore_index=ignore_index, reduction="sum")
    return loss, (labels != ignore_index).sum()


# --------------------------------------------------------------------------------------------------
# optimizers
# --------------------------------------------------------------------------------------------------
def adamw_step(p, g, m, v, lr, beta1, beta2, eps, wd, step):
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    mh = m / (1 - beta1 ** step)
    vh = v / (1 - beta2 ** step)
    p.sub_(lr * (mh / (vh.sqrt() + eps) + wd * p))


MUON_NS_COEFFS = [(3.4445, -4.7750, 2.0315)] * 8 + [(2.0, -1.5, 0.5)] * 2


def newton_schulz(g: torch.Tensor, coeffs=MUON_NS_COEFFS, eps: float = 1e-7) -> torch.Tensor:
    """Quintic Newton-Schulz orthogonalisation of a [*, n, m] batch (Gram matrix on the short side)."""
    x = g.float()
    transposed = x.shape[-2] > x.shape[-1]
    if transposed:
        x = x.transpose(-1, -2)
    x = x / x.flatten(-2).norm(dim=-1).clamp_min(eps)[..., None, None]
    for a, b, c in coeffs:
        A = x @ x.transpose(-1, -2)
        B = b * A + c * (A @ A)
        x = a * x + B @ x
    if transposed:
        x = x.transpose(-1, -2)
    return x


# --------------------------------------------------------------------------------------------------
# Subconscious PQ field / vision
# --------------------------------------------------------------------------------------------------
def pq_gather_sum(table: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """table [C,N,D], idx [T,C] -> [T,D] = sum over codebooks of the selected entries."""
    C = table.shape[0]
    out = 0
    for c in range(C):
        out = out + table[c][idx[:, c].long()].float()
    return out.to(table.dtype)


def patchify(img: torch.Tensor, patch: int, mean=None, std=None, k_pad: Optional[int] = None) -> torch.Tensor:
    """img [B,C,H,W] -> [B*gh*gw, C*P*P (padded to k_pad)], column = c*P*P + py*P + px."""
    B, C, H, W = img.shape
    x = img.float()
    if mean is not None:
        x = (x - mean.view(1, C, 1, 1)) / std.view(1, C, 1, 1)
    x = x.unfold(2, patch, patch).unfold(3, patch, patch)            # B C gh gw P P
    x = x.permute(0, 2, 3, 1, 4, 5).reshape(-1, C * patch * patch)
    if k_pad is not None and k_pad > x.shape[1]:
        x = F.pad(x, (0, k_pad - x.shape[1]))
    return x
