"""State-space variants and manifold-constrained hyper-connections (reference model/core/mamba3.py:418-1653:
trapezoidal / adaptive discretisation, complex and MIMO state spaces, gated / bidirectional / multi-head /
hierarchical SSMs, the state-space duality check, encoder / decoder / stack; model/core/blocks.py:2546-3577 mHC:
Sinkhorn-Knopp projection, manifold constraint, hyper-connection block and loss).

All recurrent variants run on the selective-scan kernel through ``models.ssm.selective_scan`` (one thread per
(sequence, channel) on the GPU; the fp32 reference loop on CPU), so none of them launches a kernel per token."""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as F_
from .norms import YvRMSNorm
from .ssm import YvMamba3Block, YvSelectiveSSM, selective_scan


class YvSSMType(str, Enum):
    SELECTIVE = "selective"
    GATED = "gated"
    BIDIRECTIONAL = "bidirectional"
    MULTI_HEAD = "multi_head"
    HIERARCHICAL = "hierarchical"


class YvSSMMode(str, Enum):
    RECURRENT = "recurrent"          # scan over time (training and prefill)
    STEP = "step"                    # one token with a carried state (decode)


@dataclass
class YvMamba3Config:
    hidden_size: int = 512
    state_dim: int = 16
    expansion_factor: int = 2
    conv_kernel: int = 3
    n_layers: int = 2
    ssm_type: YvSSMType = YvSSMType.SELECTIVE
    n_heads: int = 4
    scales: Tuple[int, ...] = (1, 4)


# ------------------------------------------------------------------------------------------------ discretisation
class YvTrapezoidalDiscretization:
    """Bilinear (trapezoidal) rule for a diagonal continuous system x' = a x + b u:
    a_bar = (1 + dt a / 2) / (1 - dt a / 2), b_bar = dt b / (1 - dt a / 2); second-order accurate, stable for a < 0."""

    @staticmethod
    def discretize(a: torch.Tensor, b: torch.Tensor, dt: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        den = 1.0 - 0.5 * dt * a
        return (1.0 + 0.5 * dt * a) / den, dt * b / den


class YvAdaptiveDiscretization(nn.Module):
    """Per-token step size from the input: dt = softplus(W x + b) clamped to [dt_min, dt_max]."""

    def __init__(self, dim: int, dt_min: float = 1e-3, dt_max: float = 0.1):
        super().__init__()
        self.proj = nn.Linear(dim, dim)
        self.dt_min, self.dt_max = dt_min, dt_max
        with torch.no_grad():
            dt = torch.exp(torch.rand(dim) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
            self.proj.bias.copy_(dt + torch.log(-torch.expm1(-dt)))          # inverse softplus
            self.proj.weight.zero_()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.softplus(self.proj(x.float())).clamp(self.dt_min, self.dt_max)


# ------------------------------------------------------------------------------------------------ SSM variants
class YvGatedSSM(nn.Module):
    """y = SSM(x) * silu(W_g x): an output gate computed from the layer input."""

    def __init__(self, hidden: int, **kw: Any):
        super().__init__()
        self.ssm = YvSelectiveSSM(hidden, **kw)
        self.gate = nn.Parameter(torch.empty(hidden, hidden).normal_(std=0.02))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.ssm(x) * F.silu(F_.linear(x, self.gate.to(x.dtype)))


class YvBidirectionalSSM(nn.Module):
    """Forward and time-reversed scans mixed by a learned sigmoid weight (encoder use: not causal)."""

    def __init__(self, hidden: int, **kw: Any):
        super().__init__()
        self.fwd, self.bwd = YvSelectiveSSM(hidden, **kw), YvSelectiveSSM(hidden, **kw)
        self.mix = nn.Parameter(torch.zeros(hidden))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        a = self.fwd(x)
        b = self.bwd(x.flip(1)).flip(1)
        w = torch.sigmoid(self.mix).to(x.dtype)
        return w * a + (1 - w) * b


class YvMultiHeadSSM(nn.Module):
    """The hidden dimension split into ``n_heads`` groups, each with its own selective SSM (its own A, B, C
    dynamics), concatenated and mixed by an output projection."""

    def __init__(self, hidden: int, n_heads: int = 4, **kw: Any):
        super().__init__()
        assert hidden % n_heads == 0
        self.h, self.dh = n_heads, hidden // n_heads
        self.heads = nn.ModuleList([YvSelectiveSSM(self.dh, **kw) for _ in range(n_heads)])
        self.out = nn.Parameter(torch.empty(hidden, hidden).normal_(std=0.02))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        parts = [ssm(x[..., i * self.dh:(i + 1) * self.dh]) for i, ssm in enumerate(self.heads)]
        return F_.linear(torch.cat(parts, -1), self.out.to(x.dtype))


class YvHierarchicalSSM(nn.Module):
    """Several time scales: scale s runs an SSM on the sequence average-pooled by s (causally: a pooled step only
    covers past and current tokens) and is upsampled back by repetition with a shift of s - 1, so that no token sees
    its future; the scales are summed with learned weights."""

    def __init__(self, hidden: int, scales: Tuple[int, ...] = (1, 4), **kw: Any):
        super().__init__()
        self.scales = tuple(scales)
        self.ssms = nn.ModuleList([YvSelectiveSSM(hidden, **kw) for _ in self.scales])
        self.w = nn.Parameter(torch.zeros(len(self.scales)))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, H = x.shape
        w = torch.softmax(self.w, 0)
        out = 0
        for i, (s, ssm) in enumerate(zip(self.scales, self.ssms)):
            if s == 1:
                y = ssm(x)
            else:
                n = S // s
                if n == 0:
                    continue
                pooled = x[:, : n * s].reshape(B, n, s, H).mean(2)
                yc = ssm(pooled).repeat_interleave(s, 1)                          # value of block j at positions j*s .. j*s+s-1
                # block j is complete at position j*s + s - 1: shift right by s - 1 and pad
                y = F.pad(yc, (0, 0, s - 1, 0))[:, :S]
                if y.shape[1] < S:
                    y = F.pad(y, (0, 0, 0, S - y.shape[1]))
            out = out + w[i].to(x.dtype) * y
        return out


class YvComplexStateSpace(nn.Module):
    """Diagonal complex state space (rotating modes): h_t = lambda * h_{t-1} + B u_t with lambda = exp(dt (-a + i w)),
    y_t = Re(C h_t) + D u_t; evaluated as a causal convolution with the kernel K_k = Re(C lambda^k B) through FFTs."""

    def __init__(self, dim: int, state_dim: int = 16, dt: float = 0.05):
        super().__init__()
        self.log_a = nn.Parameter(torch.log(0.5 + torch.rand(dim, state_dim)))
        self.w = nn.Parameter(torch.rand(dim, state_dim) * math.pi)
        self.B = nn.Parameter(torch.randn(dim, state_dim, 2) * state_dim ** -0.5)
        self.C = nn.Parameter(torch.randn(dim, state_dim, 2) * state_dim ** -0.5)
        self.D = nn.Parameter(torch.ones(dim))
        self.dt = dt

    def kernel(self, L: int) -> torch.Tensor:
        lam = torch.exp(self.dt * torch.complex(-torch.exp(self.log_a), self.w))       # [D, N], |lam| < 1
        k = torch.arange(L, device=lam.device)
        powers = lam[..., None] ** k                                                     # [D, N, L]
        cb = torch.view_as_complex(self.C.contiguous()) * torch.view_as_complex(self.B.contiguous())
        return (cb[..., None] * powers).sum(1).real                                      # [D, L]

    def forward(self, u: torch.Tensor) -> torch.Tensor:
        B, L, D = u.shape
        K = self.kernel(L)
        n = 2 * L
        y = torch.fft.irfft(torch.fft.rfft(u.float().transpose(1, 2), n=n) * torch.fft.rfft(K, n=n), n=n)[..., :L]
        return (y.transpose(1, 2) + self.D * u.float()).to(u.dtype)

    def recurrent(self, u: torch.Tensor) -> torch.Tensor:
        """The same map as an explicit recurrence (oracle for the convolutional form)."""
        B, L, D = u.shape
        lam = torch.exp(self.dt * torch.complex(-torch.exp(self.log_a), self.w))
        Bc, Cc = torch.view_as_complex(self.B.contiguous()), torch.view_as_complex(self.C.contiguous())
        h = torch.zeros(B, D, lam.shape[1], dtype=torch.complex64, device=u.device)
        ys = []
        for t in range(L):
            h = lam * h + Bc * u[:, t, :, None].float()
            ys.append((Cc * h).sum(-1).real + self.D * u[:, t].float())
        return torch.stack(ys, 1).to(u.dtype)


class YvMIMOStateSpace(nn.Module):
    """Multi-input multi-output linear state space with a shared state: h_t = A h_{t-1} + B u_t, y_t = C h_t + D u_t,
    A = diag(sigmoid) (stable), evaluated with the selective-scan op by treating every state channel as a scan
    channel with constant step."""

    def __init__(self, dim_in: int, dim_out: int, state_dim: int = 32):
        super().__init__()
        self.a = nn.Parameter(torch.randn(state_dim))
        self.B = nn.Parameter(torch.randn(state_dim, dim_in) * dim_in ** -0.5)
        self.C = nn.Parameter(torch.randn(dim_out, state_dim) * state_dim ** -0.5)
        self.D = nn.Parameter(torch.zeros(dim_out, dim_in))

    def forward(self, u: torch.Tensor) -> torch.Tensor:
        Bsz, L, _ = u.shape
        x = F.linear(u.float(), self.B)                                                  # [B, L, N] drive per state
        decay = torch.sigmoid(self.a)                                                    # A diagonal in (0, 1)
        # h_t = decay * h_{t-1} + x_t as a scan with dt = 1: exp(dt * logA) = decay, B = 1, C = 1
        N = x.shape[-1]
        A = torch.log(decay).view(N, 1)
        ones = torch.ones(Bsz, L, 1, device=u.device)
        h = selective_scan(x.contiguous(), torch.ones_like(x), A, ones, ones, torch.zeros(N, device=u.device))
        # the scan applies the zero-order-hold input factor dt * B = 1: h is the plain recurrence
        return (F.linear(h, self.C) + F.linear(u.float(), self.D)).to(u.dtype)


class YvSSDuality:
    """State-space duality: a scalar-decay SSM equals masked "attention" with the lower-triangular decay matrix
    M[t, s] = prod_{r=s+1..t} a_r.  ``attention_form`` computes that matrix form; tests compare it with the scan."""

    @staticmethod
    def attention_form(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
        """a [L] decays in (0,1); b, c [L, N]; u [L] -> y [L] with y_t = sum_s c_t . b_s (prod a_{s+1..t}) u_s."""
        L = a.shape[0]
        loga = torch.log(a).cumsum(0)
        M = torch.exp(loga[:, None] - loga[None, :]).tril()
        return ((c @ b.t()) * M) @ u

    @staticmethod
    def recurrent_form(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
        h = torch.zeros(b.shape[1])
        ys = []
        for t in range(a.shape[0]):
            h = a[t] * h + b[t] * u[t]
            ys.append((c[t] * h).sum())
        return torch.stack(ys)


# ------------------------------------------------------------------------------------------------ stacks
def _make_ssm(cfg: YvMamba3Config) -> nn.Module:
    kw = dict(state_dim=cfg.state_dim, expansion_factor=cfg.expansion_factor, conv_kernel=cfg.conv_kernel)
    t = cfg.ssm_type
    if t == YvSSMType.GATED:
        return YvGatedSSM(cfg.hidden_size, **kw)
    if t == YvSSMType.BIDIRECTIONAL:
        return YvBidirectionalSSM(cfg.hidden_size, **kw)
    if t == YvSSMType.MULTI_HEAD:
        return YvMultiHeadSSM(cfg.hidden_size, cfg.n_heads, **kw)
    if t == YvSSMType.HIERARCHICAL:
        return YvHierarchicalSSM(cfg.hidden_size, cfg.scales, **kw)
    return YvSelectiveSSM(cfg.hidden_size, **kw)


class YvMamba3Stack(nn.Module):
    """Pre-norm residual stack of SSM layers of the configured type."""

    def __init__(self, cfg: YvMamba3Config):
        super().__init__()
        self.cfg = cfg
        self.norms = nn.ModuleList([YvRMSNorm(cfg.hidden_size) for _ in range(cfg.n_layers)])
        self.layers = nn.ModuleList([_make_ssm(cfg) for _ in range(cfg.n_layers)])
        self.final = YvRMSNorm(cfg.hidden_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for n, l in zip(self.norms, self.layers):
            x = x + l(n(x))
        return self.final(x)


class YvMamba3Encoder(YvMamba3Stack):
    """Non-causal encoder: bidirectional layers."""

    def __init__(self, cfg: YvMamba3Config):
        super().__init__(YvMamba3Config(**{**cfg.__dict__, "ssm_type": YvSSMType.BIDIRECTIONAL}))


class YvMamba3Decoder(YvMamba3Stack):
    """Causal decoder: gated layers."""

    def __init__(self, cfg: YvMamba3Config):
        super().__init__(YvMamba3Config(**{**cfg.__dict__, "ssm_type": YvSSMType.GATED}))


class YvMamba3Integration(nn.Module):
    """The SSM branch as the trunk uses it: a normed selective SSM whose output is scaled by a learned sigmoid gate
    before it is fused with the attention branch (the residual is added by the fusion)."""

    def __init__(self, hidden: int, **kw: Any):
        super().__init__()
        self.norm, self.ssm = YvRMSNorm(hidden), YvSelectiveSSM(hidden, **kw)
        self.gate = nn.Parameter(torch.zeros(1))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.sigmoid(self.gate).to(x.dtype) * self.ssm(self.norm(x))


# ------------------------------------------------------------------------------------------------ mHC
class YvSinkhornKnopp:
    """Projects a positive matrix onto (approximately) doubly stochastic matrices by alternating row and column
    normalisation."""

    @staticmethod
    def project(logits: torch.Tensor, iters: int = 10) -> torch.Tensor:
        m = torch.exp(logits.float() - logits.float().amax((-1, -2), keepdim=True))
        for _ in range(iters):
            m = m / m.sum(-1, keepdim=True).clamp_min(1e-12)
            m = m / m.sum(-2, keepdim=True).clamp_min(1e-12)
        return m


class YvManifoldConstraint(nn.Module):
    """A learnable n x n stream-mixing matrix kept on the doubly stochastic manifold (Sinkhorn of its logits), so that
    mixing residual streams neither amplifies nor loses total signal; initialised near the identity."""

    def __init__(self, n_streams: int, iters: int = 10, init_scale: float = 4.0):
        super().__init__()
        self.logits = nn.Parameter(torch.eye(n_streams) * init_scale)
        self.iters = iters

    def forward(self) -> torch.Tensor:
        return YvSinkhornKnopp.project(self.logits, self.iters)


class YvMHC(nn.Module):
    """Manifold-constrained hyper-connection around a layer: ``n`` residual streams are mixed by a doubly stochastic
    matrix, the layer reads a convex combination of them and its output is written back with learned weights."""

    def __init__(self, n_streams: int = 4):
        super().__init__()
        self.mix = YvManifoldConstraint(n_streams)
        self.read = nn.Parameter(torch.zeros(n_streams))
        self.write = nn.Parameter(torch.ones(n_streams) / n_streams)

    def forward(self, streams: torch.Tensor, layer: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
        """streams [n, B, S, H]."""
        x = torch.einsum("n,n...->...", torch.softmax(self.read, 0).to(streams.dtype), streams)
        y = layer(x)
        mixed = torch.einsum("mn,n...->m...", self.mix().to(streams.dtype), streams)
        return mixed + self.write.to(streams.dtype).view(-1, 1, 1, 1) * y[None]


YvHyperConnection = YvMHC


class YvMHCBlock(nn.Module):
    """A transformer sub-block pair (attention-like ``f`` and MLP-like ``g``) each wrapped in its own mHC."""

    def __init__(self, f: nn.Module, g: nn.Module, n_streams: int = 4):
        super().__init__()
        self.f, self.g = f, g
        self.hc_f, self.hc_g = YvMHC(n_streams), YvMHC(n_streams)

    def forward(self, streams: torch.Tensor) -> torch.Tensor:
        return self.hc_g(self.hc_f(streams, self.f), self.g)


class YvMHCTransformer(nn.Module):
    """Expands the hidden state into ``n`` streams, runs mHC blocks, and collapses the streams by their mean."""

    def __init__(self, blocks: List[YvMHCBlock], n_streams: int = 4):
        super().__init__()
        self.blocks, self.n = nn.ModuleList(blocks), n_streams

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        s = x.unsqueeze(0).expand(self.n, *x.shape).contiguous()
        for b in self.blocks:
            s = b(s)
        return s.mean(0)


class YvMHCLoss(nn.Module):
    """Keeps the stream-mixing matrices close to doubly stochastic and away from collapse: row / column sum error
    plus a small entropy bonus (a permutation-like matrix mixes nothing)."""

    def __init__(self, entropy_weight: float = 1e-3):
        super().__init__()
        self.entropy_weight = entropy_weight

    def forward(self, model: nn.Module) -> torch.Tensor:
        loss = torch.zeros(())
        for m in model.modules():
            if isinstance(m, YvManifoldConstraint):
                P = m()
                err = (P.sum(-1) - 1).pow(2).mean() + (P.sum(-2) - 1).pow(2).mean()
                ent = -(P * torch.log(P.clamp_min(1e-12))).sum(-1).mean()
                loss = loss + err - self.entropy_weight * ent
        return loss
