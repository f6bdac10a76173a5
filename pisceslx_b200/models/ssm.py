"""State-space branch of the Yv backbone: selective scan op, ``YvSelectiveSSM``, ``YvMamba3Block`` and the hybrid
blocks that run it beside attention.

Reference: ``YvSelectiveSSM`` (model/core/hybrid.py:332-560: in_proj -> depthwise conv(3) -> SiLU -> x_proj ->
(dt, B, C) -> softplus(dt_proj) -> per-time-step Python loop -> gate by SiLU(z) -> out_proj), ``YvMamba3Block``
(model/core/mamba3.py:418-1653), ``YvHybridBlock`` (hybrid.py:1170-1370: FiLM -> attention || SSM -> fusion ->
residual -> norm -> MoE -> residual, learnable residual scales initialised to (2L)^-0.5 and a sigmoid gate in front
of the SSM branch) and ``YvJambaBlock`` (hybrid.py:1047).  The reference's scan is a Python loop over time steps;
here it is one CUDA kernel per direction (ops/csrc/ssm.cu) with every state kept in registers."""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import YvConfig
from ..ops import functional as F_
from ..ops import kernels
from .norms import YvFiLMModulation, YvRMSNorm


def selective_scan_reference(u, delta, A, B, C, D, h0=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 oracle: u, delta [b,l,d]; A [d,n]; B, C [b,l,n]; D [d] -> (y [b,l,d], final state [b,d,n])."""
    b, l, d = u.shape
    u, delta, A, B, C, D = (t.float() for t in (u, delta, A, B, C, D))
    h = torch.zeros(b, d, A.shape[1], dtype=torch.float32, device=u.device) if h0 is None else h0.float()
    ys = []
    for t in range(l):
        dA = torch.exp(delta[:, t, :, None] * A[None])
        h = dA * h + delta[:, t, :, None] * B[:, t, None, :] * u[:, t, :, None]
        ys.append((h * C[:, t, None, :]).sum(-1))
    return torch.stack(ys, 1) + u * D, h


class _SelectiveScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, B, C, D):
        K = kernels()
        uf, df, Af, Bf, Cf, Df = (t.float().contiguous() for t in (u, delta, A, B, C, D))
        y = torch.empty_like(uf)
        need = any(t.requires_grad for t in (u, delta, A, B, C, D))
        hs = torch.empty(*uf.shape, Af.shape[1], dtype=torch.float32, device=u.device) if need else None
        K.ssm_scan_fwd(uf, df, Af, Bf, Cf, Df, y, hs, None)
        if need:
            ctx.save_for_backward(uf, df, Af, Bf, Cf, Df, hs)
        ctx.dtypes = (u.dtype, delta.dtype, A.dtype, B.dtype, C.dtype, D.dtype)
        return y.to(u.dtype)

    @staticmethod
    def backward(ctx, dy):
        uf, df, Af, Bf, Cf, Df, hs = ctx.saved_tensors
        K = kernels()
        du, dd = torch.empty_like(uf), torch.empty_like(df)
        dA, dB, dC, dD = torch.zeros_like(Af), torch.zeros_like(Bf), torch.zeros_like(Cf), torch.zeros_like(Df)
        K.ssm_scan_bwd(uf, df, Af, Bf, Cf, Df, hs, dy.float().contiguous(), du, dd, dA, dB, dC, dD)
        return tuple(g.to(t) for g, t in zip((du, dd, dA, dB, dC, dD), ctx.dtypes))


def selective_scan(u, delta, A, B, C, D) -> torch.Tensor:
    """Differentiable selective scan; CUDA kernel for 16 states and a channel count that is a multiple of 32."""
    if u.is_cuda and A.shape[1] == 16 and u.shape[-1] % 32 == 0:
        return _SelectiveScanFn.apply(u, delta, A, B, C, D)
    return selective_scan_reference(u, delta, A, B, C, D)[0].to(u.dtype)


def selective_scan_step(u, delta, A, B, C, D, state) -> torch.Tensor:
    """One decode step (l = 1) that carries ``state [b,d,n]`` (fp32) in place."""
    if u.is_cuda and A.shape[1] == 16:
        y = torch.empty(u.shape, dtype=torch.float32, device=u.device)
        kernels().ssm_scan_fwd(u.float().contiguous(), delta.float().contiguous(), A.float().contiguous(),
                               B.float().contiguous(), C.float().contiguous(), D.float().contiguous(), y, None, state)
        return y.to(u.dtype)
    y, h = selective_scan_reference(u, delta, A, B, C, D, state)
    state.copy_(h)
    return y.to(u.dtype)


class YvSelectiveSSM(nn.Module):
    def __init__(self, hidden_size: int, state_dim: int = 16, expansion_factor: int = 2, dt_rank: Any = "auto",
                 conv_kernel: int = 3, init_std: float = 0.02):
        super().__init__()
        self.hidden_size, self.state_dim = hidden_size, state_dim
        self.d_inner = hidden_size * expansion_factor
        self.dt_rank = math.ceil(hidden_size / 16) if dt_rank == "auto" else int(dt_rank)
        self.conv_kernel = conv_kernel
        self.in_proj = nn.Parameter(torch.empty(2 * self.d_inner, hidden_size).normal_(std=init_std))
        self.conv_weight = nn.Parameter(torch.empty(self.d_inner, 1, conv_kernel).uniform_(-0.5, 0.5))
        self.conv_bias = nn.Parameter(torch.zeros(self.d_inner))
        self.x_proj = nn.Parameter(torch.empty(self.dt_rank + 2 * state_dim, self.d_inner).normal_(std=init_std))
        self.dt_proj = nn.Parameter(torch.empty(self.d_inner, self.dt_rank).normal_(std=self.dt_rank ** -0.5))
        # softplus(dt_bias) spread log-uniformly over [1e-3, 1e-1], as in the selective-scan literature
        dt = torch.exp(torch.rand(self.d_inner) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, state_dim + 1, dtype=torch.float32)).repeat(self.d_inner, 1))
        self.D = nn.Parameter(torch.ones(self.d_inner))
        self.out_proj = nn.Parameter(torch.empty(hidden_size, self.d_inner).normal_(std=init_std))

    def _conv(self, x: torch.Tensor) -> torch.Tensor:
        """Causal depthwise convolution along the sequence ([b, l, d])."""
        xt = F.pad(x.transpose(1, 2), (self.conv_kernel - 1, 0))
        return F.conv1d(xt, self.conv_weight.to(x.dtype), self.conv_bias.to(x.dtype), groups=self.d_inner).transpose(1, 2)

    def _params(self, xc: torch.Tensor):
        x_dbl = F_.linear(xc, self.x_proj)
        dt, B, C = x_dbl.split([self.dt_rank, self.state_dim, self.state_dim], dim=-1)
        dt = F.softplus(F_.linear(dt.contiguous(), self.dt_proj).float() + self.dt_bias.float())
        return dt, B.float(), C.float(), -torch.exp(self.A_log.float())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xz = F_.linear(x, self.in_proj)
        xp, z = xz.chunk(2, dim=-1)
        xc = F.silu(self._conv(xp))
        dt, B, C, A = self._params(xc)
        y = selective_scan(xc.float(), dt, A, B, C, self.D.float()).to(x.dtype)
        return F_.linear(y * F.silu(z), self.out_proj)

    # ---- incremental decoding --------------------------------------------------------------------------
    def init_state(self, batch: int, device, dtype=torch.float32) -> Dict[str, torch.Tensor]:
        return {"h": torch.zeros(batch, self.d_inner, self.state_dim, dtype=torch.float32, device=device),
                "conv": torch.zeros(batch, self.conv_kernel - 1, self.d_inner, dtype=dtype, device=device)}

    def step(self, x: torch.Tensor, state: Dict[str, torch.Tensor]) -> torch.Tensor:
        """x [b, 1, hidden]; updates ``state`` in place (SSM state and the convolution's last inputs)."""
        xz = F_.linear(x, self.in_proj)
        xp, z = xz.chunk(2, dim=-1)
        window = torch.cat([state["conv"].to(xp.dtype), xp], 1)                 # [b, k, d]
        state["conv"].copy_(window[:, 1:])
        w = self.conv_weight.to(xp.dtype).squeeze(1).t()                        # [k, d]
        xc = F.silu((window * w[None]).sum(1, keepdim=True) + self.conv_bias.to(xp.dtype))
        dt, B, C, A = self._params(xc)
        y = selective_scan_step(xc.float(), dt, A, B, C, self.D.float(), state["h"]).to(x.dtype)
        return F_.linear(y * F.silu(z), self.out_proj)


class YvMamba3Block(nn.Module):
    """Pre-norm residual block around the selective SSM (the reference's Mamba-3 block adds complex-valued states and
    MIMO heads on top of the same scan; those are not reproduced)."""

    def __init__(self, cfg: YvConfig, layer_idx: int = 0):
        super().__init__()
        ex = cfg.extra if hasattr(cfg, "extra") else {}
        self.norm = YvRMSNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.ssm = YvSelectiveSSM(cfg.hidden_size, int(ex.get("mamba_state_dim", 16)), int(ex.get("mamba_expand", 2)),
                                  init_std=cfg.initializer_range)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.ssm(self.norm(x))


class YvUnifiedFusion(nn.Module):
    """Per-channel sigmoid gate between the attention and the SSM branch, conditioned on the block input."""

    def __init__(self, hidden: int):
        super().__init__()
        self.gate = nn.Parameter(torch.zeros(hidden, hidden))
        self.bias = nn.Parameter(torch.zeros(hidden))

    def forward(self, attn_out: torch.Tensor, ssm_out: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        g = torch.sigmoid(F_.linear(x, self.gate).float() + self.bias.float()).to(x.dtype)
        return g * attn_out + (1 - g) * ssm_out


class YvHybridBlock(nn.Module):
    """FiLM -> attention || sparse-gated SSM -> fusion -> residual -> RMSNorm -> MLP / MoE -> residual."""

    def __init__(self, cfg: YvConfig, layer_idx: int, attention: nn.Module, mlp: nn.Module):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        ex = cfg.extra if hasattr(cfg, "extra") else {}
        self.norm_attention = YvRMSNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.attention = attention
        self.ssm = YvSelectiveSSM(cfg.hidden_size, int(ex.get("mamba_state_dim", 16)), int(ex.get("mamba_expand", 2)),
                                  init_std=cfg.initializer_range)
        self.fusion = YvUnifiedFusion(cfg.hidden_size)
        self.norm_fusion = YvRMSNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.mlp = mlp
        s = (2 * max(cfg.n_layer, 1)) ** -0.5
        self.residual_scale_attn = nn.Parameter(torch.tensor(s))
        self.residual_scale_ssm = nn.Parameter(torch.tensor(1.0))
        self.residual_scale_mlp = nn.Parameter(torch.tensor(s))
        self.sparse_gate_ssm = nn.Parameter(torch.zeros(()))
        self.sparsity_reg_weight = float(ex.get("ssm_sparsity_reg_weight", 1e-4))

    def sparsity_loss(self) -> torch.Tensor:
        """Parameter-only regulariser of the SSM gate; the trunk's ``sparsity_objective`` walk sums it."""
        return self.sparsity_reg_weight * torch.sigmoid(self.sparse_gate_ssm.float())

    sparsity_objective = sparsity_loss

    def forward(self, x: torch.Tensor, ctx: Any = None, film_params: Optional[Dict[str, torch.Tensor]] = None):
        """x [B, S, H] -> (x', aux)."""
        x = YvFiLMModulation.apply(x, film_params)
        n = self.norm_attention(x)
        B, S, H = x.shape
        a = self.attention(n.reshape(B * S, H), ctx).view(B, S, H) if ctx is not None else self.attention(n)
        s = torch.sigmoid(self.sparse_gate_ssm).to(x.dtype) * self.ssm(n)
        fused = self.fusion(a, self.residual_scale_ssm.to(x.dtype) * s, n)
        x = x + self.residual_scale_attn.to(x.dtype) * fused
        m = self.mlp(self.norm_fusion(x).reshape(B * S, H))
        aux = x.new_zeros((), dtype=torch.float32)
        if isinstance(m, tuple):
            m, aux = m
        return x + self.residual_scale_mlp.to(x.dtype) * m.view(B, S, H), aux


class YvJambaBlock(nn.Module):
    """Interleaving policy: one attention layer every ``attn_every`` layers, SSM layers otherwise."""

    def __init__(self, cfg: YvConfig, layer_idx: int, attention_factory, attn_every: int = 4):
        super().__init__()
        self.is_attention = (layer_idx % attn_every) == attn_every - 1
        self.norm = YvRMSNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.mixer = attention_factory() if self.is_attention else YvSelectiveSSM(cfg.hidden_size,
                                                                                init_std=cfg.initializer_range)

    def forward(self, x: torch.Tensor, ctx: Any = None) -> torch.Tensor:
        n = self.norm(x)
        if self.is_attention and ctx is not None:
            B, S, H = x.shape
            return x + self.mixer(n.reshape(B * S, H), ctx).view(B, S, H)
        return x + self.mixer(n)
