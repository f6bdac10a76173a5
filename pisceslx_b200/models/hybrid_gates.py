"""Hybrid attention / state-space plumbing beside the default block (reference model/core/hybrid.py:60-1045,
model/core/mamba3.py:1061-1420, model/core/blocks.py:1417-1470 and :3456-3520):

  * ``YvHybridMode`` / ``YvHybridConfig``       how a block combines its attention and SSM branches;
  * ``YvProgressiveHybridGate``               fixed weights early in training, learned content-dependent weights later;
  * ``YvScheduledUnifiedFusion``              the reference's scheduled form of the unified fusion (the default block's
                                              per-channel gate is ``models.ssm.YvUnifiedFusion``);
  * ``YvAdaptiveRouter``                      token-level routing between the branches with a balance loss;
  * ``YvHierarchicalFusion``                  several gated mixtures, projected and fused;
  * ``YvVKernel``                             the long-convolution form of a time-invariant diagonal SSM;
  * ``YvFlashSSM``                            projection + causal depthwise convolution + selective scan kernel;
  * ``YvSSDualityLayer``                      picks the recurrent or the convolution form by sequence length;
  * ``YvStateCache``                          recurrent and convolution state of a decoding batch;
  * ``YvUnifiedResidual``                     scaled residual + DeepNorm term + manifold-constrained stream mixing;
  * ``YvMHCLayerReplacement``                 wraps the blocks of an existing model in hyper-connections.

Device-side where the reference reads back: the training progress of the gates is a buffer that enters the weights as
a tensor (the reference calls ``current_step.item()`` every forward, hybrid.py:652), and the "one branch is enough"
shortcut of the scheduled fusion is a ``torch.where`` on the weights instead of two ``.item()`` reads.  The kernel of
``YvVKernel`` is a closed form (powers of the decays as ``exp(t log a)``) applied with an FFT convolution; the reference
builds it with a Python loop over the sequence and multiplies by NEGATIVE "decays", which alternates the sign of the
kernel from step to step (mamba3.py:1084-1091).  ``YvFlashSSM`` runs the selective-scan CUDA kernel where the reference
steps through the sequence in Python (mamba3.py:1289-1301)."""
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
from .ssm import selective_scan, selective_scan_step
from .ssm_family import YvManifoldConstraint, YvMHC, YvMHCBlock


class YvHybridMode(str, Enum):
    PARALLEL = "parallel"            # both branches on the same input, fused
    SEQUENTIAL = "sequential"        # attention, then the SSM on its output
    ROUTED = "routed"                # every token goes to one branch or both (YvAdaptiveRouter)
    ATTENTION_ONLY = "attention_only"
    SSM_ONLY = "ssm_only"


@dataclass
class YvHybridConfig:
    hidden_size: int = 2048
    n_head: int = 16
    mode: YvHybridMode = YvHybridMode.PARALLEL
    fusion: str = "unified"          # "unified" | "progressive" | "hierarchical"
    d_state: int = 16
    d_conv: int = 4
    expand: int = 2
    total_steps: int = 100000
    sequence_threshold: int = 4096
    capacity_factor: float = 1.25
    routing_temperature: float = 1.0
    num_fusion_levels: int = 3

    def build_fusion(self) -> nn.Module:
        if self.fusion == "progressive":
            return YvProgressiveHybridGate(self.hidden_size, self.total_steps, self.sequence_threshold)
        if self.fusion == "hierarchical":
            return YvHierarchicalFusion(self.hidden_size, self.num_fusion_levels)
        return YvScheduledUnifiedFusion(self.hidden_size, self.total_steps, self.sequence_threshold)


class _ScheduledWeights(nn.Module):
    """Shared by the two scheduled gates: fixed branch weights (0.7 / 0.3 for short, 0.3 / 0.7 for long sequences)
    blended with learned ones by ``sigmoid(hybrid_ratio) * progress``, progress = step / total_steps capped at 1."""

    def __init__(self, total_steps: int, sequence_threshold: int):
        super().__init__()
        self.total_steps, self.sequence_threshold = max(int(total_steps), 1), int(sequence_threshold)
        self.register_buffer("current_step", torch.zeros((), dtype=torch.float32))
        self.hybrid_ratio = nn.Parameter(torch.tensor(0.0))
        self.register_buffer("fixed_short", torch.tensor([0.7, 0.3]))
        self.register_buffer("fixed_long", torch.tensor([0.3, 0.7]))

    def blend(self, adaptive: torch.Tensor, sequence_length: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """adaptive [B, 2] (rows sum to 1) -> (attention weight [B], ssm weight [B], current ratio)."""
        if self.training and torch.is_grad_enabled():
            self.current_step += 1
        ratio = torch.sigmoid(self.hybrid_ratio.float()) * (self.current_step / self.total_steps).clamp(max=1.0)
        fixed = self.fixed_long if sequence_length > self.sequence_threshold else self.fixed_short
        w = fixed.float() * (1 - ratio) + adaptive.float() * ratio
        return w[:, 0], w[:, 1], ratio


class YvProgressiveHybridGate(_ScheduledWeights):
    """Weights from the sequence statistics (mean, spread, maximum, minimum) and the pooled content."""

    def __init__(self, d_model: int, total_steps: int = 100000, sequence_threshold: int = 4096):
        super().__init__(total_steps, sequence_threshold)
        q = max(d_model // 4, 1)
        self.seq_stats_proj = nn.Linear(4, q)
        self.content_proj = nn.Linear(d_model, q)
        self.gate_proj = nn.Sequential(nn.Linear(2 * q, max(d_model // 8, 1)), nn.SiLU(), nn.Linear(max(d_model // 8, 1), 2))

    @staticmethod
    def _compute_sequence_stats(x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        std = xf.std(1) if x.shape[1] > 1 else torch.zeros_like(xf[:, 0])
        return torch.stack([xf.mean(1).mean(-1), std.mean(-1), xf.amax(1).mean(-1), xf.amin(1).mean(-1)], -1)

    def forward(self, attention_out: torch.Tensor, ssm_out: torch.Tensor, hidden_states: torch.Tensor,
                sequence_length: Optional[int] = None) -> Dict[str, Any]:
        L = hidden_states.shape[1] if sequence_length is None else sequence_length
        feats = torch.cat([self.seq_stats_proj(self._compute_sequence_stats(hidden_states).to(hidden_states.dtype)),
                           self.content_proj(hidden_states.mean(1))], -1)
        wa, ws, ratio = self.blend(torch.softmax(self.gate_proj(feats).float(), -1), L)
        dt = attention_out.dtype
        return {"fused_output": wa.view(-1, 1, 1).to(dt) * attention_out + ws.view(-1, 1, 1).to(dt) * ssm_out,
                "attention_weight": wa, "ssm_weight": ws, "gate_type": "progressive_hybrid", "hybrid_ratio": ratio}


class YvScheduledUnifiedFusion(_ScheduledWeights):
    """Weights from the pooled content only.  In evaluation, once the learned part dominates (ratio > 0.5), a sample
    whose weight for one branch passes ``deterministic_threshold`` takes that branch alone."""

    def __init__(self, d_model: int, total_steps: int = 100000, sequence_threshold: int = 4096,
                 deterministic_mode: bool = True, deterministic_threshold: float = 0.95):
        super().__init__(total_steps, sequence_threshold)
        self.deterministic_mode, self.deterministic_threshold = deterministic_mode, deterministic_threshold
        self.content_encoder = nn.Linear(d_model, max(d_model // 4, 1), bias=False)
        self.gate = nn.Sequential(nn.Linear(max(d_model // 4, 1), max(d_model // 8, 1), bias=False), nn.SiLU(),
                                  nn.Linear(max(d_model // 8, 1), 2, bias=False))

    def forward(self, attention_out: torch.Tensor, ssm_out: torch.Tensor, hidden_states: torch.Tensor,
                sequence_length: Optional[int] = None) -> torch.Tensor:
        L = hidden_states.shape[1] if sequence_length is None else sequence_length
        adaptive = torch.softmax(self.gate(self.content_encoder(hidden_states.mean(1))).float(), -1)
        wa, ws, ratio = self.blend(adaptive, L)
        if not self.training and self.deterministic_mode:
            sure = ratio > 0.5
            only_a, only_s = sure & (wa > self.deterministic_threshold), sure & (ws > self.deterministic_threshold)
            wa = torch.where(only_a, torch.ones_like(wa), torch.where(only_s, torch.zeros_like(wa), wa))
            ws = torch.where(only_s, torch.ones_like(ws), torch.where(only_a, torch.zeros_like(ws), ws))
        dt = attention_out.dtype
        return wa.view(-1, 1, 1).to(dt) * attention_out + ws.view(-1, 1, 1).to(dt) * ssm_out


class YvAdaptiveRouter(nn.Module):
    """Token-level routing: a two-way softmax per token; each branch keeps its ``capacity_factor x S / 2`` highest
    scoring tokens (so a factor of 2 sends every token to both) and its output is weighted by the token's probability
    for it, which is what trains the router.  The reference gives each branch a capacity of ``capacity_factor x S``
    tokens, i.e. always all of them, and sums the two outputs unweighted (hybrid.py:815-833), so nothing is routed and
    the router gets no gradient from the task.  Both branch functions run on the full sequence (they need the context);
    the routing decides what is kept.  Returns (output, balance loss)."""

    def __init__(self, hidden_size: int, n_head: int, capacity_factor: float = 1.25, routing_temperature: float = 1.0):
        super().__init__()
        self.hidden_size, self.n_head = hidden_size, n_head
        self.capacity_factor, self.routing_temperature = capacity_factor, routing_temperature
        self.router = nn.Linear(hidden_size, 2, bias=False)
        self.attention_norm, self.ssm_norm = YvRMSNorm(hidden_size), YvRMSNorm(hidden_size)
        self.last_masks: Optional[Tuple[torch.Tensor, torch.Tensor]] = None

    def capacity(self, seq_len: int) -> int:
        return max(1, min(seq_len, int(math.ceil(seq_len * self.capacity_factor / 2))))

    @staticmethod
    def _compute_routing_loss(router_probs: torch.Tensor) -> torch.Tensor:
        """Both branches should carry half of the tokens on average: squared deviation of the mean probabilities."""
        mean = router_probs.float().mean(dim=(0, 1))
        return ((mean - 0.5) ** 2).sum() * 0.1

    def forward(self, x: torch.Tensor, attention_fn: Callable[[torch.Tensor], torch.Tensor],
                ssm_fn: Callable[[torch.Tensor], torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        B, S, H = x.shape
        probs = torch.softmax(self.router(x).float() / self.routing_temperature, -1)             # [B, S, 2]
        cap = self.capacity(S)
        masks = []
        for b in range(2):
            idx = probs[..., b].topk(cap, -1).indices
            masks.append(torch.zeros(B, S, device=x.device, dtype=torch.bool).scatter_(1, idx, True))
        # a token dropped by both branches keeps its better one, so that nothing passes through unprocessed
        orphan = ~(masks[0] | masks[1])
        masks[0] = masks[0] | (orphan & (probs[..., 0] >= probs[..., 1]))
        masks[1] = masks[1] | (orphan & (probs[..., 0] < probs[..., 1]))
        self.last_masks = (masks[0], masks[1])
        norm2 = lambda n, t: n(t.reshape(B * S, H)).view(B, S, H)
        a = attention_fn(norm2(self.attention_norm, x))
        s = ssm_fn(norm2(self.ssm_norm, x))
        wa = (probs[..., 0] * masks[0]).unsqueeze(-1)
        ws = (probs[..., 1] * masks[1]).unsqueeze(-1)
        tot = (wa + ws).clamp_min(1e-8)
        out = (wa / tot).to(a.dtype) * a + (ws / tot).to(s.dtype) * s
        return out, self._compute_routing_loss(probs)


class YvHierarchicalFusion(nn.Module):
    """``num_levels`` token-wise two-way gates over (attention, ssm); every level's mixture is projected, the levels are
    concatenated and fused by a two-layer MLP."""

    def __init__(self, hidden_size: int, num_levels: int = 3):
        super().__init__()
        H = hidden_size
        self.num_levels = num_levels
        self.level_gates = nn.ModuleList([nn.Sequential(nn.Linear(2 * H, max(H // 4, 1)), nn.SiLU(),
                                                        nn.Linear(max(H // 4, 1), 2)) for _ in range(num_levels)])
        self.level_projs = nn.ModuleList([nn.Linear(H, H, bias=False) for _ in range(num_levels)])
        self.final_fusion = nn.Sequential(nn.Linear(H * num_levels, H), nn.SiLU(), nn.Linear(H, H))

    def forward(self, attention_out: torch.Tensor, ssm_out: torch.Tensor,
                hidden_states: Optional[torch.Tensor] = None, sequence_length: Optional[int] = None) -> torch.Tensor:
        both = torch.cat([attention_out, ssm_out], -1)
        levels = []
        for gate, proj in zip(self.level_gates, self.level_projs):
            w = torch.softmax(gate(both).float(), -1).to(attention_out.dtype)
            levels.append(proj(w[..., :1] * attention_out + w[..., 1:] * ssm_out))
        return self.final_fusion(torch.cat(levels, -1))


# ---------------------------------------------------------------------------------------------------------------------------
class YvVKernel(nn.Module):
    """Time-invariant diagonal SSM in its convolution form: y = K * u + D u with
    K[t, d] = sum_n C[d, n] a_n**t B[n, d], a_n = exp(-exp(A_log_n) dt) in (0, 1).  The kernel is a closed form and the
    causal convolution runs as an FFT product (O(L log L)); in evaluation the kernel is cached per length."""

    def __init__(self, d_model: int, d_state: int, max_seq_len: int = 4096, dt: float = 1.0):
        super().__init__()
        self.d_model, self.d_state, self.max_seq_len = d_model, d_state, max_seq_len
        self.A_log = nn.Parameter(torch.empty(d_state).uniform_(-3.0, -1.0))
        self.log_dt = nn.Parameter(torch.tensor(math.log(dt)))
        self.B = nn.Parameter(torch.randn(d_state, d_model) * 0.1)
        self.C = nn.Parameter(torch.randn(d_model, d_state) * 0.1)
        self.D = nn.Parameter(torch.ones(d_model))
        self._kernel_cache: Optional[torch.Tensor] = None

    def decays(self) -> torch.Tensor:
        return torch.exp(-torch.exp(self.A_log.float()) * torch.exp(self.log_dt.float()))

    def _compute_kernel(self, seq_len: int, device: torch.device) -> torch.Tensor:
        """[L, d_model] fp32."""
        t = torch.arange(seq_len, device=device, dtype=torch.float32)
        powers = torch.exp(t[:, None] * torch.log(self.decays().to(device))[None, :])              # [L, N]
        return torch.einsum("ln,dn,nd->ld", powers, self.C.float(), self.B.float())

    def kernel(self, seq_len: int, device: torch.device) -> torch.Tensor:
        if self.training and torch.is_grad_enabled():
            return self._compute_kernel(seq_len, device)
        c = self._kernel_cache
        if c is None or c.shape[0] < seq_len or c.device != device:
            with torch.no_grad():
                c = self._kernel_cache = self._compute_kernel(max(seq_len, 1), device)
        return c[:seq_len]

    def train(self, mode: bool = True):
        self._kernel_cache = None
        return super().train(mode)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, L, D = x.shape
        k = self.kernel(L, x.device)
        n = 1 << (2 * L - 1).bit_length()
        y = torch.fft.irfft(torch.fft.rfft(x.float(), n=n, dim=1) * torch.fft.rfft(k, n=n, dim=0)[None], n=n, dim=1)[:, :L]
        return (y + x.float() * self.D.float()).to(x.dtype)

    def recurrent_reference(self, x: torch.Tensor) -> torch.Tensor:
        """The same map as a recurrence (tests compare the two forms).  Every channel d carries its own state of
        ``d_state`` entries: h[d, n] <- a_n h[d, n] + B[n, d] u_d, y_d = sum_n C[d, n] h[d, n]."""
        a = self.decays()
        Bt = self.B.float().t()                                                                   # [D, N]
        h = x.new_zeros(x.shape[0], self.d_model, self.d_state, dtype=torch.float32)
        ys = []
        for t in range(x.shape[1]):
            h = h * a + x[:, t].float().unsqueeze(-1) * Bt
            ys.append((h * self.C.float()).sum(-1))
        return (torch.stack(ys, 1) + x.float() * self.D.float()).to(x.dtype)


class YvStateCache:
    """Recurrent state [B, d_model, d_state] (fp32) and convolution tail [B, d_model, d_conv - 1] of a decoding batch."""

    def __init__(self, batch_size: int, d_state: int, d_model: int, device: Any = "cpu", d_conv: int = 4):
        self.batch_size, self.d_state, self.d_model, self.device, self.d_conv = batch_size, d_state, d_model, device, d_conv
        self.state = torch.zeros(batch_size, d_model, d_state, device=device, dtype=torch.float32)
        self.conv_state = torch.zeros(batch_size, d_model, max(d_conv - 1, 0), device=device)

    def update(self, new_state: torch.Tensor, new_conv_state: Optional[torch.Tensor] = None) -> None:
        self.state = new_state
        if new_conv_state is not None:
            self.conv_state = new_conv_state

    def reset(self, batch_indices: Optional[torch.Tensor] = None) -> None:
        if batch_indices is None:
            self.state.zero_()
            self.conv_state.zero_()
        else:
            self.state[batch_indices] = 0
            self.conv_state[batch_indices] = 0

    def clone(self) -> "YvStateCache":
        c = YvStateCache(self.batch_size, self.d_state, self.d_model, self.device, self.d_conv)
        c.state, c.conv_state = self.state.clone(), self.conv_state.clone()
        return c


class YvFlashSSM(nn.Module):
    """in_proj -> (u, delta, B, C); causal depthwise convolution on u; delta = softplus; selective scan; + D u; out_proj.
    ``forward`` takes whole sequences (the scan is one kernel launch); ``step`` decodes one token against a
    ``YvStateCache`` and gives what ``forward`` gives for that position."""

    def __init__(self, d_model: int, d_state: int = 16, d_conv: int = 4):
        super().__init__()
        self.d_model, self.d_state, self.d_conv = d_model, d_state, d_conv
        self.bc_width = 2 * d_state
        self.in_proj = nn.Linear(d_model, 2 * d_model + self.bc_width, bias=False)
        self.out_proj = nn.Linear(d_model, d_model, bias=False)
        self.conv_weight = nn.Parameter(torch.randn(d_model, d_conv) * (d_conv ** -0.5))
        self.conv_bias = nn.Parameter(torch.zeros(d_model))
        self.A_log = nn.Parameter(torch.empty(d_model, d_state).uniform_(-3.0, -1.0))
        self.D = nn.Parameter(torch.ones(d_model))

    def _split(self, x: torch.Tensor):
        p = self.in_proj(x)
        u, delta, bc = torch.split(p, [self.d_model, self.d_model, self.bc_width], -1)
        return u, F.softplus(delta), bc[..., :self.d_state], bc[..., self.d_state:]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, L, D = x.shape
        u, delta, Bm, Cm = self._split(x)
        u = F.conv1d(F.pad(u.transpose(1, 2), (self.d_conv - 1, 0)), self.conv_weight.to(u.dtype).unsqueeze(1),
                     self.conv_bias.to(u.dtype), groups=D).transpose(1, 2)
        A = -torch.exp(self.A_log.float())
        y = selective_scan(u.contiguous(), delta.contiguous(), A, Bm.contiguous(), Cm.contiguous(), self.D)
        return self.out_proj(y.to(x.dtype))

    def step(self, x: torch.Tensor, cache: YvStateCache) -> torch.Tensor:
        """x [B, 1, d_model]."""
        u, delta, Bm, Cm = self._split(x)
        window = torch.cat([cache.conv_state.to(u.dtype), u.transpose(1, 2)], -1)                  # [B, D, d_conv]
        cache.conv_state = window[..., 1:].detach()
        u = ((window * self.conv_weight.to(u.dtype)).sum(-1) + self.conv_bias.to(u.dtype)).unsqueeze(1)
        A = -torch.exp(self.A_log.float())
        y = selective_scan_step(u.contiguous(), delta.contiguous(), A, Bm.contiguous(), Cm.contiguous(), self.D, cache.state)
        return self.out_proj(y.to(x.dtype))


class YvSSDualityLayer(nn.Module):
    """The recurrent form (selective scan, input dependent) up to ``threshold`` tokens, the convolution form (time
    invariant, FFT) beyond it: the two sides of the state-space duality as one layer."""

    def __init__(self, d_model: int, d_state: int = 16, threshold: int = 512):
        super().__init__()
        self.threshold = threshold
        self.recurrent_mode = YvFlashSSM(d_model, d_state)
        self.conv_mode = YvVKernel(d_model, d_state)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.recurrent_mode(x) if x.shape[1] <= self.threshold else self.conv_mode(x)


# ---------------------------------------------------------------------------------------------------------------------------
class YvUnifiedResidual(nn.Module):
    """Residual connection of a sub-layer with three parts: the scaled sub-layer output (learned scale, initial value
    (2 n_layer)^-0.5), a DeepNorm term beta * scaled + alpha * hidden, and a manifold-constrained mixing of ``n_hc``
    channel groups of the updated state (a doubly stochastic matrix, so the mixing neither amplifies nor loses
    signal).  ``forward_deepnorm`` returns the DeepNorm combination alone (for post-norm blocks)."""

    def __init__(self, hidden_size: int, num_sublayers: int = 2, cfg: Any = None):
        super().__init__()
        g = lambda k, d: (getattr(cfg, k, None) if cfg is not None and getattr(cfg, k, None) is not None
                          else (getattr(cfg, "extra", {}) or {}).get(k, d) if cfg is not None else d)
        n_layer = int(getattr(cfg, "n_layer", 32)) if cfg is not None else 32
        alpha0 = float(g("residual_alpha", (2.0 * n_layer) ** -0.5 if cfg is not None else 1.0))
        self.num_sublayers = num_sublayers
        self.residual_scales = nn.ParameterList([nn.Parameter(torch.full((1,), alpha0)) for _ in range(num_sublayers)])
        self.residual_dropout = nn.Dropout(float(g("residual_dropout", 0.1)))
        self.deepnorm_beta = nn.Parameter(torch.full((num_sublayers,), float(g("deepnorm_beta", 0.13))))
        self.deepnorm_alpha = nn.Parameter(torch.full((num_sublayers,), float(g("deepnorm_alpha", 0.87))))
        self.n_hc = int(g("mhc_n_hc", 4))
        self._use_mhc = bool(g("use_mhc", True)) and hidden_size % self.n_hc == 0
        self.mhc_mix = YvManifoldConstraint(self.n_hc, int(g("mhc_sinkhorn_iters", 20))) if self._use_mhc else None
        self.mhc_scale = nn.Parameter(torch.zeros(())) if self._use_mhc else None

    def _mhc(self, x: torch.Tensor) -> torch.Tensor:
        """Mix the ``n_hc`` channel groups of x by the doubly stochastic matrix; scaled by a gate that starts at 0."""
        if not self._use_mhc:
            return torch.zeros_like(x)
        g = x.view(*x.shape[:-1], self.n_hc, -1)
        mixed = torch.einsum("mn,...nd->...md", self.mhc_mix().to(x.dtype), g).reshape(x.shape)
        return self.mhc_scale.to(x.dtype) * (mixed - x)

    def forward(self, hidden_states: torch.Tensor, sublayer_output: torch.Tensor, sublayer_idx: int = 0) -> torch.Tensor:
        standard = self.residual_scales[sublayer_idx].to(sublayer_output.dtype) * self.residual_dropout(sublayer_output)
        deepnorm = self.deepnorm_beta[sublayer_idx].to(standard.dtype) * standard + \
            self.deepnorm_alpha[sublayer_idx].to(standard.dtype) * hidden_states
        return hidden_states + standard + deepnorm + self._mhc(hidden_states + standard)

    def forward_combined(self, hidden_states: torch.Tensor, combined_output: torch.Tensor) -> torch.Tensor:
        return self.forward(hidden_states, combined_output, 0)

    def forward_deepnorm(self, hidden_states: torch.Tensor, sublayer_output: torch.Tensor, sublayer_idx: int = 0) -> torch.Tensor:
        standard = self.residual_scales[sublayer_idx].to(sublayer_output.dtype) * self.residual_dropout(sublayer_output)
        dn = self.deepnorm_beta[sublayer_idx].to(standard.dtype) * standard + \
            self.deepnorm_alpha[sublayer_idx].to(standard.dtype) * hidden_states
        return dn + self._mhc(dn)


class YvMHCLayerReplacement:
    """Upgrades existing blocks to manifold-constrained hyper-connections: a block with an attention-like and an
    MLP-like sub-module (``attention`` / ``attn`` and ``mlp`` / ``ffn``) becomes a ``YvMHCBlock`` over the SAME
    sub-modules (their weights are kept), and ``upgrade_transformer`` does that for every entry of ``model.layers`` or
    ``model.blocks``.  The upgraded blocks take and return stream tensors ``[n, B, S, H]``; ``wrap`` gives a module
    that expands a hidden state to streams, runs the upgraded blocks and collapses by the mean."""

    ATTENTION_NAMES, MLP_NAMES = ("attention", "attn", "self_attn"), ("mlp", "ffn", "feed_forward")

    @classmethod
    def _find(cls, block: nn.Module, names: Tuple[str, ...]) -> Optional[nn.Module]:
        return next((getattr(block, n) for n in names if isinstance(getattr(block, n, None), nn.Module)), None)

    @classmethod
    def replace_attention_block(cls, block: nn.Module, n_streams: int = 4) -> nn.Module:
        f, g = cls._find(block, cls.ATTENTION_NAMES), cls._find(block, cls.MLP_NAMES)
        if f is None or g is None:
            return block
        pre_f = cls._find(block, ("norm_attention", "norm1", "ln_1", "input_layernorm"))
        pre_g = cls._find(block, ("norm_mlp", "norm2", "ln_2", "post_attention_layernorm"))
        wrap = lambda norm, fn: (nn.Sequential(norm, fn) if norm is not None else fn)
        return YvMHCBlock(wrap(pre_f, f), wrap(pre_g, g), n_streams)

    @classmethod
    def upgrade_transformer(cls, model: nn.Module, n_streams: int = 4) -> Tuple[nn.Module, int]:
        """Returns (model, number of blocks upgraded)."""
        attr = "blocks" if hasattr(model, "blocks") else ("layers" if hasattr(model, "layers") else None)
        done = 0
        if attr is not None:
            blocks = getattr(model, attr)
            for i, b in enumerate(blocks):
                new = cls.replace_attention_block(b, n_streams)
                done += int(new is not b)
                blocks[i] = new
        return model, done

    @staticmethod
    def wrap(blocks: nn.ModuleList, n_streams: int = 4) -> nn.Module:
        from .ssm_family import YvMHCTransformer
        return YvMHCTransformer(list(blocks), n_streams)
