"""Mixture-of-experts: gates, experts and the DeepSeek-style layer (shared + fine-grained routed experts).

Reference parity
  * ``YvStableMoEGate`` (model/moe/gate.py:847-1247): linear gate -> softmax -> top-k -> renormalise,
    per-expert capacity with lowest-score drop by zeroing, aux-loss-free bias updated every
    ``moe_bias_update_freq`` calls (buffers, not parameters), optional LSTM load predictor; returns
    ``(weights [T,k], indices [T,k], aux)``.
  * ``YvMoEGate`` (gate.py:103-844) in its lean form: temperature, training noise, load-balance + z loss.
  * ``YvSwiGLUExpert`` (model/moe/expert.py:384-489), ``YvSharedExpert`` (:684-746),
    ``YvDeepSeekMoELayer`` (model/moe/layer.py:967-1440): output = routed + softmax-mixed shared experts.
Routed expert weights are stored stacked (``[E, 2F, H]`` / ``[E, H, F]``) for the grouped tcgen05 GEMM
and exported under the reference's per-expert key names.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import YvConfig
from ..ops import functional as F_
from ..ops import moe as moe_ops
from ..ops import reference as ref


def capacity_mask(weights: torch.Tensor, idx: torch.Tensor, probs: torch.Tensor, capacity: int,
                  counts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Vectorised capacity drop (no host sync): inside every expert keep the ``capacity`` assignments with
    the highest routing probability, zero the rest and renormalise each row."""
    T, k = idx.shape
    E = probs.shape[-1]
    if weights.is_cuda:
        # kernel path: exact selection per expert (radix select), then renormalisation through the kept weights so
        # that the gradient reaches them as in the eager form below
        if counts is None:
            counts = torch.bincount(idx.flatten().long(), minlength=E)
        _, keep = moe_ops.capacity_mask(weights, idx, probs, counts, capacity)
        w = weights * keep.to(weights.dtype)
        tot = w.sum(-1, keepdim=True)
        return torch.where(tot > 0, w / tot.clamp_min(1e-20), torch.zeros_like(w))
    e = idx.flatten().long()
    score = probs.gather(-1, idx.long()).flatten()
    # sort by expert, then by descending score; rank inside the expert = position - segment start
    key = e.double() + (1.0 - score.double().clamp(0, 1)) * 0.999999
    order = torch.argsort(key, stable=True)
    counts = torch.bincount(e, minlength=E)
    starts = torch.cumsum(counts, 0) - counts
    rank = torch.empty_like(order)
    rank[order] = torch.arange(order.numel(), device=idx.device) - starts[e[order]]
    keep = (rank < capacity).view(T, k).to(weights.dtype)
    w = weights * keep
    tot = w.sum(-1, keepdim=True)
    return torch.where(tot > 0, w / tot.clamp_min(1e-20), torch.zeros_like(w))


class YvStableMoEGate(nn.Module):
    def __init__(self, cfg: YvConfig, num_experts: Optional[int] = None, top_k: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        self.num_experts = num_experts or cfg.moe_num_experts
        self.top_k = min(top_k or cfg.moe_top_k, self.num_experts)
        self.capacity_factor = cfg.moe_capacity_factor
        self.min_capacity = cfg.moe_min_capacity
        self.drop_tokens = cfg.moe_drop_tokens
        self.aux_loss_free = cfg.moe_aux_loss_free
        self.bias_update_rate = cfg.moe_bias_update_rate
        self.bias_update_freq = max(1, cfg.moe_bias_update_freq)
        self.bias_in_combine = cfg.moe_bias_in_combine
        self.renorm_mode = int(cfg.extra.get("moe_renorm_mode", 0))
        self.gate = nn.Linear(cfg.hidden_size, self.num_experts, bias=False)
        nn.init.normal_(self.gate.weight, std=cfg.initializer_range)
        self.register_buffer("expert_bias", torch.zeros(self.num_experts, dtype=torch.float32))
        self.register_buffer("usage_counts", torch.zeros(self.num_experts, dtype=torch.int32))
        self._calls = 0
        self.recomputing = False          # set by the activation-checkpoint wrapper during recomputation
        self.last_counts: Optional[torch.Tensor] = None
        self.load_predictor: Optional[nn.LSTM] = None
        if cfg.moe_use_load_predictor:
            self.load_predictor = nn.LSTM(self.num_experts, 32, batch_first=True)
            self.load_head = nn.Linear(32, self.num_experts)
            self.register_buffer("routing_history", torch.zeros(cfg.moe_prediction_horizon, self.num_experts))

    def capacity(self, tokens: int) -> int:
        return max(int(tokens * self.capacity_factor * self.top_k / self.num_experts), self.min_capacity)

    def _predicted_adjustment(self) -> Optional[torch.Tensor]:
        if self.load_predictor is None:
            return None
        with torch.no_grad():
            h, _ = self.load_predictor(self.routing_history.unsqueeze(0))
            pred = torch.softmax(self.load_head(h[:, -1]), -1).squeeze(0)
            return 0.1 * (pred - self.routing_history.mean(0))

    def _gate_weight(self) -> torch.Tensor:
        """The gate weight as the GEMM reads it.  Without autograd (serving) an fp32 gate is cast to bf16 once and
        the copy reused until the parameter changes, instead of one cast kernel per layer per decode step."""
        w = self.gate.weight
        if torch.is_grad_enabled() or w.dtype == torch.bfloat16 or not w.is_cuda:
            return w
        key = (w.data_ptr(), w._version)
        cached = getattr(self, "_gate_bf16", None)
        if cached is None or cached[0] != key:
            cached = (key, w.detach().to(torch.bfloat16))
            self._gate_bf16 = cached
        return cached[1]

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """x [..., H] -> weights [T,k] (rows sum to 1, or 0 for fully dropped tokens), idx [T,k], aux."""
        x2 = x.reshape(-1, x.shape[-1])
        T = x2.shape[0]
        logits = F_.linear(x2, self._gate_weight(), out_fp32=True)
        adj = self._predicted_adjustment()
        if adj is not None:
            logits = logits + adj.to(logits.dtype)
        bias = self.expert_bias if self.aux_loss_free else None
        weights, idx, counts, probs = moe_ops.gate_topk(logits, bias, self.top_k, self.bias_in_combine,
                                                        self.renorm_mode)
        if self.drop_tokens:
            weights = capacity_mask(weights, idx, probs, self.capacity(T), counts)
        aux = logits.new_zeros(())
        if not self.aux_loss_free:
            p_mean = torch.softmax(logits.float(), -1).mean(0)
            f = counts.float() / max(T * self.top_k, 1)
            aux = self.cfg.moe_load_balance_alpha * self.num_experts * (f.detach() * p_mean).sum()
            aux = aux + self.cfg.moe_z_loss_alpha * torch.logsumexp(logits.float(), -1).pow(2).mean()
        self.last_counts = counts
        if self.training and not self.recomputing:
            self._track(counts, probs)
        return weights, idx, aux

    @torch.no_grad()
    def _track(self, counts: torch.Tensor, probs: torch.Tensor) -> None:
        self.usage_counts += counts.to(self.usage_counts.dtype)
        if self.load_predictor is not None:
            self.routing_history = torch.roll(self.routing_history, -1, 0)
            self.routing_history[-1] = probs.mean(0)
        self._calls += 1
        if self.aux_loss_free and self._calls % self.bias_update_freq == 0:
            self.update_bias()

    @torch.no_grad()
    def update_bias(self) -> None:
        """bias += rate * (1/E - usage), clamp +-2; then the usage window restarts."""
        moe_ops.update_gate_bias(self.expert_bias, self.usage_counts, self.bias_update_rate, 2.0)
        self.usage_counts.zero_()


class YvMoEGate(YvStableMoEGate):
    """Lean form of the reference's research gate: temperature and training-time logit noise on top of the
    stable gate; load-balance and z losses when ``moe_aux_loss_free`` is off."""

    def __init__(self, cfg: YvConfig, num_experts: Optional[int] = None, top_k: Optional[int] = None):
        super().__init__(cfg, num_experts, top_k)
        self.temperature = max(float(cfg.moe_routing_temperature), 1e-3)
        self.noise_std = float(cfg.moe_noise_std)

    def forward(self, x: torch.Tensor):
        if self.temperature == 1.0 and not (self.training and self.noise_std > 0):
            return super().forward(x)
        x2 = x.reshape(-1, x.shape[-1])
        T = x2.shape[0]
        logits = F_.linear(x2, self.gate.weight, out_fp32=True) / self.temperature
        if self.training and self.noise_std > 0 and not self.recomputing:
            logits = logits + torch.randn_like(logits) * self.noise_std
        bias = self.expert_bias if self.aux_loss_free else None
        weights, idx, counts, probs = moe_ops.gate_topk(logits, bias, self.top_k, self.bias_in_combine,
                                                        self.renorm_mode)
        if self.drop_tokens:
            weights = capacity_mask(weights, idx, probs, self.capacity(T), counts)
        aux = logits.new_zeros(())
        if not self.aux_loss_free:
            p_mean = torch.softmax(logits.float(), -1).mean(0)
            f = counts.float() / max(T * self.top_k, 1)
            aux = self.cfg.moe_load_balance_alpha * self.num_experts * (f.detach() * p_mean).sum()
        self.last_counts = counts
        if self.training and not self.recomputing:
            self._track(counts, probs)
        return weights, idx, aux


class YvSwiGLUExpert(nn.Module):
    """Dense SwiGLU FFN: down(silu(gate(x)) * up(x)); gate and up are one fused [2F, H] weight."""

    def __init__(self, hidden: int, ffn: int, init_std: float = 0.02, out_std: Optional[float] = None,
                 tp_size: int = 1, tp_group=None):
        super().__init__()
        assert ffn % tp_size == 0
        self.hidden, self.ffn, self.tp_size, self.tp_group = hidden, ffn // tp_size, tp_size, tp_group
        self.w13 = nn.Parameter(torch.empty(2 * self.ffn, hidden))
        self.w2 = nn.Parameter(torch.empty(hidden, self.ffn))
        nn.init.normal_(self.w13, std=init_std)
        nn.init.normal_(self.w2, std=out_std if out_std is not None else init_std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            from ..parallel import tp
            h = F_.swiglu(tp.allgather_linear(x, self.w13, self.tp_group))
            return tp.linear_reduce_scatter(h, self.w2, self.tp_group)
        return F_.linear(F_.swiglu(F_.linear(x, self.w13)), self.w2)

    def export_state(self, prefix: str, out: Dict[str, torch.Tensor]) -> None:
        F_ffn = self.ffn
        out[prefix + "gate_proj.weight"] = self.w13.detach()[:F_ffn].clone()
        out[prefix + "up_proj.weight"] = self.w13.detach()[F_ffn:].clone()
        out[prefix + "down_proj.weight"] = self.w2.detach().clone()

    def import_state(self, prefix: str, sd: Dict[str, torch.Tensor]) -> None:
        with torch.no_grad():
            self.w13.copy_(torch.cat([sd[prefix + "gate_proj.weight"], sd[prefix + "up_proj.weight"]], 0))
            self.w2.copy_(sd[prefix + "down_proj.weight"])


YvExpert = YvSwiGLUExpert


class YvSharedExpert(nn.Module):
    """Always-on expert (reference model/moe/expert.py:684-746 wraps one SwiGLU expert as ``.expert``)."""

    def __init__(self, hidden: int, ffn: int, init_std: float = 0.02):
        super().__init__()
        self.expert = YvSwiGLUExpert(hidden, ffn, init_std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.expert(x)
