"""``YvDeepSeekMoELayer``: shared experts + fine-grained routed experts (reference model/moe/layer.py:967-1440).

out = sum_k w_k * Expert_{idx_k}(x) + sum_s softmax(shared_expert_weight)_s * Shared_s(x)
      [+ 0.1 * previous shared output, detached, when ``moe_skip_prev_shared``]      (layer.py:741-753,942-951)

Storage is laid out for the kernels: routed experts stacked ``w13 [E_local, 2F, H]`` / ``w2 [E_local, H, F]``
(grouped tcgen05 GEMM), shared experts concatenated so the S experts run as two dense GEMMs
(``shared_w13 [S*2Fs, H]``, ``shared_w2 [H, S*Fs]``; the mixing weights scale the activations).  Expert
parallelism keeps ``E / ep`` experts per rank and exchanges tokens through ``parallel.ep``.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from ..config import YvConfig
from ..ops import functional as F_
from ..ops import moe as moe_ops
from .moe import YvMoEGate, YvStableMoEGate


class YvDeepSeekMoELayer(nn.Module):
    def __init__(self, cfg: YvConfig, layer_idx: int = 0, ep_size: int = 1, ep_rank: int = 0, ep_group=None,
                 tp_size: int = 1, tp_group=None):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        self.ep_size, self.ep_rank, self.ep_group = ep_size, ep_rank, ep_group
        self.tp_size, self.tp_group = tp_size, tp_group
        H = cfg.hidden_size
        E, F = cfg.moe_num_experts, cfg.moe_expert_intermediate_size
        assert E % ep_size == 0
        self.num_experts, self.num_local = E, E // ep_size
        self.ffn = F
        if cfg.moe_gate_type == "research":
            from .moe_gate_research import YvResearchMoEGate
            gate_cls = YvResearchMoEGate
        else:
            gate_cls = YvStableMoEGate if cfg.moe_gate_type == "stable" else YvMoEGate
        self.router = gate_cls(cfg)
        std = cfg.initializer_range
        out_std = std / math.sqrt(2 * cfg.n_layer) if cfg.use_scaled_init else std
        self.experts_w13 = nn.Parameter(torch.empty(self.num_local, 2 * F, H))
        self.experts_w2 = nn.Parameter(torch.empty(self.num_local, H, F))
        self._init_experts(std, out_std)
        # shared experts (tensor-parallel over the FFN dimension)
        self.num_shared = cfg.moe_shared_experts
        self.shared_ffn = cfg.moe_shared_intermediate_size // tp_size if self.num_shared else 0
        if self.num_shared:
            S, Fs = self.num_shared, self.shared_ffn
            self.shared_w13 = nn.Parameter(torch.empty(S * 2 * Fs, H))
            self.shared_w2 = nn.Parameter(torch.empty(H, S * Fs))
            nn.init.normal_(self.shared_w13, std=std)
            nn.init.normal_(self.shared_w2, std=out_std)
            self.shared_expert_weight = nn.Parameter(torch.zeros(S))
        self.skip_prev = cfg.moe_skip_prev_shared
        self._prev_shared: Optional[torch.Tensor] = None
        self.deterministic = bool(cfg.extra.get("moe_deterministic", False))

    def _init_experts(self, std: float, out_std: float) -> None:
        method = self.cfg.expert_init_method
        # one seed per (layer, global expert id): an EP shard holds exactly the rows the unsharded model has
        dev, dt = self.experts_w13.device, self.experts_w13.dtype
        if dev.type == "meta":
            return
        gen = torch.Generator(device=dev)
        F, H = self.ffn, self.cfg.hidden_size
        lo = self.ep_rank * self.num_local
        with torch.no_grad():
            for i in range(self.num_local):
                gen.manual_seed(1234567 + self.layer_idx * 65536 + lo + i)
                w13 = torch.randn(2 * F, H, generator=gen, device=dev, dtype=torch.float32) * std
                w2 = torch.randn(H, F, generator=gen, device=dev, dtype=torch.float32) * out_std
                if method in ("orthogonal", "hybrid"):
                    nn.init.orthogonal_(w13, gain=std * math.sqrt(H))
                self.experts_w13[i].copy_(w13.to(dt))
                self.experts_w2[i].copy_(w2.to(dt))

    # ------------------------------------------------------------------------------------------------
    def _shared(self, x: torch.Tensor) -> torch.Tensor:
        S, Fs = self.num_shared, self.shared_ffn
        T = x.shape[0]
        if self.tp_size > 1:
            from ..parallel import tp
            y1 = tp.allgather_linear(x, self.shared_w13, self.tp_group)
        else:
            y1 = F_.linear(x, self.shared_w13)
        T = y1.shape[0]
        act = F_.swiglu(y1.view(T * S, 2 * Fs)).view(T, S, Fs)
        if S > 1 or self.shared_expert_weight.requires_grad:
            sw = self.shared_expert_weight
            if torch.is_grad_enabled():
                mix = torch.softmax(sw.float(), 0).to(act.dtype)
            else:
                # serving: the mixing weights change only when the parameter does; keep them instead of running a
                # softmax and two casts per layer per decode step
                key = (sw.data_ptr(), sw._version, act.dtype)
                cached = getattr(self, "_mix_cache", None)
                if cached is None or cached[0] != key:
                    cached = (key, torch.softmax(sw.detach().float(), 0).to(act.dtype))
                    self._mix_cache = cached
                mix = cached[1]
            act = act * mix.view(1, S, 1)
        act = act.reshape(T, S * Fs)
        if self.tp_size > 1:
            from ..parallel import tp
            return tp.linear_reduce_scatter(act, self.shared_w2, self.tp_group)
        return F_.linear(act, self.shared_w2)

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """x [T, H] -> (out [T, H], aux loss)."""
        shape = x.shape
        x = x.reshape(-1, shape[-1])
        weights, idx, aux = self.router(x)
        counts = self.router.last_counts
        if self.ep_size > 1:
            from ..parallel import ep
            routed = ep.moe_experts_ep(x, self.experts_w13, self.experts_w2, weights, idx, self.num_experts,
                                       self.ep_group, fused=self.cfg.fused_comm, deterministic=self.deterministic,
                                       counts=counts)
        else:
            routed = moe_ops.moe_experts(x, self.experts_w13, self.experts_w2, weights, idx, counts,
                                         self.deterministic, fp8=getattr(self.cfg, "expert_fp8", None))
        out = routed
        if self.num_shared:
            sh = self._shared(x)
            out = out + sh
            if self.skip_prev:
                if self._prev_shared is not None and self._prev_shared.shape == sh.shape:
                    out = out + 0.1 * self._prev_shared
                self._prev_shared = sh.detach()
        return out.view(shape), aux

    # ------------------------------------------------------------------------------------------------
    # checkpoint key mapping: reference names  experts.<e>.{gate,up,down}_proj.weight,
    # shared_experts.<s>.expert.{gate,up,down}_proj.weight, shared_expert_weight, router.gate.weight
    # ------------------------------------------------------------------------------------------------
    def export_state(self, prefix: str, out: Dict[str, torch.Tensor]) -> None:
        F = self.ffn
        lo = self.ep_rank * self.num_local
        for i in range(self.num_local):
            p = f"{prefix}experts.{lo + i}."
            out[p + "gate_proj.weight"] = self.experts_w13.detach()[i, :F].clone()
            out[p + "up_proj.weight"] = self.experts_w13.detach()[i, F:].clone()
            out[p + "down_proj.weight"] = self.experts_w2.detach()[i].clone()
        if self.num_shared:
            S, Fs = self.num_shared, self.shared_ffn
            w13 = self.shared_w13.detach().view(S, 2 * Fs, -1)
            w2 = self.shared_w2.detach().view(-1, S, Fs)
            for s in range(S):
                p = f"{prefix}shared_experts.{s}.expert."
                out[p + "gate_proj.weight"] = w13[s, :Fs].clone()
                out[p + "up_proj.weight"] = w13[s, Fs:].clone()
                out[p + "down_proj.weight"] = w2[:, s].clone()
            out[prefix + "shared_expert_weight"] = self.shared_expert_weight.detach().clone()
        out[prefix + "router.gate.weight"] = self.router.gate.weight.detach().clone()
        out[prefix + "router.expert_bias"] = self.router.expert_bias.detach().clone()

    def import_state(self, prefix: str, sd: Dict[str, torch.Tensor]) -> None:
        F = self.ffn
        lo = self.ep_rank * self.num_local
        with torch.no_grad():
            for i in range(self.num_local):
                p = f"{prefix}experts.{lo + i}."
                self.experts_w13[i, :F].copy_(sd[p + "gate_proj.weight"])
                self.experts_w13[i, F:].copy_(sd[p + "up_proj.weight"])
                self.experts_w2[i].copy_(sd[p + "down_proj.weight"])
            if self.num_shared:
                S, Fs = self.num_shared, self.shared_ffn
                w13 = self.shared_w13.view(S, 2 * Fs, -1)
                w2 = self.shared_w2.view(-1, S, Fs)
                for s in range(S):
                    p = f"{prefix}shared_experts.{s}.expert."
                    w13[s, :Fs].copy_(sd[p + "gate_proj.weight"])
                    w13[s, Fs:].copy_(sd[p + "up_proj.weight"])
                    w2[:, s].copy_(sd[p + "down_proj.weight"])
                if prefix + "shared_expert_weight" in sd:
                    self.shared_expert_weight.copy_(sd[prefix + "shared_expert_weight"])
            self.router.gate.weight.copy_(sd[prefix + "router.gate.weight"])
            if prefix + "router.expert_bias" in sd:
                self.router.expert_bias.copy_(sd[prefix + "router.expert_bias"])


YvDynamicMoELayer = YvDeepSeekMoELayer
