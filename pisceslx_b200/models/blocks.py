"""Transformer block of the Yv text trunk and the activation-recomputation wrapper.

``YvTransformerBlock`` is the reference's attention + MoE block (model/core/blocks.py:1471-2545 with
``backbone_allow_legacy_blocks``): FiLM at block entry (hybrid.py:1334) -> RMSNorm -> GQA attention ->
residual -> RMSNorm -> MoE (or dense SwiGLU) -> residual.  The residual stream is carried as a pair
``(h, delta)`` with true hidden state ``h + delta`` so that each RMSNorm kernel also performs the pending
residual add.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Tuple

import torch
import torch.nn as nn

from ..config import YvConfig
from .attention import AttnContext, YvAttention
from .moe import YvSwiGLUExpert
from .moe_layer import YvDeepSeekMoELayer
from .norms import YvFiLMModulation, YvRMSNorm


class _RecomputeFn(torch.autograd.Function):
    """Activation recomputation for one block: the forward runs without a graph and keeps only the block
    inputs; the backward re-runs the block with ``recompute=True`` and back-propagates through it, so
    parameter gradients (and their post-accumulate hooks) fire layer by layer."""

    @staticmethod
    def forward(ctx, run: Callable, mask: Tuple[bool, ...], *tensors):
        ctx.run, ctx.mask = run, mask
        ctx.save_for_backward(*[t for t in tensors if t is not None])
        with torch.no_grad():
            outs = run(False, *tensors)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        saved = list(ctx.saved_tensors)
        inputs = []
        for present in ctx.mask:
            if present:
                t = saved.pop(0).detach()
                t.requires_grad_(t.is_floating_point())
                inputs.append(t)
            else:
                inputs.append(None)
        with torch.enable_grad():
            outs = ctx.run(True, *inputs)
        pairs = [(o, g) for o, g in zip(outs, grads) if o is not None and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, None) + tuple(t.grad if (t is not None and t.requires_grad) else None for t in inputs)


def recompute(run: Callable, *tensors: Optional[torch.Tensor]):
    mask = tuple(t is not None for t in tensors)
    return _RecomputeFn.apply(run, mask, *tensors)


class YvTransformerBlock(nn.Module):
    def __init__(self, cfg: YvConfig, layer_idx: int, parallel=None):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        tp = parallel.tp_size if parallel is not None else 1
        tpg = parallel.tp_group if parallel is not None else None
        ep = parallel.ep_size if parallel is not None else 1
        epr = parallel.ep_rank if parallel is not None else 0
        epg = parallel.ep_group if parallel is not None else None
        self.norm_attention = YvRMSNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.attention = YvAttention(cfg, layer_idx, tp, tpg)
        self.norm_mlp = YvRMSNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.is_moe = cfg.is_moe_layer(layer_idx)
        if self.is_moe:
            self.mlp = YvDeepSeekMoELayer(cfg, layer_idx, ep, epr, epg, tp, tpg)
        else:
            self.mlp = YvSwiGLUExpert(cfg.hidden_size, cfg.intermediate_size, cfg.initializer_range, None, tp, tpg)
        self.use_recompute = cfg.use_gradient_checkpointing
        # hybrid backbone (reference default, model/core/hybrid.py:1170-1370): a sparse-gated selective SSM beside the
        # attention branch, fused by a learned per-channel gate
        self.ssm = self.fusion = None
        if cfg.use_mamba3 and not cfg.backbone_allow_legacy_blocks:
            from .ssm import YvSelectiveSSM, YvUnifiedFusion
            assert tp == 1, "the SSM branch is not tensor-parallel"
            ex = cfg.extra
            self.ssm = YvSelectiveSSM(cfg.hidden_size, int(ex.get("mamba_state_dim", 16)),
                                      int(ex.get("mamba_expand", 2)), init_std=cfg.initializer_range)
            self.fusion = YvUnifiedFusion(cfg.hidden_size)
            self.sparse_gate_ssm = nn.Parameter(torch.zeros(()))
            self.sparsity_reg_weight = float(ex.get("ssm_sparsity_reg_weight", 1e-4))

    def sparsity_loss(self) -> Optional[torch.Tensor]:
        """Regulariser of the gate in front of the SSM branch (reference model/core/hybrid.py:1298-1307); parameters
        only, folded into the objective by the trunk's walk."""
        if self.ssm is None:
            return None
        return self.sparsity_reg_weight * torch.sigmoid(self.sparse_gate_ssm.float())

    def _body(self, recomputing: bool, h: torch.Tensor, delta: Optional[torch.Tensor], ctx: AttnContext,
              film: Optional[Dict[str, torch.Tensor]]):
        if self.is_moe:
            self.mlp.router.recomputing = recomputing
        if film is not None:
            h = h if delta is None else h + delta
            h = YvFiLMModulation.apply(h.view(film["scale"].shape[0], -1, h.shape[-1]), film).view(h.shape)
            delta = None
        if delta is None:
            n1 = self.norm_attention(h)
        else:
            n1, h = self.norm_attention(delta, residual=h)
        a = self.attention(n1, ctx)
        if self.ssm is not None and not ctx.decode:
            T, H = n1.shape
            assert T % ctx.max_len == 0, "the SSM branch needs equal-length sequences"
            s_out = self.ssm(n1.view(T // ctx.max_len, ctx.max_len, H)).reshape(T, H)
            a = self.fusion(a, torch.sigmoid(self.sparse_gate_ssm).to(a.dtype) * s_out, n1)
        n2, h = self.norm_mlp(a, residual=h)
        if self.is_moe:
            m, aux = self.mlp(n2)
        else:
            m, aux = self.mlp(n2), h.new_zeros((), dtype=torch.float32)
        if self.is_moe:
            self.mlp.router.recomputing = False
        return h, m, aux

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], ctx: AttnContext,
                film_params: Optional[Dict[str, torch.Tensor]] = None):
        """(h, delta) -> (h', delta', aux) with hidden = h + delta.  ``film_params`` None is the identity; a dict
        must carry both 'scale' and 'shift' (``ValueError`` otherwise)."""
        YvFiLMModulation.validate(film_params)
        if self.use_recompute and self.training and torch.is_grad_enabled() and h.is_cuda:
            fs = film_params["scale"] if film_params is not None else None
            fb = film_params["shift"] if film_params is not None else None

            def run(recomputing, h_, d_, fs_, fb_):
                f = None if fs_ is None else {"scale": fs_, "shift": fb_}
                return self._body(recomputing, h_, d_, ctx, f)

            return recompute(run, h, delta, fs, fb)
        if getattr(self, "measure_stored", False) and h.is_cuda and torch.is_grad_enabled():
            # bytes this layer's forward leaves allocated for its backward (read by the recompute planner)
            m0 = torch.cuda.memory_allocated(h.device)
            out = self._body(False, h, delta, ctx, film_params)
            self.stored_bytes = max(getattr(self, "stored_bytes", 0), torch.cuda.memory_allocated(h.device) - m0)
            return out
        return self._body(False, h, delta, ctx, film_params)

    # checkpoint key mapping -----------------------------------------------------------------------
    def export_state(self, prefix: str, out: Dict[str, torch.Tensor]) -> None:
        out[prefix + "norm_attention.weight"] = self.norm_attention.weight.detach().clone()
        out[prefix + "norm_mlp.weight"] = self.norm_mlp.weight.detach().clone()
        self.attention.export_state(prefix + "attention.", out)
        self.mlp.export_state(prefix + "mlp.", out)
        if self.ssm is not None:
            for n, p in self.ssm.named_parameters():
                out[prefix + "ssm." + n] = p.detach().clone()
            for n, p in self.fusion.named_parameters():
                out[prefix + "fusion." + n] = p.detach().clone()
            out[prefix + "sparse_gate_ssm"] = self.sparse_gate_ssm.detach().clone()

    def import_state(self, prefix: str, sd: Dict[str, torch.Tensor]) -> None:
        with torch.no_grad():
            self.norm_attention.weight.copy_(sd[prefix + "norm_attention.weight"])
            self.norm_mlp.weight.copy_(sd[prefix + "norm_mlp.weight"])
        self.attention.import_state(prefix + "attention.", sd)
        if self.ssm is not None and prefix + "sparse_gate_ssm" in sd:
            with torch.no_grad():
                for n, p in self.ssm.named_parameters():
                    p.copy_(sd[prefix + "ssm." + n])
                for n, p in self.fusion.named_parameters():
                    p.copy_(sd[prefix + "fusion." + n])
                self.sparse_gate_ssm.copy_(sd[prefix + "sparse_gate_ssm"])
        self.mlp.import_state(prefix + "mlp.", sd)
