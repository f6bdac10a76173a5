"""``YvModel`` (trunk) and ``YvModelForCausalLM`` (trunk + LM head + losses).

Mirrors the reference's forward contract (model/core/model.py:1979-2615): embedding -> optional
multimodal tokens prepended -> per layer FiLM parameters + block -> final RMSNorm -> LM head; the LM loss
is the shifted cross-entropy with ``ignore_index=-100`` (:2504-2509), right-aligned to the label length
when modal tokens are prepended (:2497-2498), plus the multi-token-prediction loss (:2519-2538) and the
MoE aux loss when ``moe_aux_loss_free`` is off (:2575-2578).  Padded positions have their embeddings
zeroed (:2107-2109).  The output is a dict with attribute access (``YvModelOutput``, :487).

Internally tokens are packed ``[T, H]``; the LM head and the loss are fused (``ops.loss``) so the logits of
the whole batch never exist during training.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..config import YvConfig
from ..ops import functional as F_
from ..ops.loss import linear_cross_entropy
from .attention import AttnContext
from .blocks import YvTransformerBlock
from .norms import YvRMSNorm, YvRotaryEmbedding


class YvModelOutput(dict):
    """dict with attribute access (``out.loss`` == ``out['loss']``)."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e

    def __setattr__(self, k, v):
        self[k] = v


class YvModel(nn.Module):
    def __init__(self, cfg: YvConfig, parallel=None):
        super().__init__()
        self.cfg, self.parallel = cfg, parallel
        pp_size = parallel.pp_size if parallel is not None else 1
        pp_rank = parallel.pp_rank if parallel is not None else 0
        per = math.ceil(cfg.n_layer / pp_size)
        self.layer_lo, self.layer_hi = pp_rank * per, min(cfg.n_layer, (pp_rank + 1) * per)
        self.is_first_stage, self.is_last_stage = pp_rank == 0, pp_rank == pp_size - 1
        if self.is_first_stage:
            self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
            nn.init.normal_(self.embed.weight, std=cfg.initializer_range)
        self.layers = nn.ModuleList([YvTransformerBlock(cfg, i, parallel) for i in range(self.layer_lo, self.layer_hi)])
        if self.is_last_stage:
            self.norm = YvRMSNorm(cfg.hidden_size, cfg.layer_norm_eps)
        rot = cfg.partial_rope_dim if cfg.use_partial_rope else cfg.head_dim
        if getattr(cfg, "use_mla", False) and getattr(cfg, "use_enhanced_mla", False):
            rot = min(cfg.mla_rope_dim, cfg.head_dim)        # decoupled RoPE: only the shared key slice is rotated
        scaling = "yarn" if cfg.use_dynamic_yarn else ("linear" if cfg.linear_rope_scale != 1.0 else "none")
        factor = cfg.rope_scaling_factor if cfg.use_dynamic_yarn else cfg.linear_rope_scale
        self.rotary = YvRotaryEmbedding(rot, min(cfg.max_position_embeddings, 8192), cfg.rope_theta, scaling, factor,
                                        cfg.max_position_embeddings) if cfg.use_rotary_pos_emb else None
        # optional components, attached by their builders (lazy like the reference, model.py:1276-1516)
        self.subconscious: Optional[nn.Module] = None      # YvSubconsciousSystem / YvPQKnowledgeField
        self.block_field: Optional[nn.Module] = None       # YvSubconsciousBlockField: applied once, to the embeddings
        self.block_field_diagnostics: Optional[dict] = None
        self.vision_encoder: Optional[nn.Module] = None
        self.video_encoder: Optional[nn.Module] = None
        self.audio_encoder: Optional[nn.Module] = None
        self.modal_fusion: Optional[nn.Module] = None
        self.materialized_components: List[str] = []

    # ------------------------------------------------------------------------------------------------
    def sparsity_objective(self) -> Optional[torch.Tensor]:
        """Sum of the parameter-only sparsity regularisers that this module's descendants declare through a callable
        ``sparsity_loss`` (reference model/core/model.py:1951-1976).  Each is the objective of its own gate - a learned
        scalar in front of a sparse branch - and depends on parameters only, so it is evaluated here at loss time rather
        than threaded out of every layer's forward.  It must not ride inside the routing loss: the aux-loss-free
        balancing mode keeps that lump out of the objective, which would leave the gates untrained.  ``modules()`` yields
        every submodule once, so a nested contributor is counted once.  Also callable unbound on any module tree."""
        total = None
        for module in self.modules():
            accessor = getattr(module, "sparsity_loss", None)
            if not callable(accessor):
                continue
            term = accessor()
            if not isinstance(term, torch.Tensor) or not term.requires_grad:
                continue
            total = term if total is None else total + term
        return total

    def attach(self, name: str, module: nn.Module) -> None:
        setattr(self, name, module)
        if name not in self.materialized_components:
            self.materialized_components.append(name)

    def build_context(self, batch: int, seq: int, device: torch.device, lengths: Optional[torch.Tensor] = None,
                      causal: bool = True) -> AttnContext:
        """Context for ``batch`` sequences of equal length ``seq`` (or the given per-sequence lengths)."""
        if lengths is None:
            cu = torch.arange(0, (batch + 1) * seq, seq, dtype=torch.int32, device=device)
            pos = torch.arange(seq, dtype=torch.int32, device=device).repeat(batch)
            max_len = seq
        else:
            cu = torch.zeros(batch + 1, dtype=torch.int32, device=device)
            cu[1:] = torch.cumsum(lengths.int(), 0)
            total = int(cu[-1].item())
            seq_id = torch.repeat_interleave(torch.arange(batch, device=device), lengths.long())
            pos = (torch.arange(total, device=device) - cu[:-1].long()[seq_id]).int()
            max_len = int(lengths.max().item())
        cos = sin = None
        if self.rotary is not None:
            cos, sin = self.rotary.tables(max_len, device)
        return AttnContext(positions=pos, cu_seqlens=cu, max_len=max_len, cos=cos, sin=sin, causal=causal)

    def embed_tokens(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        h = self.embed(input_ids)
        if attention_mask is not None:
            h = h * attention_mask.unsqueeze(-1).to(h.dtype)
        return h

    def run_layers(self, h: torch.Tensor, ctx: AttnContext, batch: int,
                   film_source: Optional[Any] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """h [T, H] -> (final hidden [T, H] before the last norm is applied by the caller, aux loss)."""
        delta: Optional[torch.Tensor] = None
        aux_total = h.new_zeros((), dtype=torch.float32)
        if film_source is not None:
            film_source.begin(h, batch)
        fused_film = film_source.apply_fused if h.is_cuda and getattr(film_source, "fused_ok", False) else None
        for blk in self.layers:
            film = None
            if fused_film is not None:
                # gather + projection + modulation in one kernel: the block then sees an already modulated stream
                if film_source.wants(blk.layer_idx):
                    h = fused_film(h if delta is None else h + delta)
                    delta = None
            elif film_source is not None:
                film = film_source.film_params(blk.layer_idx, h if delta is None else h + delta)
            h, delta, aux = blk(h, delta, ctx, film)
            if torch.is_grad_enabled():          # serving never reads the auxiliary loss: no add kernel per layer
                aux_total = aux_total + aux.float()
        if film_source is not None:
            film_source.end()
        return (h, delta), aux_total

    def forward(self, input_ids: Optional[torch.Tensor] = None, attention_mask: Optional[torch.Tensor] = None,
                inputs_embeds: Optional[torch.Tensor] = None, prefix_embeds: Optional[torch.Tensor] = None,
                ctx: Optional[AttnContext] = None, hidden_in: Optional[torch.Tensor] = None,
                gather_output: bool = True) -> YvModelOutput:
        """Returns ``hidden_states`` [B, S_total, H] (normalised on the last pipeline stage) and ``aux_loss``.
        With ``gather_output=False`` under sequence parallelism the states stay sharded: [B * S / tp, H], the rows of
        this tensor-parallel rank in flattened token order.

        ``prefix_embeds`` [B, P, H] (modal fusion tokens) are concatenated in front of the text embeddings.
        ``hidden_in`` feeds a non-first pipeline stage."""
        if self.is_first_stage:
            h = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids, attention_mask)
            if prefix_embeds is not None:
                h = torch.cat([prefix_embeds.to(h.dtype), h], dim=1)
            if self.block_field is not None and ctx is None:
                # one read per forward, before the first layer; only values leave through the diagnostics
                h, diag = self.block_field.read_and_modulate(h)
                self.block_field_diagnostics = {k: v for k, v in diag.items() if not torch.is_tensor(v)}
        else:
            h = hidden_in
        B, S, H = h.shape
        if ctx is None:
            ctx = self.build_context(B, S, h.device)
        flat = h.reshape(B * S, H)
        if self.parallel is not None and self.parallel.tp_size > 1 and self.cfg.sequence_parallel:
            from ..parallel import tp
            flat = tp.scatter_sequence(flat, self.parallel.tp_group)
        (hf, delta), aux = self.run_layers(flat, ctx, B, self.subconscious)
        if self.is_last_stage:
            out = self.norm(hf) if delta is None else self.norm(delta, residual=hf)[0]
        else:
            out = hf if delta is None else hf + delta
        if self.parallel is not None and self.parallel.tp_size > 1 and self.cfg.sequence_parallel:
            if not gather_output:
                return YvModelOutput(hidden_states=out, aux_loss=aux)
            from ..parallel import tp
            out = tp.gather_sequence(out, self.parallel.tp_group)
        return YvModelOutput(hidden_states=out.view(B, S, H), aux_loss=aux)


class YvModelForCausalLM(nn.Module):
    def __init__(self, cfg: YvConfig, parallel=None):
        super().__init__()
        self.cfg, self.parallel = cfg, parallel
        self.model = YvModel(cfg, parallel)
        self.tied = cfg.tie_word_embeddings and self.model.is_first_stage and self.model.is_last_stage
        if self.model.is_last_stage and not self.tied:
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size))
            nn.init.normal_(self.lm_head, std=cfg.initializer_range)
        self.num_mtp = cfg.num_mtp_heads
        if self.num_mtp > 0 and not cfg.mtp_share_embeddings and self.model.is_last_stage:
            self.mtp_heads = nn.ParameterList(
                [nn.Parameter(torch.randn(cfg.vocab_size, cfg.hidden_size) * cfg.initializer_range)
                 for _ in range(self.num_mtp)])

    @property
    def head_weight(self) -> torch.Tensor:
        return self.model.embed.weight if self.tied else self.lm_head

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """hidden [..., H] -> fp32 logits [..., V] (inference / evaluation only)."""
        return F_.linear(hidden, self.head_weight, out_fp32=True)

    def sparsity_objective(self) -> Optional[torch.Tensor]:
        """The trunk's walk over this whole model.  The contributors are looked up once per training / evaluation
        switch (the walk visits thousands of modules on a deep model and the step is launch-bound on the host).  With
        sequence-parallel tensor parallelism the gradients of replicated parameters are SUMMED over the group, because
        each rank normally holds the part of its own tokens; a parameter-only term is whole on every rank, so it is
        divided by the group size here."""
        found = self.__dict__.get("_sparsity_contributors")
        if found is None:
            found = [m for m in self.modules() if m is not self and m is not self.model
                     and callable(getattr(m, "sparsity_loss", None))]
            self.__dict__["_sparsity_contributors"] = found
        total = None
        for m in found:
            term = m.sparsity_loss()
            if isinstance(term, torch.Tensor) and term.requires_grad:
                total = term if total is None else total + term
        par = self.parallel
        if total is not None and par is not None and par.tp_size > 1 and self.cfg.sequence_parallel:
            total = total / par.tp_size
        return total

    def train(self, mode: bool = True):
        self.__dict__.pop("_sparsity_contributors", None)
        return super().train(mode)

    def forward(self, input_ids: Optional[torch.Tensor] = None, attention_mask: Optional[torch.Tensor] = None,
                labels: Optional[torch.Tensor] = None, prefix_embeds: Optional[torch.Tensor] = None,
                inputs_embeds: Optional[torch.Tensor] = None, ctx: Optional[AttnContext] = None,
                num_valid: Optional[int] = None, return_logits: Optional[bool] = None,
                return_hidden: bool = False, hidden_in: Optional[torch.Tensor] = None, **modal: Any) -> YvModelOutput:
        cfg = self.cfg
        if prefix_embeds is None and modal and self.model.modal_fusion is not None:
            prefix_embeds = self.model.modal_fusion.encode_modalities(self.model, **modal)
        par = self.parallel
        if par is not None and getattr(par, "cp_size", 1) > 1 and self.training and ctx is None and input_ids is not None:
            return self._forward_context_parallel(input_ids, attention_mask, labels)
        if self._split_head_applies(labels, prefix_embeds, return_logits, return_hidden):
            return self._forward_split_head(input_ids, attention_mask, inputs_embeds, labels, ctx, hidden_in, num_valid)
        out = self.model(input_ids, attention_mask, inputs_embeds, prefix_embeds, ctx, hidden_in)
        hidden, aux = out["hidden_states"], out["aux_loss"]
        res = YvModelOutput(aux_loss=aux, loss=None, lm_loss=None, mtp_loss=None, logits=None)
        if return_hidden:
            res["hidden_states"] = hidden
        if not self.model.is_last_stage:
            res["hidden_states"] = hidden
            return res
        if return_logits is None:
            return_logits = labels is None
        if return_logits:
            res["logits"] = self.logits(hidden)
        if labels is not None:
            B, S, H = hidden.shape
            L = labels.shape[1]
            h_txt = hidden[:, S - L:, :]                      # right-align to the labels (modal prefix skipped)
            h_in = h_txt[:, :-1, :].reshape(-1, H)
            tgt = labels[:, 1:].reshape(-1)
            nv = None
            if num_valid is not None:
                nv = num_valid
            lm_loss = linear_cross_entropy(h_in, self.head_weight, tgt, -100, nv)
            loss = lm_loss
            res["lm_loss"] = lm_loss
            if self.num_mtp > 0:
                mtp = hidden.new_zeros((), dtype=torch.float32)
                for i in range(self.num_mtp):
                    if L - 2 - i <= 0:
                        break
                    w = self.head_weight if cfg.mtp_share_embeddings else self.mtp_heads[i]
                    hi = h_txt[:, : L - 2 - i, :].reshape(-1, H)
                    ti = labels[:, 2 + i:].reshape(-1)
                    mtp = mtp + linear_cross_entropy(hi, w, ti, -100, None)
                mtp = mtp / self.num_mtp * cfg.mtp_loss_weight
                res["mtp_loss"] = mtp
                loss = loss + mtp
            if not cfg.moe_aux_loss_free:
                loss = loss + cfg.moe_aux_loss_weight * aux
            sparsity_loss = self.sparsity_objective()
            if sparsity_loss is not None:
                loss = loss + sparsity_loss
            res["loss"] = loss
        return res

    # ---- tensor parallelism: head and loss on the local token shard ----------------------------------------------
    def _split_head_applies(self, labels, prefix_embeds, return_logits, return_hidden) -> bool:
        par, cfg = self.parallel, self.cfg
        return (bool(getattr(cfg, "tp_split_head", False)) and par is not None and par.tp_size > 1 and cfg.sequence_parallel
                and self.training and labels is not None and prefix_embeds is None and not return_logits
                and not return_hidden and self.model.is_last_stage and not self.tied and self.num_mtp == 0)

    def _forward_split_head(self, input_ids, attention_mask, inputs_embeds, labels, ctx, hidden_in, num_valid):
        """The trunk's output stays sequence-sharded; every tensor-parallel rank projects ITS rows onto the vocabulary
        and sums their losses (normalised by the GLOBAL target count).  Nothing is computed twice and the final
        all-gather disappears.  The returned loss has the value of the full mean (one scalar all-reduce) and the
        gradient of the local part, which is what the sharded trunk expects: the backward of the old all-gather kept
        the local rows of an identical gradient anyway.  The head weight now receives a partial gradient per rank and
        is reduced over tensor- x data-parallel ranks like the norm weights (``parallel.zero`` reads the same flag)."""
        import torch.distributed as dist
        par, cfg = self.parallel, self.cfg
        out = self.model(input_ids, attention_mask, inputs_embeds, None, ctx, hidden_in, gather_output=False)
        h_loc, aux = out["hidden_states"], out["aux_loss"]
        B, L = labels.shape
        rows = h_loc.shape[0]
        assert rows * par.tp_size == B * L, "tp_split_head needs labels for every position (no modal prefix)"
        tgt = torch.cat([labels[:, 1:], labels.new_full((B, 1), -100)], 1).reshape(-1)
        nv = int(num_valid) if num_valid is not None else int((tgt != -100).sum().item())
        lo = par.tp_rank * rows
        local = linear_cross_entropy(h_loc, self.head_weight, tgt[lo:lo + rows].contiguous(), -100, nv)
        tot = local.detach().clone()
        dist.all_reduce(tot, group=par.tp_group)
        lm_loss = local + (tot - local.detach())
        loss = lm_loss if cfg.moe_aux_loss_free else lm_loss + cfg.moe_aux_loss_weight * aux
        sparsity_loss = self.sparsity_objective()
        if sparsity_loss is not None:
            loss = loss + sparsity_loss
        return YvModelOutput(aux_loss=aux, loss=loss, lm_loss=lm_loss, mtp_loss=None, logits=None)

    def _forward_context_parallel(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor],
                                  labels: Optional[torch.Tensor]) -> YvModelOutput:
        """Training forward with the sequence dimension split over ``parallel.cp_group``: every rank receives the FULL
        ``[B, S]`` batch (context-parallel peers read the same data), keeps tokens ``[r L, (r+1) L)`` of every
        sequence at their global positions, and computes the loss of its own positions against the globally shifted
        targets, normalised by the global target count, so that the mean over ranks is the full-sequence loss."""
        par, cfg = self.parallel, self.cfg
        W, r = par.cp_size, par.cp_rank
        B, S = input_ids.shape
        assert S % W == 0, f"sequence length {S} must be divisible by the context-parallel size {W}"
        L = S // W
        ids = input_ids[:, r * L:(r + 1) * L]
        am = attention_mask[:, r * L:(r + 1) * L] if attention_mask is not None else None
        ctx = self.model.build_context(B, L, ids.device)
        ctx.positions = ctx.positions + r * L
        if self.model.rotary is not None:
            ctx.cos, ctx.sin = self.model.rotary.tables(S, ids.device)
        ctx.cp_group = par.cp_group
        out = self.model(ids, am, None, None, ctx, None)
        hidden, aux = out["hidden_states"], out["aux_loss"]
        res = YvModelOutput(aux_loss=aux, loss=None, lm_loss=None, mtp_loss=None, logits=None)
        if labels is not None:
            tgt_full = torch.cat([labels[:, 1:], labels.new_full((B, 1), -100)], dim=1)       # target of position t is label t+1
            tgt = tgt_full[:, r * L:(r + 1) * L].reshape(-1)
            n_global = int((tgt_full != -100).sum().item()) if tgt_full.device.type == "cpu" else \
                int((tgt_full != -100).sum().item())
            lm = linear_cross_entropy(hidden.reshape(-1, hidden.shape[-1]), self.head_weight, tgt, -100, 1)
            lm = lm * (float(W) / max(n_global, 1))            # sum over local targets / (global count / ranks)
            res["lm_loss"] = res["loss"] = lm
            if not cfg.moe_aux_loss_free:
                res["loss"] = lm + cfg.moe_aux_loss_weight * aux
            sparsity_loss = self.sparsity_objective()
            if sparsity_loss is not None:
                res["loss"] = res["loss"] + sparsity_loss      # whole on every rank; the ranks' losses are averaged
        return res

    # ------------------------------------------------------------------------------------------------
    # reference-layout state dict (consolidated checkpoint key names)
    # ------------------------------------------------------------------------------------------------
    def to_reference_state_dict(self) -> Dict[str, torch.Tensor]:
        sd: Dict[str, torch.Tensor] = {}
        m = self.model
        if m.is_first_stage:
            sd["embed.weight"] = m.embed.weight.detach().clone()
        for blk in m.layers:
            blk.export_state(f"layers.{blk.layer_idx}.", sd)
        if m.is_last_stage:
            sd["norm.weight"] = m.norm.weight.detach().clone()
            sd["lm_head.weight"] = self.head_weight.detach().clone()
            if self.num_mtp > 0 and not self.cfg.mtp_share_embeddings:
                for i, w in enumerate(self.mtp_heads):
                    sd[f"mtp_heads.{i}.weight"] = w.detach().clone()
        for name in m.materialized_components:
            mod = getattr(m, name, None)
            if isinstance(mod, nn.Module):
                for k, v in mod.state_dict().items():
                    sd[f"{name}.{k}"] = v.detach().clone()
        return sd

    def load_reference_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True) -> List[str]:
        """Load a consolidated checkpoint; returns the list of keys that were not consumed."""
        m = self.model
        used = set()
        with torch.no_grad():
            if m.is_first_stage:
                m.embed.weight.copy_(sd["embed.weight"])
                used.add("embed.weight")
            for blk in m.layers:
                blk.import_state(f"layers.{blk.layer_idx}.", sd)
            if m.is_last_stage:
                m.norm.weight.copy_(sd["norm.weight"])
                used.add("norm.weight")
                if not self.tied and "lm_head.weight" in sd:
                    self.lm_head.copy_(sd["lm_head.weight"])
                used.add("lm_head.weight")
            for name in m.materialized_components:
                mod = getattr(m, name, None)
                if isinstance(mod, nn.Module):
                    sub = {k[len(name) + 1:]: v for k, v in sd.items() if k.startswith(name + ".")}
                    if sub:
                        mod.load_state_dict(sub, strict=strict)
                        used.update(name + "." + k for k in sub)
        prefixes = tuple(f"layers.{b.layer_idx}." for b in m.layers)
        return [k for k in sd if k not in used and not k.startswith(prefixes)]

    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int = 32, **kw: Any):
        from .generation import generate
        return generate(self, input_ids, max_new_tokens=max_new_tokens, **kw)

    def resize_token_embeddings(self, new_size: int) -> None:
        old = self.model.embed.weight.data
        new = torch.empty(new_size, old.shape[1], dtype=old.dtype, device=old.device).normal_(std=self.cfg.initializer_range)
        n = min(new_size, old.shape[0])
        new[:n] = old[:n]
        self.model.embed.weight = nn.Parameter(new)
        if not self.tied:
            oldh = self.lm_head.data
            newh = torch.empty(new_size, oldh.shape[1], dtype=oldh.dtype, device=oldh.device).normal_(
                std=self.cfg.initializer_range)
            newh[:n] = oldh[:n]
            self.lm_head = nn.Parameter(newh)
        self.cfg.vocab_size = new_size


def build_model(cfg: YvConfig, device: Optional[torch.device | str] = None, dtype: Optional[torch.dtype] = None,
                parallel=None, seed: int = 0) -> YvModelForCausalLM:
    """Construct the model directly on ``device`` in ``dtype`` (no fp32 staging copy)."""
    device = torch.device(device) if device is not None else torch.device("cpu")
    dtype = dtype or (torch.bfloat16 if device.type == "cuda" else torch.float32)
    prev = torch.get_default_dtype()
    torch.manual_seed(seed)
    if device.type == "cuda":
        torch.cuda.manual_seed(seed)
    try:
        torch.set_default_dtype(dtype)
        with torch.device(device):
            model = YvModelForCausalLM(cfg, parallel)
    finally:
        torch.set_default_dtype(prev)
    # routing state stays fp32 regardless of the parameter dtype
    for mod in model.modules():
        if hasattr(mod, "expert_bias"):
            mod.expert_bias.data = mod.expert_bias.data.float()
    return model
