"""Latent reasoning engines: modules that take the trunk's hidden states ``[B, S, H]`` and return thinking logits, a
reasoning loss and diagnostics (reference model/reasoning/reasoner/multipath_core.py:128-1487, cot_memory.py:95-450,
unified.py:95-801).  The prompt-level reasoners, which drive a ``generate`` callable with text, are in
``models/reasoning.py``; the classes here are the neural ones.

Built differently from the reference, on purpose:

  * **Causal.**  The thinking logits are trained with a next-token cross-entropy, so position ``t`` must not see
    positions after ``t``.  The reference runs unmasked encoder layers and pools whole sequences into the statistics
    that scale every position (multipath_core.py:566-640), which leaks the targets.  Here the abstraction layers are
    causal, every pooled statistic is a running mean over the prefix, and the bucket-sorted attention of the
    long-sequence branch masks keys by their ORIGINAL position.
  * **No host read-back.**  The reference picks the number of abstraction layers, the early exit and the branch from
    ``.item()`` values of the batch mean.  Here the depth is decided per position on the device: all layers run with
    static shapes and a position keeps its state once its budget is spent, its abstraction gain falls under the
    threshold or it has converged.  The decisions are finer (per position instead of per batch) and the module can be
    captured in a graph.
  * **Paths are attention heads before the output projection**, so pruning a path removes that head's contribution
    (the reference slices the already mixed output, where a slice is not a path).
  * **The loss does not build the logits.**  With labels the collapsed states go through the fused linear +
    cross-entropy kernel against the thinking head's weight; ``[B, S, V]`` logits are produced only on request.
    ``_compute_reasoning_loss`` also accepts logits and then evaluates the cross-entropy in bounded token chunks, which
    equals the plain mean."""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as F_
from ..ops.loss import linear_cross_entropy
from .compat import YvSwiGLU
from .norms import YvRMSNorm

IGNORE_INDEX = -100
REASONING_CE_TOKEN_CHUNK = 4096
STREAMS = ("hypothesis", "evidence", "conclusion")


def _x(cfg: Any, name: str, default: Any) -> Any:
    """Read an option from the config: attribute first, then its ``extra`` dictionary."""
    if hasattr(cfg, name) and getattr(cfg, name) is not None:
        return getattr(cfg, name)
    extra = getattr(cfg, "extra", None)
    return extra.get(name, default) if isinstance(extra, dict) else default


def prefix_mean(x: torch.Tensor) -> torch.Tensor:
    """Running mean along the sequence: out[:, t] = mean(x[:, :t+1]).  x [B, S, ...]."""
    n = torch.arange(1, x.shape[1] + 1, device=x.device, dtype=torch.float32)
    return (x.float().cumsum(1) / n.view(1, -1, *([1] * (x.dim() - 2)))).to(x.dtype)


class _HeadAttention(nn.Module):
    """Causal self-attention that returns the per-head outputs ``[B, S, heads, d]`` BEFORE the output projection."""

    def __init__(self, hidden: int, heads: int, std: float = 0.02):
        super().__init__()
        self.h, self.d = heads, hidden // heads
        self.qkv = nn.Parameter(torch.empty(3 * hidden, hidden).normal_(std=std))
        self.o = nn.Parameter(torch.empty(hidden, hidden).normal_(std=std))

    def heads_out(self, x: torch.Tensor, causal: bool = True) -> torch.Tensor:
        B, S, H = x.shape
        qkv = F_.linear(x.reshape(B * S, H), self.qkv.to(x.dtype))
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=x.device)
        o = F_.attention(qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:], cu, cu, S, S, self.h, self.h, self.d, causal)
        return o.view(B, S, self.h, self.d).to(x.dtype)

    def project(self, heads_out: torch.Tensor) -> torch.Tensor:
        B, S = heads_out.shape[:2]
        return F_.linear(heads_out.reshape(B * S, -1), self.o.to(heads_out.dtype)).view(B, S, -1)

    def forward(self, x: torch.Tensor, causal: bool = True) -> torch.Tensor:
        return self.project(self.heads_out(x, causal))


class _ReasoningLayer(nn.Module):
    """Pre-norm block: causal attention + gated feed-forward (4 x hidden), both residual."""

    def __init__(self, hidden: int, heads: int, causal: bool = True):
        super().__init__()
        self.n1, self.n2 = YvRMSNorm(hidden), YvRMSNorm(hidden)
        self.attn = _HeadAttention(hidden, heads)
        self.ffn = YvSwiGLU(hidden, 4 * hidden)
        self.causal = causal

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, H = x.shape
        x = x + self.attn(self.n1(x.reshape(B * S, H)).view(B, S, H), self.causal)
        return x + self.ffn(self.n2(x.reshape(B * S, H))).view(B, S, H)


def _mlp(sizes: List[int], final: Optional[nn.Module] = None) -> nn.Sequential:
    mods: List[nn.Module] = []
    for i in range(len(sizes) - 1):
        mods.append(nn.Linear(sizes[i], sizes[i + 1]))
        if i < len(sizes) - 2:
            mods.append(nn.ReLU())
    if final is not None:
        mods.append(final)
    return nn.Sequential(*mods)


class YvMultiPathReasoningEngine(nn.Module):
    """Hierarchical abstraction -> multi-path attention with path pruning -> hypothesis / evidence / conclusion streams
    -> convex collapse gated by a verification score -> thinking head.  See the module docstring for what is causal and
    device-side here."""

    def __init__(self, cfg: Any):
        super().__init__()
        self.cfg = cfg
        H = self.hidden_size = int(cfg.hidden_size)
        self.vocab_size = int(cfg.vocab_size)
        self.reasoning_heads = self._resolve_head_count(int(_x(cfg, "reasoning_heads", 8)))
        self.causal = bool(_x(cfg, "reasoning_causal", True))
        n_abs = int(_x(cfg, "reasoning_abstraction_layers", 3))
        self.abstraction_layers = nn.ModuleList([_ReasoningLayer(H, int(cfg.n_head), self.causal) for _ in range(n_abs)])
        self.depth_controller = _mlp([H, max(H // 4, 1), 1], nn.Sigmoid())
        self.multi_path_attention = _HeadAttention(H, self.reasoning_heads)
        self.path_pruning_controller = _mlp([H, max(H // 2, 1), self.reasoning_heads], nn.Sigmoid())
        self.chunked_attention = nn.ModuleDict({
            "lsh_proj": nn.Linear(H, max(H // 4, 8)), "chunk_q": nn.Linear(H, H), "chunk_k": nn.Linear(H, H),
            "chunk_v": nn.Linear(H, H), "output_proj": nn.Linear(H, H), "layer_norm": nn.LayerNorm(H)})
        self.fact_verifier = _mlp([2 * H, H, 1], nn.Sigmoid())
        self.meta_cognitive = nn.GRU(H, H, num_layers=2, batch_first=True)
        self.uncertainty_head = _mlp([H, max(H // 2, 1), 1], nn.Sigmoid())
        self.reasoning_streams = nn.ModuleDict({
            "hypothesis": nn.Linear(H, H), "evidence": nn.Linear(H, H), "conclusion": nn.Linear(H, H),
            "reflection": nn.Linear(H, int(_x(cfg, "react_reflection_classes", 3)))})
        self.thinking_head = nn.Linear(H, self.vocab_size, bias=False)
        nn.init.normal_(self.thinking_head.weight, std=float(_x(cfg, "initializer_range", 0.02)))
        self.long_sequence_tokens = int(_x(cfg, "reasoning_linear_attention_tokens", 512))
        self.long_sequence_layer_cap = int(_x(cfg, "reasoning_long_sequence_layer_cap", 2))
        self.keep_fraction = float(_x(cfg, "reasoning_path_keep_fraction", 0.5))
        self.gain_min = float(_x(cfg, "reasoning_abstraction_gain_min", 0.1))
        self.convergence_threshold = float(_x(cfg, "reasoning_convergence_threshold", 0.001))
        self.complexity_length_tokens = float(_x(cfg, "reasoning_complexity_length_tokens", 512))
        self.reasoning_tokens: Dict[str, Optional[int]] = {
            "start_hypothesis": None, "start_evidence": None, "start_conclusion": None,
            "hypothesis_split": None, "hypothesis_merge": None}
        self.last_depth: Optional[torch.Tensor] = None        # layers applied per position in the last call [B, S]

    # ---- reasoning tokens -----------------------------------------------------------------------------------------------
    def initialize_reasoning_tokens(self, tokenizer: Any = None) -> None:
        """Token ids of the span markers: looked up in the tokenizer when it knows them, otherwise the last five ids of
        the vocabulary."""
        names = list(self.reasoning_tokens)
        for i, name in enumerate(names):
            tid = None
            if tokenizer is not None:
                conv = getattr(tokenizer, "convert_tokens_to_ids", None) or getattr(tokenizer, "token_to_id", None)
                try:
                    tid = conv("<|" + name + "|>") if conv is not None else None
                except Exception:
                    tid = None
            self.reasoning_tokens[name] = int(tid) if isinstance(tid, int) and tid >= 0 else self.vocab_size - len(names) + i

    def resize_vocab(self, new_vocab_size: int) -> None:
        """Grow or shrink the thinking head, keeping the rows that both sizes share."""
        old = self.thinking_head
        new = nn.Linear(self.hidden_size, new_vocab_size, bias=False).to(old.weight.device, old.weight.dtype)
        nn.init.normal_(new.weight, std=0.02)
        n = min(old.weight.shape[0], new_vocab_size)
        with torch.no_grad():
            new.weight[:n] = old.weight[:n]
        self.thinking_head, self.vocab_size = new, new_vocab_size
        if any(v is not None for v in self.reasoning_tokens.values()):
            self.initialize_reasoning_tokens(None)

    # ---- geometry of paths and streams ----------------------------------------------------------------------------------
    def _resolve_head_count(self, requested: int) -> int:
        """Largest divisor of the hidden size that is at most ``requested``: paths are head subspaces."""
        if requested < 1:
            raise ValueError("reasoning_heads must be a positive integer")
        for heads in range(min(requested, self.hidden_size), 0, -1):
            if self.hidden_size % heads == 0:
                return heads
        return 1

    @staticmethod
    def _head_group_indices(heads: int, groups: int, device) -> torch.Tensor:
        """Stream that consumes each path: a balanced monotone partition (stream s owns the heads h with
        h * groups // heads == s)."""
        return (torch.arange(heads, device=device) * groups) // heads

    def _stream_weights(self, path_weights: Optional[torch.Tensor], uncertainty_scores: torch.Tensor,
                        num_streams: int) -> Tuple[torch.Tensor, str]:
        """Coefficients of the stream collapse.  With retained-path weights ``[..., heads]`` (rows sum to 1) the weight
        of a stream is the mass of its heads: a convex combination.  Without them (the long-sequence branch) a uniform
        mixture scaled by the confidence 1 - uncertainty: a contraction, rows sum to at most 1."""
        if path_weights is not None:
            groups = self._head_group_indices(path_weights.shape[-1], num_streams, path_weights.device)
            out = path_weights.new_zeros(*path_weights.shape[:-1], num_streams)
            return out.index_add_(-1, groups, path_weights), "path_partition"
        conf = (1.0 - uncertainty_scores).clamp(0.0, 1.0)
        conf = conf.reshape(conf.shape[0], -1) if conf.dim() == 3 and conf.shape[1] == 1 else conf
        if conf.dim() == 2:                                     # [B, 1]
            return conf.new_full((conf.shape[0], num_streams), 1.0 / num_streams) * conf, "uniform_confidence_scaled"
        return conf.expand(*conf.shape[:-1], num_streams) / num_streams, "uniform_confidence_scaled"

    # ---- per-position statistics ------------------------------------------------------------------------------------------
    def _position_complexity(self, h: torch.Tensor) -> torch.Tensor:
        """[B, S] in [0, 1]: length so far, spread of the prefix around its mean, and the entropy of the prefix's
        normalised state norms (how evenly the information is spread)."""
        B, S, H = h.shape
        hf = h.float()
        pos = torch.arange(1, S + 1, device=h.device, dtype=torch.float32)
        length = (pos / self.complexity_length_tokens).clamp_max(1.0).expand(B, S)
        m1 = prefix_mean(hf)
        m2 = prefix_mean(hf * hf)
        var = (m2 - m1 * m1).clamp_min(0).mean(-1)
        diversity = torch.sigmoid(var * 4.0)
        norms = hf.norm(dim=-1)
        p = norms / torch.cummax(norms, 1).values.clamp_min(1e-8)
        ent = -(p * (p + 1e-8).log())
        density = (ent.cumsum(1) / pos).clamp_min(0) / math.log(2.0)
        return (0.3 * length + 0.4 * diversity + 0.3 * density.clamp_max(1.0)).clamp(0.0, 1.0)

    @staticmethod
    def _abstraction_gain(prev: torch.Tensor, cur: torch.Tensor) -> torch.Tensor:
        """[B, S]: how far a layer moved the running summary (1 - cosine) plus the relative change of its spread."""
        a, b = prefix_mean(prev.float()), prefix_mean(cur.float())
        shift = 1.0 - F.cosine_similarity(a, b, dim=-1)
        va, vb = prev.float().var(-1), cur.float().var(-1)
        return 0.7 * shift + 0.3 * (vb - va).abs() / (va + 1e-8)

    def _abstract(self, h: torch.Tensor, long_sequence: bool) -> Tuple[torch.Tensor, torch.Tensor]:
        """Run the abstraction stack with a per-position depth.  Returns (states, layers applied per position)."""
        n = len(self.abstraction_layers)
        prior = self.depth_controller(prefix_mean(h).float().to(h.dtype)).squeeze(-1).float()        # [B, S]
        budget = 1 + torch.minimum(prior, self._position_complexity(h)).mul(n).floor()
        budget = budget.clamp(1, min(n, self.long_sequence_layer_cap) if long_sequence else n)
        active = torch.ones_like(budget, dtype=torch.bool)
        depth = torch.zeros_like(budget)
        cur = h
        for i, layer in enumerate(self.abstraction_layers):
            active = active & (budget > i)
            new = layer(cur)
            nxt = torch.where(active[..., None], new, cur)
            depth = depth + active.float()
            if i > 0:
                gain = self._abstraction_gain(cur, new)
                moved = (new.float() - cur.float()).abs().mean(-1)
                active = active & (gain >= self.gain_min) & (moved >= self.convergence_threshold)
            cur = nxt
        return cur, depth

    # ---- long-sequence branch ---------------------------------------------------------------------------------------------
    def _lsh_chunked_attention(self, states: torch.Tensor, chunk_size: int = 64, num_hashes: int = 8) -> torch.Tensor:
        """Bucket-sorted block attention.  Tokens are sorted by (bucket, position), where the bucket is the sign
        pattern of the hashed projection; attention runs inside blocks of the sorted order, a block also seeing the
        block before it, and the result returns to the original positions.

        Causal mode: a query sees the keys of ITS bucket among the ``chunk_size`` sorted entries that end at itself.
        Inside a bucket the sorted order is the positional order, so these are the most recent earlier tokens of the
        bucket plus the token itself, and the set does not move when later tokens change bucket (a block boundary does
        move then, which is why the visible set is cut by distance in the sorted order and not by the block).
        Otherwise a query sees its whole block and the previous one, whatever the buckets."""
        ca = self.chunked_attention
        B, S, H = states.shape
        dev = states.device
        hashed = ca["lsh_proj"](states)
        bits = min(num_hashes, hashed.shape[-1])
        code = ((hashed[..., :bits] > 0).long() << torch.arange(bits, device=dev)).sum(-1)          # [B, S]
        pos = torch.arange(S, device=dev).expand(B, S)
        order = torch.argsort(code * S + pos, dim=-1)
        gi = order.unsqueeze(-1).expand(B, S, H)
        q, k, v = (torch.gather(ca[n](states), 1, gi) for n in ("chunk_q", "chunk_k", "chunk_v"))
        scode = torch.gather(code, 1, order)
        nb = math.ceil(S / chunk_size)
        pad = nb * chunk_size - S
        if pad:
            z = q.new_zeros(B, pad, H)
            q, k, v = torch.cat([q, z], 1), torch.cat([k, z], 1), torch.cat([v, z], 1)
            scode = torch.cat([scode, scode.new_full((B, pad), -1)], 1)                            # pads: no bucket
        shp = (B, nb, chunk_size, H)
        bq, bk, bv = q.view(shp), k.view(shp), v.view(shp)
        bc = scode.view(B, nb, chunk_size)
        rank = torch.arange(nb * chunk_size, device=dev).view(1, nb, chunk_size).expand(B, -1, -1)  # sorted index
        prev = lambda t, fill: torch.cat([torch.full_like(t[:, :1], fill), t[:, :-1]], 1)
        wk, wv = torch.cat([prev(bk, 0.0), bk], 2), torch.cat([prev(bv, 0.0), bv], 2)
        wc, wr = torch.cat([prev(bc, -2), bc], 2), torch.cat([prev(rank, -10 ** 9), rank], 2)       # [B, nb, 2c]
        if self.causal:
            dist = rank.unsqueeze(-1) - wr.unsqueeze(-2)                                           # [B, nb, c, 2c]
            visible = (wc.unsqueeze(-2) == bc.unsqueeze(-1)) & (dist >= 0) & (dist < chunk_size) & (bc.unsqueeze(-1) >= 0)
        else:
            visible = ((wc >= 0).unsqueeze(-2) & (bc.unsqueeze(-1) >= 0)).expand(B, nb, chunk_size, 2 * chunk_size)
        scores = (bq @ wk.transpose(-2, -1)).float() / math.sqrt(H)
        scores = scores.masked_fill(~visible, float("-inf"))
        att = torch.nan_to_num(torch.softmax(scores, -1), nan=0.0).to(wv.dtype) @ wv                # pad queries: zero
        att = att.reshape(B, nb * chunk_size, H)[:, :S]
        restored = torch.empty_like(att).scatter_(1, gi, att)
        return ca["layer_norm"](ca["output_proj"](restored) + states)

    # ---- collapse and loss ------------------------------------------------------------------------------------------------
    def _efficient_path_collapse(self, reasoning_outputs: Dict[str, torch.Tensor], uncertainty_scores: torch.Tensor,
                                 verification_scores: List[torch.Tensor],
                                 path_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Weighted sum over the stream axis only; the output keeps [B, S, H].  ``path_weights`` [B, heads] or
        [B, S, heads]; ``uncertainty_scores`` [B, 1, 1] or [B, S, 1]; verification scores broadcastable to [B, S, 1]."""
        missing = [n for n in STREAMS if n not in reasoning_outputs]
        if missing:
            raise ValueError(f"the path collapse needs every reasoning stream; missing={missing}")
        w, _ = self._stream_weights(path_weights, uncertainty_scores, len(STREAMS))
        if w.dim() == 2:
            w = w[:, None, :]
        stacked = torch.stack([reasoning_outputs[n] for n in STREAMS], -1)                         # [B, S, H, streams]
        out = (stacked * w[:, :, None, :].to(stacked.dtype)).sum(-1)
        if verification_scores:
            conf = torch.stack([s if s.dim() == 3 else s[:, None, :] for s in verification_scores], 0).mean(0)
            out = out * conf.to(out.dtype)
        return out

    def _create_reasoning_masks(self, input_ids: Optional[torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Spans between the marker tokens: hypothesis = after its start marker and before the evidence marker, etc."""
        if input_ids is None:
            return {}
        if any(v is None for v in self.reasoning_tokens.values()):
            self.initialize_reasoning_tokens(None)
        t = self.reasoning_tokens
        seen = lambda name: (input_ids == t[name]).cumsum(1) > 0
        return {"hypothesis": seen("start_hypothesis") & ~seen("start_evidence"),
                "evidence": seen("start_evidence") & ~seen("start_conclusion"),
                "conclusion": seen("start_conclusion") & ~seen("hypothesis_merge")}

    def _compute_reasoning_loss(self, reasoning_outputs: Dict[str, torch.Tensor], thinking_logits: Optional[torch.Tensor],
                                uncertainty_scores: torch.Tensor, labels: Optional[torch.Tensor],
                                input_ids: Optional[torch.Tensor] = None,
                                fact_consistency: Optional[torch.Tensor] = None,
                                collapsed: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Next-token cross-entropy of the collapsed stream + per-stream cross-entropy inside the marked spans +
        an uncertainty penalty + a pull of the fact consistency towards one.  Give ``collapsed`` [B, S, H] for the
        fused projection + loss, or ``thinking_logits`` [B, S, V] for the chunked evaluation."""
        ref_t = collapsed if collapsed is not None else thinking_logits
        total = torch.zeros((), device=ref_t.device, dtype=torch.float32)
        W = self.thinking_head.weight
        if labels is not None:
            tgt = labels[:, 1:].reshape(-1)
            if collapsed is not None:
                hs = collapsed[:, :-1].reshape(-1, collapsed.shape[-1])
                count = (tgt != IGNORE_INDEX).sum()               # the divisor stays on the device
                total = total + linear_cross_entropy(hs, W, tgt, IGNORE_INDEX, 1).float() / count.clamp_min(1)
            else:
                lg = thinking_logits[:, :-1].reshape(-1, thinking_logits.shape[-1])
                valid = tgt != IGNORE_INDEX
                count = valid.sum()
                num = torch.zeros((), device=lg.device, dtype=torch.float32)
                for s in range(0, lg.shape[0], REASONING_CE_TOKEN_CHUNK):
                    e = min(s + REASONING_CE_TOKEN_CHUNK, lg.shape[0])
                    num = num + F.cross_entropy(lg[s:e].float(), tgt[s:e], ignore_index=IGNORE_INDEX, reduction="sum")
                total = total + num / count.clamp_min(1)
        if input_ids is not None and labels is not None:
            sw = float(_x(self.cfg, "reasoning_stream_loss_weight", 0.2))
            shift = labels[:, 1:]
            for name, mask in self._create_reasoning_masks(input_ids).items():
                if name not in reasoning_outputs:
                    continue
                span = mask[:, :-1] & (shift != IGNORE_INDEX)
                t_span = torch.where(span, shift, torch.full_like(shift, IGNORE_INDEX)).reshape(-1)
                hs = reasoning_outputs[name][:, :-1].reshape(-1, self.hidden_size)
                n_span = span.sum()
                ce = linear_cross_entropy(hs, W, t_span, IGNORE_INDEX, 1).float() / n_span.clamp_min(1)
                total = total + sw * torch.where(n_span > 0, ce, torch.zeros_like(ce))
        total = total + float(_x(self.cfg, "reasoning_uncertainty_weight", 0.1)) * uncertainty_scores.float().mean()
        if fact_consistency is not None:
            total = total + float(_x(self.cfg, "reasoning_consistency_weight", 0.05)) * \
                (fact_consistency.float() - 1.0).pow(2).mean()
        return total

    # ---- forward ------------------------------------------------------------------------------------------------------------
    def forward(self, hidden_states: torch.Tensor, input_ids: Optional[torch.Tensor] = None,
                labels: Optional[torch.Tensor] = None, return_logits: Optional[bool] = None) -> Dict[str, Any]:
        """hidden_states [B, S, H] -> dict with ``thinking_logits`` [B, S, V] (unless only the loss is wanted),
        ``loss``, ``uncertainty_scores`` [B, 1, 1] (the whole sequence) and ``uncertainty_per_position`` [B, S, 1],
        ``fact_consistency`` [B, S, 1], ``reasoning_outputs`` (three [B, S, H] streams), ``reflection_logits`` [B, C]
        (last position; ``reflection_per_position`` [B, S, C]), ``path_weights`` and ``collapse_rule``."""
        if not bool(_x(self.cfg, "enable_dynamic_fusion", True)):
            raise ValueError("the reasoning engine is disabled by configuration (enable_dynamic_fusion=False); "
                             "there is no stand-in path")
        B, S, H = hidden_states.shape
        if return_logits is None:
            return_logits = labels is None or not self.training
        long_sequence = S > self.long_sequence_tokens
        abstract, depth = self._abstract(hidden_states, long_sequence)
        self.last_depth = depth
        path_weights = None
        if long_sequence:
            multi = self._lsh_chunked_attention(abstract)
        else:
            heads = self.reasoning_heads
            per_head = self.multi_path_attention.heads_out(abstract, self.causal)                   # [B, S, heads, d]
            summary = prefix_mean(abstract) if self.causal else abstract.mean(1, keepdim=True).expand(B, S, H)
            importance = self.path_pruning_controller(summary).float()                              # [B, S, heads]
            keep = min(heads, max(2, int(round(heads * self.keep_fraction)))) if heads > 1 else 1
            top_v, top_i = importance.topk(keep, -1)
            path_weights = torch.zeros_like(importance).scatter_(-1, top_i, torch.softmax(top_v, -1))
            multi = self.multi_path_attention.project(per_head * path_weights[..., None].to(per_head.dtype))
        outs = {n: self.reasoning_streams[n](multi) for n in STREAMS}
        verification = [self.fact_verifier(torch.cat([abstract, multi], -1))]                       # [B, S, 1]
        pooled = prefix_mean(multi) if self.causal else multi.mean(1, keepdim=True).expand(B, S, H)
        meta, _ = self.meta_cognitive(pooled)
        reflection = self.reasoning_streams["reflection"](meta)                                     # [B, S, C]
        uncertainty = self.uncertainty_head(pooled)                                                 # [B, S, 1]
        collapsed = self._efficient_path_collapse(outs, uncertainty, verification, path_weights)
        rule = "path_partition" if path_weights is not None else "uniform_confidence_scaled"
        consistency = self.fact_verifier(torch.cat([prefix_mean(outs["hypothesis"]), prefix_mean(outs["evidence"])], -1)) \
            if self.causal else self.fact_verifier(torch.cat([outs["hypothesis"].mean(1, keepdim=True),
                                                              outs["evidence"].mean(1, keepdim=True)], -1)).expand(B, S, 1)
        loss = self._compute_reasoning_loss(outs, None, uncertainty, labels, input_ids, consistency, collapsed=collapsed)
        logits = None
        if return_logits:
            logits = F_.linear(collapsed.reshape(B * S, H), self.thinking_head.weight, out_fp32=True).view(B, S, -1)
        return {"thinking_logits": logits, "loss": loss, "uncertainty_scores": uncertainty[:, -1:, :],
                "uncertainty_per_position": uncertainty, "fact_consistency": consistency, "reasoning_outputs": outs,
                "reflection_logits": reflection[:, -1], "reflection_per_position": reflection,
                "path_weights": path_weights, "collapse_rule": rule, "collapsed_states": collapsed,
                "abstraction_depth": depth}


# ---------------------------------------------------------------------------------------------------------------------------
class YvMultiDimensionalFactVerifier(nn.Module):
    """Three scores over pooled hypothesis / evidence / conclusion states - logical consistency, knowledge accuracy,
    coherence - and a fused overall score (reference multipath_core.py:982-1076).  Inputs [B, S, H] (pooled over the
    sequence) or already pooled [B, H]."""

    def __init__(self, hidden_size: int):
        super().__init__()
        H = hidden_size
        self.logical_consistency = _mlp([2 * H, H, max(H // 2, 1), 1], nn.Sigmoid())
        self.knowledge_accuracy = _mlp([2 * H, H, max(H // 2, 1), 1], nn.Sigmoid())
        self.coherence_checker = _mlp([3 * H, H, max(H // 2, 1), 1], nn.Sigmoid())
        self.fusion_norm = nn.LayerNorm(H)
        self.fusion_in = nn.Linear(3 * H, H)
        self.fusion_out = _mlp([H, max(H // 2, 1), 1], nn.Sigmoid())
        self.default_coherence = 0.8

    @staticmethod
    def _pool(x: torch.Tensor) -> torch.Tensor:
        return x.mean(1) if x.dim() == 3 else x

    def forward(self, hypothesis: torch.Tensor, evidence: torch.Tensor,
                conclusion: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        hyp, evi = self._pool(hypothesis), self._pool(evidence)
        pair = torch.cat([hyp, evi], -1)
        logical, knowledge = self.logical_consistency(pair), self.knowledge_accuracy(pair)
        if conclusion is not None:
            coherence = self.coherence_checker(torch.cat([pair, self._pool(conclusion)], -1))
        else:
            coherence = torch.full_like(logical, self.default_coherence)
        feats = torch.cat([logical * hyp, knowledge * evi, coherence * hyp], -1)
        overall = self.fusion_out(F.relu(self.fusion_norm(self.fusion_in(feats))))
        return {"logical_consistency": logical, "knowledge_accuracy": knowledge, "coherence": coherence,
                "overall_verification": overall, "is_valid": overall > 0.5}


class YvRLDrivenMetacognition(nn.Module):
    """Actor-critic over four reasoning actions (continue / refine / verify / conclude) with a replay memory kept in
    device buffers, a context editor scored by a performance predictor (candidate search + greedy refinement, decided
    per sample with ``torch.where``), and a depth-dependent scale of the feedback (reference
    multipath_core.py:1079-1363).  The optimisers are created on the first ``update`` so that building the module costs
    no optimiser state."""

    ACTIONS = ("continue", "refine", "verify", "conclude")

    def __init__(self, hidden_size: int, action_dim: int = 4, learning_rate: float = 1e-3, gamma: float = 0.99,
                 memory_size: int = 1000):
        super().__init__()
        H = hidden_size
        self.hidden_size, self.action_dim, self.gamma, self.lr = H, action_dim, gamma, learning_rate
        self.actor_network = _mlp([H, H, max(H // 2, 1), action_dim])
        self.critic_network = _mlp([H, H, max(H // 2, 1), 1])
        self.register_buffer("memory_state", torch.zeros(memory_size, H))
        self.register_buffer("memory_action", torch.zeros(memory_size, dtype=torch.long))
        self.register_buffer("memory_reward", torch.zeros(memory_size))
        self.register_buffer("memory_next", torch.zeros(memory_size, H))
        self.register_buffer("memory_terminal", torch.ones(memory_size))
        self.memory_count = 0
        self.context_editor = nn.Sequential(nn.Linear(H, H), nn.GELU(), nn.Linear(H, H))
        self.performance_predictor = nn.Linear(H, 1)
        self.forward_consistency = nn.Linear(2 * H, 1)
        self.backward_consistency = nn.Linear(2 * H, 1)
        self.layer_entropy_scale = nn.Parameter(torch.ones(1))
        self.num_candidates, self.max_evolution_iterations, self.evolution_threshold = 3, 3, 0.01
        self.action_names = list(self.ACTIONS[:action_dim]) + [f"action_{i}" for i in range(len(self.ACTIONS), action_dim)]
        self._optimizers: Optional[Tuple[torch.optim.Optimizer, torch.optim.Optimizer]] = None

    # -- context evolution --------------------------------------------------------------------------------------------------
    def _context_evolution(self, pooled: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """One edit of a pooled context [B, H]; kept per sample only where the predicted score rises by more than the
        threshold.  Returns (context, accepted [B] bool)."""
        edited = pooled + self.context_editor(pooled)
        better = (self.performance_predictor(edited) - self.performance_predictor(pooled)).squeeze(-1) > self.evolution_threshold
        return torch.where(better[:, None], edited, pooled), better

    def _implicit_verify(self, reasoning_hidden: torch.Tensor, conclusion_hidden: torch.Tensor) -> torch.Tensor:
        pair = torch.cat([reasoning_hidden, conclusion_hidden], -1)
        return 0.5 * (torch.sigmoid(self.forward_consistency(pair)) + torch.sigmoid(self.backward_consistency(pair)))

    def tree_guided_evolution(self, hidden_states: torch.Tensor,
                              reasoning_context: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        base = reasoning_context if reasoning_context is not None else hidden_states.mean(1)
        cands, scores = [], []
        for i in range(self.num_candidates):
            v = base + torch.randn_like(base) * (0.1 * (i + 1) / self.num_candidates)
            v = v + self.context_editor(v)
            cands.append(v)
            scores.append(self.performance_predictor(v).squeeze(-1))
        scores_t = torch.stack(scores, 0)                                  # [C, B]
        best = scores_t.argmax(0)                                          # [B]
        ctx = torch.stack(cands, 0).gather(0, best.view(1, -1, 1).expand(1, -1, base.shape[-1])).squeeze(0)
        initial = scores_t.gather(0, best[None]).squeeze(0)
        accepted = torch.zeros_like(best, dtype=torch.bool)
        alive = torch.ones_like(accepted)
        for _ in range(self.max_evolution_iterations - 1):
            new, better = self._context_evolution(ctx)
            take = alive & better & (self.performance_predictor(new).squeeze(-1) > initial)
            ctx = torch.where(take[:, None], new, ctx)
            accepted, alive = accepted | take, take
        return {"evolved_context": ctx, "best_candidate_idx": best, "initial_score": initial,
                "final_score": self.performance_predictor(ctx).squeeze(-1), "accepted_refinement": accepted}

    def _layer_entropy_control(self, pooled: torch.Tensor, layer_index: int, total_layers: int) -> torch.Tensor:
        """Early layers are scaled up (explore), late layers down (commit), the middle third is left alone."""
        r = layer_index / max(total_layers - 1, 1)
        target = 1.0 + (0.33 - r) * 0.5 if r < 0.33 else (1.0 if r < 0.66 else 1.0 - (r - 0.66) * 0.5)
        return pooled * (self.layer_entropy_scale * target)

    # -- actor-critic ---------------------------------------------------------------------------------------------------------
    def select_action(self, hidden_states: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        pooled = hidden_states.mean(1) if hidden_states.dim() == 3 else hidden_states
        probs = torch.softmax(self.actor_network(pooled).float(), -1)
        action = torch.multinomial(probs, 1).squeeze(-1)
        return action, probs, self.critic_network(pooled)

    @torch.no_grad()
    def _store_transition(self, state: torch.Tensor, action: torch.Tensor, reward: Any,
                          next_state: Optional[torch.Tensor] = None) -> None:
        """state [B, H] or [H]; action [B] ids (or one-hot rows); reward scalar or [B]."""
        state = state.reshape(-1, self.hidden_size)
        n = state.shape[0]
        action = action.reshape(n, -1).argmax(-1) if action.dim() > 1 and action.shape[-1] == self.action_dim and \
            action.is_floating_point() else action.reshape(n).long()
        reward = torch.as_tensor(reward, dtype=torch.float32, device=state.device).expand(n)
        slots = (torch.arange(n, device=state.device) + self.memory_count) % self.memory_state.shape[0]
        self.memory_state[slots], self.memory_action[slots], self.memory_reward[slots] = state.float(), action, reward
        if next_state is not None:
            self.memory_next[slots], self.memory_terminal[slots] = next_state.reshape(n, -1).float(), 0.0
        else:
            self.memory_terminal[slots] = 1.0
        self.memory_count += n

    def _sample_experience(self, batch_size: int = 32):
        avail = min(self.memory_count, self.memory_state.shape[0])
        if avail <= 0:
            raise RuntimeError("no stored transition to sample")
        i = torch.randperm(avail, device=self.memory_state.device)[:min(batch_size, avail)]
        return self.memory_state[i], self.memory_action[i], self.memory_reward[i], self.memory_next[i], self.memory_terminal[i]

    def update(self, state: torch.Tensor, action: torch.Tensor, reward: Any,
               next_state: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        """Store the transition, then one critic step (TD target r + gamma V(s'), V(s') = 0 on terminal transitions)
        and one policy-gradient step on a replayed batch.  The returned values are tensors (no read-back)."""
        self._store_transition(state, action, reward, next_state)
        if self._optimizers is None:
            self._optimizers = (torch.optim.Adam(self.actor_network.parameters(), lr=self.lr),
                                torch.optim.Adam(self.critic_network.parameters(), lr=self.lr))
        opt_a, opt_c = self._optimizers
        s, a, r, s2, term = self._sample_experience()
        with torch.no_grad():
            target = r + self.gamma * (1.0 - term) * self.critic_network(s2).squeeze(-1)
        with torch.enable_grad():
            v = self.critic_network(s).squeeze(-1)
            critic_loss = F.mse_loss(v, target)
            opt_c.zero_grad()
            critic_loss.backward()
            torch.nn.utils.clip_grad_norm_(self.critic_network.parameters(), 1.0)
            opt_c.step()
            adv = (target - v.detach())
            logp = torch.log_softmax(self.actor_network(s).float(), -1).gather(1, a[:, None]).squeeze(1)
            actor_loss = -(logp * adv).mean()
            opt_a.zero_grad()
            actor_loss.backward()
            torch.nn.utils.clip_grad_norm_(self.actor_network.parameters(), 1.0)
            opt_a.step()
        return {"actor_loss": actor_loss.detach(), "critic_loss": critic_loss.detach(), "advantage": adv.mean()}

    def forward(self, hidden_states: torch.Tensor, reasoning_outputs: Optional[Dict[str, torch.Tensor]] = None,
                enable_evolution: bool = False, layer_index: Optional[int] = None,
                total_layers: Optional[int] = None) -> Dict[str, Any]:
        pooled = hidden_states.mean(1)
        out: Dict[str, Any] = {}
        if enable_evolution:
            ev = self.tree_guided_evolution(hidden_states, pooled)
            pooled = ev["evolved_context"]
            out.update(evolved=ev["accepted_refinement"], evolution_score=ev["final_score"])
        if layer_index is not None and total_layers is not None:
            pooled = self._layer_entropy_control(pooled, layer_index, total_layers)
        action, probs, value = self.select_action(hidden_states)
        out.update(selected_action=action, action_probs=probs, action_value=value, metacognitive_feedback=pooled)
        capturing = action.is_cuda and torch.cuda.is_current_stream_capturing()
        out["action_name"] = None if capturing else [self.action_names[i] for i in action.tolist()]   # names need the ids
        return out


class YvAdaptiveReasoningController(nn.Module):
    """Learned depth strategy (reference multipath_core.py:1366-1487): per sample, a complexity feature vector (mean
    state + length, spread and entropy terms) is encoded, a strategy is chosen among four and a depth predicted; a
    resource estimate scales the depth down when it exceeds the budget.  All outputs are per-sample tensors."""

    STRATEGIES = ("shallow_fast", "standard_balanced", "deep_thorough", "recursive_refine")

    def __init__(self, hidden_size: int, max_depth: int = 12, num_strategies: int = 4):
        super().__init__()
        H = hidden_size
        self.hidden_size, self.max_depth, self.num_strategies = H, max_depth, num_strategies
        self.complexity_encoder = nn.Sequential(nn.Linear(H + 3, max(H // 2, 4)), nn.ReLU(),
                                                nn.Linear(max(H // 2, 4), max(H // 4, 4)), nn.ReLU())
        self.strategy_network = _mlp([max(H // 4, 4), max(H // 8, 4), num_strategies])
        self.depth_predictor = _mlp([max(H // 4, 4), max(H // 8, 4), max_depth], nn.Sigmoid())
        self.resource_estimator = _mlp([H, max(H // 2, 1), 2], nn.Sigmoid())
        self.strategy_names = list(self.STRATEGIES[:num_strategies]) + \
            [f"strategy_{i}" for i in range(len(self.STRATEGIES), num_strategies)]

    def estimate_complexity(self, hidden_states: torch.Tensor) -> Dict[str, torch.Tensor]:
        B, S, H = hidden_states.shape
        hf = hidden_states.float()
        length = hf.new_full((B, 1), min(S / 1024.0, 1.0))
        variance = hf.var(dim=(1, 2), unbiased=False).view(B, 1)
        p = torch.softmax(hf.norm(dim=-1), -1)                                     # where the mass of the sequence sits
        density = (-(p * (p + 1e-8).log()).sum(-1, keepdim=True) / math.log(S + 1.0))
        feats = torch.cat([hf.mean(1), length, variance, density], -1).to(hidden_states.dtype)
        enc = self.complexity_encoder(feats)
        probs = torch.softmax(self.strategy_network(enc).float(), -1)
        depth_scores = self.depth_predictor(enc)
        depth = (depth_scores.float().mean(-1) * self.max_depth).floor().add(1).clamp(1, self.max_depth)
        return {"complexity_score": (0.3 * length + 0.4 * torch.sigmoid(variance) + 0.3 * density).squeeze(-1),
                "strategy_probs": probs, "strategy_index": probs.argmax(-1), "estimated_depth": depth,
                "resource_budget": self.resource_estimator(hidden_states.mean(1)), "depth_scores": depth_scores}

    def forward(self, hidden_states: torch.Tensor, budget_constraint: float = 1.0) -> Dict[str, Any]:
        a = self.estimate_complexity(hidden_states)
        usage = a["resource_budget"].float().mean(-1)                              # [B]
        over = usage > budget_constraint
        scaled = (a["estimated_depth"] * budget_constraint / usage.clamp_min(1e-6)).floor()
        depth = torch.where(over, torch.minimum(a["estimated_depth"], scaled), a["estimated_depth"]).clamp_min(1)
        return {"complexity_score": a["complexity_score"], "strategy_index": a["strategy_index"],
                "strategy_name": [self.strategy_names[i] for i in a["strategy_index"].tolist()],
                "optimal_depth": depth.long(), "strategy_probs": a["strategy_probs"], "resource_estimate": usage,
                "budget_compliance": ~over}


# ---------------------------------------------------------------------------------------------------------------------------
class YvLatentCoTReasoner(nn.Module):
    """Chain-of-thought over hidden states with an optional memory (reference cot_memory.py:95-450): memory entries
    are attended to and added, a small causal stack with a per-position depth refines the states, and heads read the
    last position: next-token logits, difficulty (5 classes), reflection type (4), confidence, an error analysis
    (type, severity, confidence) and a correction proposal conditioned on it."""

    def __init__(self, cfg: Any):
        super().__init__()
        from .compat import YvCrossAttention
        self.cfg = cfg
        H = self.hidden_size = int(cfg.hidden_size)
        self.vocab_size = int(cfg.vocab_size)
        self.causal = bool(_x(cfg, "reasoning_causal", True))
        self.reasoning_layers = nn.ModuleList([_ReasoningLayer(H, int(cfg.n_head), self.causal) for _ in range(3)])
        self.depth_controller = _mlp([H, max(H // 4, 1), 1], nn.Sigmoid())
        self.thinking_head = nn.Linear(H, self.vocab_size, bias=False)
        nn.init.normal_(self.thinking_head.weight, std=float(_x(cfg, "initializer_range", 0.02)))
        self.difficulty_head = nn.Linear(H, 5)
        self.reflection_head = nn.Linear(H, 4)
        self.confidence_head = nn.Linear(H, 1)
        self.memory_attention = YvCrossAttention(H, H, int(cfg.n_head))
        self.error_analyzer = _mlp([H, max(H // 2, 1), 3])
        self.correction_head = _mlp([H + 3, H, H])
        self.layer_norm = nn.LayerNorm(H)
        self.gain_min = float(_x(cfg, "reasoning_abstraction_gain_min", 0.1))
        self.convergence_threshold = float(_x(cfg, "reasoning_convergence_threshold", 0.001))
        self.complexity_length_tokens = float(_x(cfg, "reasoning_complexity_length_tokens", 512))
        self.long_sequence_layer_cap = len(self.reasoning_layers)
        self.last_depth: Optional[torch.Tensor] = None

    # the per-position depth machinery is the engine's
    abstraction_layers = property(lambda self: self.reasoning_layers)
    _position_complexity = YvMultiPathReasoningEngine._position_complexity
    _abstraction_gain = staticmethod(YvMultiPathReasoningEngine._abstraction_gain)
    _abstract = YvMultiPathReasoningEngine._abstract

    def sequence_complexity(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """[B]: the complexity at the last position, i.e. of the whole sequence."""
        return self._position_complexity(hidden_states)[:, -1]

    def _memory_tensor(self, memory_context: Any, like: torch.Tensor) -> Optional[torch.Tensor]:
        if memory_context is None:
            return None
        if not torch.is_tensor(memory_context):
            if len(memory_context) == 0:
                return None
            memory_context = torch.stack([torch.as_tensor(m) for m in memory_context])
        m = memory_context.to(like.device, like.dtype)
        if m.dim() == 2:
            m = m.unsqueeze(0).expand(like.shape[0], -1, -1)
        return m

    def forward(self, input_ids: Optional[torch.Tensor] = None, attention_mask: Optional[torch.Tensor] = None,
                memory_context: Any = None, labels: Optional[torch.Tensor] = None, **kwargs: Any) -> Dict[str, Any]:
        hidden = input_ids if torch.is_tensor(input_ids) and input_ids.is_floating_point() else kwargs.get("hidden_states")
        if hidden is None:
            raise ValueError("the latent reasoner needs real hidden states [B, S, H]; it never invents them")
        mem = self._memory_tensor(memory_context, hidden)
        if mem is not None:
            hidden = hidden + self.memory_attention(hidden, mem)
        states, depth = self._abstract(self.layer_norm(hidden), False)
        self.last_depth = depth
        final = states[:, -1]
        err = self.error_analyzer(final)
        out = {"thinking_logits": F_.linear(final, self.thinking_head.weight, out_fp32=True),
               "difficulty_logits": self.difficulty_head(final), "reflection_logits": self.reflection_head(final),
               "confidence_score": torch.sigmoid(self.confidence_head(final)), "reasoning_states": states,
               "reasoning_steps": [states], "correction_logits": self.correction_head(torch.cat([final, err], -1)),
               "error_analysis": err, "attention_weights": None, "final_state": final, "abstraction_depth": depth}
        if labels is not None:
            tgt = labels[:, 1:].reshape(-1)
            hs = states[:, :-1].reshape(-1, self.hidden_size)
            out["loss"] = linear_cross_entropy(hs, self.thinking_head.weight, tgt, IGNORE_INDEX, 1).float() / \
                (tgt != IGNORE_INDEX).sum().clamp_min(1)
        return out


class YvLatentUnifiedReasoner(nn.Module):
    """Routes between the chain-of-thought reasoner and the multi-path engine and returns one output format
    (reference unified.py:95-801).  ``routing``:

      * ``"length"`` (default): multi-path when the sequence is longer than ``mpr_seq_len_threshold``; decided from the
        shape, so nothing is read back from the device;
      * ``"complexity"``: also multi-path when the mean sequence complexity reaches ``mpr_threshold`` (one read-back per
        call, the reference's rule);
      * ``"blend"``: both run and each sample takes the logits of its own route (no read-back, twice the work).

    The thinking depth (1 / 3 / 5 / 10 refinement rounds) is a per-sample tensor derived from a learned complexity
    estimate and the intensity parameter; ``reason_latent`` uses it as its iteration budget."""

    def __init__(self, cfg: Any, device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.cfg = cfg
        H = int(cfg.hidden_size)
        self.cot_reasoner = YvLatentCoTReasoner(cfg)
        self.multi_path_core = YvMultiPathReasoningEngine(cfg)
        self.enable_multi_path_core = bool(_x(cfg, "enable_multi_path_core", True))
        self.mpr_threshold = float(_x(cfg, "mpr_threshold", 0.6))
        self.seq_len_threshold = int(_x(cfg, "mpr_seq_len_threshold", 512))
        self.routing = str(_x(cfg, "reasoning_routing", "length"))
        self.thinking_intensity = float(_x(cfg, "thinking_intensity", 0.5))
        self.complexity_threshold_low = float(_x(cfg, "complexity_threshold_low", 0.3))
        self.complexity_threshold_high = float(_x(cfg, "complexity_threshold_high", 0.7))
        self.complexity_estimator = _mlp([H, max(H // 4, 1), 1], nn.Sigmoid())
        self.thinking_depth_controller = nn.Parameter(torch.full((1,), self.thinking_intensity))
        self._logit_temp = nn.Parameter(torch.tensor(1.0))
        if device is not None or dtype is not None:
            self.to(device=device, dtype=dtype)

    def initialize_reasoning_tokens(self, tokenizer: Any = None) -> None:
        self.multi_path_core.initialize_reasoning_tokens(tokenizer)

    @staticmethod
    def _extract_hidden_states(input_ids: Optional[torch.Tensor], kwargs: Dict[str, Any]) -> torch.Tensor:
        if torch.is_tensor(input_ids) and input_ids.is_floating_point():
            return input_ids
        hs = kwargs.get("hidden_states")
        if torch.is_tensor(hs):
            return hs
        raise ValueError("the unified reasoner needs real hidden states (hidden_states=... or a float input); it never "
                         "invents them")

    def complexity(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """[B] in [0, 1]: 0.3 log-length + 0.3 squashed feature variance + 0.4 learned estimate."""
        S = hidden_states.shape[1]
        var = torch.sigmoid(hidden_states.float().var(-1).mean(-1))
        learned = self.complexity_estimator(hidden_states.mean(1)).squeeze(-1).float()
        return 0.3 * (math.log1p(S) / 10.0) + 0.3 * var + 0.4 * learned

    def thinking_depth(self, complexity: torch.Tensor) -> torch.Tensor:
        eff = complexity * torch.sigmoid(self.thinking_depth_controller.float())
        d = torch.full_like(eff, 10.0)
        d = torch.where(eff < 0.9, torch.full_like(eff, 5.0), d)
        d = torch.where(eff < self.complexity_threshold_high, torch.full_like(eff, 3.0), d)
        return torch.where(eff < self.complexity_threshold_low, torch.full_like(eff, 1.0), d).long()

    def _route(self, hidden_states: torch.Tensor) -> Tuple[str, Optional[torch.Tensor]]:
        if not self.enable_multi_path_core:
            return "cot", None
        if hidden_states.shape[1] > self.seq_len_threshold:
            return "multi_path", None
        if self.routing == "complexity":
            c = self.cot_reasoner.sequence_complexity(hidden_states).mean()
            return ("multi_path" if bool(c >= self.mpr_threshold) else "cot"), None
        if self.routing == "blend":
            return "blend", self.cot_reasoner.sequence_complexity(hidden_states) >= self.mpr_threshold
        return "cot", None

    def _should_use_multi_path(self, hidden_states: torch.Tensor) -> bool:
        return self._route(hidden_states)[0] != "cot"

    def forward(self, input_ids: Optional[torch.Tensor] = None, attention_mask: Optional[torch.Tensor] = None,
                memory_context: Any = None, labels: Optional[torch.Tensor] = None, **kwargs: Any) -> Dict[str, Any]:
        """Returns thinking_logits [B, V] (next token after the sequence), difficulty / reflection / correction logits,
        confidence_score [B, 1], reasoning_states, final_state, loss, thinking_depth [B] and complexity_score [B].  An
        integer ``attention_mask`` is read as the token ids (where the reasoning spans are marked)."""
        hs = self._extract_hidden_states(input_ids, kwargs)
        kwargs = {k: v for k, v in kwargs.items() if k != "hidden_states"}
        cx = self.complexity(hs)
        depth = self.thinking_depth(cx)
        if labels is None and torch.is_tensor(memory_context) and not memory_context.is_floating_point():
            labels, memory_context = memory_context, None
        ids = attention_mask if torch.is_tensor(attention_mask) and attention_mask.dtype in (torch.int32, torch.int64) \
            and attention_mask.shape == hs.shape[:2] else None
        route, per_sample = self._route(hs)
        cot = self.cot_reasoner(hs, None, memory_context, labels=labels if route != "multi_path" else None, **kwargs)
        if route == "cot":
            cot.setdefault("loss", hs.new_zeros((), dtype=torch.float32))
            cot.update(thinking_depth=depth, complexity_score=cx, route="cot")
            return cot
        core = self.multi_path_core(hs, input_ids=ids, labels=labels, return_logits=False)
        last = core["collapsed_states"][:, -1]
        logits = F_.linear(last, self.multi_path_core.thinking_head.weight, out_fp32=True) / self._logit_temp.clamp_min(1e-3)
        conf = 0.5 * cot["confidence_score"] + 0.5 * (1.0 - core["uncertainty_scores"].reshape(-1, 1))
        loss = core["loss"]
        if route == "blend":
            logits = torch.where(per_sample[:, None], logits, cot["thinking_logits"])
            conf = torch.where(per_sample[:, None], conf, cot["confidence_score"])
            if "loss" in cot:
                loss = 0.5 * (loss + cot["loss"])
        return {"thinking_logits": logits, "difficulty_logits": cot["difficulty_logits"],
                "reflection_logits": cot["reflection_logits"], "confidence_score": conf,
                "reasoning_states": core["collapsed_states"], "reasoning_steps": [], "attention_weights": None,
                "correction_logits": cot["correction_logits"], "final_state": hs.mean(1), "loss": loss,
                "thinking_depth": depth, "complexity_score": cx, "route": route, "core": core}

    @staticmethod
    def _sample_next_token(logits: torch.Tensor, temperature: float = 0.7, top_p: float = 0.9, top_k: int = 50) -> torch.Tensor:
        """logits [B, V] -> ids [B]; greedy at temperature 0, otherwise top-k then nucleus sampling."""
        if temperature <= 0:
            return logits.argmax(-1)
        lg = logits.float() / temperature
        if 0 < top_k < lg.shape[-1]:
            kth = lg.topk(top_k, -1).values[..., -1:]
            lg = lg.masked_fill(lg < kth, float("-inf"))
        if top_p < 1.0:
            sv, si = lg.sort(-1, descending=True)
            cum = torch.softmax(sv, -1).cumsum(-1)
            drop = cum - torch.softmax(sv, -1) >= top_p                # keep the first token that crosses the mass
            lg = lg.masked_fill(torch.zeros_like(drop).scatter(-1, si, drop), float("-inf"))
        return torch.multinomial(torch.softmax(lg, -1), 1).squeeze(-1)

    @torch.no_grad()
    def reason_latent(self, hidden_states: torch.Tensor, max_depth: int = 8, confidence_threshold: float = 0.85,
                      enable_self_correction: bool = True) -> Dict[str, Any]:
        """Refinement in hidden-state space with no token produced: the pooled state is fed through the chain-of-thought
        reasoner round after round.  A sample stops once its confidence passes the threshold or its own thinking depth
        is spent; a round whose confidence falls under half of the previous one is undone by blending back towards the
        starting state (counted as a correction).  Everything is per sample and stays on the device."""
        pooled = hidden_states.mean(1) if hidden_states.dim() == 3 else hidden_states
        budget = self.thinking_depth(self.complexity(hidden_states if hidden_states.dim() == 3 else pooled[:, None]))
        state = F.normalize(pooled.float(), dim=-1).to(pooled.dtype)
        B = state.shape[0]
        done = torch.zeros(B, dtype=torch.bool, device=state.device)
        prev_conf = torch.zeros(B, device=state.device)
        corrections = torch.zeros(B, dtype=torch.long, device=state.device)
        rounds = torch.zeros(B, dtype=torch.long, device=state.device)
        trace: List[torch.Tensor] = []
        for step in range(max_depth):
            out = self.cot_reasoner(state[:, None, :])
            conf = out["confidence_score"].reshape(B).float()
            live = ~done & (budget > step)
            fell = enable_self_correction & (step > 0) & (conf < 0.5 * prev_conf) & live
            blend = (conf / prev_conf.clamp_min(1e-6)).clamp_max(0.7)[:, None].to(state.dtype)
            undone = F.normalize((blend * state + (1 - blend) * pooled).float(), dim=-1).to(state.dtype)
            advanced = F.normalize((state + out["correction_logits"].to(state.dtype) * 0.1).float(), dim=-1).to(state.dtype)
            new = torch.where(fell[:, None], undone, advanced)
            state = torch.where(live[:, None], new, state)
            corrections = corrections + fell.long()
            rounds = rounds + live.long()
            prev_conf = torch.where(live & ~fell, conf, prev_conf)
            done = done | (live & ~fell & (conf >= confidence_threshold))
            trace.append(conf)
        final = self.cot_reasoner(state[:, None, :])
        return {"refined_hidden": state, "reasoning_trace": torch.stack(trace, 1), "final_confidence":
                final["confidence_score"].reshape(B), "final_difficulty": final["difficulty_logits"].softmax(-1),
                "num_iterations": rounds, "correction_count": corrections, "thinking_budget": budget}

    @torch.no_grad()
    def generate_with_thinking(self, prompt: str, tokenizer: Any, embed: Any, max_new_tokens: int = 256,
                               max_think_tokens: int = 128, temperature: float = 0.7, top_p: float = 0.9,
                               top_k: int = 50, enable_thinking: bool = True) -> str:
        """Two-phase autoregressive generation from the reasoner's own logits: a thinking span between ``<|think|>``
        and ``</|think|>`` (closed by force after ``max_think_tokens``), then the answer until end-of-sequence.
        ``embed`` maps token ids [1, S] to hidden states [1, S, H] (the trunk, or its embedding table)."""
        self.eval()
        dev = self._logit_temp.device
        open_tag, close_tag = "<|think|>", "</|think|>"
        ids = list(tokenizer.encode((open_tag if enable_thinking else "") + prompt))
        eos = getattr(tokenizer, "eos_token_id", None)
        new: List[int] = []
        thinking, n_think = enable_thinking, 0
        close_ids = list(tokenizer.encode(close_tag))
        while len(new) < max_new_tokens:
            hs = embed(torch.tensor([ids + new], device=dev))
            nxt = int(self._sample_next_token(self.forward(hidden_states=hs)["thinking_logits"], temperature, top_p, top_k)[0])
            new.append(nxt)
            if thinking:
                n_think += 1
                if close_tag in tokenizer.decode(new):
                    thinking = False
                elif n_think >= max_think_tokens:
                    new.extend(close_ids)
                    thinking = False
                continue
            if eos is not None and nxt == eos:
                break
        text = tokenizer.decode(new)
        return (open_tag + text) if enable_thinking else text


# names of the reference, for code that imports them from here
YvCoTMemoryReasoner = YvLatentCoTReasoner
YvUnifiedReasoner = YvLatentUnifiedReasoner
