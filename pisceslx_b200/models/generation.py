"""Sampling strategies and the cached generation loop.

``YvSampler`` covers the reference's strategies (model/generation/sampler.py:112-243): greedy, top-k, top-p,
top-k+top-p, typical, eta, min-p, with repetition penalty and no-repeat-ngram blocking; beam search and
contrastive search are sequence-level procedures in ``beam_search`` / ``contrastive_search``.
``generate`` is a prefill + paged-KV decode loop (the reference's ``_standard_generate`` re-runs the whole
sequence per token, model/core/model.py:1886-1896; its cached loop lives in tools/infer/core.py:1106-1144).
``YvSpeculativeDecoder`` implements draft-and-verify with the reference's threshold acceptance rule
(model/generation/speculative.py:550-568) and its back-off after three empty rounds (:855-866).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from .attention import AttnContext
from .cache import YvPagedKVCache, cache_for_model


class YvSamplingStrategy(str, Enum):
    GREEDY = "greedy"
    TOP_K = "top_k"
    TOP_P = "top_p"
    TOP_K_TOP_P = "top_k_top_p"
    TYPICAL = "typical"
    ETA = "eta"
    MIN_P = "min_p"
    BEAM = "beam"
    CONTRASTIVE = "contrastive"


@dataclass
class YvSamplingConfig:
    strategy: str = "greedy"
    temperature: float = 1.0
    top_k: int = 50
    top_p: float = 0.95
    min_p: float = 0.0
    typical_p: float = 0.95
    eta_cutoff: float = 3e-4
    repetition_penalty: float = 1.0
    no_repeat_ngram_size: int = 0
    num_beams: int = 1
    seed: Optional[int] = None


class YvSampler:
    def __init__(self, cfg: Optional[YvSamplingConfig] = None):
        self.cfg = cfg or YvSamplingConfig()
        self.gen: Optional[torch.Generator] = None

    def _generator(self, device) -> Optional[torch.Generator]:
        if self.cfg.seed is None:
            return None
        if self.gen is None or self.gen.device != device:
            self.gen = torch.Generator(device=device).manual_seed(self.cfg.seed)
        return self.gen

    @staticmethod
    def apply_repetition_penalty(logits: torch.Tensor, prev: torch.Tensor, penalty: float) -> torch.Tensor:
        if penalty == 1.0 or prev.numel() == 0:
            return logits
        g = logits.gather(-1, prev)
        g = torch.where(g > 0, g / penalty, g * penalty)
        return logits.scatter(-1, prev, g)

    @staticmethod
    def block_repeated_ngrams(logits: torch.Tensor, prev: torch.Tensor, n: int) -> torch.Tensor:
        if n <= 0 or prev.shape[1] < n:
            return logits
        for b in range(prev.shape[0]):
            seq = prev[b].tolist()
            prefix = tuple(seq[-(n - 1):]) if n > 1 else ()
            banned = [seq[i + n - 1] for i in range(len(seq) - n + 1) if tuple(seq[i:i + n - 1]) == prefix]
            if banned:
                logits[b, banned] = float("-inf")
        return logits

    def filter(self, logits: torch.Tensor) -> torch.Tensor:
        """Apply the strategy's truncation to logits [B, V]; returns filtered logits."""
        c = self.cfg
        s = c.strategy
        if s in ("top_k", "top_k_top_p") and c.top_k > 0:
            kth = torch.topk(logits, min(c.top_k, logits.shape[-1]), dim=-1).values[..., -1:]
            logits = logits.masked_fill(logits < kth, float("-inf"))
        if s in ("top_p", "top_k_top_p") and c.top_p < 1.0:
            sl, si = torch.sort(logits, descending=True, dim=-1)
            cp = torch.softmax(sl, -1).cumsum(-1)
            rm = cp - torch.softmax(sl, -1) > c.top_p
            sl = sl.masked_fill(rm, float("-inf"))
            logits = torch.full_like(logits, float("-inf")).scatter(-1, si, sl)
        if s == "min_p" or c.min_p > 0:
            p = torch.softmax(logits, -1)
            logits = logits.masked_fill(p < c.min_p * p.max(-1, keepdim=True).values, float("-inf"))
        if s == "typical":
            lp = torch.log_softmax(logits, -1)
            p = lp.exp()
            ent = -(p * lp).nansum(-1, keepdim=True)
            dev = (ent + lp).abs()
            sd, si = torch.sort(dev, dim=-1)
            cp = p.gather(-1, si).cumsum(-1)
            rm = cp - p.gather(-1, si) > c.typical_p
            keep = torch.zeros_like(rm).scatter(-1, si, ~rm)
            logits = logits.masked_fill(~keep, float("-inf"))
        if s == "eta":
            p = torch.softmax(logits, -1)
            ent = -(p * torch.log(p.clamp_min(1e-20))).sum(-1, keepdim=True)
            eta = torch.minimum(torch.full_like(ent, c.eta_cutoff), math.sqrt(c.eta_cutoff) * torch.exp(-ent))
            top = p.max(-1, keepdim=True).values
            logits = logits.masked_fill((p < eta) & (p < top), float("-inf"))
        return logits

    def sample(self, logits: torch.Tensor, prev_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits [B, V] (fp32) -> next token ids [B]."""
        c = self.cfg
        logits = logits.float()
        if prev_tokens is not None:
            logits = self.apply_repetition_penalty(logits, prev_tokens, c.repetition_penalty)
            logits = self.block_repeated_ngrams(logits, prev_tokens, c.no_repeat_ngram_size)
        if c.strategy == "greedy" or c.temperature <= 0:
            return logits.argmax(-1)
        logits = self.filter(logits / max(c.temperature, 1e-5))
        probs = torch.softmax(logits, -1)
        return torch.multinomial(probs, 1, generator=self._generator(logits.device)).squeeze(-1)


class YvSamplerFactory:
    @staticmethod
    def create(strategy: str = "greedy", **kw: Any) -> YvSampler:
        return YvSampler(YvSamplingConfig(strategy=strategy, **kw))


# --------------------------------------------------------------------------------------------------
# cached generation
# --------------------------------------------------------------------------------------------------
def _tp_size(model) -> int:
    par = getattr(model, "parallel", None)
    return par.tp_size if par is not None else 1


def _prefill(model, ids: torch.Tensor, cache: YvPagedKVCache, seq_ids: List[int]) -> torch.Tensor:
    """Run the prompt(s) [B, S] through the model, filling the cache; returns last-token logits [B, V].

    Under tensor parallelism the token rows are sharded over the ranks between the layers (sequence parallel), so the
    row count must divide by the group size: the prompts are padded at the END with tokens that are not cached
    (slot -1); causal attention keeps them out of every real token's context."""
    B, S = ids.shape
    trunk = model.model
    pad = (-S) % _tp_size(model)
    if pad:
        ids = torch.cat([ids, ids.new_zeros(B, pad)], dim=1)
    ctx = trunk.build_context(B, S + pad, ids.device)
    slots: List[int] = []
    for s in seq_ids:
        slots += cache.append_slots(s, S) + [-1] * pad
    ctx.cache = cache
    ctx.slot_map = torch.tensor(slots, dtype=torch.int32).to(ids.device)
    out = model(input_ids=ids, ctx=ctx, return_logits=False, return_hidden=True)
    return model.logits(out["hidden_states"][:, S - 1, :])


def _decode_step(model, tokens: torch.Tensor, cache: YvPagedKVCache, seq_ids: List[int]) -> torch.Tensor:
    """One token per sequence: tokens [B] -> logits [B, V].  Under tensor parallelism the batch is padded to a
    multiple of the group size with rows that read one (arbitrary) cached token and store nothing."""
    trunk = model.model
    dev = tokens.device
    slots = [cache.append_slots(s, 1)[0] for s in seq_ids]
    lens = cache.seq_lens_tensor(seq_ids)
    B = tokens.shape[0]
    pad = (-B) % _tp_size(model)
    table = cache.block_table_tensor(seq_ids)
    if pad:
        tokens = torch.cat([tokens, tokens.new_zeros(pad)])
        slots = slots + [-1] * pad
        lens = torch.cat([lens, lens.new_ones(pad)])
        table = torch.cat([table, table.new_zeros(pad, table.shape[1])], dim=0)
    Bp = B + pad
    pos = (lens - 1).int()
    cos = sin = None
    if trunk.rotary is not None:
        cos, sin = trunk.rotary.tables(max(cache.lengths[s] for s in seq_ids), dev)
    ctx = AttnContext(positions=pos, cu_seqlens=torch.arange(Bp + 1, dtype=torch.int32, device=dev), max_len=1,
                      cos=cos, sin=sin, causal=True, cache=cache,
                      slot_map=torch.tensor(slots, dtype=torch.int32).to(dev),
                      block_table=table, seq_lens=lens, decode=True)
    out = model(input_ids=tokens.view(Bp, 1), ctx=ctx, return_logits=False, return_hidden=True)
    return model.logits(out["hidden_states"][:B, -1, :])


@torch.no_grad()
def generate(model, input_ids: torch.Tensor, max_new_tokens: int = 32, sampler: Optional[YvSampler] = None,
             eos_token_id: Optional[int] = None, cache: Optional[YvPagedKVCache] = None,
             temperature: Optional[float] = None, top_k: Optional[int] = None, top_p: Optional[float] = None,
             use_speculative: bool = False, on_token: Optional[Callable[[torch.Tensor], None]] = None,
             **_: Any) -> Tuple[torch.Tensor, Dict[str, Any]]:
    """Returns ``(ids [B, S + new], stats)`` like the reference's ``model.generate`` (model.py:1667-1787)."""
    was_training = model.training
    model.eval()
    cfg = model.cfg
    B, S = input_ids.shape
    dev = input_ids.device
    if sampler is None:
        if temperature is not None and temperature > 0 and (top_k or top_p):
            sampler = YvSampler(YvSamplingConfig(strategy="top_k_top_p", temperature=temperature,
                                                 top_k=top_k or 0, top_p=top_p or 1.0))
        else:
            sampler = YvSampler()
    own_cache = cache is None
    if own_cache:
        bs = cfg.kv_cache_block_size
        blocks = B * ((S + max_new_tokens + bs - 1) // bs + 1)
        pdtype = next(model.parameters()).dtype
        cache = cache_for_model(cfg, dev, blocks, dtype=pdtype,
                                tp_size=model.parallel.tp_size if model.parallel is not None else 1)
    seq_ids = list(range(10_000_000, 10_000_000 + B))
    for s in seq_ids:
        cache.add_sequence(s)
    eos = cfg.eos_token_id if eos_token_id is None else eos_token_id
    logits = _prefill(model, input_ids, cache, seq_ids)
    out = input_ids
    done = torch.zeros(B, dtype=torch.bool, device=dev)
    steps = 0
    for _step in range(max_new_tokens):
        nxt = sampler.sample(logits, out)
        nxt = torch.where(done, torch.full_like(nxt, cfg.pad_token_id), nxt)
        out = torch.cat([out, nxt.view(B, 1)], 1)
        steps += 1
        if on_token is not None:
            on_token(nxt)
        if eos is not None and eos >= 0:
            done = done | (nxt == eos)
            if bool(done.all()):
                break
        if _step + 1 < max_new_tokens:
            logits = _decode_step(model, nxt, cache, seq_ids)
    for s in seq_ids:
        cache.free_sequence(s)
    model.train(was_training)
    return out, {"generated_tokens": steps, "prompt_tokens": S, "speculative": False}
