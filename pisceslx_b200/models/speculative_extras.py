"""Further speculative-decoding parts (reference model/generation/speculative.py:128-2050): verification strategy and
result types, a small causal draft model, the neural n-gram (DSpark) head with its decoder, and a Medusa decoder.

Where this departs from the reference, and why:
* ``YvDraftModel``: the reference stacks ``nn.TransformerEncoderLayer`` with neither a causal mask nor positions
  (speculative.py:330-377), so every position sees the future and the order of tokens is invisible - as a next-token
  model it cannot be trained to agree with a causal target.  Here it is a causal pre-norm transformer with learned
  positions and a key / value cache, so that drafting n tokens costs n single-token steps, not n re-encodings.
* DSpark candidates: the reference draws its ``dspark_parallel_candidates`` drafts one after another in a Python loop,
  reads a log-probability back per step, keeps the draft the HEAD likes best and only then asks the target
  (speculative.py:1762-1815).  Here all candidates are rows of one batch (one head call per draft position for all of
  them) and ALL of them are verified in one target forward; the candidate the TARGET accepts longest wins.  The target's
  pass is the expensive part and it is paid once either way; using its verdict on every candidate raises the accepted
  length at no extra launch.
* Medusa: the reference checks the token of head i against the target's distribution for the NEXT position only
  (speculative.py:1560-1575), whatever i is.  Here head i's token is checked against the target's distribution at the
  position it was predicted for, by appending the candidates and reading one forward - which is also the forward that
  yields the next round's hidden state, so a round is exactly one target call."""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .speculative import YvMedusaHead, YvSpeculativeConfig


class YvVerificationStrategy(str, Enum):
    STANDARD = "standard"          # one draft, sequential accept / reject with early stop
    PARALLEL = "parallel"          # one or several drafts judged in one target forward
    SEQUENTIAL = "sequential"      # token by token, a target forward each (the conservative fallback)
    MEDUSA = "medusa"              # candidates from heads on the target's own hidden state
    EAGLE = "eagle"                # feature-level drafting (drafts from the hidden state through a draft model)


@dataclass
class YvVerificationResult:
    accepted_ids: torch.Tensor
    num_accepted: int
    new_past_key_values: Optional[Any] = None
    rejection_position: int = -1
    next_token: Optional[torch.Tensor] = None
    candidate: int = 0


def _logits_and_hidden(model: Any, ids: torch.Tensor, want_hidden: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    try:
        out = model(input_ids=ids, return_logits=True, return_hidden=want_hidden) if want_hidden else model(input_ids=ids)
    except TypeError:
        out = model(ids)
    if isinstance(out, torch.Tensor):
        return out, None
    if isinstance(out, dict):
        return out["logits"], out.get("hidden_states")
    return out.logits, getattr(out, "hidden_states", None)


@torch.no_grad()
def verify_candidates(model: Any, input_ids: torch.Tensor, drafts: torch.Tensor, threshold: float = 0.0) -> YvVerificationResult:
    """input_ids [1, S], drafts [C, n]: one target forward over C rows; the candidate with the longest accepted prefix wins
    (greedy agreement when ``threshold`` is 0, else target probability of the drafted token at least ``threshold``)."""
    C, n = drafts.shape
    cand = torch.cat([input_ids.expand(C, -1), drafts], 1)
    logits = _logits_and_hidden(model, cand)[0][:, -(n + 1):].float()
    if threshold > 0:
        ok = torch.softmax(logits[:, :n], -1).gather(2, drafts.unsqueeze(-1)).squeeze(-1) >= threshold
    else:
        ok = logits[:, :n].argmax(-1) == drafts
    accepted = ok.long().cumprod(1).sum(1)                                             # [C]
    c = accepted.argmax()
    k = int(accepted[c])                                                               # the round's one read
    nxt = logits[c, k].argmax().view(1, 1)
    return YvVerificationResult(drafts[c:c + 1, :k], k, None, k if k < n else -1, nxt, int(c))


# ---- draft model -----------------------------------------------------------------------------------------------------------
class _DraftBlock(nn.Module):
    def __init__(self, hidden: int, heads: int, dropout: float):
        super().__init__()
        self.n1, self.n2 = nn.LayerNorm(hidden), nn.LayerNorm(hidden)
        self.qkv, self.o = nn.Linear(hidden, 3 * hidden, bias=False), nn.Linear(hidden, hidden, bias=False)
        self.up, self.down = nn.Linear(hidden, 4 * hidden), nn.Linear(4 * hidden, hidden)
        self.heads, self.drop = heads, nn.Dropout(dropout)

    def forward(self, x: torch.Tensor, cache: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        B, T, H = x.shape
        q, k, v = self.qkv(self.n1(x)).view(B, T, 3, self.heads, H // self.heads).permute(2, 0, 3, 1, 4)
        if cache is not None:
            k, v = torch.cat([cache[0], k], 2), torch.cat([cache[1], v], 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=cache is None and T > 1) if (cache is None or T == 1) else \
            F.scaled_dot_product_attention(q, k, v, attn_mask=torch.ones(T, k.shape[2], dtype=torch.bool, device=x.device).tril(k.shape[2] - T))
        x = x + self.drop(self.o(a.transpose(1, 2).reshape(B, T, H)))
        return x + self.drop(self.down(F.gelu(self.up(self.n2(x))))), (k, v)


class YvDraftModel(nn.Module):
    """``forward(input_ids) -> logits [B, T, V]``; ``draft(input_ids, n)`` continues greedily (or by sampling) for n tokens
    using the cache and returns (tokens [B, n], their probabilities [B, n])."""

    def __init__(self, vocab_size: int, hidden_size: int, num_layers: int, num_heads: int, max_position_embeddings: int = 2048,
                 dropout: float = 0.0, device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None):
        super().__init__()
        if hidden_size % num_heads:
            raise ValueError("hidden_size must be a multiple of num_heads")
        self.vocab_size, self.hidden_size, self.num_layers, self.num_heads = vocab_size, hidden_size, num_layers, num_heads
        self.max_position_embeddings = max_position_embeddings
        self.embed = nn.Embedding(vocab_size, hidden_size)
        self.pos = nn.Embedding(max_position_embeddings, hidden_size)
        self.blocks = nn.ModuleList([_DraftBlock(hidden_size, num_heads, dropout) for _ in range(num_layers)])
        self.norm = nn.LayerNorm(hidden_size)
        self.lm_head = nn.Linear(hidden_size, vocab_size, bias=False)
        self._init_weights()
        if device is not None or dtype is not None:
            self.to(device=device, dtype=dtype)

    def _init_weights(self) -> None:
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
                if getattr(m, "bias", None) is not None:
                    nn.init.zeros_(m.bias)

    def _run(self, input_ids: torch.Tensor, caches: Optional[List[Tuple[torch.Tensor, torch.Tensor]]] = None, offset: int = 0):
        T = input_ids.shape[1]
        pos = (torch.arange(T, device=input_ids.device) + offset).clamp_max(self.max_position_embeddings - 1)
        x = self.embed(input_ids) + self.pos(pos)
        new = []
        for i, b in enumerate(self.blocks):
            x, c = b(x, caches[i] if caches is not None else None)
            new.append(c)
        return self.lm_head(self.norm(x)), new

    def forward(self, input_ids: torch.Tensor = None, **kw: Any) -> torch.Tensor:
        return self._run(input_ids if input_ids is not None else kw["input_ids"])[0]

    @torch.no_grad()
    def draft(self, input_ids: torch.Tensor, n: int, temperature: float = 0.0, generator: Optional[torch.Generator] = None):
        logits, caches = self._run(input_ids)
        toks, probs, last, off = [], [], logits[:, -1].float(), input_ids.shape[1]
        for _ in range(n):
            p = torch.softmax(last / temperature, -1) if temperature > 0 else torch.softmax(last, -1)
            t = torch.multinomial(p, 1, generator=generator) if temperature > 0 else p.argmax(-1, keepdim=True)
            toks.append(t)
            probs.append(p.gather(1, t))
            lg, caches = self._run(t, caches, off)
            last, off = lg[:, -1].float(), off + 1
        return torch.cat(toks, 1), torch.cat(probs, 1)

    def distill_step(self, target_logits: torch.Tensor, input_ids: torch.Tensor, optimizer: torch.optim.Optimizer, temperature: float = 1.0) -> torch.Tensor:
        """One step of matching the target's next-token distributions on ``input_ids`` (KL from the target)."""
        lg = self(input_ids).float() / temperature
        tgt = torch.softmax(target_logits.detach().float() / temperature, -1)
        loss = F.kl_div(torch.log_softmax(lg, -1), tgt, reduction="batchmean") / input_ids.shape[1]
        optimizer.zero_grad(set_to_none=True)
        loss.backward()
        optimizer.step()
        return loss.detach()


# ---- DSpark ----------------------------------------------------------------------------------------------------------------
class YvNeuralDSparkHead(nn.Module):
    """Next-token logits from the last ``markov_order`` tokens: embedding -> concatenation -> MLP (the reference's
    ``YvDSparkHead`` module, speculative.py:1633-1690; ``models.speculative.YvDSparkHead`` is the parameter-free count
    table used when no trained head exists)."""

    def __init__(self, vocab_size: int, markov_order: int = 3, embed_dim: int = 256, hidden: int = 512,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.markov_order, self.vocab_size = markov_order, vocab_size
        self.embedding = nn.Embedding(vocab_size, embed_dim, device=device, dtype=dtype)
        self.predictor = nn.Sequential(nn.Linear(embed_dim * markov_order, hidden, device=device, dtype=dtype), nn.SiLU(),
                                       nn.Linear(hidden, vocab_size, bias=False, device=device, dtype=dtype))
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
                if getattr(m, "bias", None) is not None:
                    nn.init.zeros_(m.bias)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, markov_order] -> logits [B, V]."""
        return torch.nan_to_num(self.predictor(self.embedding(tokens).flatten(1)))

    def fit_step(self, sequence: torch.Tensor, optimizer: torch.optim.Optimizer) -> torch.Tensor:
        """Cross-entropy on every (order-gram -> next token) window of ``sequence`` [B, T] (e.g. text the target wrote)."""
        k = self.markov_order
        if sequence.shape[1] <= k:
            return torch.zeros((), device=sequence.device)
        ctx = sequence.unfold(1, k, 1)[:, :-1].reshape(-1, k)
        tgt = sequence[:, k:].reshape(-1)
        loss = F.cross_entropy(self(ctx).float(), tgt)
        optimizer.zero_grad(set_to_none=True)
        loss.backward()
        optimizer.step()
        return loss.detach()


class YvDSparkSpeculativeDecoder(nn.Module):
    """``speculative_generate(input_ids [1, S], max_new_tokens)``.  Config attributes read (all optional):
    ``dspark_draft_len`` 5, ``dspark_markov_order`` 3, ``dspark_confidence_threshold`` 0.7 (0 = greedy agreement),
    ``dspark_parallel_candidates`` 8, ``dspark_ngram_embed_dim`` 256, ``speculative_temperature`` / ``_top_k``."""

    def __init__(self, config: Any, model: nn.Module, tokenizer: Any = None, on_stats: Optional[Callable[[Dict[str, Any]], None]] = None,
                 markov_head: Optional[YvNeuralDSparkHead] = None):
        super().__init__()
        g = lambda k, d: (config.get(k, d) if isinstance(config, dict) else getattr(config, k, d))
        self.config, self.model, self.tokenizer, self.on_stats = config, model, tokenizer, on_stats
        self.dspark_draft_len, self.dspark_markov_order = int(g("dspark_draft_len", 5)), int(g("dspark_markov_order", 3))
        self.dspark_confidence_threshold = float(g("dspark_confidence_threshold", 0.7))
        self.dspark_parallel_candidates = int(g("dspark_parallel_candidates", 8))
        self.temperature = max(0.1, min(2.0, float(g("speculative_temperature", 0.7))))
        self.top_k = max(1, min(1000, int(g("speculative_top_k", 50))))
        mc = getattr(model, "cfg", getattr(model, "config", None))
        vocab = int(g("vocab_size", getattr(mc, "vocab_size", 65536)))
        p = next(model.parameters())
        self.markov_head = markov_head or YvNeuralDSparkHead(vocab, self.dspark_markov_order, int(g("dspark_ngram_embed_dim", 256)), device=p.device)
        self.current_draft_len = self.dspark_draft_len
        self.min_draft_len, self.max_draft_len = 1, max(int(g("dspark_max_draft_len", 12)), self.dspark_draft_len)
        self.performance_history: List[Dict[str, float]] = []
        self._ema = None

    def _apply_sampling(self, logits: torch.Tensor) -> torch.Tensor:
        logits = torch.nan_to_num(logits.float()) / self.temperature
        k = min(self.top_k, logits.shape[-1])
        kth = logits.topk(k, -1).values[..., -1:]
        return logits.masked_fill(logits < kth, float("-inf"))

    @torch.no_grad()
    def _generate_parallel_drafts(self, input_ids: torch.Tensor, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """[C, n]: C candidate continuations drawn as one batch; row 0 is the head's greedy continuation."""
        C, n, k = self.dspark_parallel_candidates, max(1, self.current_draft_len), self.dspark_markov_order
        ctx = input_ids[:, -k:]
        if ctx.shape[1] < k:
            ctx = F.pad(ctx, (k - ctx.shape[1], 0))
        ctx = ctx.expand(C, -1).clone()
        out = []
        for _ in range(n):
            lg = self._apply_sampling(self.markov_head(ctx))
            tok = torch.multinomial(torch.softmax(lg, -1), 1, generator=generator)
            tok[0] = lg[0].argmax()
            out.append(tok)
            ctx = torch.cat([ctx[:, 1:], tok], 1)
        return torch.cat(out, 1)

    def _confidence_schedule(self, num_accepted: int, draft_len: int) -> int:
        """Longer drafts while most of a draft is accepted, shorter ones when little is (a running share)."""
        share = num_accepted / max(draft_len, 1)
        self._ema = share if self._ema is None else 0.7 * self._ema + 0.3 * share
        if self._ema > 0.8:
            self.current_draft_len = min(self.current_draft_len + 1, self.max_draft_len)
        elif self._ema < 0.3:
            self.current_draft_len = max(self.current_draft_len - 1, self.min_draft_len)
        return self.current_draft_len

    @torch.no_grad()
    def _standard_generate(self, input_ids: torch.Tensor, max_new_tokens: int, eos: Optional[int]) -> torch.Tensor:
        ids = input_ids
        for _ in range(max_new_tokens):
            t = _logits_and_hidden(self.model, ids)[0][:, -1].argmax(-1, keepdim=True)
            ids = torch.cat([ids, t], 1)
            if eos is not None and eos >= 0 and int(t) == eos:
                break
        return ids

    @torch.no_grad()
    def speculative_generate(self, input_ids: torch.Tensor, max_new_tokens: int = 32, eos_token_id: Optional[int] = None,
                             generator: Optional[torch.Generator] = None) -> Tuple[torch.Tensor, Dict[str, Any]]:
        if input_ids.shape[0] != 1:
            raise ValueError("one sequence at a time (the candidates take the batch dimension)")
        was = self.model.training
        self.model.eval()
        t0 = time.perf_counter()
        ids, produced, rounds, drafted, accepted = input_ids, 0, 0, 0, 0
        while produced < max_new_tokens:
            rounds += 1
            room = max_new_tokens - produced
            if room == 1:
                ids = self._standard_generate(ids, 1, eos_token_id)
                produced += 1
                break
            drafts = self._generate_parallel_drafts(ids, generator)[:, :room - 1]
            r = verify_candidates(self.model, ids, drafts, self.dspark_confidence_threshold)
            new = torch.cat([r.accepted_ids, r.next_token], 1)
            ids = torch.cat([ids, new], 1)
            produced += new.shape[1]
            drafted += drafts.shape[1]
            accepted += r.num_accepted
            self.performance_history.append({"draft_len": drafts.shape[1], "accepted": r.num_accepted, "candidate": r.candidate})
            self._confidence_schedule(r.num_accepted, drafts.shape[1])
            if eos_token_id is not None and eos_token_id >= 0 and bool((new == eos_token_id).any()):
                cut = int((new[0] == eos_token_id).nonzero()[0]) + 1
                ids = ids[:, : ids.shape[1] - new.shape[1] + cut]
                break
        self.model.train(was)
        stats = {"generated_tokens": ids.shape[1] - input_ids.shape[1], "rounds": rounds, "drafted": drafted, "accepted": accepted,
                 "acceptance_rate": accepted / max(drafted, 1), "tokens_per_target_forward": (ids.shape[1] - input_ids.shape[1]) / max(rounds, 1),
                 "final_draft_len": self.current_draft_len, "total_time_ms": (time.perf_counter() - t0) * 1e3}
        if self.on_stats is not None:
            try:
                self.on_stats(stats)
            except Exception:
                pass
        return ids, stats


# ---- Medusa ----------------------------------------------------------------------------------------------------------------
class YvMedusaDecoder(nn.Module):
    """Heads on the target's last hidden state propose the tokens after the next one; each round is ONE target forward
    over ``[sequence, next token, proposals]`` that (a) says how many proposals the target agrees with and (b) yields
    the hidden state the next proposals come from."""

    def __init__(self, model: nn.Module, config: Optional[YvSpeculativeConfig] = None, num_heads: int = 4, medusa: Optional[YvMedusaHead] = None,
                 on_stats: Optional[Callable[[Dict[str, Any]], None]] = None):
        super().__init__()
        self.model, self.config, self.on_stats = model, config or YvSpeculativeConfig(), on_stats
        mc = getattr(model, "cfg", getattr(model, "config", None))
        self.medusa = medusa or YvMedusaHead(int(mc.hidden_size), int(mc.vocab_size), num_heads)
        self.medusa.to(next(model.parameters()).device)
        self.num_heads = len(self.medusa.heads)

    def forward(self, hidden_states: torch.Tensor) -> List[torch.Tensor]:
        return self.medusa(hidden_states)

    def train_step(self, input_ids: torch.Tensor, optimizer: torch.optim.Optimizer) -> torch.Tensor:
        """Heads only (the target is frozen): head i at position t learns token t + i + 2."""
        with torch.no_grad():
            _, h = _logits_and_hidden(self.model, input_ids, True)
        loss, n = 0.0, 0
        for i, lg in enumerate(self.medusa(h.detach().float())):
            s = i + 2
            if input_ids.shape[1] > s:
                loss = loss + F.cross_entropy(lg[:, :-s].reshape(-1, lg.shape[-1]).float(), input_ids[:, s:].reshape(-1))
                n += 1
        loss = loss / max(n, 1)
        optimizer.zero_grad(set_to_none=True)
        loss.backward()
        optimizer.step()
        return loss.detach()

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_length: Optional[int] = None, max_new_tokens: int = 32,
                 eos_token_id: Optional[int] = None) -> Tuple[torch.Tensor, Dict[str, Any]]:
        if input_ids.shape[0] != 1:
            raise ValueError("one sequence at a time")
        limit = max_length if max_length is not None else input_ids.shape[1] + max_new_tokens
        was = self.model.training
        self.model.eval()
        t0 = time.perf_counter()
        logits, hidden = _logits_and_hidden(self.model, input_ids, True)
        ids, forwards, predicted, accepted_total = input_ids, 1, 0, 0
        while ids.shape[1] < limit:
            nxt = logits[:, -1].float().argmax(-1, keepdim=True)                        # the target's own next token
            if hidden is None:
                ids = torch.cat([ids, nxt], 1)
                logits, hidden = _logits_and_hidden(self.model, ids, True)
                forwards += 1
                continue
            room = limit - ids.shape[1] - 1
            props = [lg[:, -1].float().argmax(-1, keepdim=True) for lg in self.medusa(hidden[:, -1:].float())][:max(room, 0)]
            cand = torch.cat([ids, nxt] + props, 1)
            logits_c, hidden_c = _logits_and_hidden(self.model, cand, True)
            forwards += 1
            n = len(props)
            k = 0
            if n:
                agree = logits_c[:, -(n + 1):-1].float().argmax(-1) == torch.cat(props, 1)     # position of prop i is judged by the row before it
                k = int(agree.long().cumprod(1).sum())
            predicted += n
            accepted_total += k
            keep = ids.shape[1] + 1 + k
            ids, logits, hidden = cand[:, :keep], logits_c[:, :keep], (hidden_c[:, :keep] if hidden_c is not None else None)
            if eos_token_id is not None and eos_token_id >= 0:
                new = ids[0, -(k + 1):]
                hit = (new == eos_token_id).nonzero()
                if hit.numel():
                    ids = ids[:, : ids.shape[1] - (k + 1) + int(hit[0]) + 1]
                    break
        self.model.train(was)
        gen = ids.shape[1] - input_ids.shape[1]
        stats = {"total_predicted": predicted, "accepted_tokens": accepted_total, "acceptance_rate": accepted_total / max(predicted, 1),
                 "target_forwards": forwards, "generated_tokens": gen, "speedup": gen / max(forwards - 1, 1), "total_time_ms": (time.perf_counter() - t0) * 1e3}
        if self.on_stats is not None:
            try:
                self.on_stats(stats)
            except Exception:
                pass
        return ids, stats
