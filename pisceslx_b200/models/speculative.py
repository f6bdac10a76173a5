"""Speculative decoding, beam search and contrastive search.

``YvSpeculativeDecoder`` drafts ``draft_length`` tokens and verifies them with one forward of the target model.  Two
acceptance rules: ``"threshold"`` is the reference's (model/generation/speculative.py:550-568:
``p_accept = min(1, p_target / p_draft)`` compared with ``acceptance_threshold``, greedy correction on rejection) and
``"exact"`` is the standard accept / resample rule that preserves the target distribution.  After three rounds with
no accepted token it falls back to plain decoding (reference :855-866).  Drafts come from a ``YvDSparkHead`` (an
order-k Markov table over recent tokens, reference ``YvDSparkHead``), from ``YvMedusaHead`` heads on the last hidden
state, or from the target model itself at lower depth (self-draft).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from .generation import YvSampler


@dataclass
class YvSpeculativeConfig:
    draft_length: int = 5
    acceptance_threshold: float = 0.8
    rule: str = "threshold"            # "threshold" (reference) | "exact"
    temperature: float = 0.0
    max_zero_rounds: int = 3


class YvDSparkHead:
    """Order-k Markov draft model learned online from the tokens seen so far (no parameters)."""

    def __init__(self, order: int = 3):
        self.order = order
        self.table: Dict[Tuple[int, ...], Dict[int, int]] = {}

    def observe(self, tokens: List[int]) -> None:
        for k in range(1, self.order + 1):
            for i in range(len(tokens) - k):
                ctx = tuple(tokens[i:i + k])
                nxt = tokens[i + k]
                self.table.setdefault(ctx, {})[nxt] = self.table.setdefault(ctx, {}).get(nxt, 0) + 1

    def draft(self, tokens: List[int], n: int) -> List[int]:
        out: List[int] = []
        cur = list(tokens)
        for _ in range(n):
            nxt = None
            for k in range(self.order, 0, -1):
                d = self.table.get(tuple(cur[-k:]))
                if d:
                    nxt = max(d.items(), key=lambda kv: kv[1])[0]
                    break
            if nxt is None:
                break
            out.append(nxt)
            cur.append(nxt)
        return out


class YvMedusaHead(nn.Module):
    """``n_heads`` residual MLP heads; head i predicts the token i+2 positions ahead from the last hidden state."""

    def __init__(self, hidden: int, vocab: int, n_heads: int = 4):
        super().__init__()
        self.blocks = nn.ModuleList([nn.Sequential(nn.Linear(hidden, hidden), nn.SiLU()) for _ in range(n_heads)])
        self.heads = nn.ModuleList([nn.Linear(hidden, vocab, bias=False) for _ in range(n_heads)])

    def forward(self, h: torch.Tensor) -> List[torch.Tensor]:
        return [head(h + blk(h)) for blk, head in zip(self.blocks, self.heads)]


class YvSpeculativeDecoder:
    def __init__(self, model: Any, cfg: Optional[YvSpeculativeConfig] = None, draft_model: Any = None,
                 medusa: Optional[YvMedusaHead] = None):
        self.model, self.cfg = model, cfg or YvSpeculativeConfig()
        self.draft_model, self.medusa = draft_model, medusa
        self.dspark = YvDSparkHead(getattr(model.cfg, "dspark_markov_order", 3))

    @torch.no_grad()
    def _target_probs(self, ids: torch.Tensor, n_last: int) -> torch.Tensor:
        """Probabilities of the target model for the last ``n_last`` positions (+ the next one)."""
        logits = self.model(input_ids=ids).logits[:, -n_last:, :].float()
        t = self.cfg.temperature
        return torch.softmax(logits / t, -1) if t > 0 else torch.nn.functional.one_hot(
            logits.argmax(-1), logits.shape[-1]).float()

    def _draft(self, ids: torch.Tensor) -> Tuple[List[int], Optional[torch.Tensor]]:
        n = self.cfg.draft_length
        if self.draft_model is not None:
            cur, toks, probs = ids, [], []
            for _ in range(n):
                p = torch.softmax(self.draft_model(input_ids=cur).logits[:, -1].float(), -1)
                t = int(p.argmax(-1))
                toks.append(t)
                probs.append(float(p[0, t]))
                cur = torch.cat([cur, torch.tensor([[t]], device=ids.device)], 1)
            return toks, torch.tensor(probs)
        return self.dspark.draft(ids[0].tolist(), n), None

    @torch.no_grad()
    def speculative_generate(self, input_ids: torch.Tensor, max_new_tokens: int = 32,
                             eos_token_id: Optional[int] = None) -> Tuple[torch.Tensor, Dict[str, Any]]:
        assert input_ids.shape[0] == 1, "speculative decoding runs one sequence at a time"
        self.model.eval()
        ids = input_ids
        self.dspark.observe(ids[0].tolist())
        eos = self.model.cfg.eos_token_id if eos_token_id is None else eos_token_id
        produced = accepted_total = drafted_total = rounds = zero_rounds = 0
        fallback = False
        while produced < max_new_tokens:
            rounds += 1
            draft, q = ([], None) if fallback else self._draft(ids)
            draft = draft[: max_new_tokens - produced - 1] if draft else []
            if not draft:
                p = self._target_probs(ids, 1)[0, -1]
                new = [int(p.argmax()) if self.cfg.temperature <= 0 else int(torch.multinomial(p, 1))]
            else:
                cand = torch.cat([ids, torch.tensor([draft], device=ids.device)], 1)
                P = self._target_probs(cand, len(draft) + 1)[0]           # row i judges draft[i]; last row = bonus token
                new = []
                for i, tok in enumerate(draft):
                    pt = float(P[i, tok])
                    qd = float(q[i]) if q is not None else 1.0
                    ratio = min(1.0, pt / max(qd, 1e-9))
                    if self.cfg.rule == "exact":
                        ok = bool(torch.rand(()) < ratio)
                    else:
                        ok = ratio >= self.cfg.acceptance_threshold
                    if not ok:
                        break
                    new.append(tok)
                drafted_total += len(draft)
                accepted_total += len(new)
                row = P[len(new)]
                if self.cfg.rule == "exact" and len(new) < len(draft) and q is not None and self.cfg.temperature > 0:
                    resid = row.clone()
                    resid[draft[len(new)]] = max(0.0, float(resid[draft[len(new)]]) - float(q[len(new)]))
                    row = resid / resid.sum().clamp_min(1e-9)
                    new.append(int(torch.multinomial(row, 1)))
                else:
                    new.append(int(row.argmax()))
                zero_rounds = zero_rounds + 1 if len(new) == 1 else 0
                if zero_rounds >= self.cfg.max_zero_rounds:
                    fallback = True
            ids = torch.cat([ids, torch.tensor([new], device=ids.device)], 1)
            self.dspark.observe(ids[0, -(len(new) + self.dspark.order):].tolist())
            produced += len(new)
            if eos is not None and eos >= 0 and eos in new:
                break
        stats = {"generated_tokens": produced, "rounds": rounds, "drafted": drafted_total, "accepted": accepted_total,
                 "acceptance_rate": accepted_total / max(drafted_total, 1), "fell_back": fallback, "speculative": True}
        return ids[:, : input_ids.shape[1] + max_new_tokens], stats


class YvParallelVerifier:
    """Verifies a whole draft (or several candidate drafts of equal length) in one forward pass of the target model
    (reference model/generation/speculative.py:468).  Returns, per candidate, the number of leading draft tokens that
    the target model agrees with and the token it would emit after them."""

    def __init__(self, model: Any, threshold: float = 0.0):
        self.model, self.threshold = model, threshold

    @torch.no_grad()
    def verify(self, input_ids: torch.Tensor, drafts: torch.Tensor) -> Dict[str, torch.Tensor]:
        """input_ids [1, S]; drafts [C, n] -> accepted [C], next_token [C], probs [C, n]."""
        C, n = drafts.shape
        cand = torch.cat([input_ids.expand(C, -1), drafts], 1)
        logits = self.model(input_ids=cand).logits[:, -(n + 1):, :].float()
        probs = torch.softmax(logits, -1)
        p_draft = torch.gather(probs[:, :n], 2, drafts[..., None]).squeeze(-1)          # [C, n]
        if self.threshold > 0:
            ok = p_draft >= self.threshold
        else:
            ok = logits[:, :n].argmax(-1) == drafts
        accepted = ok.long().cumprod(1).sum(1)
        nxt = torch.gather(logits.argmax(-1), 1, accepted[:, None]).squeeze(1)
        return {"accepted": accepted, "next_token": nxt, "probs": p_draft}

    def best(self, input_ids: torch.Tensor, drafts: torch.Tensor) -> Tuple[List[int], int]:
        r = self.verify(input_ids, drafts)
        c = int(r["accepted"].argmax())
        k = int(r["accepted"][c])
        return drafts[c, :k].tolist() + [int(r["next_token"][c])], k


class YvAdaptiveSpeculativeDecoder(YvSpeculativeDecoder):
    """Adjusts the draft length between generation calls from the measured acceptance rate (reference :1335): a high
    rate means drafts are cheap wins, so they get longer; a low rate shortens them.  The expected tokens per target
    forward for acceptance rate a and length n is (1 - a^(n+1)) / (1 - a); the length that maximises it per unit cost
    ``1 + n * draft_cost`` is chosen."""

    def __init__(self, model: Any, cfg: Optional[YvSpeculativeConfig] = None, draft_cost: float = 0.05,
                 min_len: int = 1, max_len: int = 16, ema: float = 0.7, **kw: Any):
        super().__init__(model, cfg, **kw)
        self.draft_cost, self.min_len, self.max_len, self.ema = draft_cost, min_len, max_len, ema
        self.rate: Optional[float] = None
        self.history: List[Dict[str, float]] = []

    def best_length(self, a: float) -> int:
        a = min(max(a, 1e-3), 0.999)
        score = lambda n: (1 - a ** (n + 1)) / (1 - a) / (1 + n * self.draft_cost)
        return max(range(self.min_len, self.max_len + 1), key=score)

    def observe(self, acceptance_rate: float) -> int:
        self.rate = acceptance_rate if self.rate is None else self.ema * self.rate + (1 - self.ema) * acceptance_rate
        self.cfg.draft_length = self.best_length(self.rate)
        self.history.append({"rate": self.rate, "draft_length": self.cfg.draft_length})
        return self.cfg.draft_length

    def speculative_generate(self, input_ids: torch.Tensor, max_new_tokens: int = 32,
                             eos_token_id: Optional[int] = None) -> Tuple[torch.Tensor, Dict[str, Any]]:
        out, stats = super().speculative_generate(input_ids, max_new_tokens, eos_token_id)
        if stats["drafted"]:
            stats["next_draft_length"] = self.observe(stats["acceptance_rate"])
        return out, stats


@torch.no_grad()
def beam_search(model: Any, input_ids: torch.Tensor, num_beams: int = 4, max_new_tokens: int = 32,
                length_penalty: float = 1.0, eos_token_id: Optional[int] = None) -> torch.Tensor:
    """Returns the best sequence [1, S + n] (reference sampler's BEAM strategy)."""
    model.eval()
    eos = model.cfg.eos_token_id if eos_token_id is None else eos_token_id
    beams: List[Tuple[torch.Tensor, float, bool]] = [(input_ids, 0.0, False)]
    for _ in range(max_new_tokens):
        cand: List[Tuple[torch.Tensor, float, bool]] = []
        for seq, score, done in beams:
            if done:
                cand.append((seq, score, True))
                continue
            lp = torch.log_softmax(model(input_ids=seq).logits[:, -1].float(), -1)[0]
            top = torch.topk(lp, num_beams)
            for v, i in zip(top.values.tolist(), top.indices.tolist()):
                cand.append((torch.cat([seq, torch.tensor([[i]], device=seq.device)], 1), score + v, i == eos))
        cand.sort(key=lambda c: c[1] / (c[0].shape[1] ** length_penalty), reverse=True)
        beams = cand[:num_beams]
        if all(d for _, _, d in beams):
            break
    return beams[0][0]


@torch.no_grad()
def contrastive_search(model: Any, input_ids: torch.Tensor, top_k: int = 4, alpha: float = 0.6,
                       max_new_tokens: int = 32) -> torch.Tensor:
    """Pick, among the top-k tokens, the one maximising (1 - alpha) * p - alpha * max cosine similarity of its
    hidden state with the context's hidden states (reference sampler's CONTRASTIVE strategy)."""
    model.eval()
    ids = input_ids
    for _ in range(max_new_tokens):
        out = model(input_ids=ids, return_logits=True, return_hidden=True)
        p = torch.softmax(out.logits[:, -1].float(), -1)[0]
        ctx_h = torch.nn.functional.normalize(out.hidden_states[0].float(), dim=-1)
        top = torch.topk(p, top_k)
        best, best_score = None, -1e9
        for prob, tok in zip(top.values.tolist(), top.indices.tolist()):
            cand = torch.cat([ids, torch.tensor([[tok]], device=ids.device)], 1)
            h = model(input_ids=cand, return_logits=False, return_hidden=True).hidden_states[0, -1].float()
            sim = float((ctx_h @ torch.nn.functional.normalize(h, dim=-1)).max())
            score = (1 - alpha) * prob - alpha * sim
            if score > best_score:
                best, best_score = tok, score
        ids = torch.cat([ids, torch.tensor([[best]], device=ids.device)], 1)
    return ids
