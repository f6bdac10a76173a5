"""Task heads on the Yv trunk (reference model/core/model.py: ``YvModelForSequenceClassification``,
``YvModelForTokenClassification``, ``YvModelForQuestionAnswering`` after ``YvModelForCausalLM`` :2617-2722) and the
speculative-decoding heads (``YvMedusaHead`` / ``YvDSparkHead``, model/generation/speculative.py)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import YvConfig
from ..ops import functional as F_
from .model import YvModel


class _HeadBase(nn.Module):
    def __init__(self, cfg: YvConfig, parallel: Any = None):
        super().__init__()
        self.cfg = cfg
        self.model = YvModel(cfg, parallel)

    def hidden(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.model(input_ids=input_ids, attention_mask=attention_mask)["hidden_states"]


class YvModelForSequenceClassification(_HeadBase):
    """Pools the hidden state of each sequence's last non-padding token and classifies it."""

    def __init__(self, cfg: YvConfig, num_labels: int, parallel: Any = None):
        super().__init__(cfg, parallel)
        self.num_labels = num_labels
        self.score = nn.Parameter(torch.empty(num_labels, cfg.hidden_size).normal_(std=cfg.initializer_range))

    def forward(self, input_ids, attention_mask=None, labels=None) -> Dict[str, torch.Tensor]:
        h = self.hidden(input_ids, attention_mask)
        B, S, _ = h.shape
        last = (attention_mask.long().sum(1) - 1).clamp_min(0) if attention_mask is not None else \
            torch.full((B,), S - 1, device=h.device, dtype=torch.long)
        pooled = h[torch.arange(B, device=h.device), last]
        logits = F_.linear(pooled, self.score).float()
        out = {"logits": logits}
        if labels is not None:
            out["loss"] = F.mse_loss(logits.squeeze(-1), labels.float()) if self.num_labels == 1 else \
                F.cross_entropy(logits, labels)
        return out


class YvModelForTokenClassification(_HeadBase):
    def __init__(self, cfg: YvConfig, num_labels: int, parallel: Any = None):
        super().__init__(cfg, parallel)
        self.classifier = nn.Parameter(torch.empty(num_labels, cfg.hidden_size).normal_(std=cfg.initializer_range))

    def forward(self, input_ids, attention_mask=None, labels=None) -> Dict[str, torch.Tensor]:
        logits = F_.linear(self.hidden(input_ids, attention_mask), self.classifier).float()
        out = {"logits": logits}
        if labels is not None:
            out["loss"] = F.cross_entropy(logits.flatten(0, 1), labels.flatten(), ignore_index=-100)
        return out


class YvModelForQuestionAnswering(_HeadBase):
    def __init__(self, cfg: YvConfig, parallel: Any = None):
        super().__init__(cfg, parallel)
        self.qa = nn.Parameter(torch.empty(2, cfg.hidden_size).normal_(std=cfg.initializer_range))

    def forward(self, input_ids, attention_mask=None, start_positions=None, end_positions=None):
        logits = F_.linear(self.hidden(input_ids, attention_mask), self.qa).float()
        start, end = logits[..., 0], logits[..., 1]
        out = {"start_logits": start, "end_logits": end}
        if start_positions is not None and end_positions is not None:
            out["loss"] = 0.5 * (F.cross_entropy(start, start_positions) + F.cross_entropy(end, end_positions))
        return out


class YvMedusaHead(nn.Module):
    """``n_heads`` residual MLP heads; head i predicts the token i + 2 positions ahead from the last hidden state."""

    def __init__(self, hidden: int, vocab: int, n_heads: int = 4, lm_head: Optional[torch.Tensor] = None):
        super().__init__()
        self.blocks = nn.ParameterList([nn.Parameter(torch.zeros(hidden, hidden)) for _ in range(n_heads)])
        self.lm_head = lm_head if lm_head is not None else nn.Parameter(torch.empty(vocab, hidden).normal_(std=0.02))

    def forward(self, h: torch.Tensor) -> List[torch.Tensor]:
        return [F_.linear(h + F.silu(F_.linear(h, w)), self.lm_head).float() for w in self.blocks]

    @torch.no_grad()
    def propose(self, h_last: torch.Tensor) -> torch.Tensor:
        """Greedy draft tokens [B, n_heads] from the last position's hidden state [B, H]."""
        return torch.stack([l.argmax(-1) for l in self.forward(h_last)], 1)


class YvDSparkHead(nn.Module):
    """Markov draft head: next-token logits from the embedding of the previous token and the last hidden state
    (one small GEMM per drafted token instead of a model step)."""

    def __init__(self, hidden: int, vocab: int, rank: int = 256):
        super().__init__()
        self.mix_h = nn.Parameter(torch.empty(rank, hidden).normal_(std=0.02))
        self.mix_e = nn.Parameter(torch.empty(rank, hidden).normal_(std=0.02))
        self.out = nn.Parameter(torch.empty(vocab, rank).normal_(std=0.02))

    def forward(self, h: torch.Tensor, prev_emb: torch.Tensor) -> torch.Tensor:
        return F_.linear(F.silu(F_.linear(h, self.mix_h) + F_.linear(prev_emb, self.mix_e)), self.out).float()

    @torch.no_grad()
    def draft(self, h_last: torch.Tensor, prev_tok: torch.Tensor, embed: nn.Module, n: int) -> torch.Tensor:
        toks = []
        for _ in range(n):
            prev_tok = self.forward(h_last, embed(prev_tok)).argmax(-1)
            toks.append(prev_tok)
        return torch.stack(toks, 1)
