"""Benchmark harness (reference tools/benchmark/*: ``performance.py`` TTFT / inter-token latency / tokens per second /
memory / FLOPs estimate :79-560, multiple-choice and generative task harnesses for MMLU / GSM8K / HumanEval-style
sets, long-context probes).  Data sets are read from local JSONL files (no downloads): multiple choice rows
``{"question", "choices": [...], "answer": index}``; generative rows ``{"prompt", "answer"}``."""
from __future__ import annotations

import json
import statistics
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch


def model_flops_per_token(cfg: Any, seq_len: int, training: bool = True) -> float:
    """Dense-equivalent FLOPs per token: 2 x active parameters (x3 with backward) + attention's 4 * S/2 * H per layer."""
    H, L = cfg.hidden_size, cfg.n_layer
    hd = H // cfg.n_head
    attn = H * (cfg.n_head + 2 * cfg.n_kv_head) * hd + cfg.n_head * hd * H
    if getattr(cfg, "moe_num_experts", 0):
        ffn = 3 * H * (cfg.moe_top_k * cfg.moe_expert_intermediate_size +
                       cfg.moe_shared_experts * cfg.moe_shared_intermediate_size)
    else:
        ffn = 3 * H * cfg.intermediate_size
    active = L * (attn + ffn) + cfg.vocab_size * H
    mm = 2.0 * active + L * 4.0 * (seq_len / 2) * H
    return mm * (3.0 if training else 1.0)


@dataclass
class PiscesLxPerformanceReport:
    ttft_ms: List[float] = field(default_factory=list)
    inter_token_ms: List[float] = field(default_factory=list)
    tokens_per_s: float = 0.0
    peak_memory_gb: float = 0.0
    model_tflops: float = 0.0

    def summary(self) -> Dict[str, Any]:
        p = lambda xs, q: sorted(xs)[min(len(xs) - 1, int(q * len(xs)))] if xs else None
        return {"ttft_p50_ms": p(self.ttft_ms, 0.5), "ttft_p95_ms": p(self.ttft_ms, 0.95),
                "itl_p50_ms": p(self.inter_token_ms, 0.5), "itl_p95_ms": p(self.inter_token_ms, 0.95),
                "tokens_per_s": self.tokens_per_s, "peak_memory_gb": self.peak_memory_gb,
                "model_tflops": self.model_tflops}


class PiscesLxPerformanceBenchmark:
    """Measures a model's generation through its public ``generate`` with a per-token callback."""

    def __init__(self, model: Any, device: Optional[torch.device] = None):
        self.model = model
        self.device = device or next(model.parameters()).device

    def _sync(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def run(self, prompts: List[torch.Tensor], max_new_tokens: int = 32) -> PiscesLxPerformanceReport:
        rep = PiscesLxPerformanceReport()
        if self.device.type == "cuda":
            torch.cuda.reset_peak_memory_stats(self.device)
        total_tokens, total_time = 0, 0.0
        for ids in prompts:
            stamps: List[float] = []

            def on_token(_t, stamps=stamps):
                self._sync()
                stamps.append(time.perf_counter())

            self._sync()
            t0 = time.perf_counter()
            self.model.generate(ids.to(self.device), max_new_tokens=max_new_tokens, eos_token_id=-1, on_token=on_token)
            self._sync()
            t1 = time.perf_counter()
            if stamps:
                rep.ttft_ms.append((stamps[0] - t0) * 1e3)
                rep.inter_token_ms += [(b - a) * 1e3 for a, b in zip(stamps, stamps[1:])]
            total_tokens += ids.shape[0] * len(stamps)
            total_time += t1 - t0
        rep.tokens_per_s = total_tokens / max(total_time, 1e-9)
        if self.device.type == "cuda":
            rep.peak_memory_gb = torch.cuda.max_memory_allocated(self.device) / 1e9
        cfg = getattr(self.model, "cfg", None)
        if cfg is not None and prompts:
            rep.model_tflops = rep.tokens_per_s * model_flops_per_token(cfg, prompts[0].shape[1], False) / 1e12
        return rep


def read_jsonl(path: str) -> List[Dict[str, Any]]:
    with open(path) as f:
        return [json.loads(l) for l in f if l.strip()]


class PiscesLxMultipleChoiceHarness:
    """Log-likelihood scoring: the choice whose continuation has the highest mean token log-probability wins."""

    def __init__(self, model: Any, tokenizer: Any):
        self.model, self.tok = model, tokenizer

    @torch.no_grad()
    def _score(self, prompt: str, cont: str) -> float:
        dev = next(self.model.parameters()).device
        p, c = self.tok.encode(prompt), self.tok.encode(cont)
        ids = torch.tensor([p + c], device=dev)
        logits = self.model(input_ids=ids, return_logits=True)["logits"].float()
        lp = torch.log_softmax(logits[0, len(p) - 1: len(p) + len(c) - 1], -1)
        return float(lp.gather(1, torch.tensor(c, device=dev)[:, None]).mean())

    def evaluate(self, rows: Iterable[Dict[str, Any]]) -> Dict[str, float]:
        n = correct = 0
        for r in rows:
            scores = [self._score(r["question"] + "\nAnswer: ", ch) for ch in r["choices"]]
            correct += int(max(range(len(scores)), key=scores.__getitem__) == int(r["answer"]))
            n += 1
        return {"accuracy": correct / max(n, 1), "n": n}


class PiscesLxGenerativeHarness:
    """Exact-match (after normalisation) on generated answers; ``extract`` pulls the answer out of the completion."""

    def __init__(self, generate: Callable[[str, int], str], extract: Optional[Callable[[str], str]] = None):
        self.generate = generate
        self.extract = extract or (lambda s: s.strip().splitlines()[0].strip() if s.strip() else "")

    @staticmethod
    def _norm(s: str) -> str:
        return "".join(ch for ch in s.lower().strip() if ch.isalnum() or ch in ".-")

    def evaluate(self, rows: Iterable[Dict[str, Any]], max_new_tokens: int = 64) -> Dict[str, float]:
        n = correct = 0
        for r in rows:
            out = self.extract(self.generate(r["prompt"], max_new_tokens))
            correct += int(self._norm(out) == self._norm(str(r["answer"])))
            n += 1
        return {"exact_match": correct / max(n, 1), "n": n}


def needle_in_haystack_rows(tokenizer: Any, context_tokens: int, depths=(0.1, 0.5, 0.9), needle: str = "The pass code is 7319.",
                            filler: str = "The sky was clear and the road was long. ") -> List[Dict[str, Any]]:
    """Long-context probe rows for the generative harness: a fact placed at a relative depth of a filler context."""
    per = max(1, len(tokenizer.encode(filler)))
    n_fill = max(1, context_tokens // per)
    rows = []
    for d in depths:
        k = int(d * n_fill)
        ctx = filler * k + needle + " " + filler * (n_fill - k)
        rows.append({"prompt": ctx + "\nWhat is the pass code? Answer: ", "answer": "7319", "depth": d})
    return rows
