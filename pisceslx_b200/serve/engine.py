"""Inference engine with continuous batching over the paged KV cache.

The reference serves one request at a time on one GPU: prefill, then a Python decode loop per request
(tools/infer/core.py:1106-1144); ``max_concurrency`` only limits HTTP handlers.  Here requests are queued, each
engine step admits waiting requests while cache blocks are free (prefill, one request at a time so that TTFT stays
low), and all running sequences decode together in one batched step (one token each) through the paged-decode
kernel.  Finished sequences release their blocks immediately.  ``generate`` / ``generate_stream`` /
``embeddings`` keep the reference engine's surface (``PiscesLxInferenceEngine``).
"""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, Dict, Iterator, List, Optional

import torch

from ..models.cache import YvPagedKVCache, cache_for_model
from ..models.generation import YvSampler, YvSamplingConfig, _decode_step, _prefill
from ..models.tokenizer import YvTokenizer


@dataclass
class YvRequest:
    request_id: int
    prompt_ids: List[int]
    max_new_tokens: int = 128
    sampling: YvSamplingConfig = field(default_factory=YvSamplingConfig)
    stop_token_ids: List[int] = field(default_factory=list)
    output_ids: List[int] = field(default_factory=list)
    arrival: float = field(default_factory=time.perf_counter)
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    finished: bool = False
    finish_reason: Optional[str] = None
    on_token: Optional[Callable[[int], None]] = None
    _next_logits: Optional[torch.Tensor] = None
    preemptions: int = 0

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token_time is None else self.first_token_time - self.arrival


@dataclass
class YvEngineConfig:
    max_num_seqs: int = 64
    num_blocks: int = 4096
    block_size: int = 64
    max_model_len: int = 131072
    eos_token_id: Optional[int] = None
    use_cuda_graphs: bool = True          # replay decode steps from CUDA graphs (one graph per batch bucket)
    graph_max_seq_len: int = 8192         # sequences longer than this decode through the eager step
    status_check_steps: int = 16          # read the kernels' status word every this many decode steps (0 = never)


class YvInferenceEngine:
    def __init__(self, model: torch.nn.Module, tokenizer: Optional[YvTokenizer] = None,
                 cfg: Optional[YvEngineConfig] = None):
        vocab = int(getattr(getattr(model, "cfg", None), "vocab_size", 0) or 0)
        self.vocab_size = vocab
        self.model, self.cfg = model.eval(), cfg or YvEngineConfig()
        self.tokenizer = tokenizer or (YvTokenizer.for_vocab(vocab) if vocab else YvTokenizer.instance())
        p = next(model.parameters())
        self.device = p.device
        tp = model.parallel.tp_size if getattr(model, "parallel", None) is not None else 1
        self.cache: YvPagedKVCache = cache_for_model(model.cfg, self.device, self.cfg.num_blocks, self.cfg.block_size,
                                                     tp_size=tp, n_layer=len(model.model.layers), dtype=p.dtype)
        self.cache.layer_offset = model.model.layer_lo
        from .graph_decode import YvDecodeGraphRunner
        self.graph = YvDecodeGraphRunner(model, self.cache, min(self.cfg.max_model_len, self.cfg.graph_max_seq_len),
                                         enabled=self.cfg.use_cuda_graphs)
        self.waiting: Deque[YvRequest] = deque()
        self.running: List[YvRequest] = []
        self._next_id = 0
        self._lock = threading.Lock()
        self.stats = {"requests": 0, "tokens_generated": 0, "prefill_tokens": 0, "steps": 0, "errors": 0,
                      "preemptions": 0, "ttft": [], "latency": []}
        self._reserved: Dict[int, int] = {}   # request id -> worst-case number of cache blocks it may ever hold
        self.eos = self.cfg.eos_token_id if self.cfg.eos_token_id is not None else model.cfg.eos_token_id

    # ---- request management ---------------------------------------------------------------------------
    def add_request(self, prompt_ids: List[int], max_new_tokens: int = 128,
                    sampling: Optional[YvSamplingConfig] = None, stop_token_ids: Optional[List[int]] = None,
                    on_token: Optional[Callable[[int], None]] = None) -> YvRequest:
        prompt_ids = list(prompt_ids)
        if not prompt_ids:
            raise ValueError("empty prompt")
        if self.vocab_size and (max(prompt_ids) >= self.vocab_size or min(prompt_ids) < 0):
            raise ValueError(f"prompt holds token ids outside the model's vocabulary of {self.vocab_size}")
        with self._lock:
            rid = self._next_id
            self._next_id += 1
        req = YvRequest(rid, list(prompt_ids), max_new_tokens, sampling or YvSamplingConfig(),
                        list(stop_token_ids or []), on_token=on_token)
        self.waiting.append(req)
        self.stats["requests"] += 1
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _finish(self, req: YvRequest, reason: str) -> None:
        req.finished, req.finish_reason, req.finish_time = True, reason, time.perf_counter()
        self.cache.free_sequence(req.request_id)
        self._reserved.pop(req.request_id, None)
        if req.ttft is not None:
            self.stats["ttft"].append(req.ttft)
        self.stats["latency"].append(req.finish_time - req.arrival)

    def _emit(self, req: YvRequest, token: int) -> None:
        req.output_ids.append(token)
        self.stats["tokens_generated"] += 1
        if req.first_token_time is None:
            req.first_token_time = time.perf_counter()
        if req.on_token is not None:
            req.on_token(token)
        if token == self.eos or token in req.stop_token_ids:
            self._finish(req, "stop")
        elif len(req.output_ids) >= req.max_new_tokens:
            self._finish(req, "length")

    # ---- admission control ---------------------------------------------------------------------------
    def _worst_case_blocks(self, req: YvRequest) -> int:
        remaining = max(req.max_new_tokens - len(req.output_ids), 0)
        total = len(req.prompt_ids) + len(req.output_ids) + remaining
        return (total + self.cfg.block_size - 1) // self.cfg.block_size

    def _owed_blocks(self) -> int:
        """Blocks that running requests may still take: their reservation minus what they already hold.  Running
        sequences allocate lazily (one block every ``block_size`` tokens), so free blocks alone overstate the room."""
        owed = 0
        for rid, need in self._reserved.items():
            owed += max(need - len(self.cache.tables.get(rid, ())), 0)
        return owed

    def _preempt_youngest(self) -> bool:
        """Give the newest running request's blocks back and put it at the head of the queue; its prompt becomes
        prompt + tokens generated so far, so it resumes by prefill where it stopped."""
        if len(self.running) <= 1:
            return False
        victim = max(self.running, key=lambda r: r.arrival)
        self.running.remove(victim)
        self.cache.free_sequence(victim.request_id)
        self._reserved.pop(victim.request_id, None)
        victim.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(victim)
        return True

    def _admit(self, req: YvRequest) -> None:
        self.cache.add_sequence(req.request_id)
        self._reserved[req.request_id] = self._worst_case_blocks(req)
        context = req.prompt_ids + req.output_ids           # non-empty output: resuming after a preemption
        ids = torch.tensor([context], dtype=torch.long, device=self.device)
        logits = _prefill(self.model, ids, self.cache, [req.request_id])
        self.stats["prefill_tokens"] += len(context)
        tok = int(YvSampler(req.sampling).sample(logits, ids)[0])
        self.running.append(req)
        self._emit(req, tok)

    # ---- one scheduler iteration ---------------------------------------------------------------------------
    @torch.no_grad()
    def step(self) -> None:
        self.stats["steps"] += 1
        # admit: prefill waiting requests while there is room for their WORST case next to what is already promised
        while self.waiting and len(self.running) < self.cfg.max_num_seqs:
            req = self.waiting[0]
            now = (len(req.prompt_ids) + len(req.output_ids) + self.cfg.block_size) // self.cfg.block_size
            need = max(self._worst_case_blocks(req), now)  # ``now``: prefill plus the first decoded token
            if need > self.cache.alloc.available() - self._owed_blocks():
                if not self.running:
                    self.waiting.popleft()
                    req.finished, req.finish_reason = True, "error: prompt does not fit the KV cache"
                    req.finish_time = time.perf_counter()
                    self.stats["errors"] += 1
                    continue
                break
            self.waiting.popleft()
            self._admit(req)
        self.running = [r for r in self.running if not r.finished]
        if not self.running:
            return
        # Safety net (reservations make it unreachable unless blocks are shared or taken behind the engine's back):
        # before ANY slot is appended, make sure every running sequence can take its next token.
        bs = self.cfg.block_size
        while True:
            new_blocks = sum(1 for r in self.running if self.cache.lengths[r.request_id] % bs == 0
                             and self.cache.lengths[r.request_id] // bs >= len(self.cache.tables[r.request_id]))
            if new_blocks <= self.cache.alloc.available() or not self._preempt_youngest():
                break
        # decode: one token for every running sequence in a single batched step
        seq_ids = [r.request_id for r in self.running]
        logits = self.graph.step([r.output_ids[-1] for r in self.running], seq_ids)
        if self.cfg.status_check_steps and self.device.type == "cuda" \
                and self.stats["steps"] % self.cfg.status_check_steps == 0:
            from ..ops import check_status
            check_status(self.device)      # a bounded wait that ran out or a bad block-table entry raises here
        greedy = all(r.sampling.strategy == "greedy" for r in self.running)
        if greedy:
            toks = logits.argmax(-1).tolist()
        else:
            toks = []
            for i, r in enumerate(self.running):
                prev = torch.tensor([r.prompt_ids + r.output_ids], dtype=torch.long, device=self.device)
                toks.append(int(YvSampler(r.sampling).sample(logits[i:i + 1], prev)[0]))
        for r, t in zip(self.running, toks):
            self._emit(r, int(t))
        self.running = [r for r in self.running if not r.finished]

    def run_until_done(self) -> None:
        while self.has_work():
            self.step()

    # ---- reference-style surface --------------------------------------------------------------------------------
    def generate(self, prompt: str, max_new_tokens: int = 128, temperature: float = 0.0, top_k: int = 0,
                 top_p: float = 1.0, **_: Any) -> Dict[str, Any]:
        strat = "greedy" if temperature <= 0 else "top_k_top_p"
        req = self.add_request(self.tokenizer.encode(prompt), max_new_tokens,
                               YvSamplingConfig(strategy=strat, temperature=max(temperature, 1e-5), top_k=top_k,
                                                top_p=top_p))
        while not req.finished:
            self.step()
        return {"text": self.tokenizer.decode(req.output_ids), "tokens": req.output_ids,
                "finish_reason": req.finish_reason, "ttft": req.ttft,
                "usage": {"prompt_tokens": len(req.prompt_ids), "completion_tokens": len(req.output_ids)}}

    def generate_stream(self, prompt: str, max_new_tokens: int = 128, **kw: Any) -> Iterator[str]:
        out: List[int] = []
        req = self.add_request(self.tokenizer.encode(prompt), max_new_tokens, on_token=out.append)
        sent = 0
        while not req.finished or sent < len(out):
            if not req.finished:
                self.step()
            while sent < len(out):
                yield self.tokenizer.decode([out[sent]])
                sent += 1

    @torch.no_grad()
    def embeddings(self, text: str) -> List[float]:
        """Mean of the final hidden states (reference tools/infer/core.py:1191-1204)."""
        ids = torch.tensor([self.tokenizer.encode(text)], dtype=torch.long, device=self.device)
        out = self.model(input_ids=ids, return_logits=False, return_hidden=True)
        return out["hidden_states"].float().mean(1)[0].tolist()

    def get_stats(self) -> Dict[str, Any]:
        s = dict(self.stats)
        tt = sorted(s.pop("ttft"))
        lat = s.pop("latency")
        s["p50_ttft"] = tt[len(tt) // 2] if tt else None
        s["mean_latency"] = sum(lat) / len(lat) if lat else None
        s["running"], s["waiting"] = len(self.running), len(self.waiting)
        s["free_blocks"] = self.cache.alloc.available()
        s["decode_graphs"] = self.graph.stats()
        return s


PiscesLxInferenceEngine = YvInferenceEngine
