"""Inference operator fronts (reference opss/infer/flash_attention.py:68-452, ring_attention.py:64-416,
speculative.py:53-417, vllm.py:66-1204): the reference's operator API over THIS framework's kernels and engine.

  * ``PiscesLxFlashAttention3Operator / Layer``   attention through ``ops.functional.attention`` (the tcgen05 / TMEM
    flash kernels on the GPU, the fp32 oracle on the CPU); a sliding window is applied as an exact mask on the oracle path.
  * ``PiscesLxRingAttentionOperator / Layer``     the sequence is cut into ``ring_size`` blocks; with a process group
    every rank holds one block and the blocks travel the ring (``parallel.cp``); in one process the blocks are visited
    in ring order and the partial results are merged by their log-sum-exp - the same arithmetic, exact, and memory
    O(block x block) instead of O(S x S).
  * ``PiscesLxSpeculativeDecodingOperator / PiscesLxAssistedDecodingOperator``   ``models.speculative`` decoders.
  * ``PiscesLxVLLMInferenceOperator``             the batch API (``generate(prompts, sampling)``) on ``YvInferenceEngine``:
    continuous batching, paged cache, prefix caching and chunked prefill are the engine's own; nothing here calls an
    external serving library."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn

from ..ops import functional as F_
from ..utils.opsc import PiscesLxOperatorInterface


# ---------------------------------------------------------------------------------------------------------------- flash attention
class PiscesLxFlashAttentionBackend(str, Enum):
    NATIVE = "native"            # this framework's kernels
    REFERENCE = "reference"      # fp32 oracle (CPU, tests)


class PiscesLxPrecisionMode(str, Enum):
    FP32 = "fp32"
    FP16 = "fp16"
    BF16 = "bf16"
    FP8_E4M3 = "fp8_e4m3"
    FP8_E5M2 = "fp8_e5m2"


@dataclass
class PiscesLxFlashAttention3Config:
    num_heads: int = 32
    num_kv_heads: Optional[int] = None
    head_dim: int = 128
    block_size: int = 128
    precision: Any = PiscesLxPrecisionMode.BF16
    causal: bool = True
    softmax_scale: Optional[float] = None
    dropout: float = 0.0
    window_size: int = -1
    backend: Any = PiscesLxFlashAttentionBackend.NATIVE

    def __post_init__(self) -> None:
        self.precision = PiscesLxPrecisionMode(getattr(self.precision, "value", self.precision))
        self.backend = PiscesLxFlashAttentionBackend(getattr(self.backend, "value", self.backend))
        self.num_kv_heads = self.num_kv_heads or self.num_heads
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.softmax_scale is None:
            self.softmax_scale = 1.0 / math.sqrt(self.head_dim)
        if self.precision in (PiscesLxPrecisionMode.FP8_E4M3, PiscesLxPrecisionMode.FP8_E5M2):
            raise ValueError("the attention kernels compute in bf16 with fp32 accumulation; fp8 is offered for GEMMs only")
        if self.dropout:
            raise ValueError("attention dropout is not implemented by the kernels")


def _windowed_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool, scale: float, window: int) -> torch.Tensor:
    """q [B, S, hq, d], k / v [B, T, hk, d]: exact masked attention in fp32 (the window counts the query's own position)."""
    B, S, hq, d = q.shape
    T, hk = k.shape[1], k.shape[2]
    g = hq // hk
    kk, vv = k.float().repeat_interleave(g, 2), v.float().repeat_interleave(g, 2)
    s = torch.einsum("bshd,bthd->bhst", q.float(), kk) * scale
    qi = torch.arange(S, device=q.device)[:, None] + (T - S)
    ki = torch.arange(T, device=q.device)[None, :]
    mask = torch.ones(S, T, dtype=torch.bool, device=q.device)
    if causal:
        mask &= ki <= qi
    if window > 0:
        mask &= ki > qi - window
    s = s.masked_fill(~mask, float("-inf"))
    return torch.einsum("bhst,bthd->bshd", torch.softmax(s, -1), vv).to(q.dtype)


class PiscesLxFlashAttention3Operator(PiscesLxOperatorInterface):
    """inputs: q [B, S, hq, d], k, v [B, T, hk, d] (or packed [T, h*d] with ``cu_seqlens``); output ``{"output": ...}``."""

    name = "flash_attention"

    def __init__(self, config: Optional[PiscesLxFlashAttention3Config] = None):
        self.config = config or PiscesLxFlashAttention3Config()

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return all(torch.is_tensor(inputs.get(k)) for k in ("q", "k", "v"))

    def attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q: Optional[torch.Tensor] = None,
               cu_k: Optional[torch.Tensor] = None, max_q: Optional[int] = None, max_k: Optional[int] = None) -> torch.Tensor:
        c = self.config
        hq, hk, d = c.num_heads, c.num_kv_heads, c.head_dim
        if q.dim() == 2:                                        # packed varlen
            return F_.attention(q, k, v, cu_q, cu_k if cu_k is not None else cu_q, int(max_q), int(max_k or max_q), hq, hk, d,
                                causal=c.causal, scale=c.softmax_scale)
        B, S = q.shape[:2]
        T = k.shape[1]
        if c.window_size > 0 or c.backend is PiscesLxFlashAttentionBackend.REFERENCE or (c.causal and S != T):
            return _windowed_reference(q, k, v, c.causal, c.softmax_scale, c.window_size)
        cq = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=q.device)
        ck = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=q.device)
        o = F_.attention(q.reshape(B * S, hq * d), k.reshape(B * T, hk * d), v.reshape(B * T, hk * d), cq, ck, S, T, hq, hk, d,
                         causal=c.causal, scale=c.softmax_scale)
        return o.view(B, S, hq, d)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        return {"output": self.attend(inputs["q"], inputs["k"], inputs["v"], inputs.get("cu_seqlens_q"), inputs.get("cu_seqlens_k"),
                                      inputs.get("max_seqlen_q"), inputs.get("max_seqlen_k"))}


class PiscesLxFlashAttention3Layer(nn.Module):
    """hidden [B, S, H] -> [B, S, H]: fused qkv projection, the operator, output projection."""

    def __init__(self, hidden_size: int, config: Optional[PiscesLxFlashAttention3Config] = None):
        super().__init__()
        self.config = c = config or PiscesLxFlashAttention3Config()
        self.op = PiscesLxFlashAttention3Operator(c)
        nq, nk = c.num_heads * c.head_dim, c.num_kv_heads * c.head_dim
        self.qkv = nn.Parameter(torch.empty(nq + 2 * nk, hidden_size).normal_(std=0.02))
        self.o = nn.Parameter(torch.empty(hidden_size, nq).normal_(std=0.02))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        c = self.config
        B, S, H = x.shape
        nq, nk = c.num_heads * c.head_dim, c.num_kv_heads * c.head_dim
        y = F_.linear(x.reshape(B * S, H), self.qkv.to(x.dtype))
        q = y[:, :nq].reshape(B, S, c.num_heads, c.head_dim)
        k = y[:, nq:nq + nk].reshape(B, S, c.num_kv_heads, c.head_dim)
        v = y[:, nq + nk:].reshape(B, S, c.num_kv_heads, c.head_dim)
        o = self.op.attend(q, k, v)
        return F_.linear(o.reshape(B * S, nq), self.o.to(x.dtype)).view(B, S, H)


# ---------------------------------------------------------------------------------------------------------------- ring attention
class PiscesLxRingTopology(str, Enum):
    RING = "ring"                        # block r sends to r + 1
    BIDIRECTIONAL = "bidirectional"      # halves of the key / value block travel both ways: half as many hops
    TREE = "tree"                        # all-gather of the blocks, then local attention (short rings)


@dataclass
class PiscesLxRingAttentionConfig:
    ring_size: int = 8
    block_size: int = 4096
    num_heads: int = 32
    num_kv_heads: Optional[int] = None
    head_dim: int = 128
    causal: bool = True
    topology: Any = PiscesLxRingTopology.RING
    max_sequence_length: int = 1048576

    def __post_init__(self) -> None:
        self.topology = PiscesLxRingTopology(getattr(self.topology, "value", self.topology))
        self.num_kv_heads = self.num_kv_heads or self.num_heads
        if self.ring_size < 1:
            raise ValueError("ring_size must be at least 1")


def merge_partial_attention(o_a: torch.Tensor, lse_a: torch.Tensor, o_b: torch.Tensor, lse_b: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Two partial attention results over disjoint key sets -> the result over their union.  o [..., d] fp32, lse [...]
    (log of the softmax denominators; -inf for an empty set)."""
    m = torch.maximum(lse_a, lse_b)
    m_safe = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    wa, wb = torch.exp(lse_a - m_safe), torch.exp(lse_b - m_safe)
    den = (wa + wb).clamp_min(1e-38)
    return (o_a * wa[..., None] + o_b * wb[..., None]) / den[..., None], m_safe + torch.log(den)


class PiscesLxRingAttentionOperator(PiscesLxOperatorInterface):
    name = "ring_attention"

    def __init__(self, config: Optional[PiscesLxRingAttentionConfig] = None):
        self.config = config or PiscesLxRingAttentionConfig()
        self.blocks_visited = 0

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return all(torch.is_tensor(inputs.get(k)) for k in ("q", "k", "v"))

    @staticmethod
    def _block(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        """q [B, Sq, h, d], k / v [B, Sk, h, d] -> (o fp32 [B, Sq, h, d], lse [B, Sq, h])."""
        s = torch.einsum("bshd,bthd->bsht", q.float(), k.float()) * scale
        if mask is not None:
            s = s.masked_fill(~mask[None, :, None, :], float("-inf"))
        lse = torch.logsumexp(s, -1)
        p = torch.exp(s - torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))[..., None])
        p = torch.where(torch.isfinite(lse)[..., None], p, torch.zeros_like(p))
        return torch.einsum("bsht,bthd->bshd", p, v.float()), lse

    def attend_local(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """One process: q, k, v [B, S, h(k), d].  Query block r meets the key blocks in the order a ring would deliver
        them (r, r - 1, ...); blocks wholly in the future of a causal query block are skipped."""
        c = self.config
        B, S, hq, d = q.shape
        g = hq // k.shape[2]
        kk, vv = k.repeat_interleave(g, 2), v.repeat_interleave(g, 2)
        R = min(c.ring_size, S)
        bounds = [(i * S) // R for i in range(R + 1)]
        scale = 1.0 / math.sqrt(d)
        out = torch.empty(B, S, hq, d, dtype=torch.float32, device=q.device)
        self.blocks_visited = 0
        for r in range(R):
            qs, qe = bounds[r], bounds[r + 1]
            acc = torch.zeros(B, qe - qs, hq, d, dtype=torch.float32, device=q.device)
            lse = torch.full((B, qe - qs, hq), float("-inf"), device=q.device)
            for hop in range(R):
                b = (r - hop) % R
                ks, ke = bounds[b], bounds[b + 1]
                if c.causal and ks >= qe:
                    continue
                mask = None
                if c.causal and ke > qs:
                    mask = torch.arange(ks, ke, device=q.device)[None, :] <= torch.arange(qs, qe, device=q.device)[:, None]
                o_b, l_b = self._block(q[:, qs:qe], kk[:, ks:ke], vv[:, ks:ke], scale, mask)
                acc, lse = merge_partial_attention(acc, lse, o_b, l_b)
                self.blocks_visited += 1
            out[:, qs:qe] = acc
        return out.to(q.dtype)

    def attend_distributed(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group: Any) -> torch.Tensor:
        """q [L, hq*d], k / v [L, hk*d]: this rank's contiguous chunk of one sequence; the blocks travel the ring."""
        from ..parallel import cp
        c = self.config
        return cp.ring_attention_train(q, k, v, group, c.num_heads, c.num_kv_heads, c.head_dim, c.causal)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        if inputs.get("group") is not None:
            return {"output": self.attend_distributed(inputs["q"], inputs["k"], inputs["v"], inputs["group"])}
        return {"output": self.attend_local(inputs["q"], inputs["k"], inputs["v"]), "blocks_visited": self.blocks_visited}


class PiscesLxRingAttentionLayer(nn.Module):
    def __init__(self, hidden_size: int, config: Optional[PiscesLxRingAttentionConfig] = None):
        super().__init__()
        self.config = c = config or PiscesLxRingAttentionConfig()
        self.op = PiscesLxRingAttentionOperator(c)
        nq, nk = c.num_heads * c.head_dim, c.num_kv_heads * c.head_dim
        self.qkv = nn.Parameter(torch.empty(nq + 2 * nk, hidden_size).normal_(std=0.02))
        self.o = nn.Parameter(torch.empty(hidden_size, nq).normal_(std=0.02))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        c = self.config
        B, S, H = x.shape
        nq, nk = c.num_heads * c.head_dim, c.num_kv_heads * c.head_dim
        y = F_.linear(x.reshape(B * S, H), self.qkv.to(x.dtype))
        q = y[:, :nq].reshape(B, S, c.num_heads, c.head_dim)
        k = y[:, nq:nq + nk].reshape(B, S, c.num_kv_heads, c.head_dim)
        v = y[:, nq + nk:].reshape(B, S, c.num_kv_heads, c.head_dim)
        o = self.op.attend_local(q, k, v)
        return F_.linear(o.reshape(B * S, nq), self.o.to(x.dtype)).view(B, S, H)


# ---------------------------------------------------------------------------------------------------------------- speculative decoding
@dataclass
class PiscesLxSpeculativeConfig:
    gamma: int = 5                           # tokens drafted per round
    draft_temperature: float = 0.8
    target_temperature: float = 0.7
    max_new_tokens: int = 512
    stop_token_id: Optional[int] = None
    early_stopping: bool = True
    acceptance_threshold: float = 0.1        # below this running acceptance rate the operator stops drafting
    fallback_to_regular: bool = True
    adaptive: bool = False


class PiscesLxSpeculativeDecodingOperator(PiscesLxOperatorInterface):
    """A target model and a drafter (a smaller model, or the n-gram / Medusa heads of ``models.speculative``).  inputs:
    {"input_ids": [1, S]}; output: the generated ids and the acceptance statistics.  The accepted tokens follow the
    target's distribution exactly (rejection sampling)."""

    name = "speculative_decoding"

    def __init__(self, target_model: Any, draft_model: Any = None, config: Optional[PiscesLxSpeculativeConfig] = None):
        from ..models.speculative import YvAdaptiveSpeculativeDecoder, YvSpeculativeConfig, YvSpeculativeDecoder
        self.config = c = config or PiscesLxSpeculativeConfig()
        scfg = YvSpeculativeConfig(draft_length=c.gamma, temperature=c.target_temperature,
                                   rule="exact" if c.target_temperature > 0 else "threshold")
        if c.adaptive:
            self.decoder = YvAdaptiveSpeculativeDecoder(target_model, scfg)
            self.decoder.draft_model = draft_model
        else:
            self.decoder = YvSpeculativeDecoder(target_model, scfg, draft_model=draft_model)
        self.target = target_model
        self.history: List[Dict[str, Any]] = []

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return torch.is_tensor(inputs.get("input_ids"))

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        c = self.config
        n = int(inputs.get("max_new_tokens", c.max_new_tokens))
        ids, stats = self.decoder.speculative_generate(inputs["input_ids"], max_new_tokens=n, eos_token_id=c.stop_token_id)
        rate = float(stats.get("acceptance_rate", 1.0))
        rec = {"acceptance_rate": rate, "generated": int(ids.shape[-1] - inputs["input_ids"].shape[-1]),
               "fell_back": bool(stats.get("fell_back", False))}
        if c.fallback_to_regular and rate < c.acceptance_threshold:
            rec["fell_back"] = True                              # drafting costs more than it saves
        self.history.append(rec)
        return {"output_ids": ids, **rec, "stats": stats}


class PiscesLxAssistedDecodingOperator(PiscesLxSpeculativeDecodingOperator):
    """Speculative decoding with an ASSISTANT model chosen per request: ``assistants`` maps a name to a draft model and
    ``inputs["assistant"]`` picks one (the first by default)."""

    name = "assisted_decoding"

    def __init__(self, target_model: Any, assistants: Dict[str, Any], config: Optional[PiscesLxSpeculativeConfig] = None):
        if not assistants:
            raise ValueError("assisted decoding needs at least one assistant model")
        self.assistants = dict(assistants)
        self._ops = {n: PiscesLxSpeculativeDecodingOperator(target_model, m, config) for n, m in self.assistants.items()}
        first = next(iter(self._ops.values()))
        self.config, self.decoder, self.target, self.history = first.config, first.decoder, target_model, []

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        name = inputs.get("assistant") or next(iter(self._ops))
        if name not in self._ops:
            raise KeyError(f"unknown assistant {name!r}; have {sorted(self._ops)}")
        out = self._ops[name].run(inputs)
        out["assistant"] = name
        self.history.append({"assistant": name, "acceptance_rate": out["acceptance_rate"]})
        return out

    def best_assistant(self) -> Optional[str]:
        """The assistant with the highest mean acceptance rate so far."""
        agg: Dict[str, List[float]] = {}
        for h in self.history:
            agg.setdefault(h["assistant"], []).append(h["acceptance_rate"])
        return max(agg, key=lambda n: sum(agg[n]) / len(agg[n])) if agg else None


# ---------------------------------------------------------------------------------------------------------------- batch engine front
@dataclass
class PiscesLxVLLMConfig:
    model_path: str = ""
    tensor_parallel_size: int = 1
    dtype: str = "bfloat16"
    seed: int = 0
    gpu_memory_utilization: float = 0.9
    max_model_len: Optional[int] = None
    max_num_seqs: int = 256
    block_size: int = 64
    num_blocks: Optional[int] = None
    enable_prefix_caching: bool = True
    enable_chunked_prefill: bool = False
    enforce_eager: bool = False


@dataclass
class PiscesLxSamplingParams:
    max_tokens: int = 128
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    stop_token_ids: List[int] = field(default_factory=list)


class PiscesLxVLLMInferenceOperator(PiscesLxOperatorInterface):
    """``generate(prompts, sampling)`` over ``YvInferenceEngine``: every prompt becomes a request, the engine batches
    them continuously, and the outputs come back in the order of the prompts.  Prompts are strings or lists of ids."""

    name = "batch_inference"

    def __init__(self, model: Optional[nn.Module] = None, config: Optional[PiscesLxVLLMConfig] = None, engine: Any = None,
                 tokenizer: Any = None):
        from .engine import YvEngineConfig, YvInferenceEngine
        self.config = c = config or PiscesLxVLLMConfig()
        if engine is None:
            if model is None:
                raise ValueError("give a model or an engine")
            torch.manual_seed(c.seed)
            ec = YvEngineConfig(max_num_seqs=c.max_num_seqs, block_size=c.block_size, use_cuda_graphs=not c.enforce_eager)
            if c.num_blocks:
                ec.num_blocks = c.num_blocks
            if c.max_model_len:
                ec.max_model_len = c.max_model_len
            engine = YvInferenceEngine(model, tokenizer, ec)
        self.engine = engine

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs.get("prompts"), (list, tuple)) and len(inputs["prompts"]) > 0

    def generate(self, prompts: Sequence[Union[str, Sequence[int]]], sampling: Optional[PiscesLxSamplingParams] = None) -> List[Dict[str, Any]]:
        from ..models.generation import YvSamplingConfig
        sp, e = sampling or PiscesLxSamplingParams(), self.engine
        strat = "greedy" if sp.temperature <= 0 else "top_k_top_p"
        reqs = []
        for p in prompts:
            ids = e.tokenizer.encode(p) if isinstance(p, str) else list(p)
            reqs.append(e.add_request(ids, sp.max_tokens, YvSamplingConfig(strategy=strat, temperature=max(sp.temperature, 1e-5),
                                                                           top_k=sp.top_k, top_p=sp.top_p), list(sp.stop_token_ids)))
        while any(not r.finished for r in reqs):
            e.step()
        return [{"request_id": r.request_id if hasattr(r, "request_id") else i, "prompt_token_ids": list(r.prompt_ids),
                 "token_ids": list(r.output_ids), "text": e.tokenizer.decode(r.output_ids), "finish_reason": r.finish_reason,
                 "ttft": r.ttft} for i, r in enumerate(reqs)]

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        sp = inputs.get("sampling_params")
        if isinstance(sp, dict):
            sp = PiscesLxSamplingParams(**sp)
        return {"outputs": self.generate(inputs["prompts"], sp), "stats": self.engine.get_stats()}
