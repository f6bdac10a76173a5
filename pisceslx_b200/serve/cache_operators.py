"""Serving operators around adapters, prompt prefixes and long prompts (reference opss/infer/vllm.py:96-900):
multi-LoRA serving, prefix caching of keys / values and chunked prefill.

Multi-LoRA, B200-first: the loaded adapters live in two slot-stacked tensors, A [S x r, in] and B [out, S x r]
(rank padded to ``max_lora_rank``, S = ``max_lora_adapters``), so that a batch whose rows use different adapters is
two dense GEMMs with K = S x r and a row mask in between -

    H = x A^T  [T, S x r];   H *= onehot(slot[t]) expanded over r;   y += (H * scale[slot]) B^T

- static shapes (loading an adapter writes into a slot, nothing is reallocated), no gather of per-row weights, no host
loop over adapters and nothing that breaks a CUDA-graph capture of the decode step.  With S x r <= hidden the extra
FLOPs stay under one base projection.  The reference hands adapter paths to vLLM's ``LoRARequest`` (vllm.py:521-560).

Prefix cache: entries are indexed by a chained hash at every ``block`` tokens, so the LONGEST cached prefix of a new
prompt is found with one dictionary probe per block and the caller learns how many tokens it covers (the reference
scans all entries and returns keys / values without their length, vllm.py:184-210).  The paged engine shares blocks
by reference count (``models/cache_policies.YvPrefixCache``); this manager is the tensor-level cache for callers
that hold keys / values themselves.

Chunked prefill: chunk boundaries fall on multiples of 128 tokens (the M tile of the tensor-core GEMMs and of the
attention kernel); every chunk attends to the cache of the chunks before it, so nothing is recomputed."""
from __future__ import annotations

import json
import os
import time
from collections import OrderedDict
from dataclasses import dataclass
from threading import Lock
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..utils.opsc import PiscesLxOperatorInterface

_FNV_OFFSET, _FNV_PRIME, _MASK64 = 1469598103934665603, 1099511628211, 0xFFFFFFFFFFFFFFFF


def _chain_hash(h: int, tokens: Sequence[int]) -> int:
    for t in tokens:
        h = ((h ^ (int(t) & 0xFFFFFFFF)) * _FNV_PRIME) & _MASK64
    return h


# ---- multi-LoRA ---------------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxMultiLoRAConfig:
    max_lora_adapters: int = 16
    max_lora_rank: int = 64
    enable_long_context: bool = False
    lora_dtype: str = "auto"

    @classmethod
    def from_adapter_path(cls, adapter_path: str) -> "PiscesLxMultiLoRAConfig":
        """Reads ``adapter_config.json`` beside the weights (keys ``r`` / ``rank``) when it exists."""
        p = os.path.join(adapter_path, "adapter_config.json") if os.path.isdir(adapter_path) else adapter_path
        rank = 64
        if os.path.isfile(p) and p.endswith(".json"):
            with open(p, encoding="utf-8") as f:
                d = json.load(f)
            rank = int(d.get("r", d.get("rank", rank)))
        return cls(max_lora_rank=max(rank, 1))


class PiscesLxMultiLoRAOperator(PiscesLxOperatorInterface):
    """Adapters for ONE projection (in_features -> out_features).  ``load_adapter(name, a [r, in], b [out, r])`` puts the
    adapter into a free slot (evicting the least recently used adapter of the lowest priority when all are taken);
    ``slots_for(names)`` turns a batch's adapter names into the slot tensor (-1 = no adapter); ``apply(x, base_out,
    slots)`` adds the adapters' contribution."""

    name = "multi_lora"

    def __init__(self, in_features: int, out_features: int, config: Optional[PiscesLxMultiLoRAConfig] = None,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None):
        self.config = c = config or PiscesLxMultiLoRAConfig()
        dt = dtype or {"auto": torch.float32, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16,
                       "float16": torch.float16, "fp32": torch.float32, "float32": torch.float32}[c.lora_dtype]
        S, r = c.max_lora_adapters, c.max_lora_rank
        self.in_features, self.out_features = in_features, out_features
        self.A = torch.zeros(S * r, in_features, device=device, dtype=dt)
        self.B = torch.zeros(out_features, S * r, device=device, dtype=dt)
        self.scale = torch.zeros(S, device=device, dtype=torch.float32)
        self.loaded_adapters: "OrderedDict[str, Dict[str, Any]]" = OrderedDict()
        self._free = list(range(S))
        self.adapter_lock = Lock()
        self.stats = {"total_requests": 0, "cache_hits": 0, "cache_misses": 0, "adapter_switches": 0, "evictions": 0}

    # -- residency ---------------------------------------------------------------------------------------------------------------
    def _evict_lru_adapter(self) -> None:
        with self.adapter_lock:
            self._evict_lru_adapter_locked()

    def load_adapter(self, adapter_name: str, a: torch.Tensor, b: torch.Tensor, alpha: Optional[float] = None, priority: int = 0,
                     path: str = "") -> int:
        r = a.shape[0]
        if a.shape != (r, self.in_features) or b.shape != (self.out_features, r):
            raise ValueError(f"adapter {adapter_name}: expected a [r, {self.in_features}] and b [{self.out_features}, r], got {tuple(a.shape)}, {tuple(b.shape)}")
        if r > self.config.max_lora_rank:
            raise ValueError(f"adapter {adapter_name}: rank {r} above max_lora_rank {self.config.max_lora_rank}")
        with self.adapter_lock:
            if adapter_name in self.loaded_adapters:
                slot = self.loaded_adapters[adapter_name]["slot"]
            else:
                if not self._free:
                    self._evict_lru_adapter_locked()
                slot = self._free.pop(0)
                self.stats["adapter_switches"] += 1
            R = self.config.max_lora_rank
            self.A[slot * R:(slot + 1) * R].zero_()
            self.B[:, slot * R:(slot + 1) * R].zero_()
            self.A[slot * R:slot * R + r].copy_(a)
            self.B[:, slot * R:slot * R + r].copy_(b)
            self.scale[slot] = (alpha / r) if alpha is not None else 1.0
            self.loaded_adapters[adapter_name] = {"slot": slot, "rank": r, "priority": priority, "path": path, "loaded_at": time.time()}
            self.loaded_adapters.move_to_end(adapter_name)
            return slot

    def _evict_lru_adapter_locked(self) -> None:
        low = min(info["priority"] for info in self.loaded_adapters.values())
        victim = next(n for n, info in self.loaded_adapters.items() if info["priority"] == low)     # oldest use first
        self._unload_locked(victim)
        self.stats["evictions"] += 1

    def _unload_locked(self, adapter_name: str) -> bool:
        info = self.loaded_adapters.pop(adapter_name, None)
        if info is None:
            return False
        slot, R = info["slot"], self.config.max_lora_rank
        self.A[slot * R:(slot + 1) * R].zero_()
        self.B[:, slot * R:(slot + 1) * R].zero_()
        self.scale[slot] = 0.0
        self._free.append(slot)
        return True

    def unload_adapter(self, adapter_name: str) -> bool:
        with self.adapter_lock:
            return self._unload_locked(adapter_name)

    def load_adapter_from_path(self, adapter_name: str, adapter_path: str, priority: int = 0, key_a: str = "lora_A", key_b: str = "lora_B") -> int:
        """A ``torch.save``d dictionary with the two matrices (and optionally ``alpha``)."""
        f = os.path.join(adapter_path, "adapter_model.pt") if os.path.isdir(adapter_path) else adapter_path
        d = torch.load(f, map_location="cpu", weights_only=True)
        return self.load_adapter(adapter_name, d[key_a], d[key_b], d.get("alpha"), priority, adapter_path)

    def get_loaded_adapters(self) -> List[str]:
        return list(self.loaded_adapters)

    # -- batch -------------------------------------------------------------------------------------------------------------------
    def slots_for(self, adapter_names: Sequence[Optional[str]]) -> torch.Tensor:
        with self.adapter_lock:
            out = []
            for n in adapter_names:
                if n is None:
                    out.append(-1)
                    continue
                info = self.loaded_adapters.get(n)
                if info is None:
                    raise KeyError(f"adapter {n} is not loaded")
                self.loaded_adapters.move_to_end(n)
                out.append(info["slot"])
        return torch.tensor(out, dtype=torch.long, device=self.A.device)

    def apply(self, x: torch.Tensor, base_out: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
        """x [T, in], base_out [T, out], slots [T] (-1 = none)."""
        S, R = self.config.max_lora_adapters, self.config.max_lora_rank
        h = x.to(self.A.dtype) @ self.A.t()                                               # [T, S*R]
        sel = (slots.unsqueeze(-1) == torch.arange(S, device=slots.device)).to(torch.float32) * self.scale   # [T, S]
        h = (h.view(-1, S, R) * sel.unsqueeze(-1).to(h.dtype)).view(-1, S * R)
        return base_out + (h @ self.B.t()).to(base_out.dtype)

    # -- front -------------------------------------------------------------------------------------------------------------------
    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return "adapter_name" in inputs and ("adapter_path" in inputs or ("lora_a" in inputs and "lora_b" in inputs) or inputs["adapter_name"] in self.loaded_adapters)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        name, priority = inputs["adapter_name"], int(inputs.get("priority", 0))
        self.stats["total_requests"] += 1
        if name in self.loaded_adapters:
            self.stats["cache_hits"] += 1
            with self.adapter_lock:
                self.loaded_adapters.move_to_end(name)
            cached, slot = True, self.loaded_adapters[name]["slot"]
        else:
            self.stats["cache_misses"] += 1
            cached = False
            if "lora_a" in inputs:
                slot = self.load_adapter(name, inputs["lora_a"], inputs["lora_b"], inputs.get("alpha"), priority, inputs.get("adapter_path", ""))
            else:
                slot = self.load_adapter_from_path(name, inputs["adapter_path"], priority)
        info = self.loaded_adapters[name]
        return {"slot": slot, "cached": cached, "adapter_info": {"name": name, "path": info["path"], "priority": info["priority"], "rank": info["rank"]}}

    def get_stats(self) -> Dict[str, Any]:
        return {**self.stats, "loaded": len(self.loaded_adapters), "free_slots": len(self._free)}

    def cleanup(self) -> None:
        for n in list(self.loaded_adapters):
            self.unload_adapter(n)


# ---- prefix cache ---------------------------------------------------------------------------------------------------------------
class PiscesLxPrefixCacheEntry:
    def __init__(self, prompt_hash: str, token_ids: Tuple[int, ...], kv_cache: Tuple[torch.Tensor, ...]):
        self.prompt_hash, self.token_ids, self.kv_cache = prompt_hash, token_ids, kv_cache
        self.cache_size = sum(t.numel() * t.element_size() for t in kv_cache if isinstance(t, torch.Tensor))
        self.hit_count, self.created_at, self.last_access = 0, time.time(), time.time()

    def hit(self) -> None:
        self.hit_count += 1
        self.last_access = time.time()

    def to_dict(self) -> Dict[str, Any]:
        return {"prompt_hash": self.prompt_hash, "token_count": len(self.token_ids), "cache_size": self.cache_size,
                "hit_count": self.hit_count, "created_at": self.created_at, "last_access": self.last_access}


class PiscesLxPrefixCacheManager:
    """``insert(token_ids, kv)`` stores the keys / values of a prompt; ``match(token_ids)`` returns the entry covering
    the longest prefix of ``token_ids`` and the number of tokens covered (the whole entry when the entry is a prefix of
    the query; a block-aligned part of it when the two only share a beginning and ``enable_substring_matching`` is
    on - the caller then slices the keys / values to that length along ``seq_dim``)."""

    def __init__(self, max_memory_bytes: Optional[int] = None, eviction_policy: str = "lru", enable_substring_matching: bool = True,
                 block: int = 16, seq_dim: int = -2):
        if eviction_policy not in ("lru", "lfu", "fifo"):
            raise ValueError(f"unknown eviction policy {eviction_policy}")
        self.cache: "OrderedDict[str, PiscesLxPrefixCacheEntry]" = OrderedDict()
        self._blocks: Dict[Tuple[int, int], str] = {}                # (tokens covered, chained hash) -> a prompt hash holding it
        self.max_memory_bytes, self.eviction_policy = max_memory_bytes, eviction_policy
        self.enable_substring_matching, self.block, self.seq_dim = enable_substring_matching, block, seq_dim
        self.lock = Lock()
        self.stats = {"hits": 0, "partial_hits": 0, "misses": 0, "evictions": 0, "memory_freed_bytes": 0, "total_accesses": 0}

    def _compute_prompt_hash(self, token_ids: Sequence[int]) -> str:
        return f"{len(token_ids)}:{_chain_hash(_FNV_OFFSET, token_ids):016x}"

    def _block_keys(self, token_ids: Sequence[int]) -> List[Tuple[int, int]]:
        h, out = _FNV_OFFSET, []
        for i in range(0, len(token_ids) - len(token_ids) % self.block, self.block):
            h = _chain_hash(h, token_ids[i:i + self.block])
            out.append((i + self.block, h))
        return out

    def match(self, token_ids: Sequence[int]) -> Tuple[Optional[PiscesLxPrefixCacheEntry], int]:
        token_ids = tuple(token_ids)
        with self.lock:
            self.stats["total_accesses"] += 1
            best: Tuple[Optional[PiscesLxPrefixCacheEntry], int] = (None, 0)
            e = self.cache.get(self._compute_prompt_hash(token_ids))
            if e is not None and e.token_ids == token_ids:
                best = (e, len(token_ids))
            elif self.enable_substring_matching:
                for covered, h in self._block_keys(token_ids):
                    ph = self._blocks.get((covered, h))
                    if ph is None:
                        break
                    ent = self.cache.get(ph)
                    if ent is None or ent.token_ids[:covered] != token_ids[:covered]:
                        break
                    best = (ent, covered)
                ent = best[0]
                if ent is not None:                                   # the unaligned tail of an entry that is a whole prefix
                    n = best[1]
                    while n < min(len(ent.token_ids), len(token_ids)) and ent.token_ids[n] == token_ids[n]:
                        n += 1
                    best = (ent, n)
            if best[0] is None:
                self.stats["misses"] += 1
                return None, 0
            best[0].hit()
            self.cache.move_to_end(best[0].prompt_hash)
            self.stats["hits" if best[1] == len(best[0].token_ids) else "partial_hits"] += 1
            return best

    def get(self, token_ids: Sequence[int]) -> Optional[Tuple[torch.Tensor, ...]]:
        """Keys / values covering the matched prefix (sliced along ``seq_dim`` when only part of an entry matches)."""
        e, n = self.match(token_ids)
        if e is None:
            return None
        if n == len(e.token_ids):
            return e.kv_cache
        return tuple(t.narrow(self.seq_dim, 0, n) if isinstance(t, torch.Tensor) else t for t in e.kv_cache)

    def insert(self, token_ids: Sequence[int], kv_cache: Tuple[torch.Tensor, ...]) -> bool:
        if not kv_cache:
            return False
        token_ids = tuple(token_ids)
        with self.lock:
            ph = self._compute_prompt_hash(token_ids)
            if ph in self.cache:
                self._drop(ph)
            self.cache[ph] = PiscesLxPrefixCacheEntry(ph, token_ids, tuple(kv_cache))
            for key in self._block_keys(token_ids):
                self._blocks[key] = ph                                # the newest holder answers for the block
            self._enforce_memory_limit()
            return ph in self.cache

    def _drop(self, ph: str) -> int:
        e = self.cache.pop(ph)
        for key in self._block_keys(e.token_ids):
            if self._blocks.get(key) == ph:
                del self._blocks[key]
                for other in self.cache.values():                     # another entry may hold the same block
                    if len(other.token_ids) >= key[0] and other.token_ids[:key[0]] == e.token_ids[:key[0]]:
                        self._blocks[key] = other.prompt_hash
                        break
        return e.cache_size

    def _victim(self) -> str:
        if self.eviction_policy == "lfu":
            return min(self.cache.values(), key=lambda e: (e.hit_count, e.last_access)).prompt_hash
        if self.eviction_policy == "fifo":
            return min(self.cache.values(), key=lambda e: e.created_at).prompt_hash
        return next(iter(self.cache))

    def _enforce_memory_limit(self) -> None:
        if self.max_memory_bytes is None:
            return
        used = sum(e.cache_size for e in self.cache.values())
        while used > self.max_memory_bytes and self.cache:
            freed = self._drop(self._victim())
            used -= freed
            self.stats["evictions"] += 1
            self.stats["memory_freed_bytes"] += freed

    def invalidate(self, prompt_hash: Optional[str] = None) -> int:
        with self.lock:
            if prompt_hash is None:
                n = len(self.cache)
                self.cache.clear()
                self._blocks.clear()
                return n
            if prompt_hash in self.cache:
                self._drop(prompt_hash)
                return 1
            return 0

    def get_memory_usage(self) -> Dict[str, Any]:
        with self.lock:
            used = sum(e.cache_size for e in self.cache.values())
        mb = 1024 * 1024
        return {"used_bytes": used, "used_mb": used / mb, "max_bytes": self.max_memory_bytes,
                "max_mb": self.max_memory_bytes / mb if self.max_memory_bytes else None, "entry_count": len(self.cache)}

    def get_stats(self) -> Dict[str, Any]:
        t = self.stats["total_accesses"]
        return {**self.stats, "hit_rate": (self.stats["hits"] + self.stats["partial_hits"]) / t if t else 0.0}

    def clear(self) -> None:
        self.invalidate(None)


class PiscesLxPrefixCachingOperator(PiscesLxOperatorInterface):
    name = "prefix_caching"

    def __init__(self, max_memory_bytes: Optional[int] = None, eviction_policy: str = "lru", enable_substring_matching: bool = True, block: int = 16):
        self.cache_manager = PiscesLxPrefixCacheManager(max_memory_bytes, eviction_policy, enable_substring_matching, block)

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        a = inputs.get("action", "lookup")
        return a in ("clear", "invalidate", "stats") or "token_ids" in inputs

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        a, m = inputs.get("action", "lookup"), self.cache_manager
        if a == "lookup":
            e, n = m.match(inputs["token_ids"])
            kv = None
            if e is not None:
                kv = e.kv_cache if n == len(e.token_ids) else tuple(t.narrow(m.seq_dim, 0, n) for t in e.kv_cache)
            return {"kv_cache": kv, "cache_hit": e is not None, "matched_tokens": n, "remaining_tokens": len(inputs["token_ids"]) - n,
                    "memory_usage": m.get_memory_usage()}
        if a == "insert":
            if inputs.get("kv_cache") is None:
                raise ValueError("kv_cache required for insert action")
            return {"inserted": m.insert(inputs["token_ids"], inputs["kv_cache"]), "memory_usage": m.get_memory_usage()}
        if a == "clear":
            m.clear()
            return {"cleared": True}
        if a == "invalidate":
            return {"invalidated_count": m.invalidate(inputs.get("prompt_hash")), "memory_usage": m.get_memory_usage()}
        if a == "stats":
            return m.get_stats()
        raise ValueError(f"Unknown action: {a}")

    def get_stats(self) -> Dict[str, Any]:
        return self.cache_manager.get_stats()

    def cleanup(self) -> None:
        self.cache_manager.clear()


# ---- chunked prefill ----------------------------------------------------------------------------------------------------------
class PiscesLxChunkedPrefillPlanner:
    """Chunk sizes for one long prompt.  ``bytes_per_token`` is the transient activation memory one prompt token costs
    (the caller measures or estimates it); with a memory budget the chunk is the largest multiple of ``align`` whose
    activations fit, between ``min_chunk_size`` and ``max_chunk_size``.  ``overlap_size`` > 0 gives every chunk a
    look-back window for models run WITHOUT a cache (the third element of a chunk is where its window starts)."""

    def __init__(self, max_chunk_size: int = 2048, min_chunk_size: int = 256, overlap_chunks: bool = False, overlap_size: int = 128,
                 memory_budget_bytes: Optional[int] = None, bytes_per_token: int = 0, align: int = 128):
        if min_chunk_size < 1 or max_chunk_size < min_chunk_size:
            raise ValueError("need 1 <= min_chunk_size <= max_chunk_size")
        self.max_chunk_size, self.min_chunk_size, self.align = max_chunk_size, min_chunk_size, max(align, 1)
        self.overlap_chunks, self.overlap_size = overlap_chunks, overlap_size
        self.memory_budget_bytes, self.bytes_per_token = memory_budget_bytes, bytes_per_token
        self.stats = {"total_requests": 0, "total_chunks": 0, "total_tokens_processed": 0, "avg_chunk_size": 0.0, "memory_saved_bytes": 0}

    def _aligned(self, n: int) -> int:
        n = max(self.min_chunk_size, min(n, self.max_chunk_size))
        return max((n // self.align) * self.align, min(self.min_chunk_size, n)) if n >= self.align else n

    def compute_optimal_chunk_size(self, seq_len: int, current_memory_usage: float = 0.0) -> int:
        size = self.max_chunk_size
        if self.memory_budget_bytes is not None and self.bytes_per_token > 0:
            free = self.memory_budget_bytes * max(0.0, 1.0 - current_memory_usage)
            size = min(size, int(free // self.bytes_per_token))
        elif current_memory_usage > 0.8:
            size = size // 2
        size = self._aligned(size)
        return seq_len if seq_len <= size else size

    def split_into_chunks(self, token_ids: Sequence[int], current_memory_usage: float = 0.0, cached_tokens: int = 0) -> List[Tuple[int, int, int]]:
        """(start, end, window_start) per chunk; ``cached_tokens`` (a prefix-cache hit) are skipped."""
        n = len(token_ids)
        size = self.compute_optimal_chunk_size(n - cached_tokens, current_memory_usage)
        chunks, start = [], cached_tokens
        while start < n:
            end = min(start + max(size, 1), n)
            window = max(start - self.overlap_size, 0) if (self.overlap_chunks and start > 0) else start
            chunks.append((start, end, window))
            start = end
        s = self.stats
        s["total_requests"] += 1
        s["total_chunks"] += len(chunks)
        s["total_tokens_processed"] += n - cached_tokens
        s["avg_chunk_size"] += ((n - cached_tokens) / max(len(chunks), 1) - s["avg_chunk_size"]) / s["total_requests"]
        s["memory_saved_bytes"] += max(n - cached_tokens - size, 0) * self.bytes_per_token
        return chunks

    def get_stats(self) -> Dict[str, Any]:
        return {**self.stats, "avg_chunk_size": round(self.stats["avg_chunk_size"], 2)}


class PiscesLxChunkedPrefillOperator(PiscesLxOperatorInterface):
    """``action="chunk"`` plans; ``action="prefill"`` also drives ``step_fn(token_chunk, start, state) -> state`` over the
    chunks in order (``state`` is whatever carries the cache; the last state is returned)."""

    name = "chunked_prefill"

    def __init__(self, max_chunk_size: int = 2048, min_chunk_size: int = 256, overlap_chunks: bool = False, overlap_size: int = 128,
                 memory_budget_bytes: Optional[int] = None, bytes_per_token: int = 0, align: int = 128):
        self.scheduler = PiscesLxChunkedPrefillPlanner(max_chunk_size, min_chunk_size, overlap_chunks, overlap_size, memory_budget_bytes, bytes_per_token, align)

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        a = inputs.get("action", "chunk")
        return a == "stats" or ("token_ids" in inputs and (a != "prefill" or callable(inputs.get("step_fn"))))

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        a = inputs.get("action", "chunk")
        if a == "stats":
            return self.scheduler.get_stats()
        if a not in ("chunk", "prefill"):
            raise ValueError(f"Unknown action: {a}")
        ids = inputs["token_ids"]
        chunks = self.scheduler.split_into_chunks(ids, float(inputs.get("current_memory_usage", 0.0)), int(inputs.get("cached_tokens", 0)))
        out = {"chunks": chunks, "chunk_count": len(chunks), "chunk_size": max((e - s for s, e, _ in chunks), default=0), "original_length": len(ids)}
        if a == "prefill":
            step_fn: Callable = inputs["step_fn"]
            state = inputs.get("state")
            for s, e, w in chunks:
                state = step_fn(ids[w:e], w, state)
            out["state"] = state
        return out

    def get_stats(self) -> Dict[str, Any]:
        return self.scheduler.get_stats()
