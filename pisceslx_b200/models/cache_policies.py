"""Cache management policies around the exact paged KV cache (reference model/core/cache.py:
``YvPagedCacheManager`` LRU / LFU / importance eviction :535-868, ``YvSSMCacheManager`` :871,
``YvSpeculativeCacheManager`` :1040, ``YvCacheCompressor`` :1404, H2O selection and compaction in
``YvUnifiedCacheManager`` :1760-2430).

The reference's cache drops or merges tokens by default.  Here the paged cache stays exact and every lossy policy is
an explicit, opt-in object that decides WHICH sequences or blocks to give up; the block pool itself
(``models.cache.YvPagedKVCache``) is untouched by them."""
from __future__ import annotations

import time
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

import torch


@dataclass
class _Entry:
    last_use: float = 0.0
    uses: int = 0
    importance: float = 0.0
    blocks: int = 0


class YvEvictionPolicy:
    """Chooses which cached sequence to drop when the pool runs dry: ``lru`` | ``lfu`` | ``importance``."""

    def __init__(self, kind: str = "lru"):
        assert kind in ("lru", "lfu", "importance")
        self.kind = kind
        self.entries: Dict[int, _Entry] = {}
        self._clock = 0.0

    def touch(self, seq_id: int, blocks: int = 0, importance: Optional[float] = None) -> None:
        self._clock += 1.0
        e = self.entries.setdefault(seq_id, _Entry())
        e.last_use, e.uses, e.blocks = self._clock, e.uses + 1, blocks or e.blocks
        if importance is not None:
            e.importance = importance

    def remove(self, seq_id: int) -> None:
        self.entries.pop(seq_id, None)

    def victim(self, protect: Iterable[int] = ()) -> Optional[int]:
        cand = [(s, e) for s, e in self.entries.items() if s not in set(protect)]
        if not cand:
            return None
        key = {"lru": lambda se: se[1].last_use, "lfu": lambda se: (se[1].uses, se[1].last_use),
               "importance": lambda se: (se[1].importance, se[1].last_use)}[self.kind]
        return min(cand, key=key)[0]


class YvPagedCacheManager:
    """Admission with eviction on top of ``YvPagedKVCache``: ``reserve`` frees victims until the request fits."""

    def __init__(self, cache, policy: Optional[YvEvictionPolicy] = None):
        self.cache, self.policy = cache, policy or YvEvictionPolicy("lru")
        self.evicted: List[int] = []

    def reserve(self, seq_id: int, n_tokens: int, protect: Iterable[int] = ()) -> bool:
        if seq_id not in self.cache.tables:
            self.cache.add_sequence(seq_id)
        protect = set(protect) | {seq_id}
        while not self.cache.can_append(seq_id, n_tokens):
            v = self.policy.victim(protect)
            if v is None:
                return False
            self.cache.free_sequence(v)
            self.policy.remove(v)
            self.evicted.append(v)
        self.policy.touch(seq_id, len(self.cache.tables[seq_id]))
        return True


class YvH2OSelector:
    """Heavy-hitter selection of which token positions to keep: the ``recent`` newest plus the ``heavy`` positions
    with the largest accumulated attention mass."""

    def __init__(self, recent: int, heavy: int):
        self.recent, self.heavy = recent, heavy

    def select(self, acc_scores: torch.Tensor) -> torch.Tensor:
        """acc_scores [T] -> sorted indices of the positions kept."""
        T = acc_scores.numel()
        if T <= self.recent + self.heavy:
            return torch.arange(T, device=acc_scores.device)
        older = acc_scores[: T - self.recent]
        keep = torch.cat([older.topk(self.heavy).indices, torch.arange(T - self.recent, T, device=acc_scores.device)])
        return keep.sort().values


class YvCacheCompressor:
    """Per-token symmetric quantisation of cache rows (int8 or fp8 e4m3) with one fp32 scale per row."""

    def __init__(self, mode: str = "int8"):
        assert mode in ("int8", "fp8")
        self.mode = mode

    def compress(self, rows: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        amax = rows.float().abs().amax(-1, keepdim=True).clamp_min(1e-12)
        if self.mode == "int8":
            s = amax / 127.0
            return torch.round(rows.float() / s).clamp(-127, 127).to(torch.int8), s
        s = amax / 448.0
        return (rows.float() / s).to(torch.float8_e4m3fn), s

    def decompress(self, q: torch.Tensor, s: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
        return (q.float() * s).to(dtype)

    def ratio(self, dtype=torch.bfloat16, row: int = 1024) -> float:
        return (row * torch.empty(0, dtype=dtype).element_size()) / (row + 4)


class YvSSMCacheManager:
    """Recurrent state per sequence and layer (SSM state + convolution window) for the state-space branch."""

    def __init__(self):
        self.states: Dict[Tuple[int, int], Dict[str, torch.Tensor]] = {}

    def get(self, seq_id: int, layer: int, init) -> Dict[str, torch.Tensor]:
        key = (seq_id, layer)
        if key not in self.states:
            self.states[key] = init()
        return self.states[key]

    def free(self, seq_id: int) -> None:
        for k in [k for k in self.states if k[0] == seq_id]:
            del self.states[k]

    def fork(self, src: int, dst: int) -> None:
        for (s, l), st in list(self.states.items()):
            if s == src:
                self.states[(dst, l)] = {k: v.clone() for k, v in st.items()}


class YvSpeculativeCacheManager:
    """Draft / verify bookkeeping: remember the committed length before drafting and roll back the rejected tail."""

    def __init__(self, cache):
        self.cache = cache
        self.marks: Dict[int, int] = {}

    def mark(self, seq_id: int) -> None:
        self.marks[seq_id] = self.cache.lengths[seq_id]

    def rollback(self, seq_id: int, accepted: int) -> None:
        """Keep ``accepted`` of the tokens appended since ``mark``; whole blocks past the new end go back to the pool."""
        new_len = self.marks[seq_id] + accepted
        bs = self.cache.cfg.block_size
        need = (new_len + bs - 1) // bs
        table = self.cache.tables[seq_id]
        while len(table) > need:
            self.cache.alloc.release(table.pop())
        self.cache.lengths[seq_id] = new_len


class YvPrefixCache:
    """Hash-of-block-contents index: requests that share a token prefix share its KV blocks (reference
    opss/infer/vllm.py prefix cache).  Blocks are reference-counted through the pool's ``share``."""

    def __init__(self, cache):
        self.cache = cache
        self.index: "OrderedDict[Tuple[int, ...], int]" = OrderedDict()
        self.hits = self.misses = 0

    def _keys(self, tokens: List[int]) -> List[Tuple[int, ...]]:
        bs = self.cache.cfg.block_size
        return [tuple(tokens[: (i + 1) * bs]) for i in range(len(tokens) // bs)]

    def match(self, seq_id: int, tokens: List[int]) -> int:
        """Attach the longest cached prefix to ``seq_id``; returns the number of tokens covered."""
        if seq_id not in self.cache.tables:
            self.cache.add_sequence(seq_id)
        covered = 0
        for key in self._keys(tokens):
            blk = self.index.get(key)
            if blk is None:
                self.misses += 1
                break
            self.cache.tables[seq_id].append(self.cache.alloc.share(blk))
            covered = len(key)
            self.hits += 1
        self.cache.lengths[seq_id] = covered
        return covered

    def publish(self, seq_id: int, tokens: List[int]) -> None:
        """Index the full blocks of a prefilled sequence (the index holds its own reference on each block)."""
        for i, key in enumerate(self._keys(tokens)):
            if key not in self.index and i < len(self.cache.tables[seq_id]):
                self.index[key] = self.cache.alloc.share(self.cache.tables[seq_id][i])

    def evict(self, n: int = 1) -> None:
        for _ in range(min(n, len(self.index))):
            _, blk = self.index.popitem(last=False)
            self.cache.alloc.release(blk)
