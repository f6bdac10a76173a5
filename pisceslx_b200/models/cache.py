"""Paged KV cache.

The reference keeps Python lists of per-layer block objects and concatenates them on every read
(model/core/cache.py:535-868, read path :824-835); its unified manager is lossy by default (H2O,
quantisation, eviction; cache.py:1886-2038).  Here the cache is two device tensors per layer
``[num_blocks, block_size, n_kv_head, head_dim]`` plus an int32 block table per sequence; the decode kernel
reads pages in place.  The cache is exact; eviction policies (LRU of whole sequences, sliding window)
are opt-in helpers that only edit block tables.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


@dataclass
class YvCacheConfig:
    block_size: int = 64
    num_blocks: int = 1024
    max_blocks_per_seq: int = 2048
    dtype: torch.dtype = torch.bfloat16
    sliding_window: Optional[int] = None      # keep only the last N tokens addressable (opt-in, lossy)


class YvBlockAllocator:
    """Free-list allocator of cache pages with reference counts (prefix sharing)."""

    def __init__(self, num_blocks: int):
        self.num_blocks = num_blocks
        self.free: List[int] = list(range(num_blocks - 1, -1, -1))
        self.refs: Dict[int, int] = {}

    def available(self) -> int:
        return len(self.free)

    def alloc(self) -> int:
        if not self.free:
            raise MemoryError("paged KV cache is out of blocks")
        b = self.free.pop()
        self.refs[b] = 1
        return b

    def share(self, b: int) -> int:
        self.refs[b] += 1
        return b

    def release(self, b: int) -> None:
        self.refs[b] -= 1
        if self.refs[b] == 0:
            del self.refs[b]
            self.free.append(b)


class YvPagedKVCache:
    """Block pool for all layers of one model replica plus per-sequence block tables (host side)."""

    def __init__(self, n_layer: int, n_kv_head: int, head_dim: int, cfg: YvCacheConfig, device: torch.device):
        self.cfg, self.device = cfg, device
        self.n_layer, self.hk, self.d = n_layer, n_kv_head, head_dim
        shape = (cfg.num_blocks, cfg.block_size, n_kv_head, head_dim)
        self.k = [torch.zeros(shape, dtype=cfg.dtype, device=device) for _ in range(n_layer)]
        self.v = [torch.zeros(shape, dtype=cfg.dtype, device=device) for _ in range(n_layer)]
        self.alloc = YvBlockAllocator(cfg.num_blocks)
        self.tables: Dict[int, List[int]] = {}       # seq id -> physical blocks
        self.lengths: Dict[int, int] = {}
        self.layer_offset = 0                         # first global layer index held by this pipeline stage

    def layer(self, idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.k[idx - self.layer_offset], self.v[idx - self.layer_offset]

    def bytes(self) -> int:
        return 2 * self.n_layer * self.k[0].numel() * self.k[0].element_size()

    # ---- sequence management (host) ---------------------------------------------------------------
    def add_sequence(self, seq_id: int) -> None:
        self.tables[seq_id] = []
        self.lengths[seq_id] = 0

    def free_sequence(self, seq_id: int) -> None:
        for b in self.tables.pop(seq_id, []):
            self.alloc.release(b)
        self.lengths.pop(seq_id, None)

    def fork(self, src: int, dst: int) -> None:
        """Share all full blocks of ``src`` with ``dst`` (prefix caching / beam search)."""
        self.tables[dst] = [self.alloc.share(b) for b in self.tables[src]]
        self.lengths[dst] = self.lengths[src]

    def can_append(self, seq_id: int, n_tokens: int) -> bool:
        need = self._blocks_needed(seq_id, n_tokens)
        return need <= self.alloc.available()

    def _blocks_needed(self, seq_id: int, n_tokens: int) -> int:
        bs = self.cfg.block_size
        have = len(self.tables[seq_id])
        total = (self.lengths[seq_id] + n_tokens + bs - 1) // bs
        return max(0, total - have)

    def append_slots(self, seq_id: int, n_tokens: int) -> List[int]:
        """Reserve room for ``n_tokens`` new tokens; returns their flat slot ids (block * block_size + offset)."""
        bs = self.cfg.block_size
        for _ in range(self._blocks_needed(seq_id, n_tokens)):
            self.tables[seq_id].append(self.alloc.alloc())
        start = self.lengths[seq_id]
        tbl = self.tables[seq_id]
        slots = [tbl[(start + i) // bs] * bs + (start + i) % bs for i in range(n_tokens)]
        self.lengths[seq_id] = start + n_tokens
        return slots

    def block_table_tensor(self, seq_ids: List[int], width: Optional[int] = None) -> torch.Tensor:
        width = width or max(1, max(len(self.tables[s]) for s in seq_ids))
        t = torch.zeros(len(seq_ids), width, dtype=torch.int32)
        for i, s in enumerate(seq_ids):
            tbl = self.tables[s]
            if self.cfg.sliding_window is not None:
                keep = (self.cfg.sliding_window + self.cfg.block_size - 1) // self.cfg.block_size + 1
                tbl = tbl[-keep:]
            t[i, : len(tbl)] = torch.tensor(tbl, dtype=torch.int32)
        return t.to(self.device, non_blocking=True)

    def seq_lens_tensor(self, seq_ids: List[int]) -> torch.Tensor:
        return torch.tensor([self.lengths[s] for s in seq_ids], dtype=torch.int32).to(self.device, non_blocking=True)

    # ---- checkpoint / restore (reference cache.py:2394-2430) ------------------------------------------------
    def state(self) -> Dict[str, object]:
        return {"tables": {k: list(v) for k, v in self.tables.items()}, "lengths": dict(self.lengths),
                "k": [t.cpu() for t in self.k], "v": [t.cpu() for t in self.v]}

    def load_state(self, st: Dict[str, object]) -> None:
        self.tables = {int(k): list(v) for k, v in st["tables"].items()}      # type: ignore[union-attr]
        self.lengths = {int(k): int(v) for k, v in st["lengths"].items()}     # type: ignore[union-attr]
        used = {b for t in self.tables.values() for b in t}
        self.alloc = YvBlockAllocator(self.cfg.num_blocks)
        self.alloc.free = [b for b in range(self.cfg.num_blocks - 1, -1, -1) if b not in used]
        self.alloc.refs = {b: sum(b in t for t in self.tables.values()) for b in used}
        for i in range(self.n_layer):
            self.k[i].copy_(st["k"][i])                                        # type: ignore[index]
            self.v[i].copy_(st["v"][i])                                        # type: ignore[index]


def cache_for_model(cfg, device: torch.device, num_blocks: int, block_size: Optional[int] = None, tp_size: int = 1,
                    n_layer: Optional[int] = None, dtype: torch.dtype = torch.bfloat16) -> YvPagedKVCache:
    cc = YvCacheConfig(block_size=block_size or cfg.kv_cache_block_size, num_blocks=num_blocks, dtype=dtype)
    return YvPagedKVCache(n_layer or cfg.n_layer, cfg.n_kv_head // tp_size, cfg.head_dim, cc, device)
