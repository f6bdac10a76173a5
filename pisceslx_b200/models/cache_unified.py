"""``YvUnifiedCacheManager``: one front for every cache a generation loop touches.

Surface of the reference's manager (model/core/cache.py:1760-2430): per-layer ``get_kv_cache`` / ``update_kv_cache``
over lists of K/V blocks, quantisation of cold blocks (int8 or clamped-fp8 values, :2174-2220), H2O heavy-hitter
selection (:2127-2172), compaction of the oldest blocks by a norm + variance importance score (:1979-2038), eviction
from the front above ``1.5 x max_cache_size`` (:1886-1952), paged sequences, SSM states, speculative drafts with an
acceptance-driven draft length, per-modality caches, a prefix trie, statistics and checkpoint / restore
(:2394-2430).

Design differences.  The reference's per-layer store is lossy by default; here every lossy step is opt-in
(``quantize_cold_blocks``, ``h2o``, ``compact``) and the default configuration returns exactly what was written.
Paged sequences delegate to ``YvPagedKVCache`` (device block pool + host block tables, read by the paged-decode
kernel), the other stores to the specialised managers in ``cache_policies`` / ``cache_extras``; this class adds the
layer-block store and the bookkeeping that ties them together.  All host-side state is guarded by one lock per
layer, so concurrent request handlers can update different layers.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .cache import YvCacheConfig as _PagedConfig
from .cache import YvPagedKVCache
from .cache_extras import YvMultimodalCacheManager, YvPLTTrieIndex
from .cache_policies import YvCacheCompressor, YvH2OSelector, YvSSMCacheManager


@dataclass
class YvUnifiedCacheConfig:
    n_layer: int = 1
    n_kv_head: int = 1
    head_dim: int = 64
    max_cache_size: int = 8192            # tokens per layer before eviction is considered
    block_tokens: int = 256               # a block is closed (and may be quantised) at this many tokens
    quantize_cold_blocks: bool = False    # lossy: closed blocks are stored as int8 (or clamped fp8 values)
    quant_mode: str = "int8"              # "int8" | "fp8"
    h2o: bool = False                     # lossy: keep recent + heavy-hitter tokens only
    h2o_recent: int = 512
    h2o_heavy: int = 512
    compact: bool = False                 # lossy: above the limit, the oldest blocks keep their most important half
    evict_factor: float = 1.5
    paged_blocks: int = 0                 # > 0: also build a paged block pool of this many blocks
    paged_block_size: int = 64
    dtype: torch.dtype = torch.float32
    device: str = "cpu"
    spec_min_draft: int = 2
    spec_max_draft: int = 8


@dataclass
class _Block:
    k: torch.Tensor                       # [B, hk, t, d] (or int8 codes when quantised)
    v: torch.Tensor
    scale_k: Optional[torch.Tensor] = None
    scale_v: Optional[torch.Tensor] = None
    quantized: bool = False
    tokens: int = 0
    created: float = field(default_factory=time.time)


class YvUnifiedCacheManager:
    def __init__(self, config: Any = None, **kw: Any):
        if isinstance(config, dict):
            config = YvUnifiedCacheConfig(**{k: v for k, v in config.items() if k in YvUnifiedCacheConfig.__dataclass_fields__})
        elif config is None:
            config = YvUnifiedCacheConfig(**kw)
        elif not isinstance(config, YvUnifiedCacheConfig):                 # a model config: take what matters
            config = YvUnifiedCacheConfig(n_layer=getattr(config, "n_layer", 1), n_kv_head=getattr(config, "n_kv_head", 1),
                                          head_dim=getattr(config, "head_dim", 64),
                                          max_cache_size=getattr(config, "max_cache_size", 8192), **kw)
        self.cfg = config
        self._layers: Dict[int, List[_Block]] = {}
        self._locks: Dict[int, threading.Lock] = {}
        self._scores: Dict[int, torch.Tensor] = {}          # accumulated attention mass per cached token (H2O)
        self._compressor = YvCacheCompressor("int8")
        self._h2o = YvHeavyHitterState(config.h2o_recent, config.h2o_heavy)
        self.ssm = YvSSMCacheManager()
        self.multimodal = YvMultimodalCacheManager()
        self.prefix = YvPLTTrieIndex(block_size=config.paged_block_size)
        self.paged: Optional[YvPagedKVCache] = None
        if config.paged_blocks > 0:
            self.paged = YvPagedKVCache(config.n_layer, config.n_kv_head, config.head_dim,
                                        _PagedConfig(num_blocks=config.paged_blocks, block_size=config.paged_block_size,
                                                     dtype=config.dtype), torch.device(config.device))
        self._generation: Dict[str, torch.Tensor] = {}
        self._drafts: Dict[int, Dict[str, torch.Tensor]] = {}
        self._accept_history: List[float] = []
        self.stats = {"updates": 0, "hits": 0, "misses": 0, "evicted_tokens": 0, "quantized_blocks": 0,
                      "compacted_tokens": 0, "h2o_dropped_tokens": 0}

    # ---- per-layer K/V ------------------------------------------------------------------------------------
    def _lock(self, layer_idx: int) -> threading.Lock:
        return self._locks.setdefault(layer_idx, threading.Lock())

    def _dense(self, b: _Block) -> Tuple[torch.Tensor, torch.Tensor]:
        if not b.quantized:
            return b.k, b.v
        shp = b.k.shape
        k = self._compressor.decompress(b.k.reshape(-1, shp[-1]), b.scale_k, self.cfg.dtype).reshape(shp)
        v = self._compressor.decompress(b.v.reshape(-1, shp[-1]), b.scale_v, self.cfg.dtype).reshape(shp)
        return k, v

    def get_kv_cache(self, layer_idx: int, past_key_values: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        """``(k, v)`` of shape ``[B, hk, S, d]`` for the layer, or ``past_key_values`` / ``None`` when nothing is stored."""
        with self._lock(layer_idx):
            blocks = self._layers.get(layer_idx)
            if not blocks:
                self.stats["misses"] += 1
                return past_key_values
            self.stats["hits"] += 1
            ks, vs = zip(*(self._dense(b) for b in blocks))
            return torch.cat(ks, dim=2), torch.cat(vs, dim=2)

    def update_kv_cache(self, layer_idx: int, key_states: torch.Tensor, value_states: torch.Tensor,
                        attention_scores: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Append ``[B, hk, t, d]`` keys / values and return the layer's full cache after the configured policies.
        ``attention_scores [B, heads, q, S_total]`` (optional) feeds the heavy-hitter statistics."""
        cfg = self.cfg
        with self._lock(layer_idx):
            blocks = self._layers.setdefault(layer_idx, [])
            self.stats["updates"] += 1
            k, v = key_states.detach(), value_states.detach()
            while k.shape[2] > 0:
                if not blocks or blocks[-1].quantized or blocks[-1].tokens >= cfg.block_tokens:
                    blocks.append(_Block(k[:, :, :0], v[:, :, :0]))
                last = blocks[-1]
                take = min(cfg.block_tokens - last.tokens, k.shape[2])
                last.k = torch.cat([last.k, k[:, :, :take]], dim=2)
                last.v = torch.cat([last.v, v[:, :, :take]], dim=2)
                last.tokens += take
                k, v = k[:, :, take:], v[:, :, take:]
                if last.tokens >= cfg.block_tokens and cfg.quantize_cold_blocks:
                    self._quantize_block(last)
            if attention_scores is not None:
                self._accumulate_scores(layer_idx, attention_scores)
            total = sum(b.tokens for b in blocks)
            if cfg.h2o and total > cfg.h2o_recent + cfg.h2o_heavy:
                self._apply_h2o(layer_idx)
            total = sum(b.tokens for b in blocks)
            if total > int(cfg.evict_factor * cfg.max_cache_size):
                if cfg.compact:
                    self._compact_blocks(layer_idx)
                self._evict_front(layer_idx)
        return self.get_kv_cache(layer_idx)

    # ---- policies (all opt-in) ----------------------------------------------------------------------------
    def _quantize_block(self, b: _Block) -> None:
        if b.quantized or b.tokens == 0:
            return
        d = b.k.shape[-1]
        if self.cfg.quant_mode == "fp8":
            # the reference's fp8 path scales into the e4m3 range, clamps and keeps the input dtype (:2188-2205)
            for name in ("k", "v"):
                t = getattr(b, name)
                s = t.abs().amax().clamp_min(1e-12) / 448.0
                q = (t / s).clamp(-448, 448)
                if hasattr(torch, "float8_e4m3fn"):
                    q = q.to(torch.float8_e4m3fn).to(t.dtype)
                setattr(b, name, q * s)
        else:
            qk, sk = self._compressor.compress(b.k.reshape(-1, d).float())
            qv, sv = self._compressor.compress(b.v.reshape(-1, d).float())
            b.k, b.v, b.scale_k, b.scale_v = qk.reshape(b.k.shape), qv.reshape(b.v.shape), sk, sv
            b.quantized = True
        self.stats["quantized_blocks"] += 1

    def _accumulate_scores(self, layer_idx: int, attn: torch.Tensor) -> None:
        mass = attn.detach().float().sum(dim=(0, 1, 2))                    # [S_total]
        old = self._scores.get(layer_idx)
        if old is None or old.numel() > mass.numel():
            old = torch.zeros(0)
        pad = torch.zeros(mass.numel() - old.numel())
        self._scores[layer_idx] = torch.cat([old, pad]) + mass.cpu()

    def _calculate_importance_scores(self, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """Per-token importance of a block: key norm plus value variance over the head dimension, averaged over batch
        and heads (reference :2160-2172)."""
        return (k.float().norm(dim=-1) + v.float().var(dim=-1, unbiased=False)).mean(dim=(0, 1))

    def _rebuild(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor) -> None:
        bt = self.cfg.block_tokens
        blocks = []
        for s in range(0, k.shape[2], bt):
            kk, vv = k[:, :, s:s + bt], v[:, :, s:s + bt]
            blocks.append(_Block(kk, vv, tokens=kk.shape[2]))
        self._layers[layer_idx] = blocks
        if self.cfg.quantize_cold_blocks:
            for b in blocks[:-1]:
                self._quantize_block(b)

    def _apply_h2o(self, layer_idx: int) -> None:
        blocks = self._layers[layer_idx]
        ks, vs = zip(*(self._dense(b) for b in blocks))
        k, v = torch.cat(ks, dim=2), torch.cat(vs, dim=2)
        S = k.shape[2]
        scores = self._scores.get(layer_idx)
        if scores is None or scores.numel() != S:
            scores = self._calculate_importance_scores(k, v).cpu()
        keep = self._h2o.select(scores)
        self.stats["h2o_dropped_tokens"] += S - keep.numel()
        self._scores[layer_idx] = scores[keep]
        self._rebuild(layer_idx, k[:, :, keep.to(k.device)], v[:, :, keep.to(k.device)])

    def _compact_blocks(self, layer_idx: int) -> None:
        """The older half of the blocks keep the more important half of their tokens, in order."""
        blocks = self._layers[layer_idx]
        n_old = len(blocks) // 2
        for b in blocks[:n_old]:
            k, v = self._dense(b)
            keep_n = max(k.shape[2] // 2, 1)
            idx = self._calculate_importance_scores(k, v).topk(keep_n).indices.sort().values
            self.stats["compacted_tokens"] += k.shape[2] - keep_n
            b.k, b.v, b.tokens, b.quantized, b.scale_k, b.scale_v = k[:, :, idx], v[:, :, idx], keep_n, False, None, None
        self._scores.pop(layer_idx, None)

    def _evict_front(self, layer_idx: int) -> None:
        blocks = self._layers[layer_idx]
        total = sum(b.tokens for b in blocks)
        while len(blocks) > 1 and total > self.cfg.max_cache_size:
            b = blocks.pop(0)
            total -= b.tokens
            self.stats["evicted_tokens"] += b.tokens
            sc = self._scores.get(layer_idx)
            if sc is not None:
                self._scores[layer_idx] = sc[b.tokens:]

    def compress_cache(self, layer_idx: Optional[int] = None) -> int:
        """Quantise every closed block now (returns how many were converted)."""
        n = 0
        for li in ([layer_idx] if layer_idx is not None else list(self._layers)):
            with self._lock(li):
                for b in self._layers.get(li, [])[:-1]:
                    if not b.quantized and self.cfg.quant_mode == "int8":
                        self._quantize_block(b)
                        n += 1
        return n

    # ---- paged sequences (exact; read by the paged-decode kernel) ---------------------------------------
    def _need_paged(self) -> YvPagedKVCache:
        if self.paged is None:
            raise RuntimeError("built without a paged pool (paged_blocks = 0)")
        return self.paged

    def allocate_paged_sequence(self, seq_id: int, initial_blocks: int = 1) -> bool:
        p = self._need_paged()
        if p.alloc.available() < initial_blocks:
            return False
        p.add_sequence(seq_id)
        return True

    def append_paged(self, seq_id: int, layer_idx: int, k: torch.Tensor, v: torch.Tensor) -> bool:
        """k, v ``[t, hk, d]``.  Slots are reserved when layer 0 appends; the other layers write the same slots."""
        p = self._need_paged()
        t = k.shape[0]
        if layer_idx == 0:
            if not p.can_append(seq_id, t):
                return False
            self._slots = {seq_id: p.append_slots(seq_id, t)}
        slots = torch.tensor(self._slots[seq_id][-t:], dtype=torch.long, device=k.device)
        kc, vc = p.layer(layer_idx)
        kc.view(-1, p.hk, p.d)[slots] = k.to(kc.dtype)
        vc.view(-1, p.hk, p.d)[slots] = v.to(vc.dtype)
        return True

    def read_paged(self, seq_id: int, layer_idx: int) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        p = self._need_paged()
        if seq_id not in p.tables:
            return None
        n, bs = p.lengths[seq_id], p.cfg.block_size
        idx = torch.tensor([p.tables[seq_id][i // bs] * bs + i % bs for i in range(n)], dtype=torch.long, device=p.device)
        kc, vc = p.layer(layer_idx)
        return kc.view(-1, p.hk, p.d)[idx], vc.view(-1, p.hk, p.d)[idx]

    def free_paged_sequence(self, seq_id: int) -> None:
        self._need_paged().free_sequence(seq_id)

    # ---- other stores ---------------------------------------------------------------------------------------
    def get_ssm_state(self, layer_idx: int, seq_id: Optional[int] = None, init=None) -> Optional[torch.Tensor]:
        st = self.ssm.get(seq_id or 0, layer_idx, init or (lambda: {"state": None}))
        return st.get("state")

    def update_ssm_state(self, layer_idx: int, state: torch.Tensor, seq_id: Optional[int] = None) -> None:
        self.ssm.get(seq_id or 0, layer_idx, lambda: {"state": None})["state"] = state.detach()

    def get_generation_cache(self, modality: str) -> Optional[torch.Tensor]:
        return self._generation.get(modality)

    def set_generation_cache(self, modality: str, cache_data: torch.Tensor) -> None:
        self._generation[modality] = cache_data

    def store_speculative_draft(self, draft_length: int, tokens: torch.Tensor, probs: Optional[torch.Tensor] = None,
                                accepted: Optional[int] = None) -> None:
        self._drafts[draft_length] = {"tokens": tokens, **({"probs": probs} if probs is not None else {})}
        if accepted is not None and draft_length > 0:
            self._accept_history.append(accepted / draft_length)
            del self._accept_history[:-64]

    def get_speculative_draft(self, draft_length: int) -> Optional[Dict[str, torch.Tensor]]:
        return self._drafts.get(draft_length)

    def get_optimal_draft_length(self) -> int:
        """Longer drafts while they are being accepted, shorter when they are not (mean acceptance of the last drafts)."""
        lo, hi = self.cfg.spec_min_draft, self.cfg.spec_max_draft
        if not self._accept_history:
            return (lo + hi) // 2
        a = sum(self._accept_history) / len(self._accept_history)
        return int(round(lo + (hi - lo) * a))

    def store_multimodal_cache(self, modality: str, cache_key: str, cache_data: torch.Tensor) -> None:
        from collections import OrderedDict
        self.multimodal.store.setdefault(modality, OrderedDict())[cache_key] = cache_data

    def get_multimodal_cache(self, modality: str, cache_key: str) -> Optional[torch.Tensor]:
        return self.multimodal.store.get(modality, {}).get(cache_key)

    def insert_plt_prefix(self, token_ids: Sequence[int], log_probs: Sequence[float], block_ids: Sequence[int]) -> None:
        self.prefix.insert(token_ids, log_probs, block_ids)

    def find_plt_prefix_match(self, token_ids: Sequence[int], context_log_probs: Optional[Sequence[float]] = None):
        return self.prefix.find_longest_match(token_ids, context_log_probs)

    # ---- bookkeeping --------------------------------------------------------------------------------------
    def clear_cache(self) -> None:
        for li in list(self._layers):
            with self._lock(li):
                self._layers[li] = []
        self._scores.clear()
        self._generation.clear()
        self._drafts.clear()

    def get_cache_stats(self) -> Dict[str, Any]:
        tokens = {li: sum(b.tokens for b in bl) for li, bl in self._layers.items()}
        nbytes = sum(b.k.numel() * b.k.element_size() + b.v.numel() * b.v.element_size()
                     for bl in self._layers.values() for b in bl)
        looked = self.stats["hits"] + self.stats["misses"]
        out = dict(self.stats, tokens_per_layer=tokens, bytes=nbytes, hit_rate=self.stats["hits"] / looked if looked else 0.0,
                   optimal_draft_length=self.get_optimal_draft_length())
        if self.paged is not None:
            out["paged_free_blocks"] = self.paged.alloc.available()
        return out

    def create_checkpoint(self) -> Dict[str, Any]:
        layers = {li: [(self._dense(b)[0].clone(), self._dense(b)[1].clone()) for b in bl] for li, bl in self._layers.items()}
        return {"layers": layers, "scores": {k: v.clone() for k, v in self._scores.items()}, "stats": dict(self.stats),
                "paged": self.paged.state() if self.paged is not None else None, "accept": list(self._accept_history)}

    def restore_checkpoint(self, checkpoint: Dict[str, Any]) -> None:
        self._layers = {int(li): [_Block(k.clone(), v.clone(), tokens=k.shape[2]) for k, v in bl]
                        for li, bl in checkpoint["layers"].items()}
        self._scores = {int(k): v.clone() for k, v in checkpoint.get("scores", {}).items()}
        self.stats.update(checkpoint.get("stats", {}))
        self._accept_history = list(checkpoint.get("accept", []))
        if checkpoint.get("paged") is not None and self.paged is not None:
            self.paged.load_state(checkpoint["paged"])


class YvHeavyHitterState(YvH2OSelector):
    """Heavy-hitter selection with the newest tokens always kept (indices returned in order)."""
