"""Further KV-cache components (reference model/core/cache.py: ``YvMultimodalCacheManager`` :1248, ``YvKVCacheRing``
:2433, ``YvLynxKVQuantizer`` :2480, ``YvSTARKVAdapter`` :2561; model/core/predictive_delta.py:65
``YvPredictiveDeltaCoder``; model/core/plt_trie.py:94 ``YvPLTTrieIndex``).

The serving engine's cache is the paged pool of ``models.cache`` read by the paged-decode kernels; the classes here
are the reference's auxiliary policies around a cache, kept host-side and allocation-light."""
from __future__ import annotations

import math
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F_
from ..quant.extras import PiscesLxSTARKVQuantizer


class YvKVCacheRing:
    """Preallocated, geometrically growing K/V buffer: appends are ``copy_`` into place instead of ``torch.cat`` per
    step.  With ``max_seq_len`` set it becomes a true ring that overwrites the oldest tokens."""

    def __init__(self, grow_factor: float = 2.0, max_seq_len: int = 0, initial: int = 256):
        self.k_buf: Optional[torch.Tensor] = None
        self.v_buf: Optional[torch.Tensor] = None
        self.pos, self.total = 0, 0
        self.grow, self.max_len, self.initial = grow_factor, max_seq_len, initial
        self.reallocations = 0

    def _ensure(self, k: torch.Tensor, need: int) -> None:
        cap = 0 if self.k_buf is None else self.k_buf.shape[-2]
        if need <= cap:
            return
        new_cap = max(need, int(max(cap, self.initial // 2) * self.grow))
        if self.max_len:
            new_cap = min(new_cap, self.max_len)
        shape = (*k.shape[:-2], new_cap, k.shape[-1])
        nk, nv = k.new_empty(shape), k.new_empty(shape)
        if self.k_buf is not None:
            nk[..., :cap, :].copy_(self.k_buf)
            nv[..., :cap, :].copy_(self.v_buf)
        self.k_buf, self.v_buf = nk, nv
        self.reallocations += 1

    def append(self, k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """k, v [..., n, D]; returns views of everything held, oldest first."""
        n = k.shape[-2]
        if self.max_len and self.pos + n > self.max_len:
            self._ensure(k, self.max_len)
            # wrap: write token by chunk at pos % max_len
            for i in range(n):
                j = (self.total + i) % self.max_len
                self.k_buf[..., j, :].copy_(k[..., i, :])
                self.v_buf[..., j, :].copy_(v[..., i, :])
            self.total += n
            self.pos = min(self.total, self.max_len)
            start = self.total % self.max_len
            order = torch.arange(start, start + self.max_len, device=k.device) % self.max_len
            return self.k_buf.index_select(-2, order), self.v_buf.index_select(-2, order)
        self._ensure(k, self.pos + n)
        self.k_buf[..., self.pos:self.pos + n, :].copy_(k)
        self.v_buf[..., self.pos:self.pos + n, :].copy_(v)
        self.pos += n
        self.total += n
        return self.k_buf[..., :self.pos, :], self.v_buf[..., :self.pos, :]

    def reset(self) -> None:
        self.pos = self.total = 0


class YvLynxKVQuantizer:
    """Anchor + residual split: a low-bit anchor stream (``anchor_bits`` per value, per-token scale) is usable at
    once; a residual stream quantised at ``residual_bits`` refines it when the entry is reused."""

    def __init__(self, anchor_bits: int = 4, residual_bits: int = 4):
        self.ab, self.rb = anchor_bits, residual_bits

    @staticmethod
    def _q(x: torch.Tensor, bits: int) -> Tuple[torch.Tensor, torch.Tensor]:
        qmax = 2 ** (bits - 1) - 1
        s = x.abs().amax(-1, keepdim=True).clamp_min(1e-8) / qmax
        return torch.round(x / s).clamp(-qmax - 1, qmax).to(torch.int8), s

    def encode(self, kv: torch.Tensor) -> Dict[str, torch.Tensor]:
        x = kv.float()
        a, sa = self._q(x, self.ab)
        r, sr = self._q(x - a.float() * sa, self.rb)
        return {"anchor": a, "anchor_scale": sa, "residual": r, "residual_scale": sr}

    @staticmethod
    def decode(c: Dict[str, torch.Tensor], refine: bool = True, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        x = c["anchor"].float() * c["anchor_scale"]
        if refine:
            x = x + c["residual"].float() * c["residual_scale"]
        return x.to(dtype)


class YvPredictiveDeltaCoder(nn.Module):
    """Stores the quantised residual between the actual compressed-KV vector and a prediction from the previous
    hidden state.  ``warmup`` mode predicts with the previous vector (no parameters)."""

    def __init__(self, hidden: int, kv_rank: int, bottleneck: int = 0, bits: int = 4, warmup: bool = False):
        super().__init__()
        self.bits, self.warmup = bits, warmup
        if bottleneck:
            self.w1 = nn.Parameter(torch.empty(bottleneck, hidden).normal_(std=0.02))
            self.w2 = nn.Parameter(torch.zeros(kv_rank, bottleneck))
        else:
            self.w1, self.w2 = None, nn.Parameter(torch.zeros(kv_rank, hidden))

    def predict(self, prev_hidden: torch.Tensor, prev_kv: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.warmup:
            return prev_kv if prev_kv is not None else prev_hidden.new_zeros(*prev_hidden.shape[:-1], self.w2.shape[0])
        h = prev_hidden
        if self.w1 is not None:
            h = torch.relu(F_.linear(h, self.w1.to(h.dtype)))
        return F_.linear(h, self.w2.to(h.dtype))

    def encode(self, kv: torch.Tensor, prev_hidden: torch.Tensor, prev_kv: Optional[torch.Tensor] = None):
        resid = kv.float() - self.predict(prev_hidden, prev_kv).float()
        qmax = 2 ** (self.bits - 1) - 1
        s = resid.abs().amax(-1, keepdim=True).clamp_min(1e-8) / qmax
        return torch.round(resid / s).clamp(-qmax - 1, qmax).to(torch.int8), s

    def decode(self, q: torch.Tensor, scale: torch.Tensor, prev_hidden: torch.Tensor,
               prev_kv: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.predict(prev_hidden, prev_kv).float() + q.float() * scale

    def training_loss(self, kv: torch.Tensor, prev_hidden: torch.Tensor) -> torch.Tensor:
        return (kv.float() - self.predict(prev_hidden).float()).pow(2).mean()


class YvDeltaCacheEntry:
    """One delta-coded block of keys / values: the quantised residuals and their scales, and (optionally) the predictions
    that were subtracted, so that the block can be rebuilt without the predictor (reference model/core/
    predictive_delta.py:443-510).  With ``pack=True`` residuals of 4 bits or fewer are held two per byte; ``residual_k`` /
    ``residual_v`` always return int8 codes."""

    def __init__(self, residual_k: torch.Tensor, residual_v: torch.Tensor, scale_k: torch.Tensor, scale_v: torch.Tensor,
                 pred_k: Optional[torch.Tensor] = None, pred_v: Optional[torch.Tensor] = None, pack: bool = False):
        self._packed = bool(pack) and residual_k.shape[-1] % 2 == 0 and residual_v.shape[-1] % 2 == 0
        self._rk = self._pack(residual_k) if self._packed else residual_k
        self._rv = self._pack(residual_v) if self._packed else residual_v
        self.scale_k, self.scale_v, self.pred_k, self.pred_v = scale_k, scale_v, pred_k, pred_v

    @staticmethod
    def _pack(q: torch.Tensor) -> torch.Tensor:
        u = (q.to(torch.int16) & 0xF).to(torch.uint8)
        return u[..., 0::2] | (u[..., 1::2] << 4)

    @staticmethod
    def _unpack(p: torch.Tensor) -> torch.Tensor:
        lo, hi = (p & 0xF).to(torch.int8), (p >> 4).to(torch.int8)
        lo, hi = torch.where(lo > 7, lo - 16, lo), torch.where(hi > 7, hi - 16, hi)
        return torch.stack([lo, hi], -1).flatten(-2)

    @property
    def residual_k(self) -> torch.Tensor:
        return self._unpack(self._rk) if self._packed else self._rk

    @property
    def residual_v(self) -> torch.Tensor:
        return self._unpack(self._rv) if self._packed else self._rv

    @classmethod
    def encode(cls, coder_k: "YvPredictiveDeltaCoder", coder_v: "YvPredictiveDeltaCoder", k: torch.Tensor, v: torch.Tensor,
               prev_hidden: torch.Tensor, prev_k: Optional[torch.Tensor] = None, prev_v: Optional[torch.Tensor] = None,
               keep_predictions: bool = False) -> "YvDeltaCacheEntry":
        qk, sk = coder_k.encode(k, prev_hidden, prev_k)
        qv, sv = coder_v.encode(v, prev_hidden, prev_v)
        pk = coder_k.predict(prev_hidden, prev_k).detach() if keep_predictions else None
        pv = coder_v.predict(prev_hidden, prev_v).detach() if keep_predictions else None
        return cls(qk, qv, sk, sv, pk, pv, pack=max(coder_k.bits, coder_v.bits) <= 4)

    def decode(self, coder_k: Optional["YvPredictiveDeltaCoder"] = None, coder_v: Optional["YvPredictiveDeltaCoder"] = None,
               prev_hidden: Optional[torch.Tensor] = None, prev_k: Optional[torch.Tensor] = None, prev_v: Optional[torch.Tensor] = None):
        """(k, v): from the stored predictions when they were kept, else from the predictors and ``prev_hidden``."""
        if self.pred_k is not None and self.pred_v is not None:
            return (self.pred_k.float() + self.residual_k.float() * self.scale_k, self.pred_v.float() + self.residual_v.float() * self.scale_v)
        if coder_k is None or coder_v is None or prev_hidden is None:
            raise ValueError("the predictions were not kept: the predictors and prev_hidden are needed to decode")
        return (coder_k.decode(self.residual_k, self.scale_k, prev_hidden, prev_k), coder_v.decode(self.residual_v, self.scale_v, prev_hidden, prev_v))

    @property
    def num_tokens(self) -> int:
        r = self._rk
        return r.shape[-2] if r.dim() >= 2 else 1

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self._rk, self._rv, self.scale_k, self.scale_v, self.pred_k, self.pred_v) if t is not None)

    def _map(self, fn) -> "YvDeltaCacheEntry":
        e = object.__new__(YvDeltaCacheEntry)
        e._packed = self._packed
        e._rk, e._rv, e.scale_k, e.scale_v = fn(self._rk), fn(self._rv), fn(self.scale_k), fn(self.scale_v)
        e.pred_k = fn(self.pred_k) if self.pred_k is not None else None
        e.pred_v = fn(self.pred_v) if self.pred_v is not None else None
        return e

    def to(self, device) -> "YvDeltaCacheEntry":
        return self._map(lambda t: t.to(device))

    def detach(self) -> "YvDeltaCacheEntry":
        return self._map(lambda t: t.detach())

    def clone(self) -> "YvDeltaCacheEntry":
        return self._map(lambda t: t.clone())


@dataclass
class _TrieNode:
    children: Dict[int, "_TrieNode"] = field(default_factory=dict)
    logp: float = 0.0               # cumulative log2-probability of the path
    block_id: Optional[int] = None  # cache block whose last token is this node
    refs: int = 0
    stamp: int = 0


class YvPLTTrieIndex:
    """Prefix trie over processed token sequences, weighted by the model's own probabilities.  Exact shared prefixes
    always match; a diverging token still matches ("close enough to share blocks") while the information lost,
    ``-log2 P`` of the substituted tokens, stays under ``distance_threshold_bits``."""

    def __init__(self, distance_threshold_bits: float = 0.0, block_size: int = 16, max_nodes: int = 1 << 20):
        self.root = _TrieNode()
        self.thr, self.bs, self.max_nodes = distance_threshold_bits, block_size, max_nodes
        self.n_nodes, self.clock = 0, 0

    def insert(self, token_ids: Sequence[int], log_probs: Sequence[float], block_ids: Sequence[int]) -> None:
        node, self.clock = self.root, self.clock + 1
        for i, t in enumerate(token_ids):
            nxt = node.children.get(t)
            if nxt is None:
                nxt = _TrieNode(logp=node.logp + log_probs[i] / math.log(2))
                node.children[t] = nxt
                self.n_nodes += 1
            nxt.stamp = self.clock
            if (i + 1) % self.bs == 0 and (i + 1) // self.bs <= len(block_ids):
                nxt.block_id = block_ids[(i + 1) // self.bs - 1]
            node = nxt
        if self.n_nodes > self.max_nodes:
            self.evict(self.n_nodes - self.max_nodes)

    def find_longest_match(self, token_ids: Sequence[int], context_log_probs: Optional[Sequence[float]] = None
                           ) -> Optional[Dict[str, Any]]:
        node, blocks, spent, depth, self.clock = self.root, [], 0.0, 0, self.clock + 1
        for i, t in enumerate(token_ids):
            nxt = node.children.get(t)
            if nxt is None and self.thr > 0 and context_log_probs is not None and len(node.children) == 1:
                # the stored continuation differs from the query token: accept it if the query token was unlikely
                # to matter, i.e. the bits needed to tell them apart fit in the remaining threshold
                cost = -context_log_probs[i] / math.log(2)
                if spent + cost <= self.thr:
                    spent += cost
                    nxt = next(iter(node.children.values()))
            if nxt is None:
                break
            nxt.stamp = self.clock
            depth = i + 1
            if nxt.block_id is not None:
                blocks.append(nxt.block_id)
            node = nxt
        if not blocks:
            return None
        return {"matched_tokens": len(blocks) * self.bs, "depth": depth, "block_ids": blocks, "distance_bits": spent}

    def acquire(self, token_ids: Sequence[int], n_tokens: int, delta: int = 1) -> None:
        node = self.root
        for t in token_ids[:n_tokens]:
            node = node.children.get(t)
            if node is None:
                return
            node.refs += delta

    def evict(self, n: int) -> List[int]:
        """Removes up to n least recently used leaves that nobody references; returns their freed block ids."""
        freed: List[int] = []
        for _ in range(n):
            best = None

            def walk(node, parent, key):
                nonlocal best
                if not node.children and parent is not None and node.refs <= 0:
                    if best is None or node.stamp < best[0].stamp:
                        best = (node, parent, key)
                for k, c in node.children.items():
                    walk(c, node, k)
            walk(self.root, None, None)
            if best is None:
                break
            node, parent, key = best
            if node.block_id is not None:
                freed.append(node.block_id)
            del parent.children[key]
            self.n_nodes -= 1
        return freed


class YvMultimodalCacheManager:
    """One namespace per modality with its own token budget and retention policy: ``text`` keeps everything,
    encoder features of ``image`` / ``audio`` / ``video`` are kept LRU under a byte budget keyed by content hash, so a
    repeated image is encoded once."""

    def __init__(self, budgets_mb: Optional[Dict[str, float]] = None):
        self.budgets = {k: v * 2 ** 20 for k, v in (budgets_mb or {"image": 512, "audio": 128, "video": 1024}).items()}
        self.store: Dict[str, "OrderedDict[str, torch.Tensor]"] = {m: OrderedDict() for m in self.budgets}
        self.bytes = {m: 0 for m in self.budgets}
        self.hits = self.misses = 0

    @staticmethod
    def content_key(t: torch.Tensor) -> str:
        import hashlib
        return hashlib.sha1(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()

    def get_or_encode(self, modality: str, raw: torch.Tensor, encode) -> torch.Tensor:
        key = self.content_key(raw)
        st = self.store[modality]
        if key in st:
            st.move_to_end(key)
            self.hits += 1
            return st[key]
        self.misses += 1
        feat = encode(raw)
        st[key] = feat
        self.bytes[modality] += feat.numel() * feat.element_size()
        while self.bytes[modality] > self.budgets[modality] and len(st) > 1:
            _, old = st.popitem(last=False)
            self.bytes[modality] -= old.numel() * old.element_size()
        return feat


class YvSTARKVAdapter:
    """Connects the salient-token KV quantiser to a cache update path: layers whose cache grows beyond
    ``activate_after`` tokens are stored compressed; reads dequantise."""

    def __init__(self, bits: int = 4, keep: int = 32, activate_after: int = 1024):
        self.q = PiscesLxSTARKVQuantizer(bits, keep)
        self.activate_after = activate_after
        self.layers: Dict[int, Dict[str, torch.Tensor]] = {}

    def update(self, layer: int, kv: torch.Tensor, attn_mass: Optional[torch.Tensor] = None) -> bool:
        if kv.shape[0] < self.activate_after:
            self.layers.pop(layer, None)
            return False
        self.layers[layer] = self.q.quantize(kv, attn_mass)
        return True

    def read(self, layer: int, dtype: torch.dtype = torch.float32) -> Optional[torch.Tensor]:
        c = self.layers.get(layer)
        return None if c is None else self.q.dequantize(c, dtype)
