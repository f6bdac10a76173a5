"""Decode steps replayed from CUDA graphs.

One decode step of a 32-layer MoE model is several hundred kernel launches for a few milliseconds of device work; at
small and medium batch the step time is the launch train plus the Python that builds block tables and contexts (the
reference decodes through Python per step as well, tools/infer/core.py:1106-1144).  ``YvDecodeGraphRunner`` captures
the whole step (embedding -> layers with cache write and paged attention -> final norm -> logits) once per batch
bucket and replays it:

* the step's inputs (token, position, cache slot, sequence length, block table) are written into a pinned host
  staging array with numpy, copied to static device tensors with two asynchronous copies, and the graph is replayed;
* batches are padded to a bucket size with rows of a reserved one-token pseudo-sequence, so that padded rows read and
  write valid cache memory and produce finite values that are simply dropped;
* the block-table width is fixed (``max_seq_len / block_size``): the split count of the paged-decode kernel depends on
  shapes only, so one graph per batch bucket serves every step.

Everything the step launches runs on the current stream, none of it synchronises with the host (expert counts and
offsets stay on the device), and tensor maps are encoded on the host at capture time against addresses in the
graph's private memory pool, so replays see the same addresses.  If capture is not possible (CPU, a parallel layout
with collectives, a sliding-window cache) or fails, the runner falls back to the eager step and says why in
``disabled_reason``."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..models.attention import AttnContext
from ..models.cache import YvPagedKVCache
from ..models.generation import _decode_step

PAD_SEQ_ID = -0x7FFFFFFF


class _Bucket:
    __slots__ = ("graph", "meta", "table", "logits", "B", "meta_host", "table_host", "meta_np", "table_np", "copied")

    def __init__(self, B: int, W: int):
        self.B = B
        self.graph: Any = None
        self.meta: Optional[torch.Tensor] = None      # int32 [4, B]: token, position, slot, seq_len
        self.table: Optional[torch.Tensor] = None     # int32 [B, W]
        self.logits: Optional[torch.Tensor] = None    # static output: overwritten by the next replay
        # pinned staging of exactly the bucket's shape, so that each host-to-device copy is one contiguous transfer
        self.meta_host = torch.zeros(4, B, dtype=torch.int32).pin_memory()
        self.table_host = torch.zeros(B, W, dtype=torch.int32).pin_memory()
        self.meta_np, self.table_np = self.meta_host.numpy(), self.table_host.numpy()
        self.copied: Optional[torch.cuda.Event] = None


class YvDecodeGraphRunner:
    def __init__(self, model: torch.nn.Module, cache: YvPagedKVCache, max_seq_len: int = 8192,
                 buckets: Sequence[int] = (1, 2, 4, 8, 16, 32, 64, 128, 256), enabled: bool = True):
        self.model, self.cache = model, cache
        self.device = cache.device
        self.bs = cache.cfg.block_size
        self.W = max(4, (max_seq_len + self.bs - 1) // self.bs)
        self.max_seq_len = self.W * self.bs
        self.bucket_sizes = sorted(buckets)
        self.buckets: Dict[int, _Bucket] = {}
        self.disabled_reason: Optional[str] = None
        self.replays = self.eager_steps = self.captures = 0
        par = getattr(model, "parallel", None)
        if not enabled:
            self.disabled_reason = "disabled by configuration"
        elif self.device.type != "cuda":
            self.disabled_reason = "no CUDA device"
        elif par is not None and getattr(par, "world_size", 1) > 1:
            self.disabled_reason = "parallel layout with collectives inside the step"
        elif cache.cfg.sliding_window is not None:
            self.disabled_reason = "sliding-window cache"
        if self.disabled_reason is None:
            # the reserved pseudo-sequence that padded rows point at: one token in one block
            cache.add_sequence(PAD_SEQ_ID)
            self._pad_slot = cache.append_slots(PAD_SEQ_ID, 1)[0]
            self._pad_block = cache.tables[PAD_SEQ_ID][0]
            rot = model.model.rotary
            self._cos, self._sin = rot.tables(self.max_seq_len, self.device) if rot is not None else (None, None)

    # ------------------------------------------------------------------------------------------------
    def _bucket_for(self, B: int) -> Optional[int]:
        for b in self.bucket_sizes:
            if b >= B:
                return b
        return None

    def _forward(self, bk: _Bucket) -> torch.Tensor:
        B = bk.B
        ctx = AttnContext(positions=bk.meta[1], cu_seqlens=self._cu[: B + 1], max_len=1, cos=self._cos, sin=self._sin,
                          causal=True, cache=self.cache, slot_map=bk.meta[2], block_table=bk.table,
                          seq_lens=bk.meta[3], decode=True)
        out = self.model(input_ids=bk.meta[0].long().view(B, 1), ctx=ctx, return_logits=False, return_hidden=True)
        return self.model.logits(out["hidden_states"][:, -1, :])

    def _capture(self, B: int) -> _Bucket:
        bk = _Bucket(B, self.W)
        bk.meta = torch.zeros(4, B, dtype=torch.int32, device=self.device)
        bk.table = torch.full((B, self.W), self._pad_block, dtype=torch.int32, device=self.device)
        bk.meta[2].fill_(self._pad_slot)
        bk.meta[3].fill_(1)
        if not hasattr(self, "_cu"):
            self._cu = torch.arange(self.bucket_sizes[-1] + 1, dtype=torch.int32, device=self.device)
        cur = torch.cuda.current_stream(self.device)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(2):                       # warm-up outside capture: lazy initialisation, autotuned paths
                self._forward(bk)
        cur.wait_stream(side)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            bk.logits = self._forward(bk)
        bk.graph = g
        self.captures += 1
        return bk

    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, last_tokens: Sequence[int], seq_ids: List[int]) -> torch.Tensor:
        """One token per running sequence -> logits [B, V].  Reserves the cache slots itself (like the eager step)."""
        B = len(seq_ids)
        Bp = self._bucket_for(B) if self.disabled_reason is None else None
        cache = self.cache
        if Bp is None or any(cache.lengths[s] + 1 > self.max_seq_len for s in seq_ids):
            self.eager_steps += 1
            return _decode_step(self.model, torch.tensor(list(last_tokens), dtype=torch.long, device=self.device),
                                cache, seq_ids)
        bk = self.buckets.get(Bp)
        if bk is None:
            try:
                bk = self._capture(Bp)
            except Exception as e:  # capture is an optimisation: fall back rather than fail the request
                self.disabled_reason = f"capture failed: {type(e).__name__}: {e}"[:300]
                torch.cuda.synchronize(self.device)
                return self.step(last_tokens, seq_ids)
            self.buckets[Bp] = bk
        if bk.copied is not None:
            bk.copied.synchronize()                  # the previous step's copies have left the staging arrays
        meta, table = bk.meta_np, bk.table_np
        for i, s in enumerate(seq_ids):
            slot = cache.append_slots(s, 1)[0]
            n = cache.lengths[s]
            tbl = cache.tables[s]
            meta[0, i], meta[1, i], meta[2, i], meta[3, i] = last_tokens[i], n - 1, slot, n
            table[i, : len(tbl)] = tbl
        if Bp > B:
            meta[0, B:Bp], meta[1, B:Bp], meta[2, B:Bp], meta[3, B:Bp] = 0, 0, self._pad_slot, 1
            table[B:Bp, 0] = self._pad_block
        bk.meta.copy_(bk.meta_host, non_blocking=True)
        bk.table.copy_(bk.table_host, non_blocking=True)
        if bk.copied is None:
            bk.copied = torch.cuda.Event()
        bk.copied.record()
        bk.graph.replay()
        self.replays += 1
        return bk.logits[:B]

    def stats(self) -> Dict[str, Any]:
        return {"graph_replays": self.replays, "eager_steps": self.eager_steps, "captures": self.captures,
                "buckets": sorted(self.buckets), "disabled_reason": self.disabled_reason}
