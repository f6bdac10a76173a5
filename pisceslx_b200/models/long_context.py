"""Long-context helpers (reference model/core/long_context.py: ``YvOOMBContext`` overlapped chunks averaged :40-114,
``YvREFORM``; ``YvMHCLiteHyperConnection``; ``YvLayerRouteAdapter``) and the trace addresser of the Subconscious block
field (``YvResonantTraceAddresser``: argmax over trace scores with a minimum dwell; ``YvResidentBlockPool`` LRU slots,
model/core/block_field.py:154-260)."""
from __future__ import annotations

from collections import OrderedDict
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as F_


class YvOOMBContext:
    """Out-of-memory-bounded context: sequences longer than ``chunk`` run through ``fn`` in overlapping windows; in
    the overlaps the outputs are blended with a linear ramp (the reference averages them)."""

    def __init__(self, chunk: int = 32768, overlap: int = 1024):
        assert 0 <= overlap < chunk
        self.chunk, self.overlap = chunk, overlap

    def windows(self, S: int) -> List[Tuple[int, int]]:
        if S <= self.chunk:
            return [(0, S)]
        step = self.chunk - self.overlap
        out, a = [], 0
        while a < S:
            b = min(S, a + self.chunk)
            out.append((a, b))
            if b == S:
                break
            a += step
        return out

    def run(self, x: torch.Tensor, fn: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
        """x [B, S, H] -> [B, S, H']."""
        S = x.shape[1]
        wins = self.windows(S)
        if len(wins) == 1:
            return fn(x)
        out = wt = None
        for a, b in wins:
            y = fn(x[:, a:b])
            if out is None:
                out = y.new_zeros(x.shape[0], S, y.shape[-1], dtype=torch.float32)
                wt = y.new_zeros(S, dtype=torch.float32)
            w = torch.ones(b - a, device=y.device)
            if a > 0 and self.overlap:
                w[: self.overlap] = torch.linspace(0, 1, self.overlap + 2, device=y.device)[1:-1]
            if b < S and self.overlap:
                w[-self.overlap:] = torch.minimum(w[-self.overlap:], torch.linspace(1, 0, self.overlap + 2, device=y.device)[1:-1])
            out[:, a:b] += y.float() * w[None, :, None]
            wt[a:b] += w
        return (out / wt[None, :, None]).to(x.dtype)


class YvREFORM(nn.Module):
    """Recall by compressed memory: past chunks are summarised into ``n_slots`` vectors by learned pooling queries;
    the current chunk cross-attends to the concatenated summaries (a bounded-size memory of an unbounded past)."""

    def __init__(self, hidden: int, n_slots: int = 16, n_head: int = 4):
        super().__init__()
        self.h, self.d = n_head, hidden // n_head
        self.pool_q = nn.Parameter(torch.randn(n_slots, hidden) * 0.02)
        self.q = nn.Parameter(torch.empty(hidden, hidden).normal_(std=0.02))
        self.kv = nn.Parameter(torch.empty(2 * hidden, hidden).normal_(std=0.02))
        self.o = nn.Parameter(torch.zeros(hidden, hidden))
        self.memory: Optional[torch.Tensor] = None

    def reset(self) -> None:
        self.memory = None

    def summarise(self, chunk: torch.Tensor) -> torch.Tensor:
        a = torch.softmax(torch.einsum("sh,bth->bst", self.pool_q.to(chunk.dtype), chunk).float() * chunk.shape[-1] ** -0.5, -1)
        return torch.einsum("bst,bth->bsh", a.to(chunk.dtype), chunk)

    def forward(self, chunk: torch.Tensor) -> torch.Tensor:
        B, S, H = chunk.shape
        out = chunk
        if self.memory is not None:
            M = self.memory.shape[1]
            q = F_.linear(chunk, self.q).view(B, S, self.h, self.d).transpose(1, 2)
            k, v = F_.linear(self.memory, self.kv).chunk(2, -1)
            k, v = k.view(B, M, self.h, self.d).transpose(1, 2), v.view(B, M, self.h, self.d).transpose(1, 2)
            a = torch.softmax(torch.matmul(q.float(), k.float().transpose(-1, -2)) * self.d ** -0.5, -1)
            r = torch.matmul(a, v.float()).to(chunk.dtype).transpose(1, 2).reshape(B, S, H)
            out = chunk + F_.linear(r, self.o)
        summ = self.summarise(chunk.detach())
        self.memory = summ if self.memory is None else torch.cat([self.memory, summ], 1)
        return out


class YvMHCLiteHyperConnection(nn.Module):
    """Hyper-connection over ``n`` parallel residual streams: read weights mix the streams into the layer input,
    write weights distribute the layer output back; initialised to behave like one plain residual stream."""

    def __init__(self, n_streams: int = 2):
        super().__init__()
        self.read = nn.Parameter(torch.zeros(n_streams))
        self.write = nn.Parameter(torch.ones(n_streams))
        self.mix = nn.Parameter(torch.eye(n_streams))

    def forward(self, streams: torch.Tensor, layer: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
        """streams [n, B, S, H] -> [n, B, S, H]."""
        x = torch.einsum("n,n...->...", torch.softmax(self.read, 0).to(streams.dtype), streams)
        y = layer(x)
        mixed = torch.einsum("mn,n...->m...", self.mix.to(streams.dtype), streams)
        return mixed + self.write.to(streams.dtype).view(-1, 1, 1, 1) * y[None]


class YvLayerRouteAdapter(nn.Module):
    """Per-layer low-rank adapter chosen by a router over ``n_routes`` adapter banks (soft mixture)."""

    def __init__(self, hidden: int, n_routes: int = 4, rank: int = 8):
        super().__init__()
        self.router = nn.Parameter(torch.zeros(n_routes, hidden))
        self.down = nn.Parameter(torch.empty(n_routes, rank, hidden).normal_(std=0.02))
        self.up = nn.Parameter(torch.zeros(n_routes, hidden, rank))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = torch.softmax(F_.linear(x, self.router.to(x.dtype)).float(), -1).to(x.dtype)       # [..., R]
        low = torch.einsum("...h,rkh->...rk", x, self.down.to(x.dtype))
        upd = torch.einsum("...rk,rhk->...rh", low, self.up.to(x.dtype))
        return x + (w[..., None] * upd).sum(-2)


class YvResonantTraceAddresser:
    """Chooses the knowledge block to address from per-block trace scores: argmax with hysteresis (a block stays
    selected for at least ``min_dwell`` steps, and a challenger must win by ``margin``)."""

    def __init__(self, min_dwell: int = 4, margin: float = 0.05):
        self.min_dwell, self.margin = min_dwell, margin
        self.current: Optional[int] = None
        self.age = 0

    def step(self, scores: torch.Tensor) -> int:
        best = int(scores.argmax())
        if self.current is None:
            self.current, self.age = best, 0
        elif best != self.current and self.age >= self.min_dwell and \
                float(scores[best]) > float(scores[self.current]) + self.margin:
            self.current, self.age = best, 0
        else:
            self.age += 1
        return self.current


class YvResidentBlockPool:
    """LRU pool of device-resident knowledge blocks backed by a host store (``fetch(block_id) -> tensor``)."""

    def __init__(self, slots: int, fetch: Callable[[int], torch.Tensor]):
        self.slots, self.fetch = slots, fetch
        self.resident: "OrderedDict[int, torch.Tensor]" = OrderedDict()
        self.loads = 0

    def get(self, block_id: int) -> torch.Tensor:
        if block_id in self.resident:
            self.resident.move_to_end(block_id)
            return self.resident[block_id]
        t = self.fetch(block_id)
        self.loads += 1
        self.resident[block_id] = t
        if len(self.resident) > self.slots:
            self.resident.popitem(last=False)
        return t
