"""Tensor-parallel GEMM + collective pairs used by ``parallel.tp`` when fused communication is on.

``allgather_gemm``      y = all_gather(x_shard) @ W      (column-parallel projections, sequence-parallel input)
``gemm_reduce_scatter`` y_shard = reduce_scatter(x @ W)  (row-parallel projections)

Each is ONE launch of the tcgen05 GEMM kernel in a communication mode (``gemm_tp``) when the shard has a whole
number of 128-row blocks:
  * all-gather -> GEMM: every rank publishes its shard in a symmetric buffer.  Inside the GEMM kernel one extra warp
    per CTA pulls the peers' shards over NVLink into the local gathered buffer, 128-row block by block, and counts
    each block complete; the TMA producer starts with the rows this rank already holds and waits (bounded) for a
    block's count before loading tiles of it, so every remote byte crosses NVLink once and the transfer is hidden
    behind the tiles of the local rows.
  * GEMM -> reduce-scatter: the kernel computes the rows owned by the other ranks first and its epilogue stores
    those tiles from registers straight into the owner's inbox (peer stores); the rank's own rows are computed last
    and stored locally.  After a flag barrier the owner adds its inbox to its own partial rows.
Shards that are not a multiple of 128 rows take the older route (copy kernel on a side stream ordered by events
against per-shard GEMM launches).
"""
from __future__ import annotations

from typing import Any, Dict, Tuple

import torch
import torch.distributed as dist

from ..ops import functional as F_
from ..ops import kernels, status_word
from . import fused as fz

_BF16 = torch.bfloat16
_SIDE: Dict[int, torch.cuda.Stream] = {}


def _side_stream(dev: torch.device) -> torch.cuda.Stream:
    s = _SIDE.get(dev.index)
    if s is None:
        s = torch.cuda.Stream(dev)
        _SIDE[dev.index] = s
    return s


_FLAGS: Dict[int, torch.Tensor] = {}


def _block_flags(dev: torch.device, blocks: int) -> torch.Tensor:
    t = _FLAGS.get(dev.index)
    if t is None or t.numel() < blocks:
        t = torch.zeros(max(blocks, 1024), dtype=torch.int32, device=dev)
        _FLAGS[dev.index] = t
    return t


def allgather_gemm(x: torch.Tensor, w: torch.Tensor, group: Any, b_mn: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [T/tp, K] local shard, w [N, K] (or [K, N] when ``b_mn``).  Returns (gathered x [T, K], y [T, N])."""
    K = kernels()
    heap = fz.heap_for(group)
    world, rank = heap.world, heap.rank
    rows, kdim = x.shape
    n_out = w.shape[1] if b_mn else w.shape[0]
    dev = x.device
    nbytes = rows * kdim * 2
    # Two publication buffers used alternately: a peer may still read call i's buffer while call i+1 publishes into
    # the other one, and the barrier of call i+1 (which every rank reaches after its kernel of call i) makes the
    # first buffer free again for call i+2.  One barrier per call instead of two.
    heap.tp_ag_calls = getattr(heap, "tp_ag_calls", 0) + 1
    pub = heap.get(f"tp_ag_pub{heap.tp_ag_calls & 1}", nbytes)
    pub_t = pub.tensor(_BF16, rows * kdim).view(rows, kdim)
    pub_t.copy_(x)
    heap.barrier()                                   # every shard is published
    xg = torch.empty(world * rows, kdim, dtype=_BF16, device=dev)
    y = torch.empty(world * rows, n_out, dtype=_BF16, device=dev)
    if rows % 128 == 0 and w.stride(-1) == 1:
        xg[rank * rows:(rank + 1) * rows].copy_(x)
        K.gemm_tp(xg, w, y, 1, pub.ptrs, _block_flags(dev, world * rows // 128), rank, rows, b_mn, 0,
                  status_word(dev))
        return xg, y
    side = _side_stream(dev)
    main = torch.cuda.current_stream(dev)
    side.wait_stream(main)
    events = {}
    order = [(rank + i) % world for i in range(world)]
    with torch.cuda.stream(side):
        for r in order[1:]:
            K.peer_copy(xg.data_ptr() + r * nbytes, pub.peer_ptrs[r], nbytes)
            ev = torch.cuda.Event()
            ev.record(side)
            events[r] = ev
    xg[rank * rows:(rank + 1) * rows].copy_(x)
    for r in order:
        if r != rank:
            main.wait_event(events[r])
        F_.gemm(xg[r * rows:(r + 1) * rows], w, b_mn=b_mn, out=y[r * rows:(r + 1) * rows])
    return xg, y


def gemm_reduce_scatter(x: torch.Tensor, w: torch.Tensor, group: Any, b_mn: bool = False) -> torch.Tensor:
    """x [T, K_local], w [N, K_local] (or [K_local, N] when ``b_mn``).  Returns the local rows of the summed
    product, [T/tp, N]."""
    K = kernels()
    heap = fz.heap_for(group)
    world, rank = heap.world, heap.rank
    T = x.shape[0]
    rows = T // world
    n_out = w.shape[1] if b_mn else w.shape[0]
    dev = x.device
    nbytes = rows * n_out * 2
    # two inboxes used alternately (same argument as for the all-gather publication buffers)
    heap.tp_rs_calls = getattr(heap, "tp_rs_calls", 0) + 1
    inbox = heap.get(f"tp_rs_inbox{heap.tp_rs_calls & 1}", world * nbytes)             # [source][rows, N]
    inbox_t = inbox.tensor(_BF16, world * rows * n_out).view(world, rows, n_out)
    if rows % 128 == 0 and n_out % 64 == 0 and rows * world == T and w.stride(-1) == 1:
        full = torch.empty(T, n_out, dtype=_BF16, device=dev)
        K.gemm_tp(x.contiguous(), w, full, 2, inbox.ptrs, None, rank, rows, b_mn, 0, status_word(dev))
        heap.barrier()                                              # every inbox is complete
        out = full[rank * rows:(rank + 1) * rows]
        for s in range(world):
            if s != rank:
                out = out + inbox_t[s]
        return out
    side = _side_stream(dev)
    main = torch.cuda.current_stream(dev)
    part = torch.empty(world, rows, n_out, dtype=_BF16, device=dev)
    order = [(rank + i) % world for i in range(1, world)] + [rank]   # remote destinations first
    for d in order:
        F_.gemm(x[d * rows:(d + 1) * rows], w, b_mn=b_mn, out=part[d])
        if d != rank:
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(side):
                side.wait_event(ev)
                K.peer_copy(inbox.peer_ptrs[d] + rank * nbytes, part[d].data_ptr(), nbytes)
    main.wait_stream(side)
    heap.barrier()                                                  # every inbox is complete
    out = part[rank]
    for s in range(world):
        if s != rank:
            out = out + inbox_t[s]
    return out
