"""Tensor-parallel GEMM + collective pairs used by ``parallel.tp`` when fused communication is on.

``allgather_gemm``      y = all_gather(x_shard) @ W      (column-parallel projections, sequence-parallel input)
``gemm_reduce_scatter`` y_shard = reduce_scatter(x @ W)  (row-parallel projections)

Both take the peer-memory route when the symmetric heap of the group is available:
  * all-gather -> GEMM: every rank publishes its shard in a symmetric buffer; the remote shards are pulled over
    NVLink by a copy kernel on a side stream, chunk by chunk, while the tcgen05 GEMM already runs on the local
    shard; the GEMM on each remote chunk is ordered after that chunk's copy by an event, so the copy of chunk
    i+1 overlaps the math on chunk i.
  * GEMM -> reduce-scatter: the GEMM is issued per destination shard (remote destinations first); each finished
    shard is pushed into the owner's inbox by the copy kernel on the side stream while the next shard is being
    computed; after a flag barrier the owner adds its inbox to the shard it computed itself.
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


def allgather_gemm(x: torch.Tensor, w: torch.Tensor, group: Any, b_mn: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [T/tp, K] local shard, w [N, K] (or [K, N] when ``b_mn``).  Returns (gathered x [T, K], y [T, N])."""
    K = kernels()
    heap = fz.heap_for(group)
    world, rank = heap.world, heap.rank
    rows, kdim = x.shape
    n_out = w.shape[1] if b_mn else w.shape[0]
    dev = x.device
    nbytes = rows * kdim * 2
    pub = heap.get("tp_ag_pub", nbytes)
    pub_t = pub.tensor(_BF16, rows * kdim).view(rows, kdim)
    heap.barrier()                                   # peers finished reading my previous publication
    pub_t.copy_(x)
    heap.barrier()                                   # every shard is published
    xg = torch.empty(world * rows, kdim, dtype=_BF16, device=dev)
    y = torch.empty(world * rows, n_out, dtype=_BF16, device=dev)
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
    inbox = heap.get("tp_rs_inbox", world * nbytes)                 # [source][rows, N]
    inbox_t = inbox.tensor(_BF16, world * rows * n_out).view(world, rows, n_out)
    heap.barrier()                                                  # owners consumed their previous inbox
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
