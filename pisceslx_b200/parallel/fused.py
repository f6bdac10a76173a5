"""Fused compute + collective paths over peer memory (NVLink 5 / NVSwitch).

Every rank of a group allocates *symmetric* buffers (same size on every rank, ``cudaMalloc`` + CUDA IPC), maps
its peers' buffers and hands the raw pointers to the kernels in ``ops/csrc/comm.cu``:

  * expert parallelism: the MoE permutation kernel stores token rows straight into the owning rank's receive
    region (dispatch), the grouped tcgen05 GEMMs run on the receive regions through a tile list, and the
    weighted un-permute loads result rows from the owners (combine).  Backward mirrors it.  Cross-rank ordering
    uses a bounded flag barrier kernel; nothing synchronises with the host.
  * ZeRO-1: the owner of a tensor pulls every peer's gradient shard, sums, scales and folds the result into the
    Muon momentum buffer / applies AdamW in the same pass; updated parameters are pulled back by the peers.
  * Subconscious PQ field: the row-sharded codebook gather reads entries from the owners' memory.

``set_enabled(False)`` (bench ``--no-fused-comm``) selects the NCCL implementations in ``parallel.tp`` /
``parallel.ep`` / ``parallel.zero`` instead - the stated baseline mode.
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import kernels, status_word

_BF16 = torch.bfloat16
_ENABLED = os.environ.get("YV_FUSED_COMM", "1") != "0"
_DTYPE_CODE = {torch.bfloat16: 0, torch.float32: 1, torch.int32: 2, torch.uint8: 3}


def set_enabled(flag: bool) -> None:
    global _ENABLED
    _ENABLED = bool(flag)


def enabled() -> bool:
    return _ENABLED and torch.cuda.is_available() and dist.is_initialized() and dist.get_backend() == "nccl"


# --------------------------------------------------------------------------------------------------
# symmetric memory
# --------------------------------------------------------------------------------------------------
class SymmBuffer:
    def __init__(self, heap: "SymmHeap", nbytes: int):
        K = kernels()
        self.heap, self.nbytes = heap, nbytes
        self.ptr, handle = K.symm_alloc(nbytes)
        handles: List[Any] = [None] * heap.world
        dist.all_gather_object(handles, handle.numpy().tobytes(), group=heap.group)
        self.peer_ptrs: List[int] = []
        for r, h in enumerate(handles):
            if r == heap.rank:
                self.peer_ptrs.append(self.ptr)
            else:
                self.peer_ptrs.append(K.symm_open(torch.frombuffer(bytearray(h), dtype=torch.uint8)))
        self.ptrs = torch.tensor(self.peer_ptrs, dtype=torch.int64)            # CPU int64 vector for the bindings

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        esz = torch.empty(0, dtype=dtype).element_size()
        numel = (self.nbytes - offset_bytes) // esz if numel is None else numel
        return kernels().symm_tensor(self.ptr + offset_bytes, numel, _DTYPE_CODE[dtype], self.heap.device.index)

    def free(self) -> None:
        K = kernels()
        for r, p in enumerate(self.peer_ptrs):
            if r != self.heap.rank:
                K.symm_close(p)
        K.symm_free(self.ptr)


class SymmHeap:
    """Symmetric allocations + the flag barrier of one process group."""

    def __init__(self, group: Any):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.buffers: Dict[str, SymmBuffer] = {}
        self.flags = SymmBuffer(self, 256)
        self.epoch = 0
        dist.barrier(group=group)

    def get(self, name: str, nbytes: int) -> SymmBuffer:
        """Named buffer, grown (re-allocated collectively) when a larger size is requested."""
        nbytes = (nbytes + 255) // 256 * 256
        buf = self.buffers.get(name)
        if buf is None or buf.nbytes < nbytes:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            if buf is not None:
                buf.free()
            buf = SymmBuffer(self, nbytes)
            self.buffers[name] = buf
            dist.barrier(group=self.group)
        return buf

    def barrier(self) -> None:
        """Device-side barrier on the current stream (bounded wait; failure lands in the status word)."""
        self.epoch += 1
        kernels().peer_barrier(self.flags.ptrs, self.rank, self.epoch, status_word(self.device))

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


_HEAPS: Dict[int, SymmHeap] = {}


def heap_for(group: Any) -> SymmHeap:
    key = id(group)
    h = _HEAPS.get(key)
    if h is None:
        h = SymmHeap(group)
        _HEAPS[key] = h
    return h


# --------------------------------------------------------------------------------------------------
# expert parallel routed experts over peer memory
# --------------------------------------------------------------------------------------------------
class _EPContext:
    """Buffers of one (group, capacity, hidden) combination."""

    def __init__(self, heap: SymmHeap, cap_rows: int, hidden: int, e_local: int):
        self.heap, self.cap, self.hidden, self.e_local = heap, cap_rows, hidden, e_local
        w = heap.world
        rows = w * cap_rows
        self.region_rows = rows
        nbytes = rows * hidden * 2
        self.x_recv = heap.get("ep_x_recv", nbytes)
        self.y_out = heap.get("ep_y_out", nbytes)
        self.dy_recv = heap.get("ep_dy_recv", nbytes)
        self.table = heap.get("ep_counts", w * e_local * 4)
        dev = heap.device
        self.x_recv_t = self.x_recv.tensor(_BF16, rows * hidden).view(rows, hidden)
        self.y_out_t = self.y_out.tensor(_BF16, rows * hidden).view(rows, hidden)
        self.dy_recv_t = self.dy_recv.tensor(_BF16, rows * hidden).view(rows, hidden)
        self.table_t = self.table.tensor(torch.int32, w * e_local)
        max_tiles = rows // 128
        self.tile_rows = torch.zeros(max_tiles, dtype=torch.int32, device=dev)
        self.tile_expert = torch.zeros(max_tiles, dtype=torch.int32, device=dev)
        self.num_tiles = torch.zeros(1, dtype=torch.int32, device=dev)
        self.seg_src = torch.zeros(w * (e_local + 1), dtype=torch.int32, device=dev)

    def valid(self) -> bool:
        """The heap grows a named buffer by freeing and re-allocating it (serving sees many token counts: a long
        prefill after a short one).  A context built before that holds pointers into freed memory."""
        b = self.heap.buffers
        return (b.get("ep_x_recv") is self.x_recv and b.get("ep_y_out") is self.y_out
                and b.get("ep_dy_recv") is self.dy_recv and b.get("ep_counts") is self.table)


_EP_CTX: Dict[Tuple[int, int, int, int], _EPContext] = {}


def _ep_context(group: Any, cap_rows: int, hidden: int, e_local: int) -> _EPContext:
    key = (id(group), cap_rows, hidden, e_local)
    ctx = _EP_CTX.get(key)
    if ctx is not None and not ctx.valid():
        ctx = None                 # a larger request re-allocated the named buffers since: the cached views are stale
    if ctx is None:
        ctx = _EPContext(heap_for(group), cap_rows, hidden, e_local)
        _EP_CTX[key] = ctx
    return ctx


class _MoEExpertsEPFused(torch.autograd.Function):
    """Expert-parallel routed experts over peer memory.

    Receive regions are sized for the worst case (every token of every source routed to this rank), but only the tiles
    that really arrived are computed and stored: the receive plan lists them expert-major, the tile count is read once
    on the host, and everything behind the receive region (up-projection output, activation, gradients) lives in
    COMPACT buffers of ``n_tiles * 128`` rows in which each local expert's rows are contiguous.  So the stored
    activations are those of the tokens this rank serves (about T * k rows when routing is balanced) instead of
    ``world`` times the bound, the element-wise kernels touch real rows only, and each weight gradient is ONE
    grouped-K GEMM over the compact buffers instead of one accumulating GEMM per source."""

    @staticmethod
    def forward(ctx, x, w13, w2, weights, idx, num_experts, group, deterministic, counts=None):
        from ..ops import moe as moe_ops
        K = kernels()
        dev = x.device
        st = status_word(dev)
        T, H = x.shape
        k = idx.shape[1]
        world = dist.get_world_size(group)
        e_local = num_experts // world
        cap = moe_ops.padded_rows_bound(T * k, e_local)
        c = _ep_context(group, cap, H, e_local)
        heap = c.heap
        rank = heap.rank
        x = x.contiguous()
        idx = idx.int().contiguous()
        if counts is None:
            counts = torch.bincount(idx.flatten().long(), minlength=num_experts)
        counts = counts.int()
        seg = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
        te_unused = torch.empty(moe_ops.padded_rows_bound(T * k, num_experts) // 128, dtype=torch.int32, device=dev)
        nt_unused = torch.empty(1, dtype=torch.int32, device=dev)
        cursor = torch.empty(num_experts, dtype=torch.int32, device=dev)
        K.moe_plan(counts, seg, te_unused, nt_unused, cursor)
        # 1. publish my per-expert padded row counts to the owners (ends with a barrier)
        K.ep_put_counts(seg, c.table.ptrs, heap.flags.ptrs, rank, e_local, heap.next_epoch(), st)
        K.ep_recv_plan(c.table_t, world, e_local, cap, c.tile_rows, c.tile_expert, c.num_tiles, c.seg_src, True)
        # 2. dispatch: the permutation writes into the owners' receive regions
        row_map = torch.empty(T, k, dtype=torch.int64, device=dev)
        K.ep_dispatch(x, idx, cursor, seg, row_map, c.x_recv.ptrs, rank, e_local, cap, st)
        K.ep_zero_pad(seg, counts, c.x_recv.ptrs, rank, e_local, cap, H)
        heap.barrier()
        # 3. local experts on the tiles that arrived, in compact buffers (one host read of the tile count)
        n_tiles = int(c.num_tiles.item())
        rows = n_tiles * 128
        F = w13.shape[1] // 2
        tile_rows = c.tile_rows[:n_tiles].clone()
        tile_expert = c.tile_expert[:max(n_tiles, 1)].clone()
        num_tiles = c.num_tiles.clone()
        seg_c = c.seg_src[:e_local + 1].clone()
        xc = torch.empty(rows, H, dtype=_BF16, device=dev)
        K.tile_gather(c.x_recv_t, tile_rows, n_tiles, xc)
        y1 = torch.empty(rows, 2 * F, dtype=_BF16, device=dev)
        act = torch.empty(rows, F, dtype=_BF16, device=dev)
        if n_tiles > 0:
            K.gemm_grouped_m(xc, w13, y1, tile_expert, num_tiles, False, 0, st)
            K.swiglu_fwd(y1, act)
            # down projection: compact activation rows in, receive-region rows out (peers read them there)
            K.gemm_grouped_m_rows(act, w2, c.y_out_t, tile_rows, tile_expert, num_tiles, False, 0, st, True)
        heap.barrier()
        # 4. combine: load my tokens' results from the owners
        out = torch.empty(T, H, dtype=_BF16, device=dev)
        wts = weights.float().contiguous()
        K.ep_combine(c.y_out.ptrs, row_map, wts, out, c.region_rows)
        need_grad = any(ctx.needs_input_grad[:4])
        if need_grad:
            ctx.save_for_backward(xc, y1, act, w13, w2, wts, row_map, seg, counts, tile_rows, tile_expert, num_tiles, seg_c)
        ctx.c, ctx.dims, ctx.w_dtype = c, (T, H, k, F, world, e_local, cap, n_tiles), weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        K = kernels()
        c = ctx.c
        heap = c.heap
        (xc, y1, act, w13, w2, wts, row_map, seg, counts, tile_rows, tile_expert, num_tiles, seg_c) = ctx.saved_tensors
        T, H, k, F, world, e_local, cap, n_tiles = ctx.dims
        dev = dout.device
        st = status_word(dev)
        rank = heap.rank
        dout = dout.contiguous()
        heap.barrier()                                   # every rank is done with the previous use of dy_recv
        dwts = torch.empty(T, k, dtype=torch.float32, device=dev)
        K.ep_combine_bwd(dout, c.y_out.ptrs, c.dy_recv.ptrs, row_map, wts, dwts, c.region_rows)
        K.ep_zero_pad(seg, counts, c.dy_recv.ptrs, rank, e_local, cap, H)
        heap.barrier()
        rows = n_tiles * 128
        dw2 = torch.zeros_like(w2) if n_tiles == 0 else torch.empty_like(w2)
        dw13 = torch.zeros_like(w13) if n_tiles == 0 else torch.empty_like(w13)
        if n_tiles > 0:
            dyc = torch.empty(rows, H, dtype=_BF16, device=dev)
            K.tile_gather(c.dy_recv_t, tile_rows, n_tiles, dyc)
            dact = torch.empty(rows, F, dtype=_BF16, device=dev)
            K.gemm_grouped_m(dyc, w2, dact, tile_expert, num_tiles, True, 0, st)
            K.gemm_grouped_k(dyc, act, dw2, seg_c, False, 0, st)             # every expert's rows are contiguous
            del dyc
            dy1 = torch.empty_like(y1)
            K.swiglu_bwd(y1, dact, dy1)
            del dact
            # the input-gradient rows go back into the receive region (already consumed) so that peers can read them
            K.gemm_grouped_m_rows(dy1, w13, c.dy_recv_t, tile_rows, tile_expert, num_tiles, True, 0, st, True)
            K.gemm_grouped_k(dy1, xc, dw13, seg_c, False, 0, st)
        heap.barrier()
        dx = torch.empty(T, H, dtype=_BF16, device=dev)
        K.ep_unpermute_sum(c.dy_recv.ptrs, row_map, dx, k, c.region_rows)
        return dx, dw13, dw2, dwts.to(ctx.w_dtype), None, None, None, None, None


def moe_experts_ep_fused(x, w13_local, w2_local, weights, idx, num_experts, group, deterministic=False, counts=None):
    """``counts`` [E] int32: the expert histogram the gate kernel produced (recomputed when omitted)."""
    return _MoEExpertsEPFused.apply(x.to(_BF16), w13_local, w2_local, weights, idx, num_experts, group, deterministic,
                                    counts)


# --------------------------------------------------------------------------------------------------
# ZeRO-1 gradient reduce-scatter fused with the optimizer fold
# --------------------------------------------------------------------------------------------------
def symmetric_flat_buffers(group: Any, name: str, numel: int, dtype: torch.dtype):
    """(param buffer, grad buffer) of ``numel`` elements in symmetric memory, as (SymmBuffer, tensor) pairs."""
    heap = heap_for(group)
    esz = torch.empty(0, dtype=dtype).element_size()
    pb = heap.get(f"zero_param_{name}", numel * esz)
    gb = heap.get(f"zero_grad_{name}", numel * esz)
    return (pb, pb.tensor(dtype, numel)), (gb, gb.tensor(dtype, numel))


def reduce_scatter_grads(g: Any, scale: float, optimizer: Any = None, sumsq: Any = None, sumsq_rep: Any = None,
                         replicated: Any = ()) -> List[str]:
    """Owner-side pull reduction of flat-group ``g``.  Tensors whose optimizer update could be fused into the
    reduction are returned by name (their gradients need no further handling).  The squared norm of every folded
    gradient is added to ``sumsq``, or to ``sumsq_rep`` for the tensors named in ``replicated`` (tensors of which
    every tensor-parallel rank holds and reduces an identical copy: the caller weights that sum by 1 / tp)."""
    K = kernels()
    heap = heap_for(g.group)
    heap.barrier()                                          # all ranks finished accumulating their gradients
    handled: List[str] = []
    ptrs = g.symm_grad.ptrs
    streaming = bool(getattr(optimizer, "_streaming", False))
    sumsq_plain = sumsq
    for n, p in g.owned():
        off = g.offsets[n]
        numel = p.numel()
        fused_done = False
        sumsq = sumsq_rep if (sumsq_rep is not None and n in replicated) else sumsq_plain
        if optimizer is not None and streaming and numel % 2 == 0 and g.flat_grad.dtype == _BF16:
            group = optimizer._group_of(p)
            state = optimizer._state_for(p, group)
            if group["use_muon"] and "momentum_buffer" not in state:
                pass                                        # quantised momentum: reduce here, fold through the optimizer
            elif group["use_muon"]:
                K.zero_reduce_fold(ptrs, g.rank, off, numel, scale, 1, None, state["momentum_buffer"].view(-1), None,
                                   group["momentum"], 0.0, 0.0, 0.0, 0.0, 0.0, 1, sumsq)
                fused_done = True
            elif p.is_contiguous():
                state["adam_step"] += 1
                b1, b2 = group["betas"]
                K.zero_reduce_fold(ptrs, g.rank, off, numel, scale, 2, p.data.view(-1), state["adam_exp_avg"].view(-1),
                                   state["adam_exp_avg_sq"].view(-1), 0.0, group["lr"], b1, b2, group["eps"],
                                   group["weight_decay"], state["adam_step"], sumsq)
                fused_done = True
        if fused_done:
            handled.append(n)
        else:
            padded = (numel + 127) // 128 * 128
            K.zero_reduce_fold(ptrs, g.rank, off, padded, scale, 0, None, None, None, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 1)
    heap.barrier()                                          # peers may overwrite their gradient buffers again
    return handled


def all_gather_params(g: Any) -> None:
    """Every rank pulls the updated parameter shards from their owners."""
    K = kernels()
    heap = heap_for(g.group)
    heap.barrier()                                          # owners finished their updates
    esz = g.flat_param.element_size()
    nbytes = g.shard * esz
    for r in range(g.world):
        if r == g.rank or nbytes == 0:
            continue
        K.peer_copy(g.symm_param.ptr + r * nbytes, g.symm_param.peer_ptrs[r] + r * nbytes, nbytes)
    heap.barrier()


# --------------------------------------------------------------------------------------------------
# row-sharded PQ codebook gather
# --------------------------------------------------------------------------------------------------
def pq_gather_sum_sharded(table_buf: SymmBuffer, idx: torch.Tensor, num_codebooks: int, rows_per_rank: int,
                          dim: int) -> torch.Tensor:
    out = torch.empty(idx.shape[0], dim, dtype=_BF16, device=idx.device)
    kernels().pq_gather_sum_peer(table_buf.ptrs, idx.int().contiguous(), out, num_codebooks, rows_per_rank,
                                 status_word(idx.device))
    return out
