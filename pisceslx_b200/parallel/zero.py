"""Data-parallel gradient reduction with ZeRO-1 ownership.

Parameters that are replicated over a data-parallel group (dense parameters over ``dp_group``, expert
parameters over ``edp_group``) are assigned *whole* to an owner rank, balanced by size - Muon needs complete
matrices, so ownership is by tensor, not by flat offset.  Gradients are accumulated locally over the
micro-batches of a step in one flat bf16 buffer laid out ``[owner 0 | owner 1 | ...]`` with equal shard
sizes; at the end of the step

    reduce-scatter(flat grads)  ->  the owner holds the summed gradients of its tensors
    owner: optimizer update of the tensors it owns (its optimizer state is the only copy: ZeRO-1)
    all-gather(flat params)     ->  every rank has the updated parameters

The parameters themselves live in a matching flat buffer, so both collectives are a single call (NCCL mode)
or a single fused kernel (``parallel.fused``: peers' gradient shards are pulled over NVLink, summed, scaled
and folded into the momentum / AdamW state in one pass).  The reference reduces gradients with DDP's
all-reduce and keeps full optimizer state on every rank (tools/train/core.py:1585-1593); its "zero_stage"
switch only swaps the optimizer class (opss/train/parallel_3d.py:413-420).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


def _is_expert_param(name: str) -> bool:
    return "experts_w13" in name or "experts_w2" in name


def _is_sequence_parallel_param(name: str) -> bool:
    """Replicated parameters that see only the local token shard (or local heads) under tensor parallelism."""
    return ("norm" in name) or ("router." in name) or name.endswith("shared_expert_weight")


def _is_tp_sharded_param(name: str) -> bool:
    """Matrices that tensor parallelism splits (each rank holds a distinct slice); every other dense parameter
    (embeddings, LM head, MTP heads) is computed on the full sequence by every tensor-parallel rank and is
    therefore replicated, gradient included."""
    return name.endswith(("attention.qkv_proj", "attention.o_proj", "mlp.shared_w13", "mlp.shared_w2"))


class _FlatGroup:
    """One replicated parameter set + its process group."""

    def __init__(self, named: List[Tuple[str, torch.nn.Parameter]], group: Any, world: int, rank: int,
                 fused: bool = False, tag: str = "g"):
        self.group, self.world, self.rank = group, world, rank
        self.named = named
        # greedy balance: biggest tensors first, each to the least loaded owner
        loads = [0] * world
        owner: Dict[str, int] = {}
        for n, p in sorted(named, key=lambda t: -t[1].numel()):
            o = min(range(world), key=lambda r: loads[r])
            owner[n] = o
            loads[o] += (p.numel() + 127) // 128 * 128
        self.owner = owner
        self.shard = max(loads) if loads else 0
        self.offsets: Dict[str, int] = {}
        cur = [r * self.shard for r in range(world)]
        for n, p in named:
            o = owner[n]
            self.offsets[n] = cur[o]
            cur[o] += (p.numel() + 127) // 128 * 128
        dev, dt = named[0][1].device, named[0][1].dtype
        self.symm_param = self.symm_grad = None
        if fused and dev.type == "cuda":
            from . import fused as fz
            (self.symm_param, self.flat_param), (self.symm_grad, self.flat_grad) = fz.symmetric_flat_buffers(
                group, tag, world * self.shard, dt)
            self.flat_grad.zero_()
        else:
            self.flat_param = torch.zeros(world * self.shard, dtype=dt, device=dev)
            self.flat_grad = torch.zeros(world * self.shard, dtype=dt, device=dev)
        for n, p in named:
            off = self.offsets[n]
            view = self.flat_param[off:off + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
        self.grad_views = {n: self.flat_grad[self.offsets[n]:self.offsets[n] + p.numel()].view(p.shape)
                           for n, p in named}

    def owned(self) -> List[Tuple[str, torch.nn.Parameter]]:
        return [(n, p) for n, p in self.named if self.owner[n] == self.rank]

    def my_grad_shard(self) -> torch.Tensor:
        return self.flat_grad[self.rank * self.shard:(self.rank + 1) * self.shard]

    def my_param_shard(self) -> torch.Tensor:
        return self.flat_param[self.rank * self.shard:(self.rank + 1) * self.shard]


class YvGradientSynchronizer:
    """Owns the flat buffers, accumulates micro-batch gradients, and runs reduce-scatter -> sharded update ->
    all-gather at the end of the step.  Works with the streaming optimizer hooks of ``optim.muon`` (gradients of
    replicated parameters are diverted into the flat buffer instead of being folded immediately)."""

    def __init__(self, model: torch.nn.Module, parallel: Any, optimizer: torch.optim.Optimizer,
                 streaming: bool = False, fused: Optional[bool] = None, prescaled: Optional[bool] = None):
        self.parallel, self.optimizer, self.streaming = parallel, optimizer, streaming
        # ``prescaled``: backward already ran on loss / micro-batches (the non-streaming trainer does), so the
        # accumulated gradient only needs 1 / dp; otherwise it needs 1 / (dp * micro-batches).
        self.prescaled = (not streaming) if prescaled is None else bool(prescaled)
        # squared norm of the reduced gradients that were consumed here (fused fold or consume_external_grad)
        # and are therefore no longer visible as ``p.grad``; reset at the first micro-batch of a step
        self.consumed_sq: Optional[torch.Tensor] = None
        self.consumed_sq_rep: Optional[torch.Tensor] = None      # same, for tensors every tensor-parallel rank reduces too
        # three replication classes (the gradient scale is 1 / (dp * micro-batches) for all of them):
        #   routed experts            replicated over tp x edp   (tensor-parallel peers hold different tokens)
        #   sequence-parallel params  replicated over tp x dp    (norm weights, router, shared-expert mix)
        #   everything else           replicated over dp         (tp-sharded matrices, embeddings, LM head)
        dense, expert, seqpar = [], [], []
        split_head = bool(getattr(getattr(model, "cfg", None), "tp_split_head", False))
        for n, p in model.named_parameters():
            if not p.requires_grad or getattr(p, "_yv_sharded", False):     # FULL_SHARD slices reduce themselves
                continue
            if _is_expert_param(n):
                expert.append((n, p))
            elif parallel.tp_size > 1 and (_is_sequence_parallel_param(n) or (split_head and n.endswith("lm_head"))):
                seqpar.append((n, p))          # partial gradient per tensor-parallel rank: reduce over tp x dp
            else:
                dense.append((n, p))
        self.groups: List[_FlatGroup] = []
        self.dp_size = parallel.dp_size

        if fused is None:
            from . import fused as fz
            fused = fz.enabled() and next(model.parameters()).is_cuda
        self.fused = fused

        def add(named, group, tag):
            if named and group is not None and dist.get_world_size(group) > 1:
                self.groups.append(_FlatGroup(named, group, dist.get_world_size(group), dist.get_rank(group),
                                              fused=bool(fused), tag=tag))

        add(dense, parallel.dp_group, "dense")
        add(expert, parallel.expert_grad_group, "expert")
        add(seqpar, parallel.stage_group, "seqpar")
        self._micro, self._total = 0, 1
        self._managed: Dict[int, Tuple[_FlatGroup, str]] = {}
        for g in self.groups:
            for n, p in g.named:
                self._managed[id(p)] = (g, n)
        # Routed experts that no group manages (expert-data-parallel size 1) still receive tokens from every
        # data-parallel rank through the dispatch, and each rank's loss is its LOCAL mean: their gradient is the
        # sum over ranks and needs the same 1 / dp as the reduced ones.
        self._local_experts = [p for n, p in expert if id(p) not in self._managed] if parallel.ep_size > 1 else []
        # unmanaged parameters that are identical on all tensor-parallel ranks: their squared norm is weighted
        # 1 / tp when the ranks' contributions are summed
        # Dense parameters that tensor parallelism does not split (embeddings, LM head, MTP heads) are computed on the
        # full sequence by every tensor-parallel rank: each of the tp data-parallel groups reduces its own identical
        # copy, so every such tensor appears tp times among "the gradients a rank alone accounts for", managed or not.
        self._tp_replicated = set()
        self._tp_replicated_names = set()
        if parallel.tp_size > 1:
            self._tp_replicated = {id(p) for n, p in dense if not _is_tp_sharded_param(n)}
            self._tp_replicated_names = {n for n, p in dense if not _is_tp_sharded_param(n)}
        self.tp_size = parallel.tp_size
        self._hooks = []
        for g in self.groups:
            for n, p in g.named:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(g, n)))
        if hasattr(optimizer, "set_external_grad_params"):
            optimizer.set_external_grad_params(set(self._managed.keys()))

    def manages(self, p: torch.nn.Parameter) -> bool:
        return id(p) in self._managed

    def consumed_sq_total(self) -> Optional[torch.Tensor]:
        """Squared norm of the reduced gradients already handed to the optimizer, with the tensor-parallel
        replicas weighted 1 / tp (None before the first step)."""
        if self.consumed_sq is None:
            return None
        return self.consumed_sq + self.consumed_sq_rep / float(self.tp_size)

    def norm_weight(self, p: torch.nn.Parameter) -> float:
        """Weight of this rank's copy of ``p`` in the global squared gradient norm."""
        return 1.0 / self.tp_size if id(p) in self._tp_replicated else 1.0

    def begin_micro_batch(self, index: int, total: int) -> None:
        self._micro, self._total = index, total
        if index == 0:
            for g in self.groups:
                g.flat_grad.zero_()
            if self.groups:
                dev = self.groups[0].flat_grad.device
                self.consumed_sq = torch.zeros(1, dtype=torch.float32, device=dev)
                self.consumed_sq_rep = torch.zeros(1, dtype=torch.float32, device=dev)

    def _make_hook(self, g: _FlatGroup, name: str):
        def hook(p: torch.nn.Parameter) -> None:
            if p.grad is None:
                return
            g.grad_views[name].add_(p.grad.to(g.flat_grad.dtype))
            p.grad = None
        return hook

    @torch.no_grad()
    def finish(self) -> None:
        """Reduce, update the owned tensors, redistribute.  Called once per optimizer step, after the last
        backward and before ``optimizer.step()``."""
        for g in self.groups:
            scale = 1.0 / self.dp_size if self.prescaled else 1.0 / (self.dp_size * self._total)
            handled: List[str] = []
            if self.fused and g.symm_grad is not None:
                from . import fused as fz
                handled = fz.reduce_scatter_grads(g, scale, self.optimizer, sumsq=self.consumed_sq,
                                                  sumsq_rep=self.consumed_sq_rep, replicated=self._tp_replicated_names)
            else:
                shard = g.my_grad_shard()
                if g.flat_grad.is_cuda:
                    dist.reduce_scatter_tensor(shard, g.flat_grad, group=g.group)
                else:
                    dist.all_reduce(g.flat_grad, group=g.group)
                shard.mul_(scale)
            # hand the reduced gradients of the owned tensors to the optimizer
            for n, p in g.owned():
                if n in handled:
                    continue
                grad = g.grad_views[n]
                if hasattr(self.optimizer, "consume_external_grad"):
                    if self.consumed_sq is not None:
                        acc = self.consumed_sq_rep if n in self._tp_replicated_names else self.consumed_sq
                        if grad.is_cuda:
                            from ..ops import kernels
                            kernels().sumsq(grad.contiguous(), acc)
                        else:
                            acc += grad.float().pow(2).sum()
                    self.optimizer.consume_external_grad(p, grad)
                else:
                    p.grad = grad
        if not self.streaming and self.dp_size > 1:
            for p in self._local_experts:
                if p.grad is not None:
                    p.grad.mul_(1.0 / self.dp_size)
        self._pending_gather = True

    @torch.no_grad()
    def global_sq_norm(self, local_sq: torch.Tensor) -> torch.Tensor:
        """Squared global gradient norm from each rank's sum over the gradients it alone accounts for: the reduced
        gradients of the tensors it owns plus the tensors no group manages (unique to the rank: tensor-parallel
        shards, local experts, its pipeline stage).  Every distinct tensor is owned by exactly one rank, so one
        all-reduce over all ranks counts each once."""
        total = local_sq.detach().float().reshape(1).clone()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(total)
        return total

    @torch.no_grad()
    def after_step(self) -> None:
        """All-gather the updated parameter shards (call after ``optimizer.step()``)."""
        for g in self.groups:
            if self.fused and g.symm_param is not None:
                from . import fused as fz
                fz.all_gather_params(g)
            elif g.flat_param.is_cuda:
                dist.all_gather_into_tensor(g.flat_param, g.my_param_shard().clone(), group=g.group)
            else:
                parts = [torch.empty_like(g.my_param_shard()) for _ in range(g.world)]
                dist.all_gather(parts, g.my_param_shard().clone(), group=g.group)
                g.flat_param.copy_(torch.cat(parts))
            for n, p in g.named:
                if p.grad is not None and g.owner[n] == g.rank:
                    p.grad = None
