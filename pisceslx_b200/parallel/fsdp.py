"""FULL_SHARD (ZeRO-3) data parallelism: parameters, gradients and optimizer state of a unit exist in full only while
the unit computes.

The reference wraps the WHOLE model as one ``FullyShardedDataParallel`` unit (tools/train/core.py:950-985; the
standalone operator opss/train/fsdp.py:219-419 does the same), so "sharded" still means the full bf16 model is
gathered at once.  Here the unit is one transformer block:

  * at wrap time the block's parameters are flattened into one padded vector; each rank keeps its ``1 / world`` slice
    as the only ``nn.Parameter`` (``flat_shard``); the original parameter slots become plain attributes;
  * forward: ``all-gather(flat_shard)`` (an autograd function), the block's weights are rebound as views of the
    gathered vector, the block runs; with ``recompute=True`` (default) the block runs under activation
    checkpointing, so neither activations nor the gathered weights outlive the forward - backward gathers again
    (this is what makes it stage 3 rather than stage 2);
  * backward of the gather is a ``reduce-scatter`` of the flat gradient, scaled ``1 / world``: every rank receives
    exactly the gradient of the slice whose optimizer state it owns;
  * the gather of unit ``i + 1`` is issued asynchronously while unit ``i`` computes (``prefetch=True``), on NCCL's own
    stream; the consumer waits on the handle.

The optimizer sees ``flat_shard`` tensors only (element-wise optimizers: AdamW; Muon needs whole matrices and uses the
ZeRO-1 ownership of ``parallel.zero`` instead).  ``full_state_dict`` reassembles reference-layout tensors.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.checkpoint import checkpoint


def _all_gather_flat(shard: torch.Tensor, group: Any, out: Optional[torch.Tensor] = None, async_op: bool = False):
    world = dist.get_world_size(group)
    full = out if out is not None else torch.empty(world * shard.numel(), dtype=shard.dtype, device=shard.device)
    if shard.is_cuda:
        h = dist.all_gather_into_tensor(full, shard.contiguous(), group=group, async_op=async_op)
    else:
        parts = list(full.view(world, -1).unbind(0))
        h = dist.all_gather(parts, shard.contiguous(), group=group, async_op=async_op)
    return full, h


class _GatherFlat(torch.autograd.Function):
    """flat_shard [S] -> full [world * S]; backward: reduce-scatter of the full gradient, mean over ranks."""

    @staticmethod
    def forward(ctx, shard: torch.Tensor, unit: "YvFullShardUnit") -> torch.Tensor:
        ctx.unit = unit
        pre = unit._take_prefetched()
        if pre is not None:
            return pre
        full, _ = _all_gather_flat(shard.detach(), unit.group)
        unit.stats["gathers"] += 1
        return full

    @staticmethod
    def backward(ctx, dfull: torch.Tensor):
        unit = ctx.unit
        world, rank = unit.world, unit.rank
        dfull = dfull.contiguous()
        S = dfull.numel() // world
        if dfull.is_cuda:
            out = torch.empty(S, dtype=dfull.dtype, device=dfull.device)
            dist.reduce_scatter_tensor(out, dfull, group=unit.group)
        else:
            dist.all_reduce(dfull, group=unit.group)
            out = dfull[rank * S:(rank + 1) * S].clone()
        unit.stats["reduce_scatters"] += 1
        return out / world, None


class YvFullShardUnit(nn.Module):
    def __init__(self, module: nn.Module, group: Any = None, recompute: bool = True, prefetch: bool = True):
        super().__init__()
        self.module = module
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.recompute, self.prefetch = recompute, prefetch
        self.next_unit: Optional["YvFullShardUnit"] = None
        self.stats = {"gathers": 0, "reduce_scatters": 0, "prefetched": 0}
        self._prefetched: Optional[Tuple[torch.Tensor, Any]] = None
        # (owner module, attribute name, shape, offset) of every parameter, in registration order
        self.slots: List[Tuple[nn.Module, str, torch.Size, int]] = []
        self.names: List[str] = []
        params = [(n, p) for n, p in module.named_parameters()]
        assert params, "a unit needs parameters"
        dtype, device = params[0][1].dtype, params[0][1].device
        off = 0
        owners = dict(module.named_modules())
        pieces = []
        for n, p in params:
            assert p.dtype == dtype, "one dtype per unit"
            owner_name, _, attr = n.rpartition(".")
            self.slots.append((owners[owner_name], attr, p.shape, off))
            self.names.append(n)
            pieces.append(p.detach().reshape(-1))
            off += p.numel()
        self.numel = off
        self.shard_size = (off + self.world - 1) // self.world
        flat = torch.zeros(self.shard_size * self.world, dtype=dtype, device=device)
        flat[:off] = torch.cat(pieces)
        self.flat_shard = nn.Parameter(flat[self.rank * self.shard_size:(self.rank + 1) * self.shard_size].clone())
        self.flat_shard._yv_sharded = True                     # data-parallel reducers must leave it alone
        for owner, attr, _, _ in self.slots:                   # the full parameters are gone from now on
            del owner._parameters[attr]
            setattr(owner, attr, None)

    # ---- binding -----------------------------------------------------------------------------------------
    def _bind(self, full: torch.Tensor) -> None:
        for owner, attr, shape, off in self.slots:
            setattr(owner, attr, full[off:off + shape.numel()].view(shape))

    def _unbind(self) -> None:
        for owner, attr, _, _ in self.slots:
            setattr(owner, attr, None)

    def start_prefetch(self) -> None:
        if self._prefetched is None and self.flat_shard.is_cuda:
            full, h = _all_gather_flat(self.flat_shard.detach(), self.group, async_op=True)
            self._prefetched = (full, h)
            self.stats["prefetched"] += 1

    def _take_prefetched(self) -> Optional[torch.Tensor]:
        if self._prefetched is None:
            return None
        full, h = self._prefetched
        self._prefetched = None
        if h is not None:
            h.wait()
        return full

    # ---- forward ---------------------------------------------------------------------------------------------
    def _run(self, shard: torch.Tensor, *args: Any, **kwargs: Any):
        full = _GatherFlat.apply(shard, self)
        if self.prefetch and self.next_unit is not None and not torch.is_grad_enabled():
            self.next_unit.start_prefetch()                    # first (no-grad) pass of a checkpointed forward
        self._bind(full)
        try:
            return self.module(*args, **kwargs)
        finally:
            self._unbind()

    def forward(self, *args: Any, **kwargs: Any):
        if self.recompute and torch.is_grad_enabled() and self.flat_shard.requires_grad:
            if self.prefetch and self.next_unit is not None:
                self.next_unit.start_prefetch()
            return checkpoint(self._run, self.flat_shard, *args, use_reentrant=False, **kwargs)
        return self._run(self.flat_shard, *args, **kwargs)

    # ---- state -----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def full_parameters(self) -> Dict[str, torch.Tensor]:
        full, _ = _all_gather_flat(self.flat_shard.detach(), self.group)
        return {n: full[off:off + shape.numel()].view(shape).clone() for n, (_, _, shape, off) in zip(self.names, self.slots)}

    @torch.no_grad()
    def load_full_parameters(self, tensors: Dict[str, torch.Tensor]) -> None:
        flat = torch.zeros(self.shard_size * self.world, dtype=self.flat_shard.dtype, device=self.flat_shard.device)
        for n, (_, _, shape, off) in zip(self.names, self.slots):
            flat[off:off + shape.numel()] = tensors[n].reshape(-1).to(flat.dtype)
        self.flat_shard.copy_(flat[self.rank * self.shard_size:(self.rank + 1) * self.shard_size])

    def __getattr__(self, name: str):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("module"), name)


def fully_shard(model: nn.Module, group: Any = None, recompute: bool = True, prefetch: bool = True) -> List[YvFullShardUnit]:
    """Wrap every transformer block of ``model`` (``model.model.layers`` or ``model.layers``) as a FULL_SHARD unit, in
    place.  Parameters outside the blocks (embeddings, final norm, LM head) stay replicated and are reduced by the
    caller like any data-parallel parameter.  Returns the units in execution order."""
    trunk = getattr(model, "model", model)
    layers = trunk.layers
    units: List[YvFullShardUnit] = []
    for i in range(len(layers)):
        u = YvFullShardUnit(layers[i], group, recompute, prefetch)
        layers[i] = u
        units.append(u)
    for a, b in zip(units, units[1:]):
        a.next_unit = b
    return units


def replicated_parameters(model: nn.Module) -> List[nn.Parameter]:
    return [p for p in model.parameters() if not getattr(p, "_yv_sharded", False)]


@torch.no_grad()
def reduce_replicated_gradients(model: nn.Module, group: Any = None) -> None:
    """Mean of the gradients of the parameters that stayed replicated (one flat all-reduce)."""
    ps = [p for p in replicated_parameters(model) if p.grad is not None]
    if not ps:
        return
    flat = torch.cat([p.grad.reshape(-1).float() for p in ps])
    dist.all_reduce(flat, group=group)
    flat /= dist.get_world_size(group)
    off = 0
    for p in ps:
        p.grad.copy_(flat[off:off + p.numel()].view_as(p.grad))
        off += p.numel()


def memory_per_rank_gb(total_params: float, unit_params: float, world: int, bytes_param: int = 2, bytes_state: int = 8) -> float:
    """Steady-state bytes per rank: 1/world of parameters, gradients and optimizer state, plus two gathered units
    (the one computing and the one being prefetched)."""
    return (total_params * (2 * bytes_param + bytes_state) / world + 2 * unit_params * bytes_param) / 1e9
