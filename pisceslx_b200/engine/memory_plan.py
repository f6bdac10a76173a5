"""Memory-aware activation recomputation: recompute only as many layers as the device's memory requires.

The reference turns ``use_gradient_checkpointing`` on for every layer of large presets (configs/train/pretrain.yaml,
tools/train/config.py:688-689) whatever the device holds.  On a 180 GB part the answer depends on the parallel
layout: one GPU holding all experts and optimizer state has no room for stored activations, while the same model
sharded over expert-parallel ranks leaves most of the memory free, and every layer that is not recomputed saves one
forward pass of that layer per micro-batch.

The planner works from measurements, in three training steps:

1. step with every layer recomputed -> peak ``P`` of the allocator;
2. if ``budget * total - P`` leaves room, the last layer runs without recomputation and reports the bytes its forward
   left allocated (``A`` = stored activations of one layer for one micro-batch);
3. ``n = floor((budget * total - P2) / A)`` further layers stop recomputing, counted from the last layer (their
   activations are the first to be freed in backward).  All ranks take the minimum of their ``n``: ranks must run the
   same sequence of collectives, and a recomputed layer runs its forward collectives twice."""
from __future__ import annotations

from typing import Any, List, Optional

import torch


class YvRecomputePlanner:
    def __init__(self, model: torch.nn.Module, device: torch.device, budget: float = 0.95, min_headroom_gb: float = 6.0,
                 group: Any = None):
        self.layers: List[Any] = list(model.model.layers)
        self.device, self.budget, self.min_headroom = device, budget, min_headroom_gb * 2 ** 30
        self.group = group
        self.stage = 0 if (device.type == "cuda" and self.layers) else 3
        self.stored_layers = 0
        self.layer_bytes: Optional[int] = None
        self.total = torch.cuda.get_device_properties(device).total_memory if device.type == "cuda" else 0

    def _agree(self, n: int) -> int:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([n], device=self.device, dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
            n = int(t.item())
        return n

    def before_step(self) -> None:
        if self.stage == 0:
            for l in self.layers:
                l.use_recompute = True
            torch.cuda.reset_peak_memory_stats(self.device)

    def after_step(self) -> None:
        """Called after the optimizer step of each of the first training steps."""
        if self.stage >= 3:
            return
        peak = torch.cuda.max_memory_allocated(self.device)
        # Memory that the caching allocator does not see (symmetric heaps of the peer-memory kernels, NCCL buffers,
        # the CUDA context) comes off the budget: device-wide usage minus what the allocator holds.
        free_now, total_now = torch.cuda.mem_get_info(self.device)
        outside = max(0, (total_now - free_now) - torch.cuda.memory_reserved(self.device))
        limit = int(self.budget * self.total) - outside
        if self.stage == 0:
            room = self._agree(1 if limit - peak > self.min_headroom else 0)
            if not room:
                self.stage = 3
                return
            last = self.layers[-1]
            last.use_recompute = False
            last.measure_stored = True
            torch.cuda.reset_peak_memory_stats(self.device)
            self.stage = 1
            return
        if self.stage == 1:
            last = self.layers[-1]
            last.measure_stored = False
            a = int(getattr(last, "stored_bytes", 0))
            self.layer_bytes = a
            n = 0
            if a > 0:
                n = max(0, (limit - peak) // a - 1)          # one layer's worth kept back for allocator fragmentation
            n = self._agree(min(int(n), len(self.layers) - 1))
            for l in self.layers[len(self.layers) - 1 - n:]:
                l.use_recompute = False
            self.stored_layers = n + 1
            self.stage = 3

    def summary(self) -> str:
        return (f"{self.stored_layers}/{len(self.layers)} layers keep their activations"
                + (f" ({self.layer_bytes / 2 ** 30:.2f} GiB each per micro-batch)" if self.layer_bytes else ""))
