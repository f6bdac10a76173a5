"""Training engine: the step loop a user drives through ``YvTrainer.train_step`` / ``fit``.

Covers the reference trainer's contract (tools/train/core.py:2877-2964: gradient accumulation with the
loss divided by the number of micro-batches, non-finite-loss abort, global-norm clipping at 1.0, LR
schedule, step result ``{loss, grad_norm, learning_rate, throughput, token_throughput, global_step,
step_time, did_step}``) and its checkpoint layout (engine.checkpoint).  Differences that matter on B200:
  * every step stages the host batch through pinned memory and an asynchronous H2D copy on a side stream,
    overlapped with the previous micro-batch;
  * step timing uses CUDA events on the compute stream (the reference reads the wall clock without a
    device synchronisation, core.py:2878,2933-2936);
  * with ``streaming_optimizer`` the optimizer consumes gradients inside backward (optim.muon), so a
    model whose weights + momentum nearly fill HBM still trains;
  * data-parallel gradient reduction goes through ``parallel.zero`` (reduce-scatter + sharded update).
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch

from ..ops import check_status
from ..optim import YvLRScheduler, YvLRSchedulerConfig, build_optimizer


class NonFiniteLossError(RuntimeError):
    pass


@dataclass
class YvTrainerConfig:
    micro_batch_size: int = 1               # sequences per forward/backward
    optimizer: str = "muon"
    lr: float = 2e-4
    weight_decay: float = 0.1
    scheduler: str = "cosine"
    warmup_steps: int = 0
    max_steps: int = 1000
    min_lr_ratio: float = 0.1
    clip_grad_norm: float = 1.0
    streaming_optimizer: bool = False       # consume gradients inside backward (memory-lean)
    track_grad_norm: bool = True
    log_steps: int = 10
    save_steps: int = 0
    output_dir: str = ".pisceslx/ckpt"
    abort_on_non_finite: bool = True
    state_dtype: Optional[str] = None       # "bf16" | "fp32" | "int8" (Muon momentum block-quantised) | None (= parameter dtype)
    recompute_policy: str = "config"        # "config": as the model config says; "auto": sized from measured memory
    sharding: str = "zero1"                 # "zero1": optimizer state by owner; "full_shard": ZeRO-3 units per block
    pipeline_schedule: str = "1f1b"         # "1f1b" | "gpipe" (used when the parallel state has pipeline stages)
    optimizer_kwargs: Dict[str, Any] = field(default_factory=dict)


class YvTrainer:
    def __init__(self, model: torch.nn.Module, cfg: YvTrainerConfig, parallel: Any = None,
                 optimizer: Optional[torch.optim.Optimizer] = None):
        self.model, self.cfg, self.parallel = model, cfg, parallel
        self.device = next(model.parameters()).device
        self.fsdp_units = []
        if cfg.sharding == "full_shard" and parallel is not None and getattr(parallel, "dp_size", 1) > 1:
            # parameters, gradients and optimizer state of every block sharded over the data-parallel group
            # (reference: FSDP FULL_SHARD, tools/train/core.py:950-985); element-wise optimizer on the shards
            if parallel.tp_size > 1 or parallel.ep_size > 1 or parallel.pp_size > 1:
                raise ValueError("sharding='full_shard' is a pure data-parallel layout (tp = ep = pp = 1)")
            if cfg.optimizer == "muon":
                raise ValueError("sharding='full_shard' shards matrices element-wise: use optimizer='adamw' "
                                 "(Muon keeps whole matrices per owner under sharding='zero1')")
            from ..parallel import fsdp
            if hasattr(model, "cfg"):
                model.cfg.use_gradient_checkpointing = False      # the units recompute themselves
            for blk in getattr(getattr(model, "model", model), "layers", []):
                if hasattr(blk, "use_recompute"):
                    blk.use_recompute = False
            self.fsdp_units = fsdp.fully_shard(model, parallel.dp_group)
        sd = {"bf16": torch.bfloat16, "fp32": torch.float32, "int8": torch.int8, None: None}[cfg.state_dtype]
        self.optimizer = optimizer or build_optimizer(model, cfg.optimizer, lr=cfg.lr, weight_decay=cfg.weight_decay,
                                                      state_dtype=sd, **cfg.optimizer_kwargs)
        self.scheduler = YvLRScheduler(self.optimizer, YvLRSchedulerConfig(
            scheduler_type=cfg.scheduler, base_lr=cfg.lr, warmup_steps=cfg.warmup_steps, total_steps=cfg.max_steps,
            min_lr_ratio=cfg.min_lr_ratio))
        self.global_step = 0
        self.best_metric = float("inf")
        self.training_stats: Dict[str, List[float]] = {"loss": [], "lr": [], "grad_norm": [], "step_time": []}
        self.callbacks: List[Callable[[Dict[str, Any]], None]] = []
        self.streaming = bool(cfg.streaming_optimizer and hasattr(self.optimizer, "attach_backward_hooks"))
        if self.streaming:
            self.optimizer.attach_backward_hooks(track_grad_norm=cfg.track_grad_norm)
        self.dp = None
        if parallel is not None and getattr(parallel, "world_size", 1) > 1:
            from ..parallel.zero import YvGradientSynchronizer
            self.dp = YvGradientSynchronizer(model, parallel, self.optimizer, streaming=self.streaming)
        self.pipeline = None
        if parallel is not None and getattr(parallel, "pp_size", 1) > 1:
            # this rank holds one stage (a contiguous slice of layers); micro-batches travel between stages over
            # NCCL point-to-point (parallel.pp).  Gradients stay in .grad until the step: no streaming optimizer.
            from ..parallel.pp import YvPipelineStage
            if self.streaming:
                raise ValueError("pipeline parallelism uses the plain optimizer step (streaming_optimizer=False)")
            mcfg = model.cfg
            self.pipeline = YvPipelineStage(model, parallel, mcfg.hidden_size, next(model.parameters()).dtype)
        self._copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.elastic_guard: Any = None                    # parallel.elastic.YvElasticGuard, set by the orchestrator
        self.recompute_planner: Any = None
        if cfg.recompute_policy == "auto" and self.device.type == "cuda" and hasattr(model, "model"):
            from .memory_plan import YvRecomputePlanner
            self.recompute_planner = YvRecomputePlanner(model, self.device)

    # ------------------------------------------------------------------------------------------------
    def _stage(self, t: torch.Tensor) -> torch.Tensor:
        """Host tensor -> device (async from pinned memory on the copy stream)."""
        if t.device == self.device:
            return t
        if self.device.type != "cuda":
            return t.to(self.device)
        if not t.is_pinned():
            t = t.pin_memory()
        self.h2d_bytes += t.numel() * t.element_size()
        with torch.cuda.stream(self._copy_stream):
            d = t.to(self.device, non_blocking=True)
        return d

    def _micro_batches(self, batch: Dict[str, torch.Tensor]):
        n = batch["input_ids"].shape[0]
        mb = max(1, min(self.cfg.micro_batch_size, n))
        chunks = [(i, min(n, i + mb)) for i in range(0, n, mb)]
        staged = None
        for ci, (a, b) in enumerate(chunks):
            cur = staged if staged is not None else {k: self._stage(v[a:b]) for k, v in batch.items()
                                                     if torch.is_tensor(v)}
            if self._copy_stream is not None:
                torch.cuda.current_stream(self.device).wait_stream(self._copy_stream)
            staged = None
            if ci + 1 < len(chunks):                      # prefetch the next micro-batch while this one runs
                a2, b2 = chunks[ci + 1]
                staged = {k: self._stage(v[a2:b2]) for k, v in batch.items() if torch.is_tensor(v)}
            yield ci, len(chunks), cur

    def train_step(self, batch: Dict[str, torch.Tensor]) -> Dict[str, Any]:
        """One optimizer step over ``batch`` (host or device tensors: input_ids [B,S], labels [B,S], optional
        attention_mask; ``images`` [B, n, 3, H, W], ``video`` and ``audio`` reach the model's modality encoders).  Returns the step result; ``loss`` is read back from the device."""
        cfg = self.cfg
        if self.elastic_guard is not None:                # peers' liveness + last step's device status, host only
            self.elastic_guard.before_step()
        if self.recompute_planner is not None:
            self.recompute_planner.before_step()
        self.model.train()
        t0 = time.perf_counter()
        ev0 = ev1 = None
        if self.device.type == "cuda":
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        labels_host = batch.get("labels", batch["input_ids"])
        total_loss = None
        tokens = int(batch["input_ids"].numel())
        n_micro = 1
        if self.pipeline is not None:
            micros = [mb for _, n_micro, mb in self._micro_batches(batch)]
            for m in micros:
                m.setdefault("labels", m["input_ids"])
            if self.dp is not None:
                self.dp.begin_micro_batch(0, len(micros))
            loss = self.pipeline.run(micros, cfg.pipeline_schedule)          # backward included, scaled 1 / n
            # the last stage knows the loss: share it with the other stages for reporting
            t = (loss.detach().float() if loss is not None else torch.zeros((), device=self.device)).reshape(1).to(self.device)
            import torch.distributed as dist
            last_stage = dist.get_global_rank(self.parallel.pp_group, self.parallel.pp_size - 1) \
                if self.parallel.pp_group is not None else 0
            dist.broadcast(t, src=last_stage, group=self.parallel.pp_group)
            total_loss, n_micro = t[0] * len(micros), len(micros)
            micro_iter = ()
        else:
            micro_iter = self._micro_batches(batch)
        for ci, n_micro, mb in micro_iter:
            lab = mb.get("labels", mb["input_ids"])
            a = ci * max(1, min(cfg.micro_batch_size, batch["input_ids"].shape[0]))
            lh = labels_host[a:a + lab.shape[0]]
            num_valid = int((lh[:, 1:] != -100).sum()) if not lh.is_cuda else None
            if self.streaming:
                self.optimizer.begin_micro_batch(ci, n_micro)
            if self.dp is not None:
                self.dp.begin_micro_batch(ci, n_micro)
            modal = {k: mb[k] for k in ("images", "video", "audio") if k in mb}      # multimodal batches
            out = self.model(input_ids=mb["input_ids"], labels=lab, attention_mask=mb.get("attention_mask"),
                             num_valid=num_valid, **modal)
            loss = out["loss"]
            (loss if self.streaming else loss / n_micro).backward()
            total_loss = loss.detach() if total_loss is None else total_loss + loss.detach()
        mean_loss = total_loss / n_micro
        grad_norm = None
        if self.dp is not None:
            self.dp.finish()
        if not self.streaming:
            if cfg.clip_grad_norm and cfg.clip_grad_norm > 0:
                grad_norm = self._clip(cfg.clip_grad_norm)
        elif getattr(self.optimizer, "sq_norm", None) is not None:
            # streaming: gradients were folded into the optimizer state as they were produced, so nothing is left
            # to clip; the norm is reported.  Locally consumed tensors contribute the sum of their per-micro-batch
            # squared norms (an upper estimate of the norm of the mean), data-parallel ones the exact reduced norm.
            sq = self.optimizer.sq_norm / float(n_micro * n_micro)
            if self.dp is not None:
                if self.dp.consumed_sq is not None:
                    sq = sq + self.dp.consumed_sq_total().to(sq.device)
                sq = self.dp.global_sq_norm(sq)
            grad_norm = sq.sqrt()
        self.optimizer.step()
        if self.dp is not None:
            self.dp.after_step()
        if not self.streaming:
            self.optimizer.zero_grad(set_to_none=True)
        lr = self.scheduler.get_last_lr()[0]
        self.scheduler.step()
        self.global_step += 1
        loss_val = float(mean_loss.item())                # D2H read of the step result
        self.d2h_bytes += 4
        if self.recompute_planner is not None:
            self.recompute_planner.after_step()
        step_ms = None
        if ev1 is not None:
            ev1.record()
            ev1.synchronize()
            step_ms = ev0.elapsed_time(ev1)
        wall = time.perf_counter() - t0
        if cfg.abort_on_non_finite and not math.isfinite(loss_val):
            raise NonFiniteLossError(f"non-finite loss {loss_val} at step {self.global_step}")
        if self.device.type == "cuda" and (self.global_step % max(cfg.log_steps, 1) == 0):
            check_status()
        dt = (step_ms / 1e3) if step_ms is not None else wall
        res = {"loss": loss_val, "grad_norm": float(grad_norm) if grad_norm is not None else None,
               "learning_rate": lr, "throughput": batch["input_ids"].shape[0] / dt, "token_throughput": tokens / dt,
               "global_step": self.global_step, "step_time": dt, "did_step": True}
        for k, v in (("loss", loss_val), ("lr", lr), ("step_time", dt)):
            self.training_stats[k].append(v)
            del self.training_stats[k][:-1000]
        for cb in self.callbacks:
            cb(res)
        return res

    def _clip(self, max_norm: float) -> torch.Tensor:
        """Global-norm clipping (reference: ``clip_grad_norm_`` at 1.0, tools/train/core.py:2857-2862).  After the
        data-parallel reduction a rank sees ``p.grad`` only for the tensors it owns plus the tensors unique to it,
        so the squared norms are summed over ALL ranks and one coefficient is applied everywhere."""
        params = [p for p in self.model.parameters() if p.grad is not None]
        distributed = self.parallel is not None and getattr(self.parallel, "world_size", 1) > 1
        if not params and not distributed:
            return torch.zeros(())
        sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        sq_rep = torch.zeros(1, dtype=torch.float32, device=self.device)     # copies shared by the tp ranks
        K = None
        if self.device.type == "cuda":
            from ..ops import kernels
            K = kernels()
        for p in params:
            acc = sq_rep if (self.dp is not None and self.dp.norm_weight(p) != 1.0) else sq
            if K is not None:
                K.sumsq(p.grad.contiguous(), acc)
            else:
                acc += p.grad.detach().float().pow(2).sum()
        if self.dp is not None:
            sq = sq + sq_rep / float(self.dp.tp_size)
        if distributed:
            if self.dp is not None:
                sq = self.dp.global_sq_norm(sq)
            else:
                torch.distributed.all_reduce(sq)
        norm = sq.sqrt()
        coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        for p in params:
            if K is not None:
                K.scale_(p.grad, coef, 1.0)
            else:
                p.grad.mul_(coef.to(p.grad.dtype))
        return norm[0]

    # ------------------------------------------------------------------------------------------------
    def fit(self, batches: Iterable[Dict[str, torch.Tensor]], max_steps: Optional[int] = None) -> Dict[str, Any]:
        from .checkpoint import save_checkpoint
        max_steps = max_steps or self.cfg.max_steps
        last: Dict[str, Any] = {}
        try:
            for batch in batches:
                if self.global_step >= max_steps:
                    break
                last = self.train_step(batch)
                if self.cfg.save_steps and self.global_step % self.cfg.save_steps == 0:
                    save_checkpoint(self, f"{self.cfg.output_dir}/checkpoint_step_{self.global_step}.pt")
        finally:
            if self.cfg.save_steps:
                save_checkpoint(self, f"{self.cfg.output_dir}/final_model.pt")
        return last
