"""Checkpoint save / load.

Consolidated format = the reference trainer's single ``torch.save`` dict (tools/train/core.py:3042-3058):
``{model_state_dict, adapter_state_dict, optimizer_state_dict, scheduler_state_dict, global_step, best_metric,
config, training_stats, materialized_components, timestamp, metadata}`` with the reference's key names in
``model_state_dict`` (``embed.weight``, ``layers.<i>.attention.q_proj.weight``,
``layers.<i>.mlp.experts.<e>.gate_proj.weight`` ...).  Files: ``checkpoint_step_<N>.pt``, ``best_model.pt``,
``final_model.pt``; the newest three step checkpoints are kept (core.py:3008-3027).  Writes go to a temporary
file and are renamed (opss/train/checkpoint.py:420-432).

Sharded format (new; the reference has no per-rank checkpoint): every rank writes
``<dir>/shard_rank<r>.pt`` with its local tensors plus ``index.json`` describing the mesh; loading into a
different mesh goes through the consolidated key space (``reshard``).  Loaders accept
``model_state_dict | model | state_dict | raw`` like the reference's inference loaders
(tools/infer/core.py:220-226).
"""
from __future__ import annotations

import glob
import json
import os
import queue
import re
import threading
import time
from typing import Any, Dict, List, Optional

import torch


def _atomic_save(obj: Any, path: str) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    tmp = f"{path}.tmp.{os.getpid()}"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def extract_state_dict(obj: Any) -> Dict[str, torch.Tensor]:
    if isinstance(obj, dict):
        for k in ("model_state_dict", "model", "state_dict"):
            if k in obj and isinstance(obj[k], dict):
                return obj[k]
    return obj


def _optimizer_state(opt: torch.optim.Optimizer) -> Dict[str, Any]:
    return opt.state_dict()


def checkpoint_dict(trainer: Any, metadata: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    model = trainer.model
    sd = model.to_reference_state_dict() if hasattr(model, "to_reference_state_dict") else model.state_dict()
    sd = {k: v.cpu() for k, v in sd.items()}
    cfg = getattr(trainer, "cfg", None)
    mcfg = getattr(model, "cfg", None)
    return {
        "model_state_dict": sd,
        "adapter_state_dict": {},
        "optimizer_state_dict": _optimizer_state(trainer.optimizer),
        "scheduler_state_dict": trainer.scheduler.state_dict() if trainer.scheduler is not None else {},
        "global_step": trainer.global_step,
        "best_metric": trainer.best_metric,
        "config": dict(cfg.__dict__) if cfg is not None else {},
        "model_config": mcfg.to_dict() if mcfg is not None else {},
        "training_stats": trainer.training_stats,
        "materialized_components": list(getattr(getattr(model, "model", model), "materialized_components", [])),
        "timestamp": time.time(),
        "metadata": metadata or {},
        "rng_state": _rng_state(),
    }


def _rng_state() -> Dict[str, Any]:
    return {"cpu": torch.get_rng_state(),
            "cuda": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else []}


def _restore_rng(state: Optional[Dict[str, Any]]) -> None:
    """Put the generators back where the checkpoint left them (dropout masks, sampled routing noise and data
    order then continue as in the uninterrupted run).  A state from a machine with another device count is
    restored as far as it matches."""
    if not state:
        return
    try:
        if state.get("cpu") is not None:
            torch.set_rng_state(state["cpu"])
        cuda = state.get("cuda") or []
        if cuda and torch.cuda.is_available():
            for i, st in enumerate(cuda[:torch.cuda.device_count()]):
                torch.cuda.set_rng_state(st, i)
    except Exception as e:                                  # a foreign or damaged state must not block a resume
        print(f"[checkpoint] warning: random-generator state not restored: {e}")


def prune_checkpoints(directory: str, keep: int = 3) -> List[str]:
    files = glob.glob(os.path.join(directory, "checkpoint_step_*.pt"))
    plain = [f for f in files if re.fullmatch(r"checkpoint_step_(\d+)\.pt", os.path.basename(f))]
    plain.sort(key=lambda f: int(re.findall(r"(\d+)", os.path.basename(f))[0]))
    removed = []
    for f in plain[:-keep] if keep > 0 else []:
        os.remove(f)
        removed.append(f)
    return removed


def save_checkpoint(trainer: Any, path: str, metadata: Optional[Dict[str, Any]] = None, keep: int = 3) -> str:
    par = getattr(trainer, "parallel", None)
    # Any multi-rank run writes per-rank shards: under tensor / expert / pipeline parallelism the weights differ
    # per rank, and under plain data parallelism the optimizer state does (ZeRO-1: the momentum and Adam moments
    # of a tensor exist only on its owner), so rank 0's state alone would silently restart (dp-1)/dp of it.
    if par is not None and par.world_size > 1:
        return save_sharded(trainer, os.path.splitext(path)[0] + "_sharded", metadata)
    if par is None or par.rank == 0:
        _atomic_save(checkpoint_dict(trainer, metadata), path)
        prune_checkpoints(os.path.dirname(os.path.abspath(path)), keep)
    return path


def load_checkpoint(trainer: Any, path: str, reset_lr: bool = False, strict: bool = True) -> Dict[str, Any]:
    """Strict model load; optimizer / scheduler state is skipped with a warning when the parameter groups do
    not match (reference core.py:3065-3122, contract pinned by tools/test/test_resume_contract.py)."""
    if not os.path.exists(path) and os.path.isdir(os.path.splitext(path)[0] + "_sharded"):
        path = os.path.splitext(path)[0] + "_sharded"
    if os.path.isdir(path):
        return load_sharded(trainer, path, reset_lr)
    ck = torch.load(path, map_location="cpu", weights_only=False)
    sd = extract_state_dict(ck)
    model = trainer.model
    trunk = getattr(model, "model", model)
    for name in ck.get("materialized_components", []) if isinstance(ck, dict) else []:
        if getattr(trunk, name, None) is None and hasattr(trunk, "materialize"):
            trunk.materialize(name)
    if hasattr(model, "load_reference_state_dict"):
        leftover = model.load_reference_state_dict(sd, strict=strict)
        if strict and leftover:
            raise RuntimeError(f"unexpected keys in checkpoint: {leftover[:8]}")
    else:
        model.load_state_dict(sd, strict=strict)
    warnings: List[str] = []
    if isinstance(ck, dict) and "optimizer_state_dict" in ck and trainer.optimizer is not None:
        saved_groups = ck["optimizer_state_dict"].get("param_groups", [])
        cur_groups = trainer.optimizer.state_dict()["param_groups"]
        same = len(saved_groups) == len(cur_groups) and all(
            len(a["params"]) == len(b["params"]) for a, b in zip(saved_groups, cur_groups))
        if same:
            trainer.optimizer.load_state_dict(ck["optimizer_state_dict"])
        else:
            warnings.append("optimizer state skipped: parameter groups differ from the checkpoint")
    if isinstance(ck, dict) and ck.get("scheduler_state_dict") and trainer.scheduler is not None:
        trainer.scheduler.load_state_dict(ck["scheduler_state_dict"], reset_lr=reset_lr)
    if isinstance(ck, dict):
        trainer.global_step = int(ck.get("global_step", 0))
        trainer.best_metric = ck.get("best_metric", trainer.best_metric)
        if ck.get("training_stats"):
            trainer.training_stats = ck["training_stats"]
        _restore_rng(ck.get("rng_state"))
    for w in warnings:
        print(f"[checkpoint] warning: {w}")
    return {"warnings": warnings, "global_step": trainer.global_step}


# --------------------------------------------------------------------------------------------------
# sharded (per-rank) format
# --------------------------------------------------------------------------------------------------
def save_sharded(trainer: Any, directory: str, metadata: Optional[Dict[str, Any]] = None) -> str:
    par = trainer.parallel
    os.makedirs(directory, exist_ok=True)
    model = trainer.model
    local = {k: v.cpu() for k, v in model.to_reference_state_dict().items()}
    shard = {"model_state_dict": local, "optimizer_state_dict": trainer.optimizer.state_dict(),
             "rank": par.rank, "tp_rank": par.tp_rank, "ep_rank": par.ep_rank, "pp_rank": par.pp_rank,
             "dp_rank": par.dp_rank, "rng_state": _rng_state(),
             "best_metric": trainer.best_metric}
    _atomic_save(shard, os.path.join(directory, f"shard_rank{par.rank}.pt"))
    if par.rank == 0:
        index = {"world_size": par.world_size, "tp": par.tp_size, "ep": par.ep_size, "pp": par.pp_size,
                 "dp": par.dp_size, "global_step": trainer.global_step,
                 "scheduler_state_dict": trainer.scheduler.state_dict(), "metadata": metadata or {},
                 "model_config": model.cfg.to_dict() if hasattr(model, "cfg") else {}, "timestamp": time.time()}
        tmp = os.path.join(directory, "index.json.tmp")
        with open(tmp, "w") as f:
            json.dump(index, f, indent=1, default=str)
        os.replace(tmp, os.path.join(directory, "index.json"))
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
    return directory


def consolidate_sharded(directory: str) -> Dict[str, torch.Tensor]:
    """Merge per-rank shards into one reference-layout state dict (tensor-parallel pieces concatenated along
    their sharded dimension, expert-parallel pieces united, data-parallel replicas deduplicated)."""
    index = json.load(open(os.path.join(directory, "index.json")))
    tp = index["tp"]
    shards = [torch.load(os.path.join(directory, f"shard_rank{r}.pt"), map_location="cpu", weights_only=False)
              for r in range(index["world_size"])]
    out: Dict[str, torch.Tensor] = {}
    col_parallel = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "gate_proj.weight", "up_proj.weight")
    row_parallel = ("o_proj.weight", "down_proj.weight")
    by_key: Dict[str, Dict[int, torch.Tensor]] = {}
    for sh in shards:
        if sh["dp_rank"] >= index["ep"]:
            continue                                   # replicas beyond the first expert-parallel row
        for k, v in sh["model_state_dict"].items():
            by_key.setdefault(k, {})
            if sh["tp_rank"] not in by_key[k] or ".experts." in k:
                by_key[k].setdefault(sh["tp_rank"], v)
    for k, parts in by_key.items():
        is_routed = ".mlp.experts." in k
        if tp > 1 and len(parts) == tp and not is_routed:
            if k.endswith(col_parallel):
                out[k] = torch.cat([parts[t] for t in range(tp)], 0)
                continue
            if k.endswith(row_parallel):
                out[k] = torch.cat([parts[t] for t in range(tp)], 1)
                continue
        out[k] = parts[min(parts)]
    return out


def load_sharded(trainer: Any, directory: str, reset_lr: bool = False) -> Dict[str, Any]:
    par = getattr(trainer, "parallel", None)
    index = json.load(open(os.path.join(directory, "index.json")))
    same_mesh = par is not None and all(index[k] == getattr(par, k + "_size") for k in ("tp", "ep", "pp", "dp"))
    warnings: List[str] = []
    if same_mesh:
        sh = torch.load(os.path.join(directory, f"shard_rank{par.rank}.pt"), map_location="cpu", weights_only=False)
        trainer.model.load_reference_state_dict(sh["model_state_dict"], strict=False)
        try:
            trainer.optimizer.load_state_dict(sh["optimizer_state_dict"])
        except Exception as e:  # mismatch degrades with a warning, like the consolidated path
            warnings.append(f"optimizer state skipped: {e}")
        _restore_rng(sh.get("rng_state"))
        trainer.best_metric = sh.get("best_metric", trainer.best_metric)
    else:
        full = consolidate_sharded(directory)
        load_full_into(trainer.model, full)
        warnings.append(f"optimizer state dropped: the checkpoint's mesh (tp {index['tp']} ep {index['ep']} pp "
                        f"{index['pp']} dp {index['dp']}) differs from the current one, and optimizer state is "
                        "stored per owner rank; momentum and Adam moments restart from zero")
    for w in warnings:
        print(f"[checkpoint] warning: {w}")
    trainer.global_step = int(index.get("global_step", 0))
    if index.get("scheduler_state_dict") and trainer.scheduler is not None:
        trainer.scheduler.load_state_dict(index["scheduler_state_dict"], reset_lr=reset_lr)
    return {"warnings": warnings, "global_step": trainer.global_step, "resharded": not same_mesh}


def load_full_into(model: Any, full: Dict[str, torch.Tensor]) -> None:
    """Load a consolidated (unsharded) state dict into a possibly sharded model: each rank slices what it owns."""
    par = getattr(model, "parallel", None)
    tp = par.tp_size if par is not None else 1
    tr = par.tp_rank if par is not None else 0
    col_parallel = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "gate_proj.weight", "up_proj.weight")
    row_parallel = ("o_proj.weight", "down_proj.weight")
    local: Dict[str, torch.Tensor] = {}
    for k, v in full.items():
        routed = ".mlp.experts." in k
        if tp > 1 and not routed and k.endswith(col_parallel):
            n = v.shape[0] // tp
            v = v[tr * n:(tr + 1) * n]
        elif tp > 1 and not routed and k.endswith(row_parallel):
            n = v.shape[1] // tp
            v = v[:, tr * n:(tr + 1) * n]
        local[k] = v
    model.load_reference_state_dict(local, strict=False)


class AsyncCheckpointWriter:
    """Background writer: ``submit`` snapshots tensors to host memory and returns; a thread does the file IO
    (reference opss/train/checkpoint.py:496-528)."""

    def __init__(self):
        self.q: "queue.Queue" = queue.Queue()
        self.errors: List[str] = []
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self) -> None:
        while True:
            item = self.q.get()
            if item is None:
                return
            obj, path = item
            try:
                _atomic_save(obj, path)
            except Exception as e:
                self.errors.append(f"{path}: {e}")
            finally:
                self.q.task_done()

    def submit(self, trainer: Any, path: str, metadata: Optional[Dict[str, Any]] = None) -> None:
        self.q.put((checkpoint_dict(trainer, metadata), path))

    def wait(self) -> None:
        self.q.join()

    def close(self) -> None:
        self.q.put(None)
