"""The checkpoint operator: typed, tagged checkpoints with metadata, retention, best / last tracking, byte-sized shards,
compression and background writes (reference opss/train/checkpoint.py:112-815).

``engine/checkpoint.py`` holds the trainer's own save / load (the consolidated and the per-rank formats); this operator is
the general front for any model / optimizer / scheduler / scaler.

The snapshot is the part that matters on a 180 GB device: the reference takes ``deepcopy(model.state_dict())`` before it
writes (checkpoint.py:349-360), which doubles the model's footprint ON the device.  Here every tensor is copied into a
pinned host buffer (kept and reused from save to save) on a copy stream of its own; the training stream only records an
event and carries on, the writer thread waits for the copies and does the file work.  Device memory use of a save is
zero, and the step that follows overlaps the copy."""
from __future__ import annotations

import gzip
import io
import json
import os
import queue
import random
import threading
import time
from dataclasses import asdict, dataclass, field
from enum import Enum
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..utils.opsc import PiscesLxOperatorInterface


class PiscesLxCheckpointType(str, Enum):
    FULL = "full"
    MODEL_ONLY = "model_only"
    WEIGHTS_ONLY = "weights_only"
    OPTIMIZER_ONLY = "optimizer_only"
    SHARDED = "sharded"


class PiscesLxCompressionType(str, Enum):
    NONE = "none"
    ZSTD = "zstd"
    GZIP = "gzip"


@dataclass
class PiscesLxCheckpointConfig:
    type: PiscesLxCheckpointType = PiscesLxCheckpointType.FULL
    save_dir: str = ".pisceslx/ckpt"
    prefix: str = "checkpoint"
    interval: int = 5000
    max_to_keep: int = 3
    compression: PiscesLxCompressionType = PiscesLxCompressionType.NONE
    save_async: bool = False
    shard_size: int = 2 * 1024 * 1024 * 1024
    save_last: bool = True
    save_best: bool = False
    best_metric: str = "loss"
    best_mode: str = "min"
    include_config: bool = True
    include_rng: bool = True
    include_cuda: bool = True
    safe_saving: bool = True

    def __post_init__(self) -> None:
        self.type = PiscesLxCheckpointType(getattr(self.type, "value", self.type))
        self.compression = PiscesLxCompressionType(getattr(self.compression, "value", self.compression))
        if self.best_mode not in ("min", "max"):
            raise ValueError("best_mode must be min or max")
        Path(self.save_dir).mkdir(parents=True, exist_ok=True)


@dataclass
class PiscesLxCheckpointMetadata:
    path: str
    type: str
    size_bytes: int
    creation_time: float
    global_step: int
    epoch: Optional[int]
    loss: Optional[float]
    metrics: Dict[str, float]
    is_best: bool
    is_last: bool


def _zstd():
    try:
        import zstandard
        return zstandard
    except ImportError:
        return None


class _PinnedSnapshot:
    """Host copies of a nested state (dictionaries, lists, tensors) in pinned buffers that are reused while the shapes stay."""

    def __init__(self) -> None:
        self._buffers: Dict[str, torch.Tensor] = {}
        self._stream: Optional["torch.cuda.Stream"] = None

    def _copy(self, key: str, t: torch.Tensor) -> torch.Tensor:
        if not t.is_cuda:
            return t.detach().clone()
        buf = self._buffers.get(key)
        if buf is None or buf.shape != t.shape or buf.dtype != t.dtype:
            buf = self._buffers[key] = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        buf.copy_(t.detach(), non_blocking=True)
        return buf

    def _walk(self, key: str, obj: Any) -> Any:
        if isinstance(obj, torch.Tensor):
            return self._copy(key, obj)
        if isinstance(obj, dict):
            return {k: self._walk(f"{key}/{k}", v) for k, v in obj.items()}
        if isinstance(obj, (list, tuple)):
            return type(obj)(self._walk(f"{key}/{i}", v) for i, v in enumerate(obj))
        return obj

    def take(self, state: Dict[str, Any]) -> Tuple[Dict[str, Any], Optional["torch.cuda.Event"]]:
        if not torch.cuda.is_available():
            return self._walk("", state), None
        if self._stream is None:
            self._stream = torch.cuda.Stream()
        self._stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._stream):
            out = self._walk("", state)
            ev = torch.cuda.Event()
            ev.record(self._stream)
        return out, ev


class PiscesLxCheckpointOperator(PiscesLxOperatorInterface):
    """``execute({"operation": "save" | "load" | "list" | "delete" | "cleanup", "tag": ..., "model": ..., ...})``; the
    ``save`` / ``load`` / ``load_model`` methods are the same calls with arguments."""

    name = "checkpoint"
    METADATA_FILE = "checkpoints.json"

    def __init__(self, config: Optional[PiscesLxCheckpointConfig] = None):
        self.config = config or PiscesLxCheckpointConfig()
        self.dir = Path(self.config.save_dir)
        self._save_lock = threading.Lock()
        self._meta: Dict[str, PiscesLxCheckpointMetadata] = {}
        self._best: Optional[float] = None
        self._snap = _PinnedSnapshot()
        self._queue: "queue.Queue" = queue.Queue()
        self._worker: Optional[threading.Thread] = None
        self.errors: List[str] = []
        self._load_metadata()

    # -- state -------------------------------------------------------------------------------------------------------------------
    def _build_state_dict(self, model: Optional[nn.Module], optimizer: Any, scheduler: Any, scaler: Any, global_step: int, epoch: Optional[int],
                          metrics: Dict[str, float]) -> Dict[str, Any]:
        c, T = self.config, PiscesLxCheckpointType
        state: Dict[str, Any] = {"epoch": epoch, "global_step": global_step, "metrics": dict(metrics), "config_type": c.type.value}
        if model is not None and c.type in (T.FULL, T.MODEL_ONLY, T.WEIGHTS_ONLY, T.SHARDED):
            state["model_state_dict"] = model.state_dict()
        if optimizer is not None and c.type in (T.FULL, T.OPTIMIZER_ONLY, T.SHARDED):
            state["optimizer_state_dict"] = optimizer.state_dict()
        if c.type in (T.FULL, T.SHARDED):
            if scheduler is not None and hasattr(scheduler, "state_dict"):
                state["scheduler_state_dict"] = scheduler.state_dict()
            if scaler is not None and hasattr(scaler, "state_dict"):
                state["scaler_state_dict"] = scaler.state_dict()
        if c.include_rng and c.type is not T.WEIGHTS_ONLY:
            import numpy
            state["random_state"] = {"python": random.getstate(), "numpy": numpy.random.get_state(), "torch": torch.get_rng_state()}
            if c.include_cuda and torch.cuda.is_available():
                state["cuda_state"] = torch.cuda.get_rng_state_all()
        if c.include_config:
            state["config"] = {"checkpoint_type": c.type.value, "save_time": time.time()}
        return state

    # -- files -------------------------------------------------------------------------------------------------------------------
    def _suffix(self) -> str:
        return {PiscesLxCompressionType.NONE: ".pt", PiscesLxCompressionType.GZIP: ".pt.gz", PiscesLxCompressionType.ZSTD: ".pt.zst"}[self.config.compression]

    def _get_checkpoint_path(self, tag: str) -> Path:
        if self.config.type is PiscesLxCheckpointType.SHARDED:
            return self.dir / tag
        return self.dir / f"{tag}{self._suffix()}"

    def _write(self, obj: Any, path: Path) -> None:
        comp = self.config.compression
        tmp = path.with_name(path.name + f".tmp.{os.getpid()}") if self.config.safe_saving else path
        if comp is PiscesLxCompressionType.NONE:
            torch.save(obj, tmp)
        else:
            buf = io.BytesIO()
            torch.save(obj, buf)
            if comp is PiscesLxCompressionType.GZIP:
                with gzip.open(tmp, "wb", compresslevel=1) as f:
                    f.write(buf.getbuffer())
            else:
                z = _zstd()
                if z is None:
                    raise RuntimeError("zstd compression asked for but the zstandard module is not installed; use gzip or none")
                with open(tmp, "wb") as f:
                    f.write(z.ZstdCompressor(level=3).compress(buf.getbuffer()))
        if tmp != path:
            os.replace(tmp, path)

    @staticmethod
    def _read(path: Path) -> Any:
        name = path.name
        if name.endswith(".gz"):
            with gzip.open(path, "rb") as f:
                return torch.load(io.BytesIO(f.read()), map_location="cpu", weights_only=False)
        if name.endswith(".zst"):
            z = _zstd()
            if z is None:
                raise RuntimeError("the checkpoint is zstd-compressed and the zstandard module is not installed")
            with open(path, "rb") as f:
                return torch.load(io.BytesIO(z.ZstdDecompressor().decompress(f.read())), map_location="cpu", weights_only=False)
        return torch.load(path, map_location="cpu", weights_only=False)

    def _save_regular(self, checkpoint_path: Path, state_dict: Dict[str, Any]) -> bool:
        self._write(state_dict, checkpoint_path)
        return True

    def _save_sharded(self, checkpoint_path: Path, state_dict: Dict[str, Any]) -> bool:
        """Model tensors go into shards of at most ``shard_size`` bytes (a tensor larger than that gets a shard of its own);
        ``index.json`` maps every tensor name to its shard; everything else goes to ``rest`` beside them."""
        checkpoint_path.mkdir(parents=True, exist_ok=True)
        model_sd = state_dict.get("model_state_dict", {})
        shards: List[Dict[str, torch.Tensor]] = [{}]
        size, index = 0, {}
        for k, v in model_sd.items():
            n = v.numel() * v.element_size() if isinstance(v, torch.Tensor) else 0
            if shards[-1] and size + n > self.config.shard_size:
                shards.append({})
                size = 0
            shards[-1][k] = v
            size += n
            index[k] = len(shards) - 1
        suffix = self._suffix()
        for i, sh in enumerate(shards):
            self._write(sh, checkpoint_path / f"shard_{i:05d}{suffix}")
        rest = {k: v for k, v in state_dict.items() if k != "model_state_dict"}
        self._write(rest, checkpoint_path / f"rest{suffix}")
        tmp = checkpoint_path / "index.json.tmp"
        tmp.write_text(json.dumps({"num_shards": len(shards), "suffix": suffix, "weight_map": index}))
        os.replace(tmp, checkpoint_path / "index.json")
        return True

    def _load_sharded(self, checkpoint_path: Path) -> Dict[str, Any]:
        idx = json.loads((checkpoint_path / "index.json").read_text())
        state = self._read(checkpoint_path / f"rest{idx['suffix']}")
        model_sd: Dict[str, torch.Tensor] = {}
        for i in range(idx["num_shards"]):
            model_sd.update(self._read(checkpoint_path / f"shard_{i:05d}{idx['suffix']}"))
        missing = set(idx["weight_map"]) - set(model_sd)
        if missing:
            raise RuntimeError(f"sharded checkpoint is missing {len(missing)} tensors, e.g. {sorted(missing)[:3]}")
        state["model_state_dict"] = model_sd
        return state

    @staticmethod
    def _size(path: Path) -> int:
        if path.is_dir():
            return sum(f.stat().st_size for f in path.iterdir() if f.is_file())
        return path.stat().st_size if path.exists() else 0

    # -- metadata ---------------------------------------------------------------------------------------------------------------
    def _is_best(self, metric_value: float) -> bool:
        if self._best is None:
            return True
        return metric_value < self._best if self.config.best_mode == "min" else metric_value > self._best

    def _update_metadata(self, tag: str, checkpoint_path: Path, state_dict: Dict[str, Any], metrics: Dict[str, float]) -> None:
        c = self.config
        best = False
        if c.save_best and c.best_metric in metrics and self._is_best(float(metrics[c.best_metric])):
            self._best, best = float(metrics[c.best_metric]), True
            for m in self._meta.values():
                m.is_best = False
        for m in self._meta.values():
            m.is_last = False
        loss = metrics.get("loss")
        self._meta[tag] = PiscesLxCheckpointMetadata(str(checkpoint_path), c.type.value, self._size(checkpoint_path), time.time(),
                                                     int(state_dict.get("global_step", 0)), state_dict.get("epoch"),
                                                     float(loss) if loss is not None else None, {k: float(v) for k, v in metrics.items()}, best, True)

    def _manage_checkpoints(self) -> List[str]:
        """Keeps the newest ``max_to_keep``; the best and (with ``save_last``) the last are never removed."""
        c = self.config
        if c.max_to_keep <= 0:
            return []
        order = sorted(self._meta.items(), key=lambda kv: (kv[1].global_step, kv[1].creation_time))
        removable = [t for t, m in order if not m.is_best and not (c.save_last and m.is_last)]
        protected = len(order) - len(removable)
        removed = []
        while removable and protected + len(removable) > c.max_to_keep:
            t = removable.pop(0)
            self._remove_files(Path(self._meta.pop(t).path))
            removed.append(t)
        self._save_metadata()
        return removed

    @staticmethod
    def _remove_files(path: Path) -> None:
        if path.is_dir():
            for f in path.iterdir():
                if f.is_file():
                    f.unlink()
            path.rmdir()
        elif path.exists():
            path.unlink()

    def _load_metadata(self) -> None:
        f = self.dir / self.METADATA_FILE
        if not f.exists():
            return
        try:
            d = json.loads(f.read_text())
        except (OSError, ValueError):
            return
        self._best = d.get("best")
        for tag, m in d.get("checkpoints", {}).items():
            if Path(m["path"]).exists():
                self._meta[tag] = PiscesLxCheckpointMetadata(**m)

    def _save_metadata(self) -> None:
        f = self.dir / self.METADATA_FILE
        tmp = f.with_suffix(".json.tmp")
        tmp.write_text(json.dumps({"best": self._best, "checkpoints": {t: asdict(m) for t, m in self._meta.items()}}, indent=1))
        os.replace(tmp, f)

    # -- operations ----------------------------------------------------------------------------------------------------------------
    def _finish_save(self, tag: str, path: Path, state: Dict[str, Any], metrics: Dict[str, float], event: Any) -> Dict[str, Any]:
        if event is not None:
            event.synchronize()
        with self._save_lock:
            if self.config.type is PiscesLxCheckpointType.SHARDED:
                self._save_sharded(path, state)
            else:
                self._save_regular(path, state)
            self._update_metadata(tag, path, state, metrics)
            removed = self._manage_checkpoints()
        return {"success": True, "path": str(path), "tag": tag, "global_step": state.get("global_step", 0), "removed": removed,
                "is_best": self._meta[tag].is_best}

    def _async_save_worker(self) -> None:
        while True:
            item = self._queue.get()
            try:
                if item is None:
                    return
                try:
                    self._finish_save(*item)
                except Exception as e:                                                  # a failed write must not end the worker
                    self.errors.append(f"{item[0]}: {e}")
            finally:
                self._queue.task_done()

    def _save_checkpoint(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        tag = inputs.get("tag") or f"{self.config.prefix}_{inputs.get('global_step', 0)}"
        metrics = dict(inputs.get("metrics") or {})
        state = self._build_state_dict(inputs.get("model"), inputs.get("optimizer"), inputs.get("scheduler"), inputs.get("scaler"),
                                       int(inputs.get("global_step", 0)), inputs.get("epoch"), metrics)
        if inputs.get("extra"):
            state["extra"] = inputs["extra"]
        path = self._get_checkpoint_path(tag)
        self.wait()                                        # the pinned buffers are reused: an earlier write must be done with them
        snap, event = self._snap.take(state)
        if self.config.save_async:
            if self._worker is None or not self._worker.is_alive():
                self._worker = threading.Thread(target=self._async_save_worker, daemon=True)
                self._worker.start()
            self._queue.put((tag, path, snap, metrics, event))
            return {"success": True, "path": str(path), "tag": tag, "global_step": state["global_step"], "pending": True}
        return self._finish_save(tag, path, snap, metrics, event)

    def wait(self) -> None:
        """Blocks until every queued save is on disk."""
        self._queue.join()

    def _load_checkpoint(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        self.wait()
        tag = inputs["tag"]
        path = Path(self._meta[tag].path) if tag in self._meta else self._find(tag)
        state = self._load_sharded(path) if path.is_dir() else self._read(path)
        strict = bool(inputs.get("strict", True))
        loaded = []
        for key, obj_key in (("model_state_dict", "model"), ("optimizer_state_dict", "optimizer"), ("scheduler_state_dict", "scheduler"),
                             ("scaler_state_dict", "scaler")):
            obj = inputs.get(obj_key)
            if obj is not None and key in state:
                obj.load_state_dict(state[key], strict=strict) if obj_key == "model" else obj.load_state_dict(state[key])
                loaded.append(obj_key)
        if inputs.get("restore_rng") and "random_state" in state:
            import numpy
            rs = state["random_state"]
            random.setstate(rs["python"])
            numpy.random.set_state(rs["numpy"])
            torch.set_rng_state(rs["torch"])
            if "cuda_state" in state and torch.cuda.is_available() and len(state["cuda_state"]) == torch.cuda.device_count():
                torch.cuda.set_rng_state_all(state["cuda_state"])
        return {"success": True, "state": state, "loaded": loaded, "global_step": state.get("global_step", 0), "epoch": state.get("epoch")}

    def _find(self, tag: str) -> Path:
        for cand in (self.dir / tag, self.dir / f"{tag}.pt", self.dir / f"{tag}.pt.gz", self.dir / f"{tag}.pt.zst"):
            if cand.exists():
                return cand
        raise FileNotFoundError(f"no checkpoint {tag!r} under {self.dir}")

    def _list_checkpoints(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        items = sorted(self._meta.items(), key=lambda kv: kv[1].global_step)
        return {"checkpoints": [dict(asdict(m), tag=t) for t, m in items], "count": len(items),
                "best": next((t for t, m in items if m.is_best), None), "last": next((t for t, m in items if m.is_last), None)}

    def _delete_checkpoint(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        self.wait()
        tag = inputs["tag"]
        with self._save_lock:
            m = self._meta.pop(tag, None)
            if m is None:
                return {"deleted": False, "tag": tag}
            self._remove_files(Path(m.path))
            self._save_metadata()
        return {"deleted": True, "tag": tag}

    def _cleanup_old_checkpoints(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        self.wait()
        keep = inputs.get("keep")
        with self._save_lock:
            old = self.config.max_to_keep
            if keep is not None:
                self.config.max_to_keep = int(keep)
            try:
                removed = self._manage_checkpoints()
            finally:
                self.config.max_to_keep = old
        return {"removed": removed, "remaining": len(self._meta)}

    # -- front -------------------------------------------------------------------------------------------------------------------
    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        op = inputs.get("operation")
        if op is None:
            return False
        if op in ("load", "delete"):
            return "tag" in inputs
        return op in ("save", "list", "cleanup")

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        return {"save": self._save_checkpoint, "load": self._load_checkpoint, "list": self._list_checkpoints,
                "delete": self._delete_checkpoint, "cleanup": self._cleanup_old_checkpoints}[inputs["operation"]](inputs)

    def should_save(self, global_step: int) -> bool:
        return self.config.interval > 0 and global_step > 0 and global_step % self.config.interval == 0

    def save(self, tag: Optional[str] = None, model: Optional[nn.Module] = None, optimizer: Any = None, scheduler: Any = None, scaler: Any = None,
             global_step: int = 0, epoch: Optional[int] = None, metrics: Optional[Dict[str, float]] = None) -> Dict[str, Any]:
        return self._save_checkpoint({"tag": tag, "model": model, "optimizer": optimizer, "scheduler": scheduler, "scaler": scaler,
                                      "global_step": global_step, "epoch": epoch, "metrics": metrics or {}})

    def load(self, tag: str) -> Dict[str, Any]:
        return self._load_checkpoint({"tag": tag})["state"]

    def load_model(self, tag: str, model: nn.Module, strict: bool = True) -> bool:
        return "model" in self._load_checkpoint({"tag": tag, "model": model, "strict": strict})["loaded"]

    def shutdown(self) -> None:
        self.wait()
        if self._worker is not None and self._worker.is_alive():
            self._queue.put(None)
            self._worker.join(timeout=30)
        self._worker = None
