"""Run management: on-disk run records, control channel, heartbeat, crash detection and recovery, GPU allocation.

Mirrors ``opss/run`` of the reference: ``.pisceslx/runs/<id>/{spec.json,state.json,events.jsonl,metrics.jsonl,
control.jsonl,artifacts.json}`` (store.py:57-210) written atomically under a file lock (lock.py), a controller that
spawns detached ``manage.py`` processes (controller.py:347), control messages polled by the training process
(tools/train/run_reporter.py:183-258), a heartbeat monitor that raises alerts on silence (monitor.py:326-413), crash
detection = state says running but the pid is gone (recovery.py:259-293), newest-checkpoint discovery (:295-410),
restart bookkeeping (:452-499), a state guard with a content signature (state_guard.py:420-424), a task queue with
priorities (queue.py) and a GPU allocation scheduler over ``nvidia-smi``/NVML readings (gpu_scheduler.py).
"""
from __future__ import annotations

import fcntl
import glob
import hashlib
import heapq
import json
import os
import re
import signal
import subprocess
import sys
import threading
import time
import uuid
from contextlib import contextmanager
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterator, List, Optional


def pisces_home() -> Path:
    return Path(os.environ.get("PISCESLX_HOME", ".pisceslx"))


class PiscesLxRunIdFactory:
    @staticmethod
    def new(prefix: str = "run") -> str:
        return f"{prefix}-{time.strftime('%Y%m%d-%H%M%S')}-{uuid.uuid4().hex[:6]}"


class PiscesLxFileLock:
    def __init__(self, path: Path):
        self.path = Path(path)

    @contextmanager
    def hold(self) -> Iterator[None]:
        self.path.parent.mkdir(parents=True, exist_ok=True)
        with open(self.path, "a+") as f:
            fcntl.flock(f, fcntl.LOCK_EX)
            try:
                yield
            finally:
                fcntl.flock(f, fcntl.LOCK_UN)


def _atomic_write_json(path: Path, obj: Any) -> None:
    tmp = path.with_suffix(path.suffix + f".tmp{os.getpid()}")
    with open(tmp, "w") as f:
        json.dump(obj, f, indent=1, default=str)
    os.replace(tmp, path)


class PiscesLxStateFileCorruptedError(RuntimeError):
    pass


class PiscesLxStateGuard:
    """Protected state file: the JSON body carries a truncated SHA-256 of its content."""

    @staticmethod
    def sign(state: Dict[str, Any]) -> str:
        body = json.dumps({k: v for k, v in state.items() if k != "_sig"}, sort_keys=True, default=str)
        return hashlib.sha256(body.encode()).hexdigest()[:16]

    @classmethod
    def seal(cls, state: Dict[str, Any]) -> Dict[str, Any]:
        s = dict(state)
        s["_sig"] = cls.sign(s)
        return s

    @classmethod
    def verify(cls, state: Dict[str, Any]) -> Dict[str, Any]:
        if "_sig" in state and state["_sig"] != cls.sign(state):
            raise PiscesLxStateFileCorruptedError("state.json content does not match its signature")
        return state


class PiscesLxRunStore:
    def __init__(self, root: Optional[Path] = None):
        self.root = Path(root) if root else pisces_home() / "runs"

    def run_dir(self, run_id: str) -> Path:
        return self.root / run_id

    def _lock(self, run_id: str) -> PiscesLxFileLock:
        return PiscesLxFileLock(self.run_dir(run_id) / ".lock")

    def init_run(self, run_id: str, spec: Dict[str, Any], state: Optional[Dict[str, Any]] = None) -> Path:
        d = self.run_dir(run_id)
        d.mkdir(parents=True, exist_ok=True)
        with self._lock(run_id).hold():
            _atomic_write_json(d / "spec.json", spec)
            _atomic_write_json(d / "state.json", PiscesLxStateGuard.seal(
                state or {"status": "pending", "created": time.time(), "pid": None, "restarts": 0}))
            for name in ("events.jsonl", "metrics.jsonl", "control.jsonl"):
                (d / name).touch()
            _atomic_write_json(d / "artifacts.json", {"checkpoints": []})
        return d

    def read_state(self, run_id: str) -> Dict[str, Any]:
        with open(self.run_dir(run_id) / "state.json") as f:
            return PiscesLxStateGuard.verify(json.load(f))

    def update_state(self, run_id: str, **kw: Any) -> Dict[str, Any]:
        with self._lock(run_id).hold():
            st = self.read_state(run_id)
            st.update(kw)
            st["updated"] = time.time()
            _atomic_write_json(self.run_dir(run_id) / "state.json", PiscesLxStateGuard.seal(st))
        return st

    def _append(self, run_id: str, name: str, rec: Dict[str, Any]) -> None:
        with self._lock(run_id).hold():
            with open(self.run_dir(run_id) / name, "a") as f:
                f.write(json.dumps(rec, default=str) + "\n")

    def append_event(self, run_id: str, kind: str, **kw: Any) -> None:
        self._append(run_id, "events.jsonl", {"ts": time.time(), "kind": kind, **kw})

    def append_metrics(self, run_id: str, **kw: Any) -> None:
        self._append(run_id, "metrics.jsonl", {"ts": time.time(), **kw})

    def send_control(self, run_id: str, command: str, **kw: Any) -> None:
        self._append(run_id, "control.jsonl", {"ts": time.time(), "command": command, **kw})

    def read_jsonl(self, run_id: str, name: str, start: int = 0) -> List[Dict[str, Any]]:
        p = self.run_dir(run_id) / name
        if not p.exists():
            return []
        out = []
        with open(p) as f:
            for i, line in enumerate(f):
                if i >= start and line.strip():
                    out.append(json.loads(line))
        return out

    def list_runs(self) -> List[str]:
        return sorted(p.name for p in self.root.glob("*") if (p / "state.json").exists()) if self.root.exists() else []

    def add_artifact(self, run_id: str, path: str, kind: str = "checkpoint") -> None:
        with self._lock(run_id).hold():
            p = self.run_dir(run_id) / "artifacts.json"
            a = json.load(open(p))
            a.setdefault("checkpoints", []).append({"path": path, "kind": kind, "ts": time.time()})
            _atomic_write_json(p, a)


class PiscesLxTrainingRunReporter:
    """Trainer callback: writes metrics, polls the control channel (pause / resume / stop / save_ckpt_now /
    adjust_lr), keeps the heartbeat fresh."""

    def __init__(self, store: PiscesLxRunStore, run_id: str, trainer: Any = None):
        self.store, self.run_id, self.trainer = store, run_id, trainer
        self._seen = 0
        self.stop_requested = False
        self.paused = False
        self.heartbeat = PiscesLxHeartbeatMonitor(store, run_id)

    def __call__(self, step_result: Dict[str, Any]) -> None:
        self.store.append_metrics(self.run_id, step=step_result.get("global_step"), loss=step_result.get("loss"),
                                  lr=step_result.get("learning_rate"), grad_norm=step_result.get("grad_norm"),
                                  throughput=step_result.get("token_throughput"))
        self.heartbeat.beat()
        self.poll_control()

    def poll_control(self) -> None:
        msgs = self.store.read_jsonl(self.run_id, "control.jsonl", self._seen)
        self._seen += len(msgs)
        for m in msgs:
            cmd = m.get("command")
            if cmd == "stop":
                self.stop_requested = True
            elif cmd == "pause":
                self.paused = True
            elif cmd == "resume":
                self.paused = False
            elif cmd == "adjust_lr" and self.trainer is not None:
                for g in self.trainer.optimizer.param_groups:
                    g["lr"] = float(m.get("lr", g["lr"]))
            elif cmd == "save_ckpt_now" and self.trainer is not None:
                from .checkpoint import save_checkpoint
                path = f"{self.trainer.cfg.output_dir}/checkpoint_step_{self.trainer.global_step}_{m.get('reason', 'manual')}.pt"
                save_checkpoint(self.trainer, path, keep=0)
                self.store.add_artifact(self.run_id, path)
            self.store.append_event(self.run_id, "control", command=cmd)


class PiscesLxHeartbeatMonitor:
    def __init__(self, store: PiscesLxRunStore, run_id: str, timeout_s: float = 120.0):
        self.store, self.run_id, self.timeout_s = store, run_id, timeout_s

    def beat(self) -> None:
        self.store.update_state(self.run_id, heartbeat=time.time(), pid=os.getpid(), status="running")

    def is_stale(self, now: Optional[float] = None) -> bool:
        st = self.store.read_state(self.run_id)
        hb = st.get("heartbeat")
        return st.get("status") == "running" and hb is not None and ((now or time.time()) - hb) > self.timeout_s


@dataclass
class PiscesLxCheckpointInfo:
    path: str
    step: int
    mtime: float


class PiscesLxTaskRecovery:
    def __init__(self, store: PiscesLxRunStore, max_restarts: int = 3):
        self.store, self.max_restarts = store, max_restarts

    def check_crashed(self, run_id: str) -> bool:
        st = self.store.read_state(run_id)
        if st.get("status") != "running" or not st.get("pid"):
            return False
        try:
            os.kill(int(st["pid"]), 0)
            return False
        except (ProcessLookupError, PermissionError):
            return True

    @staticmethod
    def _readable(path: str) -> bool:
        """A ``torch.save`` file is a zip archive whose directory sits at the end: a file cut short in mid-write
        has none, so opening the archive (no tensor is read) tells the two apart."""
        if os.path.isdir(path):
            return os.path.exists(os.path.join(path, "meta.json")) or bool(os.listdir(path))
        import zipfile
        try:
            with zipfile.ZipFile(path) as z:
                return len(z.namelist()) > 0
        except (zipfile.BadZipFile, OSError):
            return False

    @staticmethod
    def find_latest_checkpoint(directory: str, validate: bool = False) -> Optional[PiscesLxCheckpointInfo]:
        best: Optional[PiscesLxCheckpointInfo] = None
        for f in glob.glob(os.path.join(directory, "checkpoint_step_*.pt")) + glob.glob(
                os.path.join(directory, "checkpoint_step_*_sharded")):
            m = re.search(r"checkpoint_step_(\d+)", os.path.basename(f))
            if not m:
                continue
            if os.path.isfile(f) and os.path.getsize(f) == 0:
                continue                                   # a truncated file is not a checkpoint
            if validate and not PiscesLxTaskRecovery._readable(f):
                continue
            info = PiscesLxCheckpointInfo(f, int(m.group(1)), os.path.getmtime(f))
            if best is None or info.step > best.step:
                best = info
        return best

    def restart_task(self, run_id: str) -> bool:
        st = self.store.read_state(run_id)
        n = int(st.get("restarts", 0))
        if n >= self.max_restarts:
            self.store.update_state(run_id, status="failed", reason="max restarts reached")
            return False
        self.store.update_state(run_id, status="pending", restarts=n + 1, pid=None)
        self.store.append_event(run_id, "restart", attempt=n + 1)
        return True


class PiscesLxRunController:
    def __init__(self, store: Optional[PiscesLxRunStore] = None):
        self.store = store or PiscesLxRunStore()

    def spawn(self, run_id: str, argv: List[str], env: Optional[Dict[str, str]] = None) -> int:
        d = self.store.run_dir(run_id)
        log = open(d / "output.log", "a")
        proc = subprocess.Popen([sys.executable] + argv, stdout=log, stderr=subprocess.STDOUT, start_new_session=True,
                                env={**os.environ, **(env or {})})
        self.store.update_state(run_id, status="running", pid=proc.pid, started=time.time())
        self.store.append_event(run_id, "spawn", pid=proc.pid, argv=argv)
        return proc.pid

    def stop(self, run_id: str, grace_s: float = 10.0) -> None:
        self.store.send_control(run_id, "stop")
        st = self.store.read_state(run_id)
        pid = st.get("pid")
        if not pid:
            return
        t0 = time.time()
        while time.time() - t0 < grace_s:
            try:
                os.kill(int(pid), 0)
            except ProcessLookupError:
                break
            time.sleep(0.2)
        else:
            try:
                os.killpg(os.getpgid(int(pid)), signal.SIGTERM)
            except ProcessLookupError:
                pass
        self.store.update_state(run_id, status="interrupted")


@dataclass(order=True)
class PiscesLxTask:
    priority: int
    created: float
    task_id: str = field(compare=False)
    spec: Dict[str, Any] = field(compare=False, default_factory=dict)


class PiscesLxTaskQueue:
    def __init__(self):
        self._heap: List[PiscesLxTask] = []
        self._lock = threading.Lock()

    def submit(self, spec: Dict[str, Any], priority: int = 10) -> str:
        t = PiscesLxTask(priority, time.time(), PiscesLxRunIdFactory.new("task"), spec)
        with self._lock:
            heapq.heappush(self._heap, t)
        return t.task_id

    def pop(self) -> Optional[PiscesLxTask]:
        with self._lock:
            return heapq.heappop(self._heap) if self._heap else None

    def __len__(self) -> int:
        return len(self._heap)


@dataclass
class PiscesLxGPUInfo:
    index: int
    memory_total_mb: int
    memory_used_mb: int
    utilization: int


class PiscesLxGPUAllocationScheduler:
    """Picks the least-loaded GPUs from a reading of the devices.  ``reader`` returns the readings (the default
    asks NVML / nvidia-smi; tests pass a fake).  Nothing here changes a device setting."""

    def __init__(self, reader: Optional[Callable[[], List[PiscesLxGPUInfo]]] = None):
        self.reader = reader or self._read_nvidia_smi
        self.allocations: Dict[str, List[int]] = {}

    @staticmethod
    def _read_nvidia_smi() -> List[PiscesLxGPUInfo]:
        try:
            out = subprocess.run(["nvidia-smi", "--query-gpu=index,memory.total,memory.used,utilization.gpu",
                                  "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10).stdout
        except Exception:
            return []
        gpus = []
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) == 4:
                gpus.append(PiscesLxGPUInfo(int(f[0]), int(f[1]), int(f[2]), int(f[3]) if f[3].isdigit() else 0))
        return gpus

    def allocate(self, run_id: str, count: int, min_free_mb: int = 0) -> List[int]:
        taken = {i for v in self.allocations.values() for i in v}
        free = [g for g in self.reader() if g.index not in taken and g.memory_total_mb - g.memory_used_mb >= min_free_mb]
        free.sort(key=lambda g: (g.memory_used_mb, g.utilization))
        if len(free) < count:
            raise RuntimeError(f"only {len(free)} GPUs satisfy the request for {count}")
        ids = [g.index for g in free[:count]]
        self.allocations[run_id] = ids
        return ids

    def release(self, run_id: str) -> None:
        self.allocations.pop(run_id, None)
