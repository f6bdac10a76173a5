"""Run management beyond the store itself (reference opss/run: ``PiscesLxRunAttacher`` attacher.py, ``PiscesLxRunManager``
/ ``PiscesLxRunCleaner`` / ``PiscesLxResourceMonitor`` monitor.py, ``PiscesLxStateReader`` state_guard.py,
``PiscesLxResourceRequirements`` / ``PiscesLxTaskResourceGrant`` / ``PiscesLxResourceLimits`` resources.py,
``PiscesLxRunCLI`` cli.py).  Everything works on the run directories of ``engine.runstore.PiscesLxRunStore``; GPU
figures come from read-only NVML queries through ``utils.monitor``."""
from __future__ import annotations

import json
import os
import shutil
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterator, List, Optional

from .runstore import PiscesLxRunStore, PiscesLxStateGuard


# ------------------------------------------------------------------------------------------------ attach / follow
class PiscesLxRunAttacher:
    """Follows a run's ``events.jsonl`` and ``metrics.jsonl`` like ``tail -f``: each ``poll`` returns the records
    appended since the previous one; ``attach`` loops until the run reaches a final status."""

    FINAL = ("completed", "failed", "stopped", "cancelled")

    def __init__(self, store: PiscesLxRunStore, run_id: str):
        self.store, self.run_id = store, run_id
        self._events_off = self._metrics_off = 0

    def poll(self) -> Dict[str, List[Dict[str, Any]]]:
        ev = self.store.read_jsonl(self.run_id, "events.jsonl", self._events_off)
        me = self.store.read_jsonl(self.run_id, "metrics.jsonl", self._metrics_off)
        self._events_off += len(ev)
        self._metrics_off += len(me)
        return {"events": ev, "metrics": me}

    def attach(self, sink: Callable[[str, Dict[str, Any]], None], poll_interval_s: float = 0.5, follow: bool = True,
               max_idle_polls: int = 0) -> int:
        seen = idle = 0
        while True:
            got = self.poll()
            for kind in ("events", "metrics"):
                for rec in got[kind]:
                    sink(kind, rec)
                    seen += 1
            status = self.store.read_state(self.run_id).get("status")
            idle = 0 if (got["events"] or got["metrics"]) else idle + 1
            if not follow or status in self.FINAL or (max_idle_polls and idle >= max_idle_polls):
                return seen
            time.sleep(poll_interval_s)


# ------------------------------------------------------------------------------------------------ listing / cleaning
class PiscesLxRunManager:
    def __init__(self, store: Optional[PiscesLxRunStore] = None):
        self.store = store or PiscesLxRunStore()

    def list(self, status: Optional[str] = None) -> List[Dict[str, Any]]:
        out = []
        for rid in self.store.list_runs():
            try:
                st = self.store.read_state(rid)
            except Exception as e:
                st = {"status": "corrupted", "error": str(e)}
            if status is None or st.get("status") == status:
                out.append({"run_id": rid, **{k: st.get(k) for k in ("status", "step", "updated", "pid")}})
        return sorted(out, key=lambda r: r.get("updated") or 0, reverse=True)

    def summary(self) -> Dict[str, int]:
        counts: Dict[str, int] = {}
        for r in self.list():
            counts[str(r["status"])] = counts.get(str(r["status"]), 0) + 1
        return counts


class PiscesLxRunCleaner:
    """Deletes run directories that are older than ``max_age_days`` or beyond the newest ``max_runs``, never the
    ones whose status is in ``keep_statuses`` (running, paused by default)."""

    def __init__(self, store: PiscesLxRunStore, max_age_days: float = 30.0, max_runs: int = 1000,
                 keep_statuses: Optional[List[str]] = None, clock: Callable[[], float] = time.time):
        self.store, self.max_age, self.max_runs, self.clock = store, max_age_days * 86400.0, max_runs, clock
        self.keep = set(keep_statuses if keep_statuses is not None else ["running", "paused"])

    def candidates(self) -> List[str]:
        rows = []
        for rid in self.store.list_runs():
            try:
                st = self.store.read_state(rid)
            except Exception:
                st = {"status": "corrupted"}
            ts = st.get("updated") or self.store.run_dir(rid).stat().st_mtime
            rows.append((ts, rid, st.get("status")))
        rows.sort(reverse=True)
        now, out = self.clock(), []
        for i, (ts, rid, status) in enumerate(rows):
            if status in self.keep:
                continue
            if i >= self.max_runs or now - ts > self.max_age:
                out.append(rid)
        return out

    def clean(self, dry_run: bool = False) -> List[str]:
        victims = self.candidates()
        if not dry_run:
            for rid in victims:
                shutil.rmtree(self.store.run_dir(rid), ignore_errors=True)
        return victims


# ------------------------------------------------------------------------------------------------ read-only access
class PiscesLxUnauthorizedWriteError(PermissionError):
    pass


class PiscesLxStateReader:
    """Read-only view of run state for other subsystems (the server's ``/v1/runs``, monitors): reads verify the
    state file's seal; every write method refuses."""

    def __init__(self, store: Optional[PiscesLxRunStore] = None):
        self.store = store or PiscesLxRunStore()

    def read_state(self, run_id: str) -> Optional[Dict[str, Any]]:
        try:
            return self.store.read_state(run_id)
        except FileNotFoundError:
            return None

    def read_records(self, run_id: str, name: str = "events.jsonl", last: int = 50) -> List[Dict[str, Any]]:
        return self.store.read_jsonl(run_id, name)[-last:]

    def write_state(self, *a: Any, **k: Any) -> None:
        raise PiscesLxUnauthorizedWriteError("PiscesLxStateReader is read-only; state is written by the run's owner "
                                             "through PiscesLxRunStore")

    update_state = append_event = send_control = write_state


# ------------------------------------------------------------------------------------------------ resources
@dataclass
class PiscesLxResourceRequirements:
    gpu_count: int = 1
    gpu_memory_mb: int = 24000
    cpu_cores: int = 4
    memory_mb: int = 32000
    storage_mb: int = 0

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PiscesLxResourceRequirements":
        return cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d})


@dataclass
class PiscesLxTaskResourceGrant:
    task_id: str
    gpus: List[int]
    cpu_cores: int
    memory_mb: int
    granted_at: float = field(default_factory=time.time)


class PiscesLxResourceLimits:
    """Admission control for queued tasks on one node: a task is granted GPUs (those with enough free memory and not
    granted to another task), CPU cores and host memory, or is told what is short."""

    def __init__(self, gpus: Callable[[], List[Dict[str, Any]]], cpu_cores: Optional[int] = None,
                 memory_mb: Optional[int] = None):
        import psutil
        self.read_gpus = gpus
        self.cpu_total = cpu_cores if cpu_cores is not None else (os.cpu_count() or 1)
        self.mem_total = memory_mb if memory_mb is not None else int(psutil.virtual_memory().total / 2 ** 20)
        self.grants: Dict[str, PiscesLxTaskResourceGrant] = {}

    def _used(self) -> Dict[str, Any]:
        g = [i for gr in self.grants.values() for i in gr.gpus]
        return {"gpus": set(g), "cpu": sum(gr.cpu_cores for gr in self.grants.values()),
                "mem": sum(gr.memory_mb for gr in self.grants.values())}

    def check_available(self, req: PiscesLxResourceRequirements) -> Dict[str, Any]:
        used = self._used()
        free_gpus = [g["index"] for g in self.read_gpus()
                     if g["index"] not in used["gpus"]
                     and (g["memory_total_gb"] - g["memory_used_gb"]) * 1024 >= req.gpu_memory_mb]
        short = []
        if len(free_gpus) < req.gpu_count:
            short.append(f"gpus: need {req.gpu_count} with {req.gpu_memory_mb} MB free, have {len(free_gpus)}")
        if self.cpu_total - used["cpu"] < req.cpu_cores:
            short.append(f"cpu cores: need {req.cpu_cores}, have {self.cpu_total - used['cpu']}")
        if self.mem_total - used["mem"] < req.memory_mb:
            short.append(f"host memory: need {req.memory_mb} MB, have {self.mem_total - used['mem']} MB")
        return {"ok": not short, "short": short, "gpus": free_gpus[: req.gpu_count]}

    def allocate(self, task_id: str, req: PiscesLxResourceRequirements) -> Optional[PiscesLxTaskResourceGrant]:
        chk = self.check_available(req)
        if not chk["ok"]:
            return None
        grant = PiscesLxTaskResourceGrant(task_id, chk["gpus"], req.cpu_cores, req.memory_mb)
        self.grants[task_id] = grant
        return grant

    def release(self, task_id: str) -> Optional[PiscesLxTaskResourceGrant]:
        return self.grants.pop(task_id, None)

    def utilization(self) -> Dict[str, Any]:
        u = self._used()
        return {"gpus_granted": sorted(u["gpus"]), "cpu_cores_granted": u["cpu"], "cpu_cores_total": self.cpu_total,
                "memory_mb_granted": u["mem"], "memory_mb_total": self.mem_total, "tasks": sorted(self.grants)}


@dataclass
class PiscesLxResourceSnapshot:
    time: float
    host: Dict[str, Any]
    gpus: List[Dict[str, Any]]
    process: Optional[Dict[str, Any]] = None

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


class PiscesLxResourceMonitor:
    """Periodic resource snapshots of the node and, optionally, of one process (a training run's pid), with
    callbacks; the history is bounded."""

    def __init__(self, system_monitor: Any = None, history: int = 512):
        if system_monitor is None:
            from ..utils.monitor import PiscesLxSystemMonitor
            system_monitor = PiscesLxSystemMonitor()
        self.sys, self.max_history = system_monitor, history
        self.history: List[PiscesLxResourceSnapshot] = []
        self.callbacks: List[Callable[[PiscesLxResourceSnapshot], None]] = []

    def add_callback(self, cb: Callable[[PiscesLxResourceSnapshot], None]) -> None:
        self.callbacks.append(cb)

    def snapshot(self, pid: Optional[int] = None) -> PiscesLxResourceSnapshot:
        import psutil
        vm = psutil.virtual_memory()
        host = {"cpu_percent": psutil.cpu_percent(interval=None), "memory_percent": vm.percent,
                "memory_used_gb": vm.used / 1e9}
        proc = None
        if pid is not None:
            try:
                p = psutil.Process(pid)
                proc = {"pid": pid, "rss_gb": p.memory_info().rss / 1e9, "cpu_percent": p.cpu_percent(interval=None),
                        "threads": p.num_threads(), "status": p.status()}
            except psutil.Error:
                proc = {"pid": pid, "status": "gone"}
        snap = PiscesLxResourceSnapshot(time.time(), host, self.sys.gpus(), proc)
        self.history.append(snap)
        del self.history[:-self.max_history]
        for cb in self.callbacks:
            cb(snap)
        return snap

    def last_snapshot(self) -> Optional[PiscesLxResourceSnapshot]:
        return self.history[-1] if self.history else None


# ------------------------------------------------------------------------------------------------ CLI
class PiscesLxRunCLI:
    """``manage.py action <list|status|logs|pause|resume|stop|clean>`` on the run store."""

    def __init__(self, store: Optional[PiscesLxRunStore] = None, out: Callable[[str], None] = print):
        self.store, self.out = store or PiscesLxRunStore(), out

    def run(self, argv: List[str]) -> int:
        if not argv:
            self.out("usage: action <list|status|logs|pause|resume|stop|clean> [run_id]")
            return 2
        cmd, rest = argv[0], argv[1:]
        if cmd == "list":
            for r in PiscesLxRunManager(self.store).list():
                self.out(f"{r['run_id']}\t{r['status']}\tstep={r['step']}")
            return 0
        if cmd == "clean":
            victims = PiscesLxRunCleaner(self.store).clean(dry_run="--dry-run" in rest)
            self.out(f"removed {len(victims)} run(s)")
            return 0
        if not rest:
            self.out(f"{cmd}: run id required")
            return 2
        rid = rest[0]
        if rid not in self.store.list_runs():
            self.out(f"unknown run {rid}")
            return 1
        if cmd == "status":
            self.out(json.dumps(self.store.read_state(rid), indent=1, default=str))
        elif cmd == "logs":
            PiscesLxRunAttacher(self.store, rid).attach(lambda k, r: self.out(f"[{k}] {json.dumps(r, default=str)}"), follow=False)
        elif cmd in ("pause", "resume", "stop"):
            self.store.send_control(rid, cmd)
            self.out(f"sent {cmd} to {rid}")
        else:
            self.out(f"unknown command {cmd}")
            return 2
        return 0
