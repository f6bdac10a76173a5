"""In-job failure detection: rank heartbeats over the rendezvous store, a liveness check the trainer runs between
steps (before its next launch), the status-word check that turns a bounded device-side wait that ran out into a
host exception, and a host-memory guard.

The reference has process-level liveness only: ``PiscesLxHeartbeatMonitor`` (opss/run/monitor.py:326-413) writes
beats into the run store and ``PiscesLxTaskRecovery.check_crashed`` (opss/run/recovery.py:259-293) probes the pid; a
rank failure inside a job ends the whole torchrun group.  Here every rank publishes a counter under
``hb/<rank>`` in the job's key-value store from a host thread; peers read the counters on the host, so a rank that
raised, exited or never joined is seen without touching the GPU, and the survivors stop launching collectives,
write a checkpoint marker and leave.  Failures are injected on the host only (a fake store that drops keys, a rank
that stops beating); no kernel is ever made to fault."""
from __future__ import annotations

import os
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch

from ..ops import KernelStatusError, check_status


class YvRankFailure(RuntimeError):
    def __init__(self, ranks: List[int], reason: str):
        super().__init__(f"rank(s) {ranks} {reason}")
        self.ranks, self.reason = ranks, reason


class CommTimeout(RuntimeError):
    """A bounded wait inside one of the peer-memory kernels ran out (status bit 4) or a pipeline wait did (bit 1)."""


class DictStore:
    """In-process stand-in for the rendezvous store (same ``set`` / ``get`` / ``add`` surface); ``drop`` names keys
    whose writes are lost, which is how tests make a message disappear."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()
        self.drop: set = set()

    def set(self, k: str, v: Any) -> None:
        if k in self.drop:
            return
        with self._lock:
            self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        with self._lock:
            if k not in self._d:
                raise KeyError(k)
            return self._d[k]

    def add(self, k: str, n: int) -> int:
        with self._lock:
            v = int(self._d.get(k, b"0")) + n
            if k not in self.drop:
                self._d[k] = str(v).encode()
            return v

    def check(self, keys: List[str]) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


@dataclass
class YvHeartbeatConfig:
    interval_s: float = 1.0
    timeout_s: float = 10.0
    join_timeout_s: float = 60.0
    prefix: str = "hb"


class YvRankHeartbeat:
    """Publishes ``<prefix>/<rank>`` = "<counter>:<status>" every ``interval_s`` from a daemon thread."""

    def __init__(self, store: Any, rank: int, cfg: Optional[YvHeartbeatConfig] = None):
        self.store, self.rank, self.cfg = store, rank, cfg or YvHeartbeatConfig()
        self._count = 0
        self._status = "ok"
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def key(self, rank: Optional[int] = None) -> str:
        return f"{self.cfg.prefix}/{self.rank if rank is None else rank}"

    def beat(self) -> None:
        self._count += 1
        self.store.set(self.key(), f"{self._count}:{self._status}")

    def start(self) -> "YvRankHeartbeat":
        self.beat()
        self._thread = threading.Thread(target=self._run, daemon=True, name=f"yv-heartbeat-{self.rank}")
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.cfg.interval_s):
            try:
                self.beat()
            except Exception:
                return                                     # the store went away with the job

    def report(self, status: str) -> None:
        """Publish a terminal status ("failed: ...", "left") at once so peers need not wait for the timeout."""
        self._status = status
        try:
            self.beat()
        except Exception:
            pass

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.cfg.interval_s + 1.0)


class YvFailureDetector:
    """Host-side view of the peers' heartbeats.  ``check()`` is called between steps; it raises ``YvRankFailure``
    when a peer reported a failure, left, never joined within ``join_timeout_s`` or stopped beating for
    ``timeout_s``."""

    def __init__(self, store: Any, rank: int, world: int, cfg: Optional[YvHeartbeatConfig] = None,
                 clock: Callable[[], float] = time.monotonic):
        self.store, self.rank, self.world, self.cfg, self.clock = store, rank, world, cfg or YvHeartbeatConfig(), clock
        self._t0 = clock()
        self._last: Dict[int, int] = {}
        self._last_change: Dict[int, float] = {}

    def _read(self, r: int) -> Optional[str]:
        key = f"{self.cfg.prefix}/{r}"
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def poll(self) -> Dict[int, str]:
        """rank -> "ok" | "missing" | "stale" | reported status."""
        now = self.clock()
        out: Dict[int, str] = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            if v is None:
                out[r] = "missing" if now - self._t0 > self.cfg.join_timeout_s else "ok"
                continue
            cnt_s, _, status = v.partition(":")
            cnt = int(cnt_s)
            if status != "ok":
                out[r] = status
                continue
            if self._last.get(r) != cnt:
                self._last[r], self._last_change[r] = cnt, now
            out[r] = "stale" if now - self._last_change.get(r, now) > self.cfg.timeout_s else "ok"
        return out

    def check(self) -> None:
        bad = {r: s for r, s in self.poll().items() if s != "ok"}
        if bad:
            raise YvRankFailure(sorted(bad), "; ".join(f"{r}: {s}" for r, s in sorted(bad.items())))


def check_device_status(device: Optional[torch.device] = None) -> None:
    """Read (and clear) the per-device kernel status word; a wait that ran out becomes ``CommTimeout``."""
    try:
        check_status(device)
    except KernelStatusError as e:
        if e.status_bits & (1 | 4):
            raise CommTimeout(str(e)) from e
        raise


class YvElasticGuard:
    """Bundles heartbeat + detector + status check for the trainer.

    ``before_step()`` runs on the host before anything is launched: peers' liveness first, then the device status of
    the previous step.  On failure it calls ``on_failure`` (by default: write ``failure_rank<r>.json`` beside the
    checkpoints so that the controller's recovery finds the newest checkpoint and re-spawns) and re-raises; the
    caller must not launch further collectives."""

    def __init__(self, store: Any, rank: int, world: int, cfg: Optional[YvHeartbeatConfig] = None,
                 device: Optional[torch.device] = None, on_failure: Optional[Callable[[BaseException], None]] = None,
                 output_dir: Optional[str] = None):
        self.cfg = cfg or YvHeartbeatConfig()
        self.heartbeat = YvRankHeartbeat(store, rank, self.cfg)
        self.detector = YvFailureDetector(store, rank, world, self.cfg)
        self.rank, self.device, self.output_dir = rank, device, output_dir
        self.on_failure = on_failure or self._default_on_failure
        self.failed: Optional[BaseException] = None

    def start(self) -> "YvElasticGuard":
        self.heartbeat.start()
        return self

    def _default_on_failure(self, exc: BaseException) -> None:
        if self.output_dir:
            import json
            os.makedirs(self.output_dir, exist_ok=True)
            with open(os.path.join(self.output_dir, f"failure_rank{self.rank}.json"), "w") as f:
                json.dump({"rank": self.rank, "error": repr(exc), "time": time.time()}, f)

    def before_step(self) -> None:
        try:
            self.detector.check()
            if self.device is not None and self.device.type == "cuda":
                check_device_status(self.device)
        except (YvRankFailure, CommTimeout) as e:
            self.failed = e
            self.heartbeat.report(f"failed: {type(e).__name__}")
            self.on_failure(e)
            raise

    def leave(self, status: str = "left") -> None:
        """Called between steps with nothing in flight: tell the peers, then stop beating."""
        self.heartbeat.report(status)
        self.heartbeat.stop()

    def guard(self, fn: Callable[[], Any]) -> Any:
        """Run one step; an exception on this rank is published before it propagates."""
        try:
            return fn()
        except BaseException as e:
            self.heartbeat.report(f"failed: {type(e).__name__}")
            raise


class PiscesLxHostMemoryBudget:
    """Aborts a run whose resident set passes the budget, after the caller's ``on_abort`` wrote its emergency
    checkpoint (reference tools/train/core.py:2775-2799)."""

    def __init__(self, limit_gb: float, reader: Optional[Callable[[], float]] = None):
        self.limit_gb = limit_gb
        self.reader = reader or self._rss_gb

    @staticmethod
    def _rss_gb() -> float:
        import psutil
        return psutil.Process().memory_info().rss / 2 ** 30

    def guard(self, step: int, on_abort: Optional[Callable[[int], None]] = None) -> None:
        used = self.reader()
        if used > self.limit_gb:
            if on_abort is not None:
                on_abort(step)
            raise MemoryError(f"host memory {used:.1f} GiB over the budget of {self.limit_gb:.1f} GiB at step {step}")
