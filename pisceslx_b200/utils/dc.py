"""Platform utilities: logger, metrics, tracing, paths, determinism, device resolution, memory budgets.

Own implementations of what the reference wraps around the ``dmsc`` middleware (utils/dc.py:166-661) and of its
small platform modules (utils/paths.py, seed.py, device.py, host_memory.py, vram_controller.py):

``PiscesLxLogger``       ``ts | LEVEL | name | event=... | msg`` lines to stderr and to
                         ``$PISCESLX_HOME/logs/<name>/output.log``.
``PiscesLxMetrics``      counters / gauges / histograms with a Prometheus text export.
``PiscesLxTracing``      host spans with a Chrome-trace (``chrome://tracing``) exporter, optionally mirrored to NVTX
                         ranges so that Nsight timelines carry the same names.
``PiscesLxPaths``        directory layout under ``.pisceslx``.
``PiscesLxDeterminism``  seeding of python / numpy / torch.
``PiscesLxDeviceResolver`` picks the device and dtype.
``PiscesLxHostMemoryBudget`` / ``PiscesLxVramController``  abort-before-OOM guards (reference core.py:2775-2799).
"""
from __future__ import annotations

import contextlib
import json
import os
import random
import shutil
import sys
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, Iterator, List, Optional

import torch


from .paths import PiscesLxPaths, _home  # noqa: F401,E402  (defined in utils/paths.py)
from .seed import PiscesLxDeterminism  # noqa: F401,E402  (defined in utils/seed.py)


class PiscesLxLogger:
    LEVELS = {"DEBUG": 10, "INFO": 20, "WARNING": 30, "ERROR": 40}

    def __init__(self, name: str, file_path: Optional[str] = None, enable_file: bool = False, level: str = "INFO"):
        self.name, self.level = name, self.LEVELS.get(level.upper(), 20)
        self.file = None
        if enable_file or file_path:
            p = Path(file_path) if file_path else PiscesLxPaths().logs(name.replace(".", "_")) / "output.log"
            p.parent.mkdir(parents=True, exist_ok=True)
            self.file = open(p, "a")
        self._lock = threading.Lock()

    def _emit(self, level: str, msg: str, event: Optional[str], kw: Dict[str, Any]) -> None:
        if self.LEVELS[level] < self.level:
            return
        extra = " ".join(f"{k}={v}" for k, v in kw.items())
        line = f"{time.strftime('%Y-%m-%dT%H:%M:%S')} | {level} | {self.name} | event={event or '-'} | {msg} {extra}".rstrip()
        with self._lock:
            print(line, file=sys.stderr)
            if self.file:
                self.file.write(line + "\n")
                self.file.flush()

    def debug(self, msg: str, event: Optional[str] = None, **kw: Any) -> None:
        self._emit("DEBUG", msg, event, kw)

    def info(self, msg: str, event: Optional[str] = None, **kw: Any) -> None:
        self._emit("INFO", msg, event, kw)

    def warning(self, msg: str, event: Optional[str] = None, **kw: Any) -> None:
        self._emit("WARNING", msg, event, kw)

    def error(self, msg: str, event: Optional[str] = None, **kw: Any) -> None:
        self._emit("ERROR", msg, event, kw)


class PiscesLxMetrics:
    def __init__(self):
        self.counters: Dict[str, float] = {}
        self.gauges: Dict[str, float] = {}
        self.hist: Dict[str, List[float]] = {}
        self._lock = threading.Lock()

    def inc(self, name: str, v: float = 1.0) -> None:
        with self._lock:
            self.counters[name] = self.counters.get(name, 0.0) + v

    def set(self, name: str, v: float) -> None:
        with self._lock:
            self.gauges[name] = v

    def observe(self, name: str, v: float) -> None:
        with self._lock:
            self.hist.setdefault(name, []).append(v)
            del self.hist[name][:-10000]

    def quantile(self, name: str, q: float) -> Optional[float]:
        h = sorted(self.hist.get(name, []))
        return h[min(len(h) - 1, int(q * len(h)))] if h else None

    def prometheus(self) -> str:
        out = []
        for k, v in self.counters.items():
            out += [f"# TYPE {k} counter", f"{k} {v}"]
        for k, v in self.gauges.items():
            out += [f"# TYPE {k} gauge", f"{k} {v}"]
        for k, h in self.hist.items():
            out += [f"# TYPE {k} summary", f"{k}_count {len(h)}", f"{k}_sum {sum(h)}"]
            for q in (0.5, 0.9, 0.99):
                out.append(f'{k}{{quantile="{q}"}} {self.quantile(k, q)}')
        return "\n".join(out) + "\n"


class PiscesLxTracing:
    """Host spans -> Chrome trace; ``nvtx=True`` also pushes an NVTX range for every span."""

    def __init__(self, nvtx: bool = False):
        self.events: List[Dict[str, Any]] = []
        self.nvtx = nvtx and torch.cuda.is_available()
        self._t0 = time.perf_counter()

    @contextlib.contextmanager
    def span(self, name: str, **args: Any) -> Iterator[None]:
        ts = (time.perf_counter() - self._t0) * 1e6
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            if self.nvtx:
                torch.cuda.nvtx.range_pop()
            dur = (time.perf_counter() - self._t0) * 1e6 - ts
            self.events.append({"name": name, "ph": "X", "ts": ts, "dur": dur, "pid": os.getpid(),
                                "tid": threading.get_ident() % 100000, "args": args})

    def export_chrome_trace(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"traceEvents": self.events, "displayTimeUnit": "ms"}, f)


class PiscesLxDeviceResolver:
    @staticmethod
    def resolve(device: Optional[str] = None) -> torch.device:
        if device:
            return torch.device(device)
        if torch.cuda.is_available():
            return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        return torch.device("cpu")

    @staticmethod
    def default_dtype(device: torch.device) -> torch.dtype:
        return torch.bfloat16 if device.type == "cuda" else torch.float32

    @staticmethod
    def describe() -> Dict[str, Any]:
        d: Dict[str, Any] = {"cuda": torch.cuda.is_available(), "devices": []}
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            d["devices"].append({"index": i, "name": p.name, "sm": f"{p.major}{p.minor}", "sms": p.multi_processor_count,
                                 "memory_gb": p.total_memory / 1e9})
        return d


class MemoryBudgetExceeded(RuntimeError):
    pass


class PiscesLxHostMemoryBudget:
    def __init__(self, max_fraction: float = 0.92):
        self.max_fraction = max_fraction

    def usage(self) -> float:
        import psutil
        return psutil.virtual_memory().percent / 100.0

    def guard(self, step: int = 0) -> None:
        u = self.usage()
        if u > self.max_fraction:
            raise MemoryBudgetExceeded(f"host memory at {u:.0%} (> {self.max_fraction:.0%}) at step {step}")


class PiscesLxVramController:
    def __init__(self, max_fraction: float = 0.97, device: Optional[torch.device] = None):
        self.max_fraction, self.device = max_fraction, device

    def usage(self) -> float:
        if not torch.cuda.is_available():
            return 0.0
        free, total = torch.cuda.mem_get_info(self.device)
        return 1.0 - free / total

    def check_and_adjust(self) -> bool:
        """True when memory is above the budget after releasing the allocator's cached blocks."""
        if self.usage() <= self.max_fraction:
            return False
        torch.cuda.empty_cache()
        return self.usage() > self.max_fraction
