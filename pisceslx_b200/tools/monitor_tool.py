"""The ``manage.py monitor`` tool as classes (reference tools/monitor: config, context manager, data manager, stats
collector, alert manager, display utilities, runner / orchestrator): periodic snapshots from
``utils.monitor.PiscesLxSystemMonitor`` (read-only NVML and psutil queries), rolling statistics and alert rules from
``utils.alerts``, a bounded history on disk, and a plain-text table renderer."""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

from ..utils.alerts import PiscesLxAlert, PiscesLxAlertManager, PiscesLxAlertRule, PiscesLxStatsCollector


@dataclass
class PiscesLxToolsMonitorConfig:
    interval_s: float = 2.0
    history_path: Optional[str] = None
    max_history: int = 2000
    rules: List[PiscesLxAlertRule] = field(default_factory=PiscesLxAlertManager.default_rules)


class PiscesLxMonitorDataManager:
    """Bounded in-memory history, optionally mirrored to a JSONL file (rewritten when it exceeds twice the bound)."""

    def __init__(self, path: Optional[str] = None, max_history: int = 2000):
        self.path, self.max_history = path, max_history
        self.rows: List[Dict[str, Any]] = []
        self._written = 0

    def add(self, row: Dict[str, Any]) -> None:
        self.rows.append(row)
        del self.rows[:-self.max_history]
        if self.path:
            os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
            self._written += 1
            if self._written > 2 * self.max_history:
                with open(self.path, "w") as f:
                    f.writelines(json.dumps(r, default=str) + "\n" for r in self.rows)
                self._written = len(self.rows)
            else:
                with open(self.path, "a") as f:
                    f.write(json.dumps(row, default=str) + "\n")

    def last(self, n: int = 1) -> List[Dict[str, Any]]:
        return self.rows[-n:]


class PiscesLxToolsMonitorDisplayUtils:
    @staticmethod
    def bar(frac: float, width: int = 20) -> str:
        k = max(0, min(width, int(round(frac * width))))
        return "[" + "#" * k + "." * (width - k) + "]"

    @staticmethod
    def table(rows: List[List[str]]) -> str:
        w = [max(len(str(r[i])) for r in rows) for i in range(len(rows[0]))]
        return "\n".join("  ".join(str(c).ljust(w[i]) for i, c in enumerate(r)).rstrip() for r in rows)


class PiscesLxToolsMonitorDisplay:
    def render(self, snap: Dict[str, Any], alerts: List[PiscesLxAlert]) -> str:
        U = PiscesLxToolsMonitorDisplayUtils
        rows = [["gpu", "memory", "", "util", "sm MHz", "power W"]]
        for g in snap.get("gpus", []):
            frac = g.get("memory_used_frac", g["memory_used_gb"] / max(g["memory_total_gb"], 1e-9))
            rows.append([str(g["index"]), f"{g['memory_used_gb']:.1f}/{g['memory_total_gb']:.0f} GB", U.bar(frac),
                         f"{g.get('utilization', 0)}%", str(g.get("sm_mhz", "-")), f"{g.get('power_w', 0):.0f}"])
        host = snap.get("host", {})
        out = U.table(rows) + f"\nhost: cpu {host.get('cpu_percent', 0):.0f}%  memory {host.get('memory_percent', 0):.0f}%"
        for a in alerts:
            out += f"\n! {a.severity}: {a.rule}: {a.message}"
        return out


class PiscesLxToolsMonitorRunner:
    """One monitoring loop: snapshot -> derived fields -> statistics -> alerts -> history -> display."""

    def __init__(self, system_monitor: Any = None, config: Optional[PiscesLxToolsMonitorConfig] = None,
                 out: Callable[[str], None] = print, sleep: Callable[[float], None] = time.sleep):
        if system_monitor is None:
            from ..utils.monitor import PiscesLxSystemMonitor
            system_monitor = PiscesLxSystemMonitor()
        self.sys, self.cfg, self.out, self.sleep = system_monitor, config or PiscesLxToolsMonitorConfig(), out, sleep
        self.data = PiscesLxMonitorDataManager(self.cfg.history_path, self.cfg.max_history)
        self.stats = PiscesLxStatsCollector()
        self.alerts = PiscesLxAlertManager(self.cfg.rules)
        self.display = PiscesLxToolsMonitorDisplay()

    def snapshot(self) -> Dict[str, Any]:
        gpus = self.sys.gpus()
        for g in gpus:
            g["memory_used_frac"] = g["memory_used_gb"] / max(g["memory_total_gb"], 1e-9)
            g["thermal_throttle"] = int(bool(g.get("throttle_reasons", 0) & 0x60))       # hw / sw thermal slowdown bits
        host = self.sys.host() if hasattr(self.sys, "host") else {}
        return {"time": time.time(), "gpus": gpus, "host": host}

    def tick(self) -> Dict[str, Any]:
        snap = self.snapshot()
        for g in snap["gpus"]:
            self.stats.add(f"gpu{g['index']}.memory_used_frac", g["memory_used_frac"])
            self.stats.add(f"gpu{g['index']}.utilization", g.get("utilization", 0))
        fired = self.alerts.evaluate(snap)
        self.data.add(snap)
        self.out(self.display.render(snap, fired))
        return {"snapshot": snap, "alerts": fired}

    def run(self, iterations: int = 0) -> int:
        n = 0
        while iterations == 0 or n < iterations:
            self.tick()
            n += 1
            if iterations == 0 or n < iterations:
                self.sleep(self.cfg.interval_s)
        return n


PiscesLxToolsMonitorOrchestrator = PiscesLxToolsMonitorImpl = PiscesLxToolsMonitorRunner
PiscesLxMonitorAlertManager, PiscesLxMonitorStatsCollector = PiscesLxAlertManager, PiscesLxStatsCollector


# ---- context, cache and configuration helpers of the monitor (reference tools/monitor/context_utils.py, alert_manager.py:30-45, config.py:31-41) ----
class PiscesLxMonitorCache:
    """A small key-value store with an optional time-to-live per entry and a directory per cache name."""

    def __init__(self, root: Optional[str] = None, clock: Callable[[], float] = time.time):
        self._data: Dict[str, Any] = {}
        self._expiry: Dict[str, float] = {}
        self._root, self._clock = root or os.path.join(os.path.expanduser("~"), ".pisceslx", "cache"), clock

    def get_cache_dir(self, name: str) -> str:
        d = os.path.join(self._root, name)
        os.makedirs(d, exist_ok=True)
        return d

    def get(self, key: str, default: Any = None) -> Any:
        t = self._expiry.get(key)
        if t is not None and self._clock() >= t:
            self._data.pop(key, None)
            self._expiry.pop(key, None)
        return self._data.get(key, default)

    def set(self, key: str, value: Any, ttl: Optional[float] = None) -> None:
        self._data[key] = value
        if ttl is not None:
            self._expiry[key] = self._clock() + ttl
        else:
            self._expiry.pop(key, None)

    def __len__(self) -> int:
        return len(self._data)


class PiscesLxCoreEnhancedCacheManager(PiscesLxMonitorCache):
    """The alert side's cache: entries live 300 s unless told otherwise."""

    def set(self, key: str, value: Any, ttl: Optional[float] = 300.0) -> None:
        super().set(key, value, ttl)


class PiscesLxCoreConfigManager:
    def __init__(self, data: Optional[Dict[str, Any]] = None):
        self._data = dict(data or {})

    def get(self, key: str, default: Any = None) -> Any:
        cur: Any = self._data
        for part in key.split("."):
            if not isinstance(cur, dict) or part not in cur:
                return default
            cur = cur[part]
        return cur

    def set(self, key: str, value: Any) -> None:
        cur = self._data
        *path, leaf = key.split(".")
        for part in path:
            cur = cur.setdefault(part, {})
        cur[leaf] = value


class PiscesLxMonitorContext:
    """Shared values and event hooks of one monitor; a hook that raises is dropped from that event, not from the list."""

    def __init__(self) -> None:
        self._ctx: Dict[str, Any] = {}
        self._hooks: List[Callable[[str, Dict[str, Any]], None]] = []
        self.hook_errors: List[str] = []

    def set_context(self, key: str, value: Any) -> None:
        self._ctx[key] = value

    def get_context(self, key: str, default: Any = None) -> Any:
        return self._ctx.get(key, default)

    def add_hook(self, hook: Callable[[str, Dict[str, Any]], None]) -> None:
        self._hooks.append(hook)

    def emit_event(self, event_type: str, data: Optional[Dict[str, Any]] = None, **kwargs: Any) -> int:
        payload = {**(data or {}), **kwargs}
        n = 0
        for h in list(self._hooks):
            try:
                h(event_type, payload)
                n += 1
            except Exception as e:
                self.hook_errors.append(f"{event_type}: {type(e).__name__}: {e}")
        return n


class PiscesLxMonitorUtils:
    """The helpers a monitor asks for: cache, device list (read-only NVML through ``utils.monitor``), filesystem, logger."""

    def __init__(self, cache: Optional[PiscesLxMonitorCache] = None, system_monitor: Any = None, logger: Any = None):
        self._cache, self._sys, self._logger = cache or PiscesLxMonitorCache(), system_monitor, logger

    def get_cache_manager(self) -> PiscesLxMonitorCache:
        return self._cache

    def get_device_manager(self) -> Any:
        if self._sys is None:
            from ..utils.monitor import PiscesLxSystemMonitor
            self._sys = PiscesLxSystemMonitor()
        return self._sys

    def get_fs_manager(self) -> Any:
        from ..utils.core import PiscesLxFilesystem
        return PiscesLxFilesystem()

    def PiscesLxLogger(self) -> Any:
        if self._logger is None:
            import logging
            self._logger = logging.getLogger("PiscesLx.Tools.Monitor")
        return self._logger


class PiscesLxMonitorContextManager(PiscesLxMonitorContext):
    def __init__(self) -> None:
        super().__init__()
        self._utils = PiscesLxMonitorUtils()

    def set_utils(self, cache_manager: Any = None, device_manager: Any = None, fs_manager: Any = None, logger: Any = None) -> None:
        self._utils = PiscesLxMonitorUtils(cache_manager or self._utils._cache, device_manager or self._utils._sys, logger or self._utils._logger)
        self._fs = fs_manager

    def get_cache_manager(self) -> Any:
        return self._utils.get_cache_manager()

    def get_device_manager(self) -> Any:
        return self._utils.get_device_manager()

    def get_fs_manager(self) -> Any:
        return getattr(self, "_fs", None) or self._utils.get_fs_manager()

    def PiscesLxLogger(self) -> Any:
        return self._utils.PiscesLxLogger()
