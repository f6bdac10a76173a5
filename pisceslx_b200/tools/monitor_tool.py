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
