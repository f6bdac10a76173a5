"""Alert rules and rolling statistics for the monitor (reference tools/monitor/alert_manager.py,
tools/monitor/stats_collector.py): threshold rules over monitor snapshots with a hold time and a cool-down, so that
one noisy sample neither fires nor floods."""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, Dict, List, Optional


@dataclass
class PiscesLxAlertRule:
    name: str
    metric: str                          # dotted path into the snapshot, e.g. "gpus.0.memory_used_frac"
    op: str                              # ">" | "<" | ">=" | "<=" | "=="
    threshold: float
    hold_s: float = 0.0                  # the condition must hold this long before the alert fires
    cooldown_s: float = 300.0
    severity: str = "warning"


@dataclass
class PiscesLxAlert:
    rule: str
    severity: str
    value: float
    time: float
    message: str


def _lookup(snapshot: Any, path: str) -> Optional[float]:
    cur = snapshot
    for part in path.split("."):
        if isinstance(cur, (list, tuple)):
            if not part.isdigit() or int(part) >= len(cur):
                return None
            cur = cur[int(part)]
        elif isinstance(cur, dict):
            if part not in cur:
                return None
            cur = cur[part]
        else:
            return None
    try:
        return float(cur)
    except (TypeError, ValueError):
        return None


_OPS: Dict[str, Callable[[float, float], bool]] = {
    ">": lambda a, b: a > b, "<": lambda a, b: a < b, ">=": lambda a, b: a >= b, "<=": lambda a, b: a <= b,
    "==": lambda a, b: a == b}


class PiscesLxAlertManager:
    def __init__(self, rules: List[PiscesLxAlertRule], sinks: Optional[List[Callable[[PiscesLxAlert], None]]] = None,
                 clock: Callable[[], float] = time.time):
        self.rules, self.sinks, self.clock = rules, sinks or [], clock
        self._since: Dict[str, float] = {}
        self._last_fired: Dict[str, float] = {}
        self.history: List[PiscesLxAlert] = []

    def evaluate(self, snapshot: Dict[str, Any]) -> List[PiscesLxAlert]:
        now, fired = self.clock(), []
        for r in self.rules:
            v = _lookup(snapshot, r.metric)
            if v is None or not _OPS[r.op](v, r.threshold):
                self._since.pop(r.name, None)
                continue
            start = self._since.setdefault(r.name, now)
            if now - start < r.hold_s:
                continue
            if now - self._last_fired.get(r.name, float("-inf")) < r.cooldown_s:
                continue
            self._last_fired[r.name] = now
            a = PiscesLxAlert(r.name, r.severity, v, now, f"{r.metric} = {v:g} {r.op} {r.threshold:g}")
            fired.append(a)
            self.history.append(a)
            for s in self.sinks:
                s(a)
        return fired

    @staticmethod
    def default_rules() -> List[PiscesLxAlertRule]:
        return [PiscesLxAlertRule("gpu_memory_high", "gpus.0.memory_used_frac", ">", 0.97, hold_s=30),
                PiscesLxAlertRule("gpu_thermal_throttle", "gpus.0.thermal_throttle", ">=", 1, severity="critical"),
                PiscesLxAlertRule("host_memory_high", "host.memory_percent", ">", 92, hold_s=60),
                PiscesLxAlertRule("throughput_drop", "train.tokens_per_s_ratio", "<", 0.7, hold_s=120)]


class PiscesLxStatsCollector:
    """Rolling window per metric with mean / min / max / p50 / p95 and the ratio of the latest value to the window
    mean (the input of a "throughput dropped" rule)."""

    def __init__(self, window: int = 256):
        self.window = window
        self.series: Dict[str, Deque[float]] = {}

    def add(self, name: str, value: float) -> None:
        self.series.setdefault(name, deque(maxlen=self.window)).append(float(value))

    def summary(self, name: str) -> Dict[str, float]:
        s = sorted(self.series.get(name, ()))
        if not s:
            return {}
        q = lambda p: s[min(len(s) - 1, int(p * (len(s) - 1) + 0.5))]
        mean = sum(s) / len(s)
        last = self.series[name][-1]
        return {"n": len(s), "mean": mean, "min": s[0], "max": s[-1], "p50": q(0.5), "p95": q(0.95), "last": last,
                "last_over_mean": last / mean if mean else 0.0}
