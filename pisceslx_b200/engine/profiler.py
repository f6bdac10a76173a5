"""Step profiler: CUDA-event timing of named phases, peak-memory deltas, tokens/s, an optional per-kernel table from
the PyTorch profiler, and a Chrome-trace of the host spans.

The reference's ``PiscesLxProfilingOperator`` (opss/train/profiler.py:67-539) wraps forward in wall-clock timers and
is wired to trainer actions it does not implement (tools/train/core.py:2882-2953), so it is inert in practice.  This
one implements the ``start_step`` / ``end_step`` actions the trainer calls, times on the device, and is a trainer
callback."""
from __future__ import annotations

import contextlib
import json
import time
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional

import torch

from ..utils.dc import PiscesLxTracing


@dataclass
class PiscesLxProfilingConfig:
    warmup_steps: int = 2
    profile_kernels: bool = False
    nvtx: bool = False
    max_records: int = 1000


class PiscesLxProfilingOperator:
    def __init__(self, cfg: Optional[PiscesLxProfilingConfig] = None, device: Optional[torch.device] = None):
        self.cfg = cfg or PiscesLxProfilingConfig()
        self.device = device or (torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu"))
        self.cuda = self.device.type == "cuda"
        self.tracing = PiscesLxTracing(nvtx=self.cfg.nvtx)
        self.records: List[Dict[str, Any]] = []
        self._open: Dict[str, Any] = {}
        self._step = 0
        self._phase_events: List[Any] = []

    # ---- trainer-facing actions ------------------------------------------------------------------------
    def execute(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        action = inputs.get("action")
        if action == "start_step":
            self.start_step()
            return {"status": "SUCCESS"}
        if action == "end_step":
            return {"status": "SUCCESS", "record": self.end_step(inputs.get("tokens", 0))}
        if action == "summary":
            return {"status": "SUCCESS", "summary": self.summary()}
        return {"status": "FAILED", "error": f"unknown action {action!r}"}

    def start_step(self) -> None:
        self._step += 1
        self._open = {"wall": time.perf_counter()}
        if self.cuda:
            torch.cuda.reset_peak_memory_stats(self.device)
            self._open["mem0"] = torch.cuda.memory_allocated(self.device)
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._open["ev0"] = ev
        self._phase_events = []

    @contextlib.contextmanager
    def phase(self, name: str) -> Iterator[None]:
        """Device-timed sub-range of the current step (forward, backward, optimizer ...)."""
        with self.tracing.span(name, step=self._step):
            if self.cuda:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                yield
                b.record()
                self._phase_events.append((name, a, b))
            else:
                t0 = time.perf_counter()
                yield
                self._phase_events.append((name, t0, time.perf_counter()))

    def end_step(self, tokens: int = 0) -> Dict[str, Any]:
        rec: Dict[str, Any] = {"step": self._step, "tokens": tokens}
        if self.cuda:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            ev1.synchronize()
            rec["step_ms"] = self._open["ev0"].elapsed_time(ev1)
            rec["peak_memory_gb"] = torch.cuda.max_memory_allocated(self.device) / 1e9
            rec["memory_delta_gb"] = (torch.cuda.memory_allocated(self.device) - self._open["mem0"]) / 1e9
            rec["phases_ms"] = {n: a.elapsed_time(b) for n, a, b in self._phase_events}
        else:
            rec["step_ms"] = (time.perf_counter() - self._open["wall"]) * 1e3
            rec["phases_ms"] = {n: (b - a) * 1e3 for n, a, b in self._phase_events}
        if tokens:
            rec["tokens_per_s"] = tokens / (rec["step_ms"] / 1e3)
        if self._step > self.cfg.warmup_steps:
            self.records.append(rec)
            del self.records[:-self.cfg.max_records]
        return rec

    # ---- analysis -----------------------------------------------------------------------------------------
    def summary(self) -> Dict[str, Any]:
        if not self.records:
            return {"steps": 0}
        ms = sorted(r["step_ms"] for r in self.records)
        phases: Dict[str, float] = {}
        for r in self.records:
            for k, v in r.get("phases_ms", {}).items():
                phases[k] = phases.get(k, 0.0) + v
        total = sum(phases.values()) or 1.0
        out = {"steps": len(ms), "step_ms_p50": ms[len(ms) // 2], "step_ms_min": ms[0], "step_ms_max": ms[-1],
               "phase_share": {k: v / total for k, v in phases.items()}}
        tps = [r["tokens_per_s"] for r in self.records if "tokens_per_s" in r]
        if tps:
            out["tokens_per_s_mean"] = sum(tps) / len(tps)
        if phases:
            out["bottleneck"] = max(phases.items(), key=lambda kv: kv[1])[0]
        return out

    def kernel_table(self, fn, row_limit: int = 25) -> str:
        """Run ``fn`` once under the PyTorch profiler and return the per-kernel device-time table."""
        from torch.profiler import ProfilerActivity, profile
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if self.cuda else [])
        with profile(activities=acts) as prof:
            fn()
            if self.cuda:
                torch.cuda.synchronize()
        return prof.key_averages().table(sort_by="cuda_time_total" if self.cuda else "cpu_time_total", row_limit=row_limit)

    def export(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"records": self.records, "summary": self.summary()}, f, indent=1)

    def export_chrome_trace(self, path: str) -> None:
        self.tracing.export_chrome_trace(path)

    def __call__(self, step_result: Dict[str, Any]) -> None:       # trainer callback form
        pass
