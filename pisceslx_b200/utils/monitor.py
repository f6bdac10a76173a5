"""System / GPU monitor: host CPU and memory through psutil, GPU memory, utilisation, clocks, power and throttle
reasons through NVML (read-only queries; no device setting is ever changed).  Reference: ``PiscesLxSystemMonitor``
(utils/dc.py:1307) and ``opss/run/monitor.py:94-323``."""
from __future__ import annotations

import time
from typing import Any, Dict, List


class PiscesLxSystemMonitor:
    def __init__(self, nvml: Any = None):
        self.nvml = nvml

    def _nvml(self):
        if self.nvml is not None:
            return self.nvml
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
        except Exception:
            self.nvml = False
        return self.nvml

    def gpus(self) -> List[Dict[str, Any]]:
        n = self._nvml()
        if not n:
            return []
        out = []
        for i in range(n.nvmlDeviceGetCount()):
            h = n.nvmlDeviceGetHandleByIndex(i)
            mem = n.nvmlDeviceGetMemoryInfo(h)
            util = n.nvmlDeviceGetUtilizationRates(h)
            rec = {"index": i, "memory_used_gb": mem.used / 1e9, "memory_total_gb": mem.total / 1e9,
                   "utilization": util.gpu}
            try:
                rec["sm_mhz"] = n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)
                rec["sm_max_mhz"] = n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)
                rec["power_w"] = n.nvmlDeviceGetPowerUsage(h) / 1000.0
                rec["throttle_reasons"] = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(h))
            except Exception:
                pass
            out.append(rec)
        return out

    def snapshot(self) -> Dict[str, Any]:
        import psutil
        vm = psutil.virtual_memory()
        return {"ts": time.time(), "cpu_percent": psutil.cpu_percent(interval=None), "host_memory_used_gb": vm.used / 1e9,
                "host_memory_total_gb": vm.total / 1e9, "gpus": self.gpus()}
