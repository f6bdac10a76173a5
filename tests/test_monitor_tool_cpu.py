"""CPU test of the monitor tool with a fake system monitor."""
from __future__ import annotations

import json

from pisceslx_b200.tools.monitor_tool import (PiscesLxMonitorDataManager, PiscesLxToolsMonitorConfig,
                                              PiscesLxToolsMonitorDisplayUtils, PiscesLxToolsMonitorRunner)
from pisceslx_b200.utils.alerts import PiscesLxAlertRule


class FakeSys:
    def __init__(self):
        self.used = 20.0

    def gpus(self):
        return [{"index": 0, "memory_used_gb": self.used, "memory_total_gb": 180.0, "utilization": 97, "sm_mhz": 1550,
                 "power_w": 990.0, "throttle_reasons": 0x4}]

    def host(self):
        return {"cpu_percent": 12.0, "memory_percent": 40.0}


def test_monitor_runner_history_alerts_and_display(tmp_path):
    assert PiscesLxToolsMonitorDisplayUtils.bar(0.5, 10) == "[#####.....]"
    assert PiscesLxToolsMonitorDisplayUtils.table([["a", "bb"], ["ccc", "d"]]) == "a    bb\nccc  d"
    lines, slept = [], []
    sysm = FakeSys()
    cfg = PiscesLxToolsMonitorConfig(interval_s=0.5, history_path=str(tmp_path / "mon" / "history.jsonl"), max_history=3,
                                     rules=[PiscesLxAlertRule("mem", "gpus.0.memory_used_frac", ">", 0.9, cooldown_s=0.0)])
    run = PiscesLxToolsMonitorRunner(sysm, cfg, out=lines.append, sleep=slept.append)
    assert run.run(iterations=2) == 2 and slept == [0.5]
    assert "20.0/180 GB" in lines[0] and "97%" in lines[0] and "host: cpu 12%" in lines[0] and "!" not in lines[0]
    sysm.used = 175.0
    out = run.tick()
    assert len(out["alerts"]) == 1 and "! warning: mem" in lines[-1] and out["snapshot"]["gpus"][0]["thermal_throttle"] == 0
    for _ in range(5):
        run.tick()
    assert len(run.data.rows) == 3 and run.stats.summary("gpu0.memory_used_frac")["max"] > 0.97
    stored = [json.loads(l) for l in open(cfg.history_path)]
    assert 3 <= len(stored) <= 8 and stored[-1]["gpus"][0]["memory_used_gb"] == 175.0
    dm = PiscesLxMonitorDataManager(None, 2)
    for i in range(4):
        dm.add({"i": i})
    assert dm.last(2) == [{"i": 2}, {"i": 3}]
