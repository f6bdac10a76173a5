"""CPU tests of run management: attacher, manager, cleaner, read-only state reader, resource admission, monitor, CLI."""
from __future__ import annotations

import os
import time

import pytest

from pisceslx_b200.engine.runmgmt import (PiscesLxResourceLimits, PiscesLxResourceMonitor, PiscesLxResourceRequirements,
                                          PiscesLxRunAttacher, PiscesLxRunCLI, PiscesLxRunCleaner, PiscesLxRunManager,
                                          PiscesLxStateReader, PiscesLxUnauthorizedWriteError)
from pisceslx_b200.engine.runstore import PiscesLxRunStore


def _store(tmp_path):
    st = PiscesLxRunStore(tmp_path / "runs")
    for i, status in enumerate(["running", "completed", "failed"]):
        rid = f"run-{i}"
        st.init_run(rid, {"stage": "pretrain"})
        st.update_state(rid, status=status, step=10 * i)
    return st


def test_attacher_follows_new_records(tmp_path):
    st = _store(tmp_path)
    at = PiscesLxRunAttacher(st, "run-0")
    st.append_event("run-0", "started")
    st.append_metrics("run-0", loss=2.5)
    got = at.poll()
    assert [e["kind"] for e in got["events"]] == ["started"] and got["metrics"][0]["loss"] == 2.5
    assert at.poll() == {"events": [], "metrics": []}
    st.append_event("run-0", "checkpoint")
    seen = []
    n = at.attach(lambda kind, rec: seen.append((kind, rec.get("kind"))), follow=False)
    assert n == 1 and seen == [("events", "checkpoint")]
    st.update_state("run-1", status="completed")
    assert PiscesLxRunAttacher(st, "run-1").attach(lambda k, r: None, poll_interval_s=0.01) == 0      # final status ends it


def test_manager_cleaner_and_state_reader(tmp_path):
    st = _store(tmp_path)
    mgr = PiscesLxRunManager(st)
    assert {r["run_id"] for r in mgr.list()} == {"run-0", "run-1", "run-2"}
    assert [r["run_id"] for r in mgr.list("failed")] == ["run-2"] and mgr.summary() == {"running": 1, "completed": 1, "failed": 1}
    now = time.time()
    old = PiscesLxRunCleaner(st, max_age_days=1.0, clock=lambda: now + 3 * 86400)
    assert sorted(old.candidates()) == ["run-1", "run-2"]            # the running one is never a candidate
    assert sorted(old.clean(dry_run=True)) == ["run-1", "run-2"] and len(st.list_runs()) == 3
    few = PiscesLxRunCleaner(st, max_age_days=365, max_runs=1, keep_statuses=[])
    victims = few.clean()
    assert len(victims) == 2 and len(st.list_runs()) == 1
    rd = PiscesLxStateReader(st)
    left = st.list_runs()[0]
    assert rd.read_state(left)["status"] in ("running", "completed", "failed") and rd.read_state("nope") is None
    with pytest.raises(PiscesLxUnauthorizedWriteError):
        rd.update_state(left, status="hacked")
    with pytest.raises(PiscesLxUnauthorizedWriteError):
        rd.send_control(left, "stop")


def test_resource_admission_and_monitor():
    gpus = [{"index": i, "memory_total_gb": 180.0, "memory_used_gb": 170.0 if i == 1 else 2.0} for i in range(4)]
    lim = PiscesLxResourceLimits(lambda: gpus, cpu_cores=16, memory_mb=64000)
    req = PiscesLxResourceRequirements(gpu_count=2, gpu_memory_mb=100_000, cpu_cores=8, memory_mb=30000)
    assert PiscesLxResourceRequirements.from_dict({**req.to_dict(), "junk": 1}) == req
    a = lim.allocate("task-a", req)
    assert a.gpus == [0, 2]                                          # GPU 1 has too little free memory
    b = lim.check_available(req)
    assert not b["ok"] and any("gpus" in s for s in b["short"])      # only GPU 3 is left
    assert lim.allocate("task-b", req) is None
    small = PiscesLxResourceRequirements(gpu_count=1, gpu_memory_mb=50_000, cpu_cores=8, memory_mb=30000)
    assert lim.allocate("task-c", small).gpus == [3]
    assert "cpu cores" in " ".join(lim.check_available(small)["short"])
    u = lim.utilization()
    assert u["gpus_granted"] == [0, 2, 3] and u["cpu_cores_granted"] == 16 and u["tasks"] == ["task-a", "task-c"]
    assert lim.release("task-a").task_id == "task-a" and lim.release("task-a") is None

    class FakeSys:
        def gpus(self):
            return gpus
    mon = PiscesLxResourceMonitor(FakeSys(), history=2)
    got = []
    mon.add_callback(got.append)
    for _ in range(3):
        s = mon.snapshot(pid=os.getpid())
    assert len(mon.history) == 2 and len(got) == 3 and s.process["pid"] == os.getpid() and s.process["rss_gb"] > 0
    assert mon.last_snapshot().to_dict()["gpus"][1]["memory_used_gb"] == 170.0
    assert mon.snapshot(pid=2 ** 22 + 12345).process["status"] == "gone"


def test_run_cli(tmp_path):
    st = _store(tmp_path)
    lines = []
    cli = PiscesLxRunCLI(st, out=lines.append)
    assert cli.run([]) == 2
    assert cli.run(["list"]) == 0 and sum("run-" in l for l in lines) == 3
    assert cli.run(["status", "run-2"]) == 0 and '"failed"' in lines[-1]
    assert cli.run(["pause", "run-0"]) == 0 and st.read_jsonl("run-0", "control.jsonl")[-1]["command"] == "pause"
    st.append_event("run-0", "hello")
    assert cli.run(["logs", "run-0"]) == 0 and "hello" in lines[-1]
    assert cli.run(["status", "nope"]) == 1 and cli.run(["status"]) == 2 and cli.run(["frobnicate", "run-0"]) == 2
    assert cli.run(["clean", "--dry-run"]) == 0 and len(st.list_runs()) == 3
