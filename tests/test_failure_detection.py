"""Failure detection without faulting anything: failures are made on the host (a rank that raises, leaves, never
joins, or whose store writes are dropped), gloo ranks run on CPU, and the one GPU case lets a bounded device-side
wait run out on a flag that nothing sets and reads the status word afterwards."""
import json
import os
import socket
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pisceslx_b200.parallel.elastic import (CommTimeout, DictStore, PiscesLxHostMemoryBudget, YvElasticGuard,
                                            YvFailureDetector, YvHeartbeatConfig, YvRankFailure, YvRankHeartbeat)


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class _Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def test_detector_sees_stale_missing_and_reported_ranks():
    store, clock = DictStore(), _Clock()
    cfg = YvHeartbeatConfig(interval_s=0.01, timeout_s=5.0, join_timeout_s=20.0)
    hb1, hb2 = YvRankHeartbeat(store, 1, cfg), YvRankHeartbeat(store, 2, cfg)
    det = YvFailureDetector(store, 0, 4, cfg, clock=clock)
    hb1.beat(); hb2.beat()
    assert det.poll() == {1: "ok", 2: "ok", 3: "ok"}            # rank 3 has not joined yet: still inside the grace
    clock.t = 4.0
    hb1.beat()
    assert det.poll()[2] == "ok"
    clock.t = 6.0                                               # rank 2 silent for 6 s > 5 s
    hb1.beat()
    st = det.poll()
    assert st[1] == "ok" and st[2] == "stale"
    clock.t = 21.0
    hb1.beat()
    assert det.poll()[3] == "missing"
    hb1.report("failed: ValueError")
    with pytest.raises(YvRankFailure) as ei:
        det.check()
    assert ei.value.ranks == [1, 2, 3] and "ValueError" in ei.value.reason


def test_dropped_heartbeat_messages_are_detected():
    store, clock = DictStore(), _Clock()
    cfg = YvHeartbeatConfig(timeout_s=2.0)
    hb = YvRankHeartbeat(store, 1, cfg)
    det = YvFailureDetector(store, 0, 2, cfg, clock=clock)
    hb.beat()
    det.check()
    store.drop.add("hb/1")                                      # the network loses every later beat of rank 1
    for t in (1.0, 2.5):
        clock.t = t
        hb.beat()
    with pytest.raises(YvRankFailure):
        det.check()


def test_guard_writes_failure_marker_and_publishes_own_exception(tmp_path):
    store = DictStore()
    cfg = YvHeartbeatConfig(interval_s=0.02, timeout_s=0.2)
    g0 = YvElasticGuard(store, 0, 2, cfg, output_dir=str(tmp_path)).start()
    g1 = YvElasticGuard(store, 1, 2, cfg).start()
    g0.before_step()
    with pytest.raises(ZeroDivisionError):
        g1.guard(lambda: 1 / 0)                                 # rank 1's step raises on the host
    g1.heartbeat.stop()
    with pytest.raises(YvRankFailure):
        g0.before_step()
    assert json.load(open(tmp_path / "failure_rank0.json"))["rank"] == 0
    assert store.get("hb/0").decode().endswith("failed: YvRankFailure")
    g0.heartbeat.stop()


def test_host_memory_budget_aborts_after_emergency_checkpoint():
    calls = []
    PiscesLxHostMemoryBudget(10.0, reader=lambda: 5.0).guard(1, calls.append)
    with pytest.raises(MemoryError):
        PiscesLxHostMemoryBudget(10.0, reader=lambda: 11.0).guard(7, calls.append)
    assert calls == [7]


# ---------------------------------------------------------------------------------------------- gloo ranks
def _worker_rank_leaves(rank: int, world: int, port: int, out_dir: str) -> None:
    """Rank 1 leaves between steps (nothing in flight); rank 0 learns of it on the host before its next collective."""
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=__import__("datetime").timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    cfg = YvHeartbeatConfig(interval_s=0.05, timeout_s=1.0)
    guard = YvElasticGuard(store, rank, world, cfg, output_dir=out_dir).start()
    x = torch.ones(4)
    steps_done = 0
    try:
        for step in range(50):
            if rank == 1 and step == 3:
                guard.leave("left")
                break
            guard.before_step()
            if rank == 0 and step >= 3:                         # give the peer's last word time to land
                t0 = time.time()
                while time.time() - t0 < 3.0:
                    guard.before_step()
                    time.sleep(0.05)
            dist.all_reduce(x)
            steps_done += 1
    except YvRankFailure as e:
        with open(os.path.join(out_dir, f"seen_{rank}.json"), "w") as f:
            json.dump({"ranks": e.ranks, "reason": e.reason, "steps": steps_done}, f)
    guard.heartbeat.stop()
    if rank == 0:
        time.sleep(0.5)                                         # keep the store up until the peer is gone


def test_gloo_rank_leaving_is_seen_on_host_before_next_collective(tmp_path):
    port = _free_port()
    mp.spawn(_worker_rank_leaves, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    seen = json.load(open(tmp_path / "seen_0.json"))
    assert seen["ranks"] == [1] and "left" in seen["reason"] and seen["steps"] == 3
    assert (tmp_path / "failure_rank0.json").exists()


def _worker_collective_timeout(rank: int, world: int, port: int, out_dir: str) -> None:
    """Rank 1 never joins the second collective; rank 0's short process-group timeout ends it with an error."""
    import datetime
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=datetime.timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=2))
    x = torch.ones(4)
    dist.all_reduce(x)
    if rank == 1:
        time.sleep(5.0)                                         # withholds its contribution, then exits
        return
    t0 = time.time()
    try:
        dist.all_reduce(x)
        result = "completed"
    except Exception as e:                                      # gloo raises RuntimeError on timeout
        result = type(e).__name__
    with open(os.path.join(out_dir, "timeout.json"), "w") as f:
        json.dump({"result": result, "waited": time.time() - t0}, f)


def test_gloo_short_timeout_ends_collective_with_error(tmp_path):
    port = _free_port()
    mp.spawn(_worker_collective_timeout, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r = json.load(open(tmp_path / "timeout.json"))
    assert r["result"] != "completed" and r["waited"] < 4.5


# ---------------------------------------------------------------------------------------------- recovery of artefacts
def test_truncated_checkpoint_is_skipped_by_recovery(tmp_path):
    from pisceslx_b200.engine.runstore import PiscesLxTaskRecovery
    good = {"model_state_dict": {"w": torch.ones(2)}, "global_step": 10}
    torch.save(good, tmp_path / "checkpoint_step_10.pt")
    torch.save(good, tmp_path / "checkpoint_step_20.pt")
    raw = (tmp_path / "checkpoint_step_20.pt").read_bytes()
    (tmp_path / "checkpoint_step_20.pt").write_bytes(raw[: len(raw) // 2])           # a crash in mid-write
    info = PiscesLxTaskRecovery.find_latest_checkpoint(str(tmp_path), validate=True)
    assert info.step == 10


def test_data_loader_exception_reaches_the_trainer_loop():
    from pisceslx_b200.data.prefetch import PiscesLxPrefetchLoader

    def gen():
        yield {"input_ids": torch.zeros(1, 4, dtype=torch.long)}
        raise OSError("shard unreadable")

    it = iter(PiscesLxPrefetchLoader(gen(), depth=2, device=torch.device("cpu")))
    next(it)
    with pytest.raises(OSError):
        next(it)


# ---------------------------------------------------------------------------------------------- GPU: bounded wait
@pytest.mark.gpu
def test_bounded_peer_wait_runs_out_and_context_stays_usable():
    """Two flag arrays in this GPU's own memory stand for two ranks; nothing ever writes rank 1's slot in rank 0's
    array, so rank 0's barrier wait runs out after its limit, sets the peer-timeout bit and returns."""
    from pisceslx_b200.ops import KernelStatusError, check_status, kernels, status_word
    from pisceslx_b200.parallel.elastic import check_device_status
    dev = torch.device("cuda", 0)
    flags0 = torch.zeros(64, dtype=torch.int32, device=dev)
    flags1 = torch.zeros(64, dtype=torch.int32, device=dev)
    ptrs = torch.tensor([flags0.data_ptr(), flags1.data_ptr()], dtype=torch.int64)
    st = status_word(dev)
    st.zero_()
    t0 = time.time()
    kernels().peer_barrier(ptrs, 0, 1, st)
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 0.5 < waited < 10.0
    assert int(flags1[0]) == 1 and int(flags0[0]) == 1          # its own arrivals were posted
    with pytest.raises(CommTimeout):
        check_device_status(dev)
    check_status(dev)                                           # cleared by the read above
    # the context is intact: a kernel of the same extension runs and gives the right answer
    x = torch.randn(256, 512, device=dev, dtype=torch.bfloat16)
    w = torch.randn(128, 512, device=dev, dtype=torch.bfloat16)
    from pisceslx_b200.ops import functional as F_
    y = F_.linear(x, w)
    assert torch.allclose(y.float(), x.float() @ w.float().t(), atol=0.5, rtol=2e-2)
    # with the peer's flag present the same barrier passes at once
    flags0[1] = 2
    kernels().peer_barrier(ptrs, 0, 2, st)
    torch.cuda.synchronize()
    check_device_status(dev)
