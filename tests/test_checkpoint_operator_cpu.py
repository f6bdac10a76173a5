"""Checkpoint operator: types, retention, best / last, sharding, compression, background writes, metadata reload."""
import json
import random

import pytest
import torch
import torch.nn as nn

from pisceslx_b200.engine.checkpoint_operator import (PiscesLxCheckpointConfig, PiscesLxCheckpointOperator, PiscesLxCheckpointType,
                                                      PiscesLxCompressionType)


def _setup():
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(8, 16), nn.Linear(16, 4))
    opt = torch.optim.AdamW(m.parameters(), lr=1e-2)
    m(torch.randn(2, 8)).sum().backward()
    opt.step()
    sch = torch.optim.lr_scheduler.StepLR(opt, 10)
    return m, opt, sch


def test_full_save_load_round_trip_with_rng(tmp_path):
    m, opt, sch = _setup()
    op = PiscesLxCheckpointOperator(PiscesLxCheckpointConfig(save_dir=str(tmp_path)))
    r = op.execute({"operation": "save", "model": m, "optimizer": opt, "scheduler": sch, "global_step": 7, "epoch": 1, "metrics": {"loss": 0.5}})
    assert r.is_success() and r.output["tag"] == "checkpoint_7" and (tmp_path / "checkpoint_7.pt").exists()
    a, pa = torch.rand(3), random.random()
    m2, opt2, sch2 = _setup()
    with torch.no_grad():
        for p in m2.parameters():
            p.add_(1.0)
    out = op.execute({"operation": "load", "tag": "checkpoint_7", "model": m2, "optimizer": opt2, "scheduler": sch2, "restore_rng": True}).output
    assert out["loaded"] == ["model", "optimizer", "scheduler"] and out["global_step"] == 7 and out["epoch"] == 1
    assert all(torch.equal(x, y) for x, y in zip(m.state_dict().values(), m2.state_dict().values()))
    assert torch.equal(torch.rand(3), a) and random.random() == pa                   # the generator states came back
    st = opt2.state_dict()["state"]
    assert torch.equal(st[0]["exp_avg"], opt.state_dict()["state"][0]["exp_avg"])
    assert not op.execute({"operation": "load"}).is_success() and not op.execute({}).is_success()
    assert not op.execute({"operation": "load", "tag": "nope"}).is_success()


def test_snapshot_is_taken_at_save_time(tmp_path):
    m, opt, _ = _setup()
    op = PiscesLxCheckpointOperator(PiscesLxCheckpointConfig(save_dir=str(tmp_path), save_async=True))
    w0 = m[0].weight.detach().clone()
    r = op.save("a", model=m, global_step=1)
    with torch.no_grad():
        m[0].weight.zero_()                                                          # training goes on while the write is pending
    assert r.get("pending")
    op.wait()
    assert torch.equal(op.load("a")["model_state_dict"]["0.weight"], w0) and op.errors == []
    op.shutdown()


def test_types_select_contents(tmp_path):
    m, opt, sch = _setup()
    for t, has_model, has_opt, has_sched in ((PiscesLxCheckpointType.MODEL_ONLY, True, False, False), (PiscesLxCheckpointType.WEIGHTS_ONLY, True, False, False),
                                              (PiscesLxCheckpointType.OPTIMIZER_ONLY, False, True, False), ("full", True, True, True)):
        op = PiscesLxCheckpointOperator(PiscesLxCheckpointConfig(type=t, save_dir=str(tmp_path / str(getattr(t, "value", t)))))
        op.save("x", model=m, optimizer=opt, scheduler=sch)
        s = op.load("x")
        assert ("model_state_dict" in s) == has_model and ("optimizer_state_dict" in s) == has_opt and ("scheduler_state_dict" in s) == has_sched
        assert ("random_state" in s) == (getattr(t, "value", t) != "weights_only")


def test_retention_keeps_best_and_last(tmp_path):
    m, _, _ = _setup()
    op = PiscesLxCheckpointOperator(PiscesLxCheckpointConfig(save_dir=str(tmp_path), max_to_keep=2, save_best=True))
    for step, loss in ((1, 0.9), (2, 0.2), (3, 0.5), (4, 0.6), (5, 0.7)):
        out = op.save(model=m, global_step=step, metrics={"loss": loss})
    ls = op.execute({"operation": "list"}).output
    assert [c["tag"] for c in ls["checkpoints"]] == ["checkpoint_2", "checkpoint_5"] and ls["best"] == "checkpoint_2" and ls["last"] == "checkpoint_5"
    assert out["removed"] == ["checkpoint_4"] and not (tmp_path / "checkpoint_3.pt").exists()
    # a new operator on the same folder sees the same records
    op2 = PiscesLxCheckpointOperator(PiscesLxCheckpointConfig(save_dir=str(tmp_path), max_to_keep=2, save_best=True))
    assert op2.execute({"operation": "list"}).output["count"] == 2 and op2._best == 0.2
    assert op2.execute({"operation": "delete", "tag": "checkpoint_5"}).output["deleted"]
    assert not op2.execute({"operation": "delete", "tag": "checkpoint_5"}).output["deleted"]
    op.save(model=m, global_step=6)
    assert op.execute({"operation": "cleanup", "keep": 1}).output["remaining"] <= 2
    assert op.should_save(5000) and not op.should_save(5001) and not op.should_save(0)
    with pytest.raises(ValueError):
        PiscesLxCheckpointConfig(save_dir=str(tmp_path), best_mode="median")


def test_sharded_by_bytes_and_gzip(tmp_path):
    m, opt, _ = _setup()
    cfg = PiscesLxCheckpointConfig(type="sharded", save_dir=str(tmp_path), shard_size=600, compression=PiscesLxCompressionType.GZIP)
    op = PiscesLxCheckpointOperator(cfg)
    op.save("s", model=m, optimizer=opt, global_step=3)
    d = tmp_path / "s"
    idx = json.loads((d / "index.json").read_text())
    assert idx["num_shards"] >= 2 and set(idx["weight_map"]) == set(m.state_dict()) and (d / "shard_00000.pt.gz").exists()
    m2, _, _ = _setup()
    with torch.no_grad():
        m2[1].bias.fill_(9.0)
    assert op.load_model("s", m2) and torch.equal(m2[1].bias, m[1].bias)
    assert "optimizer_state_dict" in op.load("s")
    (d / f"shard_{idx['num_shards'] - 1:05d}.pt.gz").unlink()
    assert not op.execute({"operation": "load", "tag": "s"}).is_success()
    assert op.execute({"operation": "delete", "tag": "s"}).output["deleted"] and not d.exists()


def test_zstd_reports_missing_module_or_works(tmp_path):
    m, _, _ = _setup()
    op = PiscesLxCheckpointOperator(PiscesLxCheckpointConfig(save_dir=str(tmp_path), compression="zstd"))
    r = op.execute({"operation": "save", "tag": "z", "model": m})
    try:
        import zstandard  # noqa: F401
        assert r.is_success() and torch.equal(op.load("z")["model_state_dict"]["0.bias"], m[0].bias)
    except ImportError:
        assert not r.is_success() and "zstandard" in r.error
