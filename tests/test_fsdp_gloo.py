"""FULL_SHARD (ZeRO-3) units on two Gloo ranks reproduce single-process training."""
import json
import os
import socket
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, {root!r})
    import torch
    import torch.distributed as dist
    from pisceslx_b200 import YvConfig
    from pisceslx_b200.models import build_model
    from pisceslx_b200.parallel import fsdp
    out = sys.argv[1]
    world = int(os.environ["WORLD_SIZE"])
    if world > 1:
        dist.init_process_group("gloo")
    rank = dist.get_rank() if world > 1 else 0
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    cfg.n_layer = 3
    cfg.use_gradient_checkpointing = False
    cfg.extra["moe_deterministic"] = True
    model = build_model(cfg, "cpu", torch.float32, seed=7)
    n_before = sum(p.numel() for p in model.parameters())
    units = fsdp.fully_shard(model, None) if world > 1 else []
    n_after = sum(p.numel() for p in model.parameters())
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.0)
    g = torch.Generator().manual_seed(0)
    data = torch.randint(0, 512, (3, 4, 32), generator=g)
    losses = []
    for s in range(3):
        b = data[s]
        if world > 1:
            b = b[rank * 2:(rank + 1) * 2]
        loss = model(input_ids=b, labels=b)["loss"]
        loss.backward()
        if world > 1:
            fsdp.reduce_replicated_gradients(model)
        opt.step(); opt.zero_grad(set_to_none=True)
        l = loss.detach().double().reshape(1)
        if world > 1:
            dist.all_reduce(l); l /= world
        losses.append(float(l))
    res = {{"losses": losses, "n_before": n_before, "n_after": n_after}}
    if world > 1:
        full = units[0].full_parameters()
        res["unit0_keys"] = sorted(full)[:3]
        res["stats"] = units[1].stats
        res["shard"] = units[0].flat_shard.numel()
        res["unit_numel"] = units[0].numel
        # no-grad forward (evaluation) works on the sharded model too
        with torch.no_grad():
            res["eval_loss"] = float(model(input_ids=data[0][:2], labels=data[0][:2])["loss"])
    if rank == 0:
        json.dump(res, open(out, "w"))
    if world > 1:
        dist.destroy_process_group()
""")


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _run(tmp_path, world, tag):
    script = tmp_path / "fsdp_worker.py"
    script.write_text(WORKER.format(root=ROOT))
    out = tmp_path / f"{tag}.json"
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script), str(out)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT))
    logs = [p.communicate(timeout=500)[0].decode()[-3000:] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(logs)
    return json.load(open(out))


@pytest.mark.timeout(900)
def test_full_shard_matches_single_process(tmp_path):
    single = _run(tmp_path, 1, "single")
    sharded = _run(tmp_path, 2, "sharded")
    for a, b in zip(single["losses"], sharded["losses"]):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (single["losses"], sharded["losses"])
    # each rank holds half of every block (padded) plus the replicated embeddings / head
    assert sharded["n_after"] < sharded["n_before"]
    assert sharded["shard"] == (sharded["unit_numel"] + 1) // 2
    # three training steps: one gather in forward and one in the recomputation of backward, one reduce-scatter each
    assert sharded["stats"]["reduce_scatters"] == 3 and sharded["stats"]["gathers"] >= 6
    assert abs(sharded["eval_loss"]) < 20
