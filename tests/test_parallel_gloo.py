"""Multi-process CPU tests (Gloo, world_size 2): the parallel layouts must reproduce the single-process model.

Each case spawns its ranks as child processes that train the tiny Yv text MoE (4 layers, hidden 256, 4q/2kv
heads, 8 routed experts top-2 + 1 shared expert) for a few AdamW steps and write their losses; the parent
compares them with a single-process run on the same global batch."""
import json
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, {root!r})
    import torch
    from pisceslx_b200 import YvConfig
    from pisceslx_b200.models import build_model
    from pisceslx_b200.parallel.state import init_parallel, destroy_parallel
    from pisceslx_b200.engine.trainer import YvTrainer, YvTrainerConfig
    tp, ep, steps, out = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    torch.manual_seed(0)
    cp, pp = int(os.environ.get("YV_TEST_CP", "1")), int(os.environ.get("YV_TEST_PP", "1"))
    par = init_parallel(tp=tp, ep=ep, cp=cp, pp=pp, backend="gloo", device=torch.device("cpu"), timeout_s=120)
    cfg = YvConfig.tiny_text_moe(vocab_size=1024)
    cfg.n_layer = 2
    cfg.context_parallel = cp
    if os.environ.get("YV_TEST_UNTIED") == "1":
        cfg.tie_word_embeddings = False
    cfg.tp_split_head = os.environ.get("YV_TEST_SPLIT_HEAD") == "1"
    cfg.context_parallel_mode = os.environ.get("YV_TEST_CP_MODE", "allgather")
    cfg.use_gradient_checkpointing = False
    cfg.extra["moe_deterministic"] = True
    model = build_model(cfg, "cpu", torch.float32, parallel=par if par.world_size > 1 else None, seed=7)
    full = torch.load(sys.argv[5])
    from pisceslx_b200.engine.checkpoint import load_full_into
    load_full_into(model, full)
    clip, batch = float(os.environ.get("YV_TEST_CLIP", "0")), int(os.environ.get("YV_TEST_BATCH", "4"))
    tr = YvTrainer(model, YvTrainerConfig(micro_batch_size=2, optimizer="adamw", lr=1e-3, max_steps=100,
                                          clip_grad_norm=clip, sharding=os.environ.get("YV_TEST_SHARDING", "zero1")),
                   parallel=par if par.world_size > 1 else None)
    g = torch.Generator().manual_seed(0)
    data = torch.randint(0, 1024, (steps, batch, 32), generator=g)
    losses, norms = [], []
    for s in range(steps):
        b = data[s]
        if par.data_size > 1:
            per = b.shape[0] // par.data_size
            b = b[par.data_rank * per:(par.data_rank + 1) * per]
        res = tr.train_step({{"input_ids": b, "labels": b}})
        losses.append(res["loss"])
        norms.append(res["grad_norm"] or 0.0)
    if par.world_size > 1:
        t = torch.tensor(losses, dtype=torch.float64)
        torch.distributed.all_reduce(t, group=par.dp_group) if par.dp_size > 1 else None
        losses = (t / par.dp_size).tolist()
    if par.rank == 0:
        json.dump(losses, open(out, "w"))
        json.dump(norms, open(out + ".norms", "w"))
    destroy_parallel()
""")


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(tmp_path, world, tp, ep, steps, init_path, tag, extra_env=None):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    out = tmp_path / f"loss_{tag}.json"
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2", **(extra_env or {}))
        procs.append(subprocess.Popen([sys.executable, str(script), str(tp), str(ep), str(steps), str(out),
                                       str(init_path)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        logs.append(o.decode()[-3000:])
    assert all(p.returncode == 0 for p in procs), "\n".join(logs)
    return json.load(open(out))


@pytest.fixture(scope="module")
def init_weights(tmp_path_factory):
    sys.path.insert(0, ROOT)
    from pisceslx_b200 import YvConfig
    from pisceslx_b200.models import build_model
    cfg = YvConfig.tiny_text_moe(vocab_size=1024)
    cfg.n_layer = 2
    m = build_model(cfg, "cpu", torch.float32, seed=7)
    p = tmp_path_factory.mktemp("init") / "full.pt"
    torch.save(m.to_reference_state_dict(), p)
    return p


@pytest.mark.timeout(900)
@pytest.mark.parametrize("tp,ep", [(1, 4), (2, 2)])
def test_four_rank_layouts_match_single_process(tmp_path, init_weights, tp, ep):
    # the layouts of a four-GPU node: tp1 x ep4 x dp4 (experts over all ranks) and tp2 x ep2 x dp2
    steps = 3
    single = _run(tmp_path, 1, 1, 1, steps, init_weights, "single4")
    multi = _run(tmp_path, 4, tp, ep, steps, init_weights, f"w4tp{tp}ep{ep}")
    assert len(single) == len(multi) == steps
    for a, b in zip(single, multi):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (single, multi)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("tp,ep", [(1, 2), (2, 1)])
def test_parallel_matches_single_process(tmp_path, init_weights, tp, ep):
    steps = 4
    single = _run(tmp_path, 1, 1, 1, steps, init_weights, "single")
    multi = _run(tmp_path, 2, tp, ep, steps, init_weights, f"tp{tp}ep{ep}")
    assert len(single) == len(multi) == steps
    for a, b in zip(single, multi):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (single, multi)
    assert single[-1] < single[0]


@pytest.mark.timeout(900)
def test_clipping_and_accumulation_under_data_parallel(tmp_path, init_weights):
    """Global-norm clipping at 1.0 with two micro-batches per rank: the data-parallel run must report the same
    gradient norm and the same losses as one process on the same global batch (every rank applies one global
    coefficient; the accumulated gradient is divided by the micro-batch count exactly once)."""
    steps = 3
    env = {"YV_TEST_CLIP": "1.0", "YV_TEST_BATCH": "8"}
    single = _run(tmp_path, 1, 1, 1, steps, init_weights, "clip_single", env)
    n_single = json.load(open(str(tmp_path / "loss_clip_single.json") + ".norms"))
    for tp, ep in [(1, 2), (2, 1)]:
        multi = _run(tmp_path, 2, tp, ep, steps, init_weights, f"clip_tp{tp}ep{ep}", env)
        n_multi = json.load(open(str(tmp_path / f"loss_clip_tp{tp}ep{ep}.json") + ".norms"))
        assert all(n > 0 for n in n_single)
        for a, b in zip(n_single, n_multi):
            assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (tp, ep, n_single, n_multi)
        for a, b in zip(single, multi):
            assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (single, multi)


RESUME_WORKER = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, {root!r})
    import torch
    from pisceslx_b200 import YvConfig
    from pisceslx_b200.models import build_model
    from pisceslx_b200.parallel.state import init_parallel, destroy_parallel
    from pisceslx_b200.engine.trainer import YvTrainer, YvTrainerConfig
    from pisceslx_b200.engine.checkpoint import save_checkpoint, load_checkpoint
    out, ckdir = sys.argv[1], sys.argv[2]
    par = init_parallel(tp=1, ep=1, backend="gloo", device=torch.device("cpu"), timeout_s=120)
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    cfg.n_layer = 2
    cfg.use_gradient_checkpointing = False
    cfg.extra["moe_deterministic"] = True

    def make(seed):
        model = build_model(cfg, "cpu", torch.float32, parallel=par, seed=seed)
        return YvTrainer(model, YvTrainerConfig(micro_batch_size=2, optimizer="adamw", lr=1e-3, max_steps=100,
                                                clip_grad_norm=1.0), parallel=par)

    g = torch.Generator().manual_seed(par.dp_rank)
    data = torch.randint(0, 512, (3, 2, 32), generator=g)
    a = make(7)
    for s in range(2):
        a.train_step({{"input_ids": data[s], "labels": data[s]}})
    path = save_checkpoint(a, os.path.join(ckdir, "checkpoint_step_2.pt"))
    ra = a.train_step({{"input_ids": data[2], "labels": data[2]}})
    sum_a = float(sum(p.double().sum() for p in a.model.parameters()))
    b = make(99)                                            # different weights, empty optimizer state
    info = load_checkpoint(b, os.path.join(ckdir, "checkpoint_step_2.pt"))
    rb = b.train_step({{"input_ids": data[2], "labels": data[2]}})
    sum_b = float(sum(p.double().sum() for p in b.model.parameters()))
    json.dump({{"path": path, "loss_a": ra["loss"], "loss_b": rb["loss"], "sum_a": sum_a, "sum_b": sum_b,
               "step_b": b.global_step, "warnings": info["warnings"]}}, open(out + f".{{par.rank}}", "w"))
    destroy_parallel()
""")


@pytest.mark.timeout(600)
def test_data_parallel_resume_is_bit_equal(tmp_path):
    """ZeRO-1 keeps each tensor's optimizer state on its owner only: a 2-rank data-parallel run must save every
    rank's state and continue after a reload exactly like the uninterrupted run."""
    script = tmp_path / "resume_worker.py"
    script.write_text(RESUME_WORKER.format(root=ROOT))
    out, port = tmp_path / "resume.json", _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script), str(out), str(tmp_path / "ck")], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    logs = [p.communicate(timeout=500)[0].decode()[-3000:] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(logs)
    for r in range(2):
        res = json.load(open(str(out) + f".{r}"))
        assert res["path"].endswith("_sharded") and os.path.isfile(os.path.join(res["path"], f"shard_rank{r}.pt"))
        assert res["warnings"] == [] and res["step_b"] == 3
        assert res["loss_a"] == res["loss_b"] and res["sum_a"] == res["sum_b"], res


@pytest.mark.timeout(900)
def test_trainer_full_shard_matches_single_process(tmp_path, init_weights):
    """``sharding='full_shard'`` through the trainer (two data-parallel ranks, clipping on, two micro-batches per
    rank): same losses and gradient norms as one process."""
    steps = 3
    env = {"YV_TEST_CLIP": "1.0", "YV_TEST_BATCH": "8"}
    single = _run(tmp_path, 1, 1, 1, steps, init_weights, "fs_single", env)
    n_single = json.load(open(str(tmp_path / "loss_fs_single.json") + ".norms"))
    multi = _run(tmp_path, 2, 1, 1, steps, init_weights, "fs_multi", dict(env, YV_TEST_SHARDING="full_shard"))
    n_multi = json.load(open(str(tmp_path / "loss_fs_multi.json") + ".norms"))
    for a, b in zip(n_single, n_multi):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (n_single, n_multi)
    for a, b in zip(single, multi):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (single, multi)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world,cp,mode", [(2, 2, "allgather"), (4, 2, "allgather"), (2, 2, "ring")])
def test_context_parallel_training_matches_single_process(tmp_path, init_weights, world, cp, mode):
    """Sequences split over context-parallel ranks (K / V all-gathered per layer, loss of local positions against the
    globally shifted targets): same losses and gradient norm as one process; with 4 ranks two data shards x cp 2."""
    steps = 3
    env = {"YV_TEST_CLIP": "1.0", "YV_TEST_BATCH": "4"}
    single = _run(tmp_path, 1, 1, 1, steps, init_weights, f"cp_single{world}", env)
    n_single = json.load(open(str(tmp_path / f"loss_cp_single{world}.json") + ".norms"))
    multi = _run(tmp_path, world, 1, 1, steps, init_weights, f"cp_w{world}", dict(env, YV_TEST_CP=str(cp), YV_TEST_CP_MODE=mode))
    n_multi = json.load(open(str(tmp_path / f"loss_cp_w{world}.json") + ".norms"))
    for a, b in zip(single, multi):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (single, multi)
    for a, b in zip(n_single, n_multi):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (n_single, n_multi)


@pytest.mark.timeout(900)
def test_pipeline_parallel_through_the_trainer_matches_single_process(tmp_path, init_weights):
    """Two pipeline stages driven by ``YvTrainer.train_step`` (1F1B over two micro-batches, clipping with the norm summed
    over stages, AdamW per stage): same losses and gradient norms as one process."""
    steps = 3
    env = {"YV_TEST_CLIP": "1.0", "YV_TEST_BATCH": "4"}
    single = _run(tmp_path, 1, 1, 1, steps, init_weights, "pp_single", env)
    n_single = json.load(open(str(tmp_path / "loss_pp_single.json") + ".norms"))
    multi = _run(tmp_path, 2, 1, 1, steps, init_weights, "pp_w2", dict(env, YV_TEST_PP="2"))
    n_multi = json.load(open(str(tmp_path / "loss_pp_w2.json") + ".norms"))
    for a, b in zip(single, multi):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (single, multi)
    for a, b in zip(n_single, n_multi):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (n_single, n_multi)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world,tp,ep,split", [(2, 2, 1, "1"), (4, 2, 2, "1"), (4, 2, 2, "0")])
def test_tensor_parallel_head_on_the_local_token_shard_matches_single_process(tmp_path, init_weights, world, tp, ep, split):
    """``tp_split_head``: every tensor-parallel rank runs the LM head and the loss on its own token rows (no final
    all-gather, no duplicated head work); the head weight's partial gradients are reduced over tp x dp.  Losses and
    clipped gradient norms over three steps equal the single process.  The run without the flag on tp 2 x dp 2 pins
    the norm accounting of the tensors that every tensor-parallel rank reduces a copy of (embeddings, head)."""
    steps = 3
    env = {"YV_TEST_CLIP": "1.0", "YV_TEST_BATCH": "4", "YV_TEST_UNTIED": "1"}
    single = _run(tmp_path, 1, 1, 1, steps, init_weights, f"sh_single{world}", env)
    n_single = json.load(open(str(tmp_path / f"loss_sh_single{world}.json") + ".norms"))
    multi = _run(tmp_path, world, tp, ep, steps, init_weights, f"sh_w{world}", dict(env, YV_TEST_SPLIT_HEAD=split))
    n_multi = json.load(open(str(tmp_path / f"loss_sh_w{world}.json") + ".norms"))
    for a, b in zip(single, multi):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (single, multi)
    for a, b in zip(n_single, n_multi):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (n_single, n_multi)
