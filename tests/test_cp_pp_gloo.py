"""Gloo (CPU, world_size 2) tests of context parallelism (exact ring attention, all-gather attention with gradients,
zig-zag layout) and pipeline parallelism (two stages, 1F1B and GPipe) against single-process references."""
import json
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CP_WORKER = textwrap.dedent("""
    import json, sys, math
    sys.path.insert(0, {root!r})
    import torch, torch.distributed as dist
    from pisceslx_b200.parallel.state import init_parallel
    from pisceslx_b200.parallel import cp
    from pisceslx_b200.ops import reference as ref
    par = init_parallel(backend="gloo", device=torch.device("cpu"), timeout_s=120)
    W, r = par.world_size, par.rank
    torch.manual_seed(0)
    hq, hk, d, S = 4, 2, 16, 64
    q = torch.randn(S, hq * d); k = torch.randn(S, hk * d); v = torch.randn(S, hk * d)
    cu = torch.tensor([0, S], dtype=torch.int32)
    res = {{}}
    for causal in (True, False):
        full = ref.attention_varlen(q.view(S, hq, d), k.view(S, hk, d), v.view(S, hk, d), cu, None, causal, 1 / math.sqrt(d)).reshape(S, hq * d)
        L = S // W
        sl = slice(r * L, (r + 1) * L)
        o = cp.ring_attention(q[sl], k[sl], v[sl], dist.group.WORLD, hq, hk, d, causal=causal, fused=False)
        res[f"ring_{{causal}}"] = float((o - full[sl]).abs().max())
        # differentiable all-gather variant, contiguous layout
        ql, kl, vl = (t[sl].clone().requires_grad_(True) for t in (q, k, v))
        o2 = cp.allgather_attention(ql, kl, vl, dist.group.WORLD, hq, hk, d, causal=causal)
        res[f"ag_{{causal}}"] = float((o2 - full[sl]).abs().max())
        w = torch.randn(S, hq * d, generator=torch.Generator().manual_seed(1))
        (o2 * w[sl]).sum().backward()
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        fo = ref.attention_varlen(qf.view(S, hq, d), kf.view(S, hk, d), vf.view(S, hk, d), cu, None, causal, 1 / math.sqrt(d)).reshape(S, hq * d)
        (fo * w).sum().backward()
        res[f"ag_dk_{{causal}}"] = float((kl.grad - kf.grad[sl]).abs().max())
        res[f"ag_dq_{{causal}}"] = float((ql.grad - qf.grad[sl]).abs().max())
        # zig-zag layout
        half = S // (2 * W)
        rows = torch.cat([torch.arange(r * half, (r + 1) * half), torch.arange((2 * W - 1 - r) * half, (2 * W - r) * half)])
        o3 = cp.allgather_attention(q[rows], k[rows], v[rows], dist.group.WORLD, hq, hk, d, causal=causal, zigzag=True)
        res[f"zz_{{causal}}"] = float((o3 - full[rows]).abs().max())
    if r == 0:
        json.dump(res, open(sys.argv[1], "w"))
    dist.barrier(); dist.destroy_process_group()
""")

PP_WORKER = textwrap.dedent("""
    import json, sys
    sys.path.insert(0, {root!r})
    import torch, torch.distributed as dist
    from pisceslx_b200 import YvConfig
    from pisceslx_b200.models import build_model
    from pisceslx_b200.parallel.state import init_parallel
    from pisceslx_b200.parallel.pp import YvPipelineStage
    from pisceslx_b200.engine.checkpoint import load_full_into
    schedule = sys.argv[2]
    par = init_parallel(pp=2, backend="gloo", device=torch.device("cpu"), timeout_s=120)
    cfg = YvConfig.tiny_text_moe(vocab_size=512); cfg.n_layer = 4; cfg.use_gradient_checkpointing = False
    cfg.hidden_size = 64; cfg.head_dim = 16; cfg.moe_expert_intermediate_size = 32; cfg.moe_shared_intermediate_size = 64
    model = build_model(cfg, "cpu", torch.float32, parallel=par, seed=5)
    full = torch.load(sys.argv[3])
    load_full_into(model, full)
    model.train()
    g = torch.Generator().manual_seed(0)
    micro = [dict(input_ids=(t := torch.randint(0, 512, (2, 16), generator=g)), labels=t) for _ in range(4)]
    stage = YvPipelineStage(model, par, cfg.hidden_size, torch.float32)
    loss = stage.run(micro, schedule)
    grads = {{n: float(p.grad.norm()) for n, p in model.named_parameters() if p.grad is not None}}
    out = {{"rank": par.rank, "loss": float(loss) if loss is not None else None, "grads": grads}}
    json.dump(out, open(sys.argv[1] + f".{{par.rank}}", "w"))
    dist.barrier(); dist.destroy_process_group()
""")


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn(script_text, tmp_path, world, args):
    script = tmp_path / "w.py"
    script.write_text(script_text.format(root=ROOT))
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)] + [str(a) for a in args], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    logs = []
    for p in procs:
        o, _ = p.communicate(timeout=600)
        logs.append(o.decode()[-3000:])
    assert all(p.returncode == 0 for p in procs), "\n".join(logs)


@pytest.mark.timeout(900)
def test_context_parallel_is_exact(tmp_path):
    out = tmp_path / "cp.json"
    _spawn(CP_WORKER, tmp_path, 2, [out])
    res = json.load(open(out))
    for k, v in res.items():
        assert v < 2e-5, (k, v, res)


@pytest.mark.timeout(900)
@pytest.mark.parametrize("schedule", ["1f1b", "gpipe"])
def test_pipeline_two_stages_match_single(tmp_path, schedule):
    sys.path.insert(0, ROOT)
    from pisceslx_b200 import YvConfig
    from pisceslx_b200.models import build_model
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    cfg.n_layer, cfg.use_gradient_checkpointing = 4, False
    cfg.hidden_size, cfg.head_dim, cfg.moe_expert_intermediate_size, cfg.moe_shared_intermediate_size = 64, 16, 32, 64
    ref_model = build_model(cfg, "cpu", torch.float32, seed=5)
    init = tmp_path / "full.pt"
    torch.save(ref_model.to_reference_state_dict(), init)
    g = torch.Generator().manual_seed(0)
    micro = [torch.randint(0, 512, (2, 16), generator=g) for _ in range(4)]
    ref_model.train()
    total = 0.0
    for t in micro:
        l = ref_model(input_ids=t, labels=t).loss / len(micro)
        l.backward()
        total += float(l)
    out = tmp_path / "pp.json"
    _spawn(PP_WORKER, tmp_path, 2, [out, schedule, init])
    r0, r1 = json.load(open(str(out) + ".0")), json.load(open(str(out) + ".1"))
    assert abs(r1["loss"] - total) < 1e-4
    ref_grads = {n: float(p.grad.norm()) for n, p in ref_model.named_parameters() if p.grad is not None}
    # stage 0 holds layers 0-1 + embedding, stage 1 layers 2-3 + head; local layer indices restart at 0 per stage
    assert abs(r0["grads"]["model.embed.weight"] - ref_grads["model.embed.weight"]) < 1e-4 * max(1, ref_grads["model.embed.weight"])
    assert abs(r1["grads"]["lm_head"] - ref_grads["lm_head"]) < 1e-4 * max(1, ref_grads["lm_head"])
    assert abs(r1["grads"]["model.layers.0.attention.o_proj"] - ref_grads["model.layers.2.attention.o_proj"]) < 1e-4
