"""Serving layout "tensor-parallel attention x expert-parallel experts on the same ranks" (ep_over_tp), two Gloo ranks:
logits and engine output equal the single-process model."""
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
    from pisceslx_b200.engine.checkpoint import load_full_into
    from pisceslx_b200.serve.engine import YvEngineConfig, YvInferenceEngine
    world = int(os.environ["WORLD_SIZE"])
    par = init_parallel(tp=world, ep_over_tp=True, backend="gloo", device=torch.device("cpu"), timeout_s=120)
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    cfg.n_layer = 2
    cfg.use_gradient_checkpointing = False
    cfg.extra["moe_deterministic"] = True
    cfg.fused_comm = False
    model = build_model(cfg, "cpu", torch.float32, parallel=par if world > 1 else None, seed=7).eval()
    load_full_into(model, torch.load(sys.argv[2]))
    moe = model.model.layers[0].mlp
    ids = torch.randint(0, 512, (2, 16), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        logits = model(input_ids=ids)["logits"]
    eng = YvInferenceEngine(model, cfg=YvEngineConfig(max_num_seqs=4, num_blocks=32, block_size=8, eos_token_id=-1,
                                                      use_cuda_graphs=False))
    prompts = [[5, 6, 7, 8, 9, 10, 11, 12], [9, 10, 3, 4], [11, 12, 13, 14, 15, 16]]
    reqs = [eng.add_request(p, max_new_tokens=6) for p in prompts]
    eng.run_until_done()
    if par.rank == 0:
        json.dump({{"logits_sum": float(logits.double().sum()), "logits_0": logits[0, -1, :8].tolist(),
                   "tokens": [r.output_ids for r in reqs], "local_experts": moe.num_local, "ep": moe.ep_size,
                   "tp": par.tp_size, "shared_ffn": moe.shared_ffn}}, open(sys.argv[1], "w"))
    if world > 1:
        destroy_parallel()
""")


def _run(tmp_path, world, init, tag):
    script = tmp_path / "w.py"
    script.write_text(WORKER.format(root=ROOT))
    out = tmp_path / f"{tag}.json"
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script), str(out), str(init)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT))
    logs = [p.communicate(timeout=500)[0].decode()[-3000:] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(logs)
    return json.load(open(out))


@pytest.mark.timeout(900)
def test_tp_attention_with_ep_experts_on_the_same_ranks(tmp_path):
    sys.path.insert(0, ROOT)
    from pisceslx_b200 import YvConfig
    from pisceslx_b200.models import build_model
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    cfg.n_layer = 2
    init = tmp_path / "full.pt"
    torch.save(build_model(cfg, "cpu", torch.float32, seed=7).to_reference_state_dict(), init)
    one = _run(tmp_path, 1, init, "one")
    two = _run(tmp_path, 2, init, "two")
    assert two["tp"] == 2 and two["ep"] == 2 and two["local_experts"] == one["local_experts"] // 2
    assert two["shared_ffn"] == one["shared_ffn"] // 2
    assert abs(one["logits_sum"] - two["logits_sum"]) < 1e-3 * max(1.0, abs(one["logits_sum"]))
    for a, b in zip(one["logits_0"], two["logits_0"]):
        assert abs(a - b) < 1e-4
    assert one["tokens"] == two["tokens"]
