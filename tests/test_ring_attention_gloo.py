"""Differentiable ring attention on Gloo ranks: output and all three gradients equal full attention on one process."""
import json
import os
import socket
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, math, os, sys
    sys.path.insert(0, {root!r})
    import torch
    import torch.distributed as dist
    from pisceslx_b200.parallel import cp
    out, causal = sys.argv[1], sys.argv[2] == "1"
    dist.init_process_group("gloo")
    W, r = dist.get_world_size(), dist.get_rank()
    hq, hk, d, S = 4, 2, 16, 8 * W
    g = torch.Generator().manual_seed(5)
    q = torch.randn(S, hq * d, generator=g, dtype=torch.float64).float()
    k = torch.randn(S, hk * d, generator=g, dtype=torch.float64).float()
    v = torch.randn(S, hk * d, generator=g, dtype=torch.float64).float()
    w = torch.randn(S, hq * d, generator=g, dtype=torch.float64).float()          # d(loss)/d(out)
    # single-process oracle
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    qq = qf.view(S, hq, d).transpose(0, 1)
    kk = kf.view(S, hk, d).transpose(0, 1).repeat_interleave(hq // hk, 0)
    vv = vf.view(S, hk, d).transpose(0, 1).repeat_interleave(hq // hk, 0)
    s = qq @ kk.transpose(1, 2) / math.sqrt(d)
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
    ref = (torch.softmax(s, -1) @ vv).transpose(0, 1).reshape(S, hq * d)
    (ref * w).sum().backward()
    # ring over the ranks
    L = S // W
    sl = slice(r * L, (r + 1) * L)
    ql, kl, vl = (t[sl].clone().requires_grad_(True) for t in (q, k, v))
    o = cp.ring_attention_train(ql, kl, vl, dist.group.WORLD, hq, hk, d, causal=causal)
    (o * w[sl]).sum().backward()
    err = lambda a, b: float((a - b).abs().max())
    e = torch.tensor([err(o, ref[sl]), err(ql.grad, qf.grad[sl]), err(kl.grad, kf.grad[sl]), err(vl.grad, vf.grad[sl])],
                     dtype=torch.float64)
    dist.all_reduce(e, op=dist.ReduceOp.MAX)
    if r == 0:
        json.dump({{"errs": e.tolist()}}, open(out, "w"))
    dist.barrier()
""")


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world,causal", [(2, True), (4, True), (3, False)])
def test_ring_attention_forward_and_backward_match_full_attention(tmp_path, world, causal):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    out = tmp_path / "out.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(script), str(out), "1" if causal else "0"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-3000:])
    errs = json.load(open(out))["errs"]
    assert max(errs) < 2e-5, errs
