"""Worker of the multi-GPU tests (launched by torchrun, one rank per GPU).

Trains a small Yv text MoE (kernel-friendly sizes) for a few steps in the requested layout, once with the fused
peer-memory collectives and once with the NCCL implementations, and writes the losses of every mode to a JSON
file; the parent test compares them with each other and with a single-GPU run of the same global batch."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from pisceslx_b200 import YvConfig
from pisceslx_b200.engine.checkpoint import load_full_into
from pisceslx_b200.engine.trainer import YvTrainer, YvTrainerConfig
from pisceslx_b200.models import build_model
from pisceslx_b200.ops import check_status
from pisceslx_b200.parallel import fused as fz
from pisceslx_b200.parallel.state import init_parallel


def small_cfg() -> YvConfig:
    cfg = YvConfig(vocab_size=4096, hidden_size=512, n_layer=2, n_head=8, n_kv_head=4, head_dim=64, rope_theta=1e4,
                   moe_num_experts=8, moe_top_k=2, moe_shared_experts=1, moe_expert_intermediate_size=256,
                   moe_shared_intermediate_size=512, intermediate_size=512, tie_word_embeddings=False,
                   max_position_embeddings=4096)
    cfg.use_gradient_checkpointing = True
    return cfg


def run(par, full_sd, fused: bool, steps: int, streaming: bool):
    fz.set_enabled(fused)
    cfg = small_cfg()
    cfg.fused_comm = fused
    model = build_model(cfg, par.device, torch.bfloat16, parallel=par if par.world_size > 1 else None, seed=3)
    load_full_into(model, full_sd)
    tr = YvTrainer(model, YvTrainerConfig(micro_batch_size=2, optimizer="muon", lr=2e-3, max_steps=100, clip_grad_norm=0.0,
                                          streaming_optimizer=streaming, track_grad_norm=False),
                   parallel=par if par.world_size > 1 else None)
    g = torch.Generator().manual_seed(0)
    data = torch.randint(0, cfg.vocab_size, (steps, 4, 256), generator=g)
    losses = []
    for s in range(steps):
        b = data[s]
        if par.dp_size > 1:
            per = b.shape[0] // par.dp_size
            b = b[par.dp_rank * per:(par.dp_rank + 1) * per]
        b = b.to(par.device)
        losses.append(tr.train_step({"input_ids": b, "labels": b})["loss"])
    torch.cuda.synchronize()
    check_status()
    t = torch.tensor(losses, dtype=torch.float64, device=par.device)
    if par.world_size > 1 and par.dp_size > 1:
        dist.all_reduce(t, group=par.dp_group)
        t /= par.dp_size
    return t.tolist()


def determinism(par, iters: int = 100) -> dict:
    """The flag / epoch protocols of the fused kernels, repeated: with the deterministic row order every repetition
    must reproduce the first one bit for bit and leave the status word clear (a race between a peer's stores and the
    consumer's loads, or a flag observed one epoch early, shows up as a differing or corrupted tile)."""
    from pisceslx_b200.ops import moe as moe_ops
    from pisceslx_b200.parallel import fused_tp as ft
    dev = par.device
    fz.set_enabled(True)
    res = {}
    torch.manual_seed(100 + par.rank)
    if par.ep_size > 1:
        T, H, E, F, k = 512, 512, 8, 256, 2
        e_loc = E // par.ep_size
        x = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
        w13 = (torch.randn(e_loc, 2 * F, H, device=dev) * 0.05).bfloat16()
        w2 = (torch.randn(e_loc, H, F, device=dev) * 0.05).bfloat16()
        wts, idx, _, _ = moe_ops.gate_topk(torch.randn(T, E, device=dev), None, k)
        first, mism = None, 0
        for _ in range(iters):
            y = fz.moe_experts_ep_fused(x, w13, w2, wts, idx, E, par.ep_group, deterministic=True)
            if first is None:
                first = y.clone()
            elif not torch.equal(y, first):
                mism += 1
        res["ep_mismatches"] = mism
        res["ep_finite"] = bool(torch.isfinite(first.float()).all())
    if par.tp_size > 1:
        rows, H, N = 256, 512, 1024
        xs = torch.randn(rows, H, device=dev).bfloat16()
        wc = (torch.randn(N // par.tp_size, H, device=dev) * 0.05).bfloat16()
        xf = torch.randn(rows * par.tp_size, H // par.tp_size, device=dev).bfloat16()
        wr = (torch.randn(H, H // par.tp_size, device=dev) * 0.05).bfloat16()
        f_ag = f_rs = None
        m_ag = m_rs = 0
        for _ in range(iters):
            a = ft.allgather_gemm(xs, wc, par.tp_group)[1]
            b = ft.gemm_reduce_scatter(xf, wr, par.tp_group)
            if f_ag is None:
                f_ag, f_rs = a.clone(), b.clone()
            else:
                m_ag += int(not torch.equal(a, f_ag))
                m_rs += int(not torch.equal(b, f_rs))
        res["ag_mismatches"], res["rs_mismatches"] = m_ag, m_rs
    torch.cuda.synchronize()
    check_status()
    res["iters"] = iters
    t = torch.tensor([float(v) for k, v in sorted(res.items()) if k.endswith("mismatches")], device=dev)
    if t.numel():
        dist.all_reduce(t)                                   # any rank's mismatch counts
        for (k, _), v in zip([(k, v) for k, v in sorted(res.items()) if k.endswith("mismatches")], t.tolist()):
            res[k] = int(v)
    return res


def ep_regrow(par) -> dict:
    """The fused expert-parallel layer at a small, a large and again the small token count (what a serving engine
    does: short prompt, long prefill, decode).  The large call re-allocates the symmetric buffers; the small call
    after it must not use views of the freed ones.  Every call is compared with the NCCL path."""
    from pisceslx_b200.parallel import ep as epm
    torch.manual_seed(11 + par.rank)
    dev, E, H, F, k = par.device, 8, 512, 256, 2
    e_local = E // par.ep_size
    w13 = (torch.randn(e_local, 2 * F, H, device=dev) * 0.05).bfloat16()
    w2 = (torch.randn(e_local, H, F, device=dev) * 0.05).bfloat16()
    errs = []
    for T in (16, 4096, 16, 9000, 64):
        x = torch.randn(T, H, device=dev).bfloat16()
        idx = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)]).int()
        wts = torch.softmax(torch.randn(T, k, device=dev), -1)
        with torch.no_grad():
            fz.set_enabled(True)
            a = epm.moe_experts_ep(x, w13, w2, wts, idx, E, par.ep_group, fused=True)
            fz.set_enabled(False)
            b = epm.moe_experts_ep(x, w13, w2, wts, idx, E, par.ep_group, fused=False)
        torch.cuda.synchronize()
        errs.append(float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)))
    check_status()
    t = torch.tensor(errs, dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"rel_err": t.tolist()}


def main() -> None:
    tp, ep, out_path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    par = init_parallel(tp=tp, ep=ep, timeout_s=120)
    if os.environ.get("YV_MULTI_MODE") == "ep_regrow":
        res = ep_regrow(par)
        if par.rank == 0:
            json.dump(res, open(out_path, "w"))
        dist.barrier()
        dist.destroy_process_group()
        return
    if os.environ.get("YV_MULTI_MODE") == "determinism":
        res = determinism(par, int(os.environ.get("YV_MULTI_ITERS", "100")))
        if par.rank == 0:
            json.dump(res, open(out_path, "w"))
        dist.barrier()
        dist.destroy_process_group()
        return
    torch.manual_seed(0)
    ref_model = build_model(small_cfg(), "cpu", torch.float32, seed=3)
    full_sd = ref_model.to_reference_state_dict()
    res = {}
    if par.world_size == 1:
        for streaming in (False, True):
            res["stream" if streaming else "plain"] = run(par, full_sd, False, 3, streaming)
        json.dump(res, open(out_path, "w"))
        return
    for streaming in (False, True):
        for fused in (False, True):
            key = f"{'fused' if fused else 'nccl'}_{'stream' if streaming else 'plain'}"
            res[key] = run(par, full_sd, fused, 3, streaming)
    if par.rank == 0:
        json.dump(res, open(out_path, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
