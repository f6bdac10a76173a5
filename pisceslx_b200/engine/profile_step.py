"""Per-kernel device time of one training step, split into the part that repeats per micro-batch and the part that
runs once per optimizer step.

    python -m pisceslx_b200.engine.profile_step --layers 32 --micro-batch 2                 (one GPU)
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m pisceslx_b200.engine.profile_step --ep 2                                        (one process per GPU)

A full-size step is tens of seconds and hundreds of thousands of launches, too much to trace.  A step is n identical
micro-batches (forward, backward with the gradients folded into the optimizer state) plus a fixed part (Newton-Schulz
and the parameter update, data-parallel reduction and parameter gather), so a one-micro-batch step and a
two-micro-batch step are traced with the PyTorch profiler (CUDA activities) and their difference per kernel name is
the cost of one micro-batch, the remainder the fixed part.  Kernels are also grouped into phases by name.  The
reference times a step with the host clock and no device synchronisation (tools/train/core.py:2878,2933-2936) and its
profiler hook is inert (opss/train/profiler.py:245-345).
"""
from __future__ import annotations

import argparse
import json
import os
from collections import defaultdict
from typing import Dict, Tuple

import torch

PHASES = (
    ("attention", ("attn_fwd", "attn_bwd", "attn_delta", "rope")),
    ("newton_schulz", ("gemm_batched", "frob_", "ns_poly", "muon_apply", "dequant_q8")),
    ("momentum_fold/adamw", ("momentum", "adamw", "zero_reduce_fold", "sumsq")),
    ("expert_parallel comm", ("ep_dispatch", "ep_combine", "ep_unpermute", "flag_barrier", "peer_copy", "nccl")),
    ("moe routing/permute", ("gate_topk", "moe_", "swiglu", "histogram")),
    ("loss", ("ce_kernel", "ce_")),
    ("norm/elementwise", ("rmsnorm", "film", "elementwise", "vectorized", "copy", "Memcpy", "Memset", "fill", "cat")),
    ("gemm", ("gemm",)),
)


def phase_of(name: str) -> str:
    for phase, keys in PHASES:
        if any(k in name for k in keys):
            return phase
    return "other"


def trace(trainer, ids: torch.Tensor) -> Tuple[Dict[str, float], Dict[str, int], float]:
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        res = trainer.train_step({"input_ids": ids, "labels": ids})
        torch.cuda.synchronize()
    ms, cnt = defaultdict(float), defaultdict(int)
    for e in prof.key_averages():
        if e.self_device_time_total > 0:
            ms[e.key] += e.self_device_time_total / 1e3
            cnt[e.key] += e.count
    return ms, cnt, res["step_time"] * 1e3


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--micro-batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--state-dtype", default="int8")
    ap.add_argument("--recompute", default="all", choices=["all", "none"], help="layers recomputed in backward")
    ap.add_argument("--no-fused-comm", action="store_true")
    ap.add_argument("--top", type=int, default=28)
    ap.add_argument("--json", default="")
    a = ap.parse_args()

    from .. import YvConfig
    from ..models import build_model
    from ..ops import load_extension
    from ..parallel.state import init_parallel
    from .trainer import YvTrainer, YvTrainerConfig

    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    load_extension()
    par = init_parallel(tp=a.tp, ep=a.ep) if world > 1 else init_parallel()
    dev = par.device
    cfg = YvConfig.yv_7b_moe(vocab_size=154856, n_layer=a.layers)
    cfg.tensor_parallel, cfg.expert_parallel, cfg.fused_comm = a.tp, a.ep, not a.no_fused_comm
    cfg.use_gradient_checkpointing = a.recompute == "all"
    model = build_model(cfg, dev, torch.bfloat16, parallel=par if world > 1 else None, seed=1)
    tr = YvTrainer(model, YvTrainerConfig(micro_batch_size=a.micro_batch, optimizer="muon", lr=2e-4, streaming_optimizer=True,
                                          clip_grad_norm=0.0, track_grad_norm=False, max_steps=1000,
                                          state_dtype=a.state_dtype), parallel=par if world > 1 else None)
    g = torch.Generator().manual_seed(1 + par.dp_rank)
    ids = torch.randint(0, 154856, (2 * a.micro_batch, a.seq), generator=g).to(dev)
    for _ in range(2):
        tr.train_step({"input_ids": ids, "labels": ids})
    ms1, c1, t1 = trace(tr, ids[: a.micro_batch])
    ms2, c2, t2 = trace(tr, ids)
    if par.rank != 0:
        return
    per_micro = {k: ms2.get(k, 0.0) - ms1.get(k, 0.0) for k in set(ms1) | set(ms2)}
    fixed = {k: ms1.get(k, 0.0) - per_micro[k] for k in per_micro}
    tokens = a.micro_batch * a.seq
    tot_m, tot_f = sum(per_micro.values()), sum(fixed.values())
    print(f"layers {a.layers}  micro-batch {a.micro_batch} x {a.seq}  tp {a.tp} ep {a.ep} world {world}  recompute {a.recompute}  "
          f"momentum {a.state_dtype}")
    print(f"step (1 micro-batch) {t1:.1f} ms, step (2 micro-batches) {t2:.1f} ms")
    print(f"per micro-batch: {tot_m:.1f} ms of kernels ({tokens / max(tot_m, 1e-9) * 1e3:.0f} tokens/s if that were all); "
          f"fixed per step: {tot_f:.1f} ms")
    phases_m, phases_f = defaultdict(float), defaultdict(float)
    for k in per_micro:
        phases_m[phase_of(k)] += per_micro[k]
        phases_f[phase_of(k)] += fixed[k]
    print("\nphase                       per micro-batch ms     share   | fixed per step ms")
    for ph in sorted(set(phases_m) | set(phases_f), key=lambda p: -phases_m[p]):
        print(f"{ph:28s}{phases_m[ph]:14.2f}  {100 * phases_m[ph] / max(tot_m, 1e-9):8.1f}%   | {phases_f[ph]:12.2f}")
    print("\nkernels, per micro-batch (launches = second trace minus first):")
    for k in sorted(per_micro, key=lambda k: -per_micro[k])[: a.top]:
        print(f"{per_micro[k]:10.2f} ms {100 * per_micro[k] / max(tot_m, 1e-9):5.1f}% {c2.get(k, 0) - c1.get(k, 0):6d}  {k[:120]}")
    print("\nkernels, fixed per step:")
    for k in sorted(fixed, key=lambda k: -fixed[k])[: max(a.top // 2, 8)]:
        print(f"{fixed[k]:10.2f} ms {100 * fixed[k] / max(tot_f, 1e-9):5.1f}% {2 * c1.get(k, 0) - c2.get(k, 0):6d}  {k[:120]}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"per_micro_ms": per_micro, "fixed_ms": fixed, "step1_ms": t1, "step2_ms": t2}, f, indent=1)


if __name__ == "__main__":
    main()
