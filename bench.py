#!/usr/bin/env python
"""Flagship benchmark: training tokens/s of the Yv 7B-class text MoE (32 layers, hidden 4096, 32q/8kv heads of
128, 64 routed experts FFN 1408 top-6 + 2 shared experts FFN 2816, vocabulary = tokenizer size 154 856), bf16,
sequence length 4096, Muon on 2-D weights + AdamW elsewhere, synthetic uniform-random token ids and random-init
weights.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run)
    python bench.py --impl reference ...                     (the reference arm)

One JSON line is printed by rank 0.  ``value`` is device-timed (CUDA events around exactly K optimizer steps,
barrier + synchronize on both sides, max over ranks) with the step's inputs already on the device; ``e2e`` is the
same K steps through ``YvTrainer.train_step`` with each step's token ids copied from pinned host memory and the
loss read back.  Every step's input (tokens x hidden activations, 80 GB of weights) is far larger than L2.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

VOCAB = 154856
SEQ = 4096


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seqs-per-gpu", type=int, default=0, help="sequences per GPU per optimizer step (0 = default)")
    ap.add_argument("--micro-batch", type=int, default=0, help="sequences per forward/backward (0 = default)")
    ap.add_argument("--layers", type=int, default=32, help="debug only: anything but 32 is reported as invalid")
    ap.add_argument("--tp", type=int, default=0)
    ap.add_argument("--ep", type=int, default=0)
    ap.add_argument("--no-fused-comm", action="store_true", help="NCCL-only collectives (the stated baseline mode)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--state-dtype", default="int8", choices=["int8", "bf16"],
                    help="Muon momentum storage: int8 block-quantised (stochastic rounding) or bf16")
    ap.add_argument("--expert-fp8", default="", choices=["", "mx"],
                    help="routed experts' forward products in block-scaled e4m3 (a labelled fp8 line, never the headline)")
    ap.add_argument("--ref-limit", type=int, default=300, help="seconds given to the reference's full-size attempt")
    ap.add_argument("--no-ref-context", action="store_true", help="skip the reduced-layer context run of the reference")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------------
def _run_reference_child(extra, out_path, limit_s, port_shift=0):
    """Run ``baseline/run_reference.py`` as a child of this rank (same RANK / LOCAL_RANK / WORLD_SIZE, so the N
    children form the reference's own process group) and return its JSON line, or a reason string."""
    env = dict(os.environ)
    if port_shift and env.get("MASTER_PORT"):
        env["MASTER_PORT"] = str(int(env["MASTER_PORT"]) + port_shift)
    env.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    env.setdefault("YV_STANDIN_INFO", "1")                   # the reference's own info log lines go to the child's log
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "run_reference.py"), "--out", out_path] + extra
    log = open(out_path + ".log", "w")
    proc = subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT, env=env, cwd=ROOT)
    try:
        proc.wait(timeout=limit_s)
    except subprocess.TimeoutExpired:
        proc.kill()                                          # the exact child this rank started
        proc.wait()
        return (f"stock reference path did not finish within {limit_s} s (killed); its own log says: "
                + _reference_log_digest(out_path + ".log"))
    finally:
        log.close()
    try:
        with open(out_path) as f:
            return json.loads(f.read().strip().splitlines()[-1])
    except Exception:
        tail = ""
        try:
            tail = open(out_path + ".log").read()[-400:].replace("\n", " ")
        except OSError:
            pass
        return f"stock reference path exited with code {proc.returncode} and no result: {tail}"


def _reference_log_digest(path: str) -> str:
    """The reference's parameter-count line and its last log line, from the child's captured output."""
    try:
        lines = [l.strip() for l in open(path, errors="replace").read().splitlines() if l.strip()]
    except OSError:
        return "(no log)"
    keep = [l for l in lines if "total parameters" in l][:1]
    if lines and (not keep or lines[-1] != keep[0]):
        keep.append(lines[-1])
    return " | ".join(l[:300] for l in keep) or "(empty log)"


def reference_arm(args) -> None:
    """Train the UNMODIFIED reference (plain copy under ``baseline/_ref``) through its own trainer on the benchmark's
    model and data shape (``baseline/run_reference.py`` says which reference calls are driven), first at the full
    configuration; when that fails on its own (its model does not fit host or device memory), the captured reason is
    reported as ``unavailable`` together with a labelled context run of the same path at 4 of the 32 layers, which is
    NOT the benchmark configuration and carries ``same_config: false``."""
    import tempfile
    rank = int(os.environ.get("RANK", "0"))
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "tools")):
        # where an unpacked reference source tree may be found when ``baseline/_ref`` is empty
        src = os.environ.get("YV_REFERENCE_SRC", os.path.join(os.sep, "root", "reference"))
        if os.path.isdir(os.path.join(src, "tools")):        # a plain copy is the whole installation: pure Python
            import shutil
            import time as _time
            if rank == 0:                                    # one rank copies into a side folder and renames it in
                tmp_dir = ref_dir + ".partial"
                shutil.rmtree(tmp_dir, ignore_errors=True)
                os.makedirs(tmp_dir)
                for name in ("manage.py", "configs", "utils", "third_party", "opss", "tools", "model", "tokenizer"):
                    s_, d_ = os.path.join(src, name), os.path.join(tmp_dir, name)
                    (shutil.copytree if os.path.isdir(s_) else shutil.copy)(s_, d_)
                if os.path.isdir(ref_dir):
                    shutil.rmtree(ref_dir, ignore_errors=True)
                os.rename(tmp_dir, ref_dir)
            else:
                t_end = _time.time() + 300
                while not os.path.isdir(os.path.join(ref_dir, "tools")) and _time.time() < t_end:
                    _time.sleep(0.5)
        else:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "no copy of the reference under baseline/_ref "
                                  f"and no source tree at {src} to copy it from"}))
            return
    tmp = tempfile.mkdtemp(prefix="yv_ref_arm_")
    seqs = args.seqs_per_gpu or 64
    full = ["--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup),
            "--seqs-per-gpu", str(seqs), "--micro-batch", "1"]
    if args.layers != 32:
        full += ["--layers", str(args.layers)]
    res = _run_reference_child(full, os.path.join(tmp, f"full_{rank}.json"), limit_s=args.ref_limit)
    if isinstance(res, dict) and "unavailable" not in res:
        if rank == 0:
            print(json.dumps(res))
        return
    reason = res if isinstance(res, str) else res.get("unavailable", "unknown")
    out = {"impl": "reference", "unavailable": reason}
    if not args.no_ref_context and args.layers == 32:
        ctx = _run_reference_child(["--gpus", str(args.gpus), "--steps", str(min(args.steps, 2)), "--warmup", "1",
                                    "--seqs-per-gpu", "8", "--micro-batch", "1", "--layers", "4"],
                                   os.path.join(tmp, f"ctx_{rank}.json"), limit_s=600, port_shift=7)
        out["context_reduced"] = {"note": "same reference path at 4 of 32 layers, 8 sequences per GPU per step: "
                                  "context only, not the benchmark configuration; compare with "
                                  "`bench.py --layers 4 --seqs-per-gpu 8` of this framework",
                                  "result": ctx}
    if rank == 0:
        print(json.dumps(out))


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs (read-only queries)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def layout_for(n: int, args):
    """(tp, ep) per world size: the named layout TP2 x EP4 at 8 GPUs, expert parallel over all ranks below."""
    if args.tp or args.ep:
        return max(args.tp, 1), max(args.ep, 1)
    return {1: (1, 1), 2: (1, 2), 4: (1, 4), 8: (2, 4)}.get(n, (1, n))


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    import torch
    import torch.distributed as dist

    from pisceslx_b200 import YvConfig
    from pisceslx_b200.engine.trainer import YvTrainer, YvTrainerConfig
    from pisceslx_b200.models import build_model
    from pisceslx_b200.ops import check_status, load_extension
    from pisceslx_b200.parallel.state import init_parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        # convenience: re-exec under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29577", os.path.abspath(__file__)] + sys.argv[1:]
        os.execv(sys.executable, cmd)
    load_extension()
    tp, ep = layout_for(world, args)
    par = init_parallel(tp=tp, ep=ep) if world > 1 else init_parallel()
    dev = par.device
    rank = par.rank

    cfg = YvConfig.yv_7b_moe(vocab_size=VOCAB, n_layer=args.layers)
    cfg.tensor_parallel, cfg.expert_parallel = tp, ep
    cfg.fused_comm = not args.no_fused_comm
    cfg.use_gradient_checkpointing = True
    if args.expert_fp8:
        cfg.expert_fp8 = args.expert_fp8
    seqs = args.seqs_per_gpu or 64            # 64 per GPU = the named global batch of 512 sequences on 8 GPUs
    micro = args.micro_batch or (2 if world == 1 else 4)
    model = build_model(cfg, dev, torch.bfloat16, parallel=par if world > 1 else None, seed=1234)
    tcfg = YvTrainerConfig(micro_batch_size=micro, optimizer="muon", lr=2e-4, weight_decay=0.1, warmup_steps=10,
                           max_steps=10_000, streaming_optimizer=True, clip_grad_norm=0.0, log_steps=1,
                           track_grad_norm=False, recompute_policy="auto", state_dtype=args.state_dtype)
    trainer = YvTrainer(model, tcfg, parallel=par if world > 1 else None)

    # tensor-parallel peers work on the same sequences: batch size and seed follow the data-parallel rank
    seqs_rank = seqs * tp
    g = torch.Generator().manual_seed(1000 + par.dp_rank)
    n_batches = max(args.steps, 1)
    host_batches = [torch.randint(0, VOCAB, (seqs_rank, SEQ), generator=g, dtype=torch.int64).pin_memory()
                    for _ in range(min(n_batches, 4))]
    dev_batches = [b.to(dev) for b in host_batches]

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def run(batches, count):
        last = None
        for i in range(count):
            b = batches[i % len(batches)]
            last = trainer.train_step({"input_ids": b, "labels": b})
        return last

    # ---- warm-up (untimed) ----
    run(dev_batches, args.warmup)
    while trainer.recompute_planner is not None and trainer.recompute_planner.stage < 3:
        run(dev_batches, 1)                      # the recompute plan needs two measured steps before it is final
    check_status()

    # ---- kernel launch census over one untimed step ----
    # A step is n_micro identical micro-batches plus a fixed part (optimizer, collectives); counting a one- and a
    # two-micro-batch step under the profiler gives both terms without tracing a full-size step.
    launches_per_step = None
    try:
        from torch.profiler import ProfilerActivity, profile

        def census(n_micro: int) -> int:
            small = dev_batches[0][: micro * n_micro]
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                trainer.train_step({"input_ids": small, "labels": small})
                torch.cuda.synchronize(dev)
            return sum(e.count for e in prof.key_averages() if "yv::" in e.key)

        l1, l2 = census(1), census(2)
        n_micro_step = (seqs_rank + micro - 1) // micro
        launches_per_step = (l1 - (l2 - l1)) + (l2 - l1) * n_micro_step
    except Exception:
        launches_per_step = None

    # ---- timed: device-resident inputs ----
    sampler = ClockSampler(dev.index or 0)
    sync()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = run(dev_batches, args.steps)
    e1.record()
    sync()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    t_ms = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms = float(t_ms.item())
    tokens_per_step = seqs_rank * SEQ * par.dp_size
    value = tokens_per_step * args.steps / (ms / 1e3)

    # ---- timed: end to end through the public trainer API from pinned host memory ----
    e2e = None
    if not args.skip_e2e:
        # a step takes tens of seconds at this size: the end-to-end pass runs at most three of them
        e2e_steps = max(1, min(args.steps, 3))
        trainer.h2d_bytes = trainer.d2h_bytes = 0
        sync()
        e0.record()
        run(host_batches, e2e_steps)
        e1.record()
        sync()
        ems = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ems, op=dist.ReduceOp.MAX)
        e2e = {"value": tokens_per_step * e2e_steps / (float(ems.item()) / 1e3), "unit": "tokens/s",
               "steps": e2e_steps,
               "h2d_bytes_per_step": trainer.h2d_bytes // e2e_steps,
               "d2h_bytes_per_step": trainer.d2h_bytes // e2e_steps}
    check_status()

    if rank == 0:
        par_name = "single" if world == 1 else f"tp{tp}xep{ep}xdp{par.dp_size}"
        out = {
            "metric": "train tokens/sec/box Yv-7B MoE", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / max(args.steps, 1),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if not args.expert_fp8 else "bf16 + mxfp8 expert forward",
            "data": "synthetic uniform-random token ids, random-init weights",
            "config": {"model": "Yv 7B-class text MoE: 32L h4096 32q/8kv hd128, 64 experts ffn1408 top6 + 2 shared "
                                "ffn2816, vocab 154856" + ("" if args.layers == 32 else f" [INVALID: {args.layers} layers]")
                                + (f" [fp8 line, not the headline: routed experts' forward in {args.expert_fp8} e4m3]"
                                   if args.expert_fp8 else ""),
                       "global_batch": seqs_rank * par.dp_size, "seq_len": SEQ,
                       "micro_batch": micro, "parallelism": par_name, "optimizer": "Muon(2-D)+AdamW, "
                       + ("int8 block-scaled Muon momentum (128-element blocks, stochastic rounding), bf16 AdamW moments, "
                          if args.state_dtype == "int8" else "bf16 states, ") + "gradients consumed inside backward", "activation_recompute": ("per layer, sized from measured memory: " + trainer.recompute_planner.summary())
                       if trainer.recompute_planner is not None else "per layer",
                       "l2": "inputs larger than L2 (80 GB of weights and >1 GB of activations per layer)",
                       "fused_comm": bool(cfg.fused_comm) if world > 1 else None},
            "clocks": clocks, "e2e": e2e,
            "gpu_launches": (launches_per_step * args.steps) if launches_per_step is not None else None,
            "loss": last["loss"] if last else None,
            "max_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9,
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
