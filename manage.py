#!/usr/bin/env python
"""Command line entry point: ``python manage.py <command> [flags]``.

Commands follow the reference CLI (manage.py:195-209): setup, train, infer, serve, test, monitor, download,
benchmark, help, action, dev, cache, publish.  ``train --distributed`` re-executes itself under
``torch.distributed.run`` with one rank per GPU (reference manage.py:1462-1498); ``infer`` is the one-shot
generation entry the reference's run CLI expects (opss/run/cli.py:338); ``action`` manages background runs
(submit / status / logs / control / recover / list)."""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

COMMANDS = ["setup", "train", "infer", "serve", "test", "monitor", "download", "benchmark", "help", "action", "dev",
            "cache", "publish", "check"]


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="manage.py", description="pisceslx_b200 management CLI")
    p.add_argument("command", choices=COMMANDS)
    p.add_argument("subcommand", nargs="?", default=None)
    p.add_argument("target", nargs="?", default=None)
    # model / data
    p.add_argument("--model_size", default="0.01B")
    p.add_argument("--model_config", default=None)
    p.add_argument("--train_config", default=None)
    p.add_argument("--stage", default="pretrain")
    p.add_argument("--dataset", default="synthetic")
    p.add_argument("--seq_len", type=int, default=None)
    p.add_argument("--batch_size", type=int, default=None)
    p.add_argument("--micro_batch_size", type=int, default=None)
    p.add_argument("--max_steps", type=int, default=None)
    p.add_argument("--lr", type=float, default=None)
    p.add_argument("--optimizer", default=None)
    p.add_argument("--resume_ckpt", default=None)
    p.add_argument("--reset_lr", action="store_true")
    p.add_argument("--output_dir", default=None)
    p.add_argument("--save_steps", type=int, default=None)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--device", default=None)
    p.add_argument("--dtype", default=None, choices=[None, "bf16", "fp32"])
    # distributed
    p.add_argument("--distributed", action="store_true")
    p.add_argument("--world_size", type=int, default=None)
    p.add_argument("--tensor_parallel", type=int, default=None)
    p.add_argument("--expert_parallel", type=int, default=None)
    p.add_argument("--pipeline_parallel", type=int, default=None)
    p.add_argument("--master_addr", default="127.0.0.1")
    p.add_argument("--master_port", type=int, default=29511)
    p.add_argument("--no_fused_comm", action="store_true")
    # runs
    p.add_argument("--run_id", default=None)
    p.add_argument("--run_dir", default=None)
    p.add_argument("--dry_run", action="store_true")
    # inference / serving
    p.add_argument("--ckpt", default=None)
    p.add_argument("--prompt", default="Hello")
    p.add_argument("--max_new_tokens", type=int, default=32)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top_k", type=int, default=0)
    p.add_argument("--top_p", type=float, default=1.0)
    p.add_argument("--speculative", action="store_true")
    p.add_argument("--infer_mode", default="standard")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--kv_blocks", type=int, default=1024)
    # test / benchmark
    p.add_argument("--quick", action="store_true")
    p.add_argument("--gpu", action="store_true")
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--gpus", type=int, default=1)
    return p


def _relaunch_distributed(args, argv) -> int:
    import torch
    n = args.world_size or max(torch.cuda.device_count(), 1)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           args.master_addr, "--master-port", str(args.master_port), os.path.abspath(__file__)] + argv
    return subprocess.run(cmd).returncode


def cmd_train(args, argv) -> int:
    if args.distributed and "LOCAL_RANK" not in os.environ:
        return _relaunch_distributed(args, argv)
    from pisceslx_b200.engine.orchestrator import PiscesLxTrainOrchestrator
    return PiscesLxTrainOrchestrator(args).run(args)


def cmd_infer(args, argv) -> int:
    from pisceslx_b200.engine.orchestrator import PiscesLxInferOrchestrator
    return PiscesLxInferOrchestrator(args).run(args)


def cmd_serve(args, argv) -> int:
    from pisceslx_b200.serve.server import PiscesLxBackendServer
    PiscesLxBackendServer(args).run()
    return 0


def cmd_test(args, argv) -> int:
    marker = "gpu" if args.gpu else "not gpu"
    extra = ["-k", "not gloo"] if args.quick else []
    return subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests"), "-x", "-q", "-m", marker] + extra).returncode


def cmd_benchmark(args, argv) -> int:
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", str(args.gpus), "--steps", str(args.steps),
           "--warmup", str(args.warmup)]
    return subprocess.run(cmd).returncode


def cmd_action(args, argv) -> int:
    from pisceslx_b200.engine.runstore import (PiscesLxRunController, PiscesLxRunIdFactory, PiscesLxRunStore,
                                               PiscesLxTaskRecovery)
    store = PiscesLxRunStore()
    sub = args.subcommand or "list"
    if sub == "list":
        for r in store.list_runs():
            print(r, store.read_state(r).get("status"))
        return 0
    if sub == "submit":
        run_id = args.run_id or PiscesLxRunIdFactory.new()
        child = [os.path.abspath(__file__), args.target or "train", "--run_id", run_id] + [a for a in argv[2:] if a != args.target]
        store.init_run(run_id, {"argv": child, "created": time.time()})
        if args.dry_run:
            print(json.dumps({"run_id": run_id, "argv": child}))
            return 0
        pid = PiscesLxRunController(store).spawn(run_id, child)
        print(json.dumps({"run_id": run_id, "pid": pid}))
        return 0
    if sub == "clean":
        from pisceslx_b200.engine.runmgmt import PiscesLxRunCleaner
        victims = PiscesLxRunCleaner(store).clean(dry_run=bool(args.dry_run))
        print(json.dumps({"removed" if not args.dry_run else "would_remove": victims}))
        return 0
    run_id = args.target or args.run_id
    if not run_id:
        print("run id required", file=sys.stderr)
        return 2
    if sub == "attach":
        from pisceslx_b200.engine.runmgmt import PiscesLxRunAttacher
        PiscesLxRunAttacher(store, run_id).attach(lambda kind, rec: print(f"[{kind}] {json.dumps(rec, default=str)}", flush=True))
        return 0
    if sub == "status":
        print(json.dumps(store.read_state(run_id), indent=1))
    elif sub == "logs":
        p = store.run_dir(run_id) / "output.log"
        print(p.read_text()[-8000:] if p.exists() else "")
    elif sub == "metrics":
        for m in store.read_jsonl(run_id, "metrics.jsonl")[-20:]:
            print(json.dumps(m))
    elif sub in ("stop", "pause", "resume", "save_ckpt_now"):
        store.send_control(run_id, sub)
    elif sub == "recover":
        rec = PiscesLxTaskRecovery(store)
        if rec.check_crashed(run_id) and rec.restart_task(run_id):
            spec = json.load(open(store.run_dir(run_id) / "spec.json"))
            PiscesLxRunController(store).spawn(run_id, spec["argv"])
            print("restarted")
        else:
            print("nothing to recover")
    else:
        print(f"unknown action {sub}", file=sys.stderr)
        return 2
    return 0


def cmd_help(args, argv) -> int:
    build_parser().print_help()
    print("\ncommands:", ", ".join(COMMANDS))
    return 0


def cmd_check(args, argv) -> int:
    from pisceslx_b200.utils.check import run_checks
    return run_checks(ROOT)


def cmd_setup(args, argv) -> int:
    """Build the sm_100a extension in-tree."""
    from pisceslx_b200.ops.build import build
    print(build(verbose=True))
    return 0


def cmd_monitor(args, argv) -> int:
    from pisceslx_b200.utils.monitor import PiscesLxSystemMonitor
    print(json.dumps(PiscesLxSystemMonitor().snapshot(), indent=1))
    return 0


def cmd_cache(args, argv) -> int:
    from pisceslx_b200.utils.paths import PiscesLxPaths
    paths = PiscesLxPaths()
    if args.subcommand == "clear":
        n = paths.clear_cache()
        print(f"removed {n} cache files")
    else:
        print(json.dumps(paths.describe(), indent=1))
    return 0


def cmd_publish(args, argv) -> int:
    from pisceslx_b200.engine.loader import load_model_for_inference, save_pretrained
    model = load_model_for_inference(args.model_size, args.ckpt, args.device or "cpu", args.model_config)
    out = args.output_dir or "export"
    save_pretrained(model, out)
    print(f"exported to {out}")
    return 0


def cmd_download(args, argv) -> int:
    print("no network in this environment: place datasets under data/ and point --dataset at them", file=sys.stderr)
    return 1


def cmd_dev(args, argv) -> int:
    from pisceslx_b200.engine.verify import PiscesLxCheckpointVerifier
    if args.subcommand == "verify_checkpoint" and args.ckpt:
        rep = PiscesLxCheckpointVerifier().verify(args.ckpt, args.model_size, args.model_config)
        print(json.dumps(rep, indent=1))
        return 0 if rep["ok"] else 1
    print("dev subcommands: verify_checkpoint --ckpt <file>")
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    args, _unknown = build_parser().parse_known_args(argv)
    handlers = {"train": cmd_train, "infer": cmd_infer, "serve": cmd_serve, "test": cmd_test, "benchmark": cmd_benchmark,
                "action": cmd_action, "help": cmd_help, "check": cmd_check, "setup": cmd_setup, "monitor": cmd_monitor,
                "cache": cmd_cache, "publish": cmd_publish, "download": cmd_download, "dev": cmd_dev}
    return int(handlers[args.command](args, argv) or 0)


if __name__ == "__main__":
    sys.exit(main())
