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
            "cache", "plxs", "publish", "check", "mcp"]


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
    # ---- names the reference CLI uses (manage.py:487-1427); aliases map onto the options above ----
    p.add_argument("--config", dest="model_config", default=argparse.SUPPRESS, help="model YAML (alias of --model_config)")
    p.add_argument("--model", dest="model_size", default=argparse.SUPPRESS, help="model preset (alias of --model_size)")
    p.add_argument("--model_path", dest="ckpt", default=argparse.SUPPRESS, help="checkpoint (alias of --ckpt)")
    p.add_argument("--model_name_or_path", default=None, help="base weight to adapt: turns the run into an adapter run")
    p.add_argument("--run_name", default=None)
    p.add_argument("--control_interval", type=float, default=0.5)
    p.add_argument("--log_level", default="INFO")
    p.add_argument("--log_interval", type=int, default=None)
    p.add_argument("--train_mode", default="standard", choices=["standard", "preference", "quant_export"])
    p.add_argument("--sharding", default=None, choices=[None, "zero1", "full_shard"])
    p.add_argument("--state_dtype", default=None, choices=[None, "bf16", "fp32", "int8"])
    p.add_argument("--context_parallel", type=int, default=None)
    # preference / RL stage
    p.add_argument("--rlhf", action="store_true", help="run the preference stage (same as --train_mode preference)")
    p.add_argument("--rlhf_dataset", default=None)
    p.add_argument("--rlhf_epochs", type=int, default=1)
    p.add_argument("--rlhf_lr", type=float, default=1e-5)
    p.add_argument("--rlhf_batch_size", type=int, default=4)
    p.add_argument("--rlhf_mini_batch_size", type=int, default=2)
    p.add_argument("--rlhf_accum_steps", type=int, default=1)
    p.add_argument("--rlhf_max_length", type=int, default=512)
    p.add_argument("--rlhf_max_samples", type=int, default=None)
    # distillation
    p.add_argument("--distill", action="store_true")
    p.add_argument("--distill_alpha", type=float, default=0.5)
    p.add_argument("--distill_temperature", type=float, default=2.0)
    p.add_argument("--teacher_model", default=None)
    p.add_argument("--teacher_name", default=None)
    p.add_argument("--teacher_type", default="local")
    p.add_argument("--teacher_api_key", default=None)
    # quantisation
    p.add_argument("--quant", default=None, help="post-training quantisation method for export / serving (rtn, gptq, awq, smoothquant)")
    p.add_argument("--quant_bits", type=int, default=4)
    p.add_argument("--no_quant", action="store_true")
    p.add_argument("--force_quant", action="store_true")
    p.add_argument("--force_lora", action="store_true")
    p.add_argument("--save", default=None, help="output path of --train_mode quant_export")
    # serving
    p.add_argument("--serve_config", default=None)
    p.add_argument("--workers", type=int, default=1)
    p.add_argument("--max_concurrency", type=int, default=64)
    p.add_argument("--request_timeout", type=float, default=300.0)
    p.add_argument("--cors_origins", default="*")
    p.add_argument("--api_key", default=None)
    p.add_argument("--disable_agent_intercept", action="store_true")
    p.add_argument("--disable_opss", action="store_true")
    # monitor / benchmark / download / misc
    p.add_argument("--monitor_mode", default="once", choices=["once", "loop"])
    p.add_argument("--update_interval", type=float, default=2.0)
    p.add_argument("--max_samples", type=int, default=None)
    p.add_argument("--benchmark", default=None, help="evaluation suite: mmlu, gsm8k, aime, humaneval, needle, ...")
    p.add_argument("--perf", action="store_true", help="throughput / latency benchmark instead of an evaluation suite")
    p.add_argument("--selftest", action="store_true")
    p.add_argument("--list", action="store_true")
    p.add_argument("--info", action="store_true")
    p.add_argument("--mirror", default=None, help="directory or file:// URL of a staged dataset mirror")
    # MCP service / studio
    p.add_argument("--mcp_action", default="status", choices=["status", "list", "start", "call"])
    p.add_argument("--mcp_host", default="127.0.0.1")
    p.add_argument("--mcp_port", type=int, default=3141)
    p.add_argument("--plxs_port", type=int, default=3140)
    p.add_argument("--frontend_port", type=int, default=3000)
    p.add_argument("--no_frontend", action="store_true")
    # publishing
    p.add_argument("--publish_action", default="export", choices=["export", "docker", "register", "hub", "all"])
    p.add_argument("--publish_config", default=None)
    p.add_argument("--publish_model_path", default=None)
    p.add_argument("--publish_model_size", default=None)
    p.add_argument("--publish_output_dir", default=None)
    p.add_argument("--publish_export_format", default="safetensors")
    p.add_argument("--publish_export_quantize", action="store_true")
    p.add_argument("--publish_quant_bits", type=int, default=8)
    p.add_argument("--publish_generate_checksum", action="store_true", default=True)
    p.add_argument("--publish_no_checksum", action="store_true")
    p.add_argument("--publish_checksum_algorithms", default="sha256")
    p.add_argument("--publish_metadata_name", default=None)
    p.add_argument("--publish_metadata_version", default=None)
    p.add_argument("--publish_metadata_author", default=None)
    p.add_argument("--publish_metadata_description", default=None)
    p.add_argument("--publish_metadata_license", default=None)
    p.add_argument("--publish_base_image", default=None)
    p.add_argument("--publish_port", type=int, default=8000)
    p.add_argument("--publish_env_vars", default=None)
    p.add_argument("--publish_health_check", action="store_true", default=True)
    p.add_argument("--publish_no_health_check", action="store_true")
    p.add_argument("--publish_template", default=None)
    p.add_argument("--publish_registry", default=None)
    p.add_argument("--publish_registry_namespace", default=None)
    p.add_argument("--publish_registry_repo", default=None)
    p.add_argument("--publish_registry_tag", default="latest")
    p.add_argument("--publish_username", default=None)
    p.add_argument("--publish_password", default=None)
    p.add_argument("--publish_retry_count", type=int, default=3)
    p.add_argument("--publish_retry_delay", type=float, default=2.0)
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
    if args.rlhf or args.train_mode == "preference":
        from pisceslx_b200.engine.orchestrator import PiscesLxPreferenceOrchestrator
        return PiscesLxPreferenceOrchestrator(args).run(args)
    if args.train_mode == "quant_export":
        from pisceslx_b200.engine.orchestrator import run_quant_export
        return run_quant_export(args)
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
    if args.selftest or args.benchmark or args.list:
        from pisceslx_b200.tools import benchmark_suites as suites
        if args.list:
            print("\n".join(sorted(suites.available_suites())))
            return 0
        if args.selftest:
            rep = suites.selftest()
            print(json.dumps(rep, indent=1, default=str))
            return 0 if rep.get("ok", True) else 1
        from pisceslx_b200.engine.loader import load_model_for_inference
        model = load_model_for_inference(args.model_size, args.ckpt, args.device or "cpu", args.model_config)
        print(json.dumps(suites.run_suite(args.benchmark, model, max_samples=args.max_samples), indent=1, default=str))
        return 0
    if args.perf:
        from pisceslx_b200.engine.loader import load_model_for_inference
        from pisceslx_b200.tools.benchmark import PiscesLxPerformanceBenchmark
        model = load_model_for_inference(args.model_size, args.ckpt, args.device or "cpu", args.model_config)
        print(json.dumps(PiscesLxPerformanceBenchmark(model).run().__dict__, indent=1, default=str))
        return 0
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
    if args.monitor_mode == "loop":
        from pisceslx_b200.tools.monitor_tool import PiscesLxToolsMonitorConfig, PiscesLxToolsMonitorRunner
        cfg = PiscesLxToolsMonitorConfig()
        cfg.interval_s = float(args.update_interval)
        PiscesLxToolsMonitorRunner(config=cfg).run(iterations=int(args.steps) if args.dry_run else 0)
        return 0
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
    """export -> docker context -> local registry -> hub preparation, as ``--publish_action`` asks."""
    from pisceslx_b200.engine.loader import load_model_for_inference
    from pisceslx_b200.tools.publish_pipeline import PiscesLxPublishConfig, PiscesLxPublishOrchestrator
    cfg = PiscesLxPublishConfig(output_dir=args.publish_output_dir or args.output_dir or "publish_out")
    act = args.publish_action
    cfg.docker.enabled = act in ("docker", "all")
    if act in ("register", "all") or args.publish_registry:
        cfg.registry.root = args.publish_registry or os.path.join(cfg.output_dir, "_registry")
    if act in ("hub", "all") and args.publish_registry_repo:
        cfg.hub.repo_id = "/".join(x for x in (args.publish_registry_namespace, args.publish_registry_repo) if x)
    for field_name, val in (("name", args.publish_metadata_name), ("version", args.publish_metadata_version),
                            ("author", args.publish_metadata_author), ("description", args.publish_metadata_description),
                            ("license", args.publish_metadata_license)):
        if val is not None and hasattr(cfg.metadata, field_name):
            setattr(cfg.metadata, field_name, val)
    if args.publish_no_checksum and hasattr(cfg.checksum, "enabled"):
        cfg.checksum.enabled = False
    if hasattr(cfg.checksum, "algorithm"):
        cfg.checksum.algorithm = args.publish_checksum_algorithms.split(",")[0]
    if args.publish_base_image and hasattr(cfg.docker, "base_image"):
        cfg.docker.base_image = args.publish_base_image
    if hasattr(cfg.docker, "port"):
        cfg.docker.port = args.publish_port
    model = load_model_for_inference(args.publish_model_size or args.model_size, args.publish_model_path or args.ckpt,
                                     args.device or "cpu", args.model_config)
    print(json.dumps(PiscesLxPublishOrchestrator(cfg).run(model), indent=1, default=str))
    return 0


def cmd_download(args, argv) -> int:
    """Datasets of ``configs/dataset.yaml`` (or ``--dataset NAME``) from a staged mirror or, where a hub client and
    the network exist, from the hubs; resumable."""
    from pisceslx_b200.data.acquire import (PiscesLxToolsDataConfigLoader, PiscesLxToolsDataDatasetDownload,
                                            PiscesLxToolsDataDownloadConfig, PiscesLxToolsDatasetItem)
    if args.dataset and args.dataset != "synthetic":
        cfg = PiscesLxToolsDataDownloadConfig([PiscesLxToolsDatasetItem(args.dataset)])
    else:
        path = os.path.join(ROOT, "configs", "dataset.yaml")
        cfg = PiscesLxToolsDataConfigLoader(path).load() if os.path.exists(path) else PiscesLxToolsDataDownloadConfig()
    cfg.mirror = args.mirror or cfg.mirror
    if args.output_dir:
        cfg.data_dir = args.output_dir
    if args.list or args.dry_run:
        print(json.dumps({"datasets": [d.name for d in cfg.datasets], "data_dir": cfg.data_dir, "mirror": cfg.mirror}))
        return 0
    rep = PiscesLxToolsDataDatasetDownload().download(cfg, args.max_samples)
    print(json.dumps(rep, indent=1))
    return 1 if rep["failed"] and not rep["completed"] and not rep["skipped"] else 0


def cmd_mcp(args, argv) -> int:
    from pisceslx_b200.third_party.mcp_service import MCPPlaza
    plaza = MCPPlaza()
    if args.mcp_action in ("status", "list"):
        tools = plaza.registry.list() if hasattr(plaza, "registry") and hasattr(plaza.registry, "list") else []
        print(json.dumps({"host": args.mcp_host, "port": args.mcp_port, "tools": tools}, default=str))
        return 0
    print(json.dumps({"action": args.mcp_action, "note": "the MCP service runs inside `manage.py serve` (routes under /v1/tools)"}))
    return 0


def cmd_plxs(args, argv) -> int:
    """Studio back end: the inference service on ``--plxs_port``.  The graphical front end of the reference's studio is
    a separate web application and is not part of this package (``--no_frontend`` is implied)."""
    args.port = args.plxs_port
    if args.dry_run:
        print(json.dumps({"backend": f"http://{args.host}:{args.plxs_port}", "frontend": None}))
        return 0
    return cmd_serve(args, argv)


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
                "cache": cmd_cache, "publish": cmd_publish, "download": cmd_download, "dev": cmd_dev, "mcp": cmd_mcp,
                "plxs": cmd_plxs}
    return int(handlers[args.command](args, argv) or 0)


if __name__ == "__main__":
    sys.exit(main())
