#!/usr/bin/env python
"""Reference arm: trains the UNMODIFIED reference (a plain copy under ``baseline/_ref``) on the benchmark's
model and data shape through the reference's own trainer, and prints the benchmark's JSON line.

Path driven (all reference code): ``PiscesLxTrainOrchestrator`` (tools/train/orchestrator.py:135) with the same
configuration steps as its ``run`` (``:998-1057``: model YAML -> top-level config -> CLI overrides -> flagship
memory/convergence policy -> MoE overrides), the same process-group set-up (``:1077-1100``),
``initialize_training(YvModel, cfg=...)`` (``:1492``: ``PiscesLxTrainingOperator.initialize_model`` with its
DDP / FSDP decision, optimizer and scheduler), then ``trainer.train_step(batch)`` (tools/train/core.py:2877) per
micro-batch.  Only the dataset is replaced: batches of uniform-random token ids in the collator's format
``{input_ids, attention_mask, labels}`` are made on the host, pinned, and handed to ``train_step`` (which copies
them to the device itself, core.py:1920-1924).  No module of ``pisceslx_b200`` is imported here.

The one missing third-party import (``dmsc``, a logging middleware) is satisfied by ``baseline/standin/dmsc``,
which lives outside the reference copy.  Any failure of the stock path (host- or device-memory refusal included)
is reported as ``{"impl": "reference", "unavailable": "<exception text>"}`` with exit code 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
VOCAB = 154856


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--seqs-per-gpu", type=int, default=64, help="sequences per GPU per optimizer step")
    ap.add_argument("--micro-batch", type=int, default=1, help="sequences per train_step call")
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--vocab", type=int, default=VOCAB)
    ap.add_argument("--optimizer", default="", help="override optimizer.name (default: what the reference picks)")
    ap.add_argument("--grad-ckpt", default="on", choices=["on", "off"],
                    help="activation checkpointing (the reference's policy default is on)")
    ap.add_argument("--cpu", action="store_true", help="host-only smoke run of the path (tiny shapes)")
    ap.add_argument("--out", default="", help="also write the JSON line to this file")
    return ap.parse_args()


def model_yaml(a) -> dict:
    """Benchmark model as reference YvConfig fields: legacy attention + MoE block, no SSM branch.

    The reference builds routed and shared experts with ONE width (``intermediate_size``, model/moe/layer.py:625,
    :665-700), so the two shared experts of FFN 2816 are expressed as four of FFN 1408: same parameters and FLOPs.
    """
    heads = max(a.hidden // 128, 1)
    return {
        "vocab_size": a.vocab, "hidden_size": a.hidden, "n_layer": a.layers, "n_head": heads,
        "n_kv_head": max(heads // 4, 1), "head_dim": a.hidden // heads,
        "intermediate_size": max(1408 * a.hidden // 4096, 8),
        "max_position_embeddings": a.seq, "rope_theta": 10000.0,
        "moe_num_experts": a.experts, "moe_top_k": min(6, a.experts), "moe_shared_experts": 4,
        "moe_fine_grained": False, "moe_num_sub_experts": 1, "moe_aux_loss_free": True,
        "backbone_allow_legacy_blocks": True, "use_mamba3": False, "use_subconscious": False,
        "use_subconscious_blocks": False, "num_mtp_heads": 0, "tie_word_embeddings": False,
        "use_gradient_checkpointing": a.grad_ckpt == "on", "vram_gradient_checkpointing": a.grad_ckpt == "on",
        # the legacy block passes a keyword its own YvPhiBalancing does not take (model/core/blocks.py:1707-1714)
        "use_phi_balancing": False,
        # plain causal GQA as the benchmark names it: key pruning (DSA), KV condensation (LCA) and the Duo streaming
        # window off.  (With the Duo window shorter than the sequence the reference concatenates K of two lengths
        # along the head axis and raises, model/core/attention.py:5512-5523.)
        "dsa_sparse_ratio": 0.0, "use_lca": False, "duo_attention_buffer_size": max(a.seq, 1024),
        "duo_attention_retrieval_ratio": 1.0,
        # its "fused" dispatch adds fp32 rows into a bf16 buffer under autocast and raises
        # (opss/infer/fused_moe.py:119); the plain per-expert loop (model/moe/layer.py:915-936) runs
        "use_fused_moe": False,
    }


def emit(obj, out_path=""):
    line = json.dumps(obj)
    print(line, flush=True)
    if out_path:
        try:
            with open(out_path, "w") as f:
                f.write(line + "\n")
        except OSError:
            pass


def short(exc: BaseException) -> str:
    text = f"{type(exc).__name__}: {exc}".replace("\n", " ")
    return text[:600]


def start_host_memory_watchdog(out_path: str, floor_gb: float = 0.0) -> None:
    """The reference builds the whole model in host memory first (tools/train/core.py:883).  If that drives the
    machine close to exhaustion, report it and leave before the kernel's OOM killer takes the box down."""
    import threading

    try:
        import psutil
    except ImportError:
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    floor_gb = floor_gb or (12.0 + 4.0 * world)             # every rank builds at the same time

    def watch():
        while True:
            avail = psutil.virtual_memory().available / 2 ** 30
            if avail < floor_gb:
                if int(os.environ.get("RANK", "0")) == 0:
                    emit({"impl": "reference", "unavailable": "stock reference path failed: host memory exhausted while "
                          f"the reference built the model on the CPU ({avail:.1f} GB left of "
                          f"{psutil.virtual_memory().total / 2 ** 30:.0f} GB)"}, out_path)
                os._exit(0)
            time.sleep(0.1)

    threading.Thread(target=watch, daemon=True).start()


def run(a) -> dict:
    import tempfile

    import yaml

    sys.path.insert(0, os.path.join(HERE, "standin"))
    sys.path.insert(0, REF)
    os.chdir(REF)                      # the reference resolves configs/ and tokenizer/ relative to the cwd
    os.environ.setdefault("PISCESLX_HOME", tempfile.mkdtemp(prefix="plx_ref_home_"))
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = os.environ.get("LOCAL_RANK")
    use_cuda = torch.cuda.is_available() and not a.cpu
    if local_rank is not None and world > 1:
        # same defaults as tools/train/orchestrator.py:1077-1100
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        os.environ.setdefault("TORCH_NCCL_AVOID_RECORD_STREAMS", "1")
        dist.init_process_group(backend="nccl" if use_cuda else "gloo")
        if use_cuda:
            torch.cuda.set_device(int(local_rank))
    rank = dist.get_rank() if dist.is_initialized() else 0

    from model import YvConfig, YvModel
    from tools.train.orchestrator import PiscesLxTrainOrchestrator

    cfg_dir = tempfile.mkdtemp(prefix="plx_ref_cfg_")
    cfg_path = os.path.join(cfg_dir, "bench.yaml")
    with open(cfg_path, "w") as f:
        yaml.safe_dump(model_yaml(a), f)

    n_micro = max(a.seqs_per_gpu // a.micro_batch, 1)
    params = {"model_size": "bench", "config": cfg_path, "seq_len": a.seq, "stage": None, "dataset": "synthetic",
              "batch_size": a.micro_batch, "gradient_accumulation_steps": n_micro,
              "max_steps": a.steps + a.warmup, "device": "cuda" if use_cuda else "cpu"}
    orch = PiscesLxTrainOrchestrator(None)
    tc = orch.train_config
    model_cfg = YvConfig.from_yaml(cfg_path)
    orch._seed_training_moe_defaults_from_model_config(model_cfg)
    orch._apply_top_level_config(model_cfg)
    try:
        tc.apply_cli_overrides(params)
    except Exception:
        pass
    orch._apply_flagship_memory_and_convergence_policy(model_cfg, params)
    model_cfg = orch._apply_training_moe_overrides_to_model_config(model_cfg)
    tc.max_steps = a.steps + a.warmup
    tc.data.sequence_length = a.seq
    tc.data.batch_size = a.micro_batch
    tc.gradient_accumulation_steps = n_micro
    tc.gradient_checkpointing = a.grad_ckpt == "on"
    if a.optimizer:
        tc.optimizer.name = a.optimizer
    if not use_cuda:                    # host-only smoke run: what the reference's CPU tier accepts
        tc.device = "cpu"
        for name in ("mixed_precision", "vram_mixed_precision"):
            if hasattr(tc, name):
                setattr(tc, name, "none")
        for name in ("use_flash_attention", "vram_flash_attention", "flash_attention"):
            if hasattr(tc, name):
                setattr(tc, name, False)

    orch.initialize_training(model_class=YvModel, train_dataloader_factory=lambda *x, **k: None,
                             val_dataloader_factory=None, cfg=model_cfg, modalities={"text"})
    trainer = orch.trainer
    n_params = sum(p.numel() for p in trainer.model.parameters())

    gen = torch.Generator().manual_seed(1234 + rank)

    def host_batch():
        ids = torch.randint(0, a.vocab, (a.micro_batch, a.seq), generator=gen, dtype=torch.long)
        if use_cuda:
            ids = ids.pin_memory()
        return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids.clone()}

    def one_step():
        loss = 0.0
        for _ in range(n_micro):
            out = trainer.train_step(host_batch())
            loss = out["loss"]
        return loss

    def fence():
        if dist.is_initialized():
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()

    for _ in range(a.warmup):
        one_step()
    fence()
    if use_cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    loss = 0.0
    for _ in range(a.steps):
        loss = one_step()
    if use_cuda:
        e1.record()
    fence()
    ms = e0.elapsed_time(e1) if use_cuda else (time.perf_counter() - t0) * 1e3
    if dist.is_initialized():
        t = torch.tensor([ms], dtype=torch.float64, device="cuda" if use_cuda else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tokens = a.steps * world * n_micro * a.micro_batch * a.seq
    value = tokens / (ms / 1e3)
    full = (a.layers == 32 and a.hidden == 4096 and a.experts == 64 and a.vocab == VOCAB and a.seq == 4096)
    wrapper = type(trainer.model).__name__
    return {"impl": "reference", "metric": "train tokens/sec/box Yv-7B MoE", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": str(getattr(tc, "mixed_precision", "bf16")), "data": "synthetic uniform-random token ids, "
            "random-init weights", "same_config": bool(full),
            "config": {"model": f"reference YvModel legacy blocks: {a.layers}L h{a.hidden} {a.experts} experts "
                                f"ffn{model_yaml(a)['intermediate_size']} top6 + 4 shared (= 2 x 2816), vocab {a.vocab}",
                       "global_batch": world * n_micro * a.micro_batch, "seq_len": a.seq, "micro_batch": a.micro_batch,
                       "parallelism": f"{wrapper} x{world}", "optimizer": str(tc.optimizer.name),
                       "parameters": n_params},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": n_micro * a.micro_batch * a.seq * 8 * 3,
                    "d2h_bytes_per_step": 4 * n_micro},
            "loss": float(loss)}


def main():
    a = parse_args()
    start_host_memory_watchdog(a.out)
    try:
        emit(run(a), a.out)
    except BaseException as exc:            # SystemExit from the reference included
        traceback.print_exc(file=sys.stderr)
        rank = int(os.environ.get("RANK", "0"))
        if rank == 0:
            emit({"impl": "reference", "unavailable": "stock reference path failed: " + short(exc)}, a.out)
    finally:
        try:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:
            pass


if __name__ == "__main__":
    main()
