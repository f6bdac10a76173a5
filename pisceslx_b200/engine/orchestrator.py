"""Train / infer orchestrators behind ``manage.py``.

``PiscesLxTrainOrchestrator.run(args)`` follows the reference flow (tools/train/orchestrator.py:881-1811): model
YAML -> nested ``training_config`` / ``distributed`` sections -> stage YAML (``configs/train/<stage>.yaml``) -> CLI
overrides (later wins; unknown keys are ignored), process group from the torchrun environment, dataset + collator,
trainer, optional resume, run-store reporting, checkpoints ``checkpoint_step_<N>.pt`` / ``final_model.pt``.
``PiscesLxInferOrchestrator.run(args)`` is the one-shot generation entry (tools/infer/orchestrator.py:85-244).
"""
from __future__ import annotations

import json
import os
import time
from pathlib import Path
from typing import Any, Dict, Optional

import torch
import yaml

from ..config import YvConfig
from .loader import REPO_ROOT, attach_optional_components, load_model_for_inference, resolve_model_config
from .runstore import PiscesLxRunIdFactory, PiscesLxRunStore, PiscesLxTrainingRunReporter
from .trainer import YvTrainer, YvTrainerConfig


def load_stage_config(stage: str, path: Optional[str] = None) -> Dict[str, Any]:
    p = Path(path) if path else REPO_ROOT / "configs" / "train" / f"{stage}.yaml"
    if not p.exists():
        p = REPO_ROOT / "configs" / "train" / "default.yaml"
    return yaml.safe_load(p.read_text()) or {}


def build_trainer_config(model_cfg: YvConfig, stage_cfg: Dict[str, Any], args: Any) -> YvTrainerConfig:
    tc = dict(model_cfg.extra.get("training_config") or {})
    opt = dict(stage_cfg.get("optimizer") or {})
    sch = dict(stage_cfg.get("scheduler") or {})
    cfg = YvTrainerConfig(
        micro_batch_size=int(stage_cfg.get("micro_batch_size", tc.get("micro_batch_size", 1))),
        optimizer=str(opt.get("name", tc.get("optimizer", "muon"))),
        lr=float(opt.get("lr", tc.get("lr", 2e-4))),
        weight_decay=float(opt.get("weight_decay", tc.get("weight_decay", 0.1))),
        scheduler=str(sch.get("type", "cosine")),
        warmup_steps=max(1, int(sch.get("warmup_steps", tc.get("warmup_steps", 1)))),
        min_lr_ratio=max(0.1, float(sch.get("min_lr_ratio", 0.1))),
        max_steps=int(stage_cfg.get("max_steps", 1000)),
        clip_grad_norm=float(stage_cfg.get("clip_grad_norm", 1.0)),
        save_steps=int(stage_cfg.get("save_steps", 1000)),
        log_steps=int(stage_cfg.get("log_steps", 10)),
    )
    for name in ("micro_batch_size", "max_steps", "lr", "optimizer", "save_steps", "output_dir"):
        v = getattr(args, name, None)
        if v is not None:
            setattr(cfg, name, v)
    return cfg


class PiscesLxTrainOrchestrator:
    CONTROL_SYNC_STEPS = 10            # multi-rank runs agree on stop / pause every this many steps

    def __init__(self, args: Any):
        self.args = args

    @staticmethod
    def apply_policy(model_cfg: YvConfig, stage_cfg: Dict[str, Any], tcfg: YvTrainerConfig, args: Any, par: Any,
                     seq_len: int) -> list:
        """Run the convergence and memory rule sets (``engine.policy``) over the merged configuration layers and copy
        their decisions into the trainer configuration; explicit command-line values are left alone."""
        from .policy import YvTrainingPlan, apply_convergence_policy, apply_memory_policy
        plan = YvTrainingPlan.from_layers(model_cfg.extra.get("training_config"), stage_cfg, stage=str(args.stage))
        plan.max_steps = tcfg.max_steps
        plan.optimizer = tcfg.optimizer
        notes = apply_convergence_policy(plan, model_cfg, getattr(args, "model_name_or_path", None),
                                         getattr(args, "resume_ckpt", None))
        tcfg.scheduler, tcfg.warmup_steps, tcfg.min_lr_ratio = plan.scheduler, plan.warmup_steps, plan.min_lr_ratio
        if getattr(args, "save_steps", None) is None and stage_cfg.get("save_steps") is None:
            tcfg.save_steps = plan.save_steps
        tcfg.log_steps = tcfg.log_steps or plan.log_steps
        if plan.gradient_checkpointing is False:
            model_cfg.use_gradient_checkpointing = False
        if par.device.type == "cuda":
            plan.streaming_optimizer = tcfg.streaming_optimizer
            notes += apply_memory_policy(plan, model_cfg, tp=par.tp_size, ep=par.ep_size, dp=par.dp_size, seq_len=seq_len)
            tcfg.streaming_optimizer = tcfg.streaming_optimizer or plan.streaming_optimizer
            if tcfg.state_dtype is None:
                tcfg.state_dtype = plan.state_dtype
            if tcfg.streaming_optimizer:
                tcfg.clip_grad_norm = 0.0                    # gradients are folded as produced: nothing left to clip
            tcfg.recompute_policy = plan.recompute_policy
            if getattr(args, "micro_batch_size", None) is None and "micro_batch_size" not in stage_cfg:
                tcfg.micro_batch_size = plan.micro_batch_size
        return notes

    @staticmethod
    def _sync_control(reporter: Any, par: Any) -> bool:
        """Broadcast rank 0's stop / pause state; paused ranks wait here together.  Returns True to stop."""
        import torch.distributed as dist
        while True:
            if reporter is not None:
                reporter.poll_control()
            flags = torch.tensor([int(bool(reporter and reporter.stop_requested)), int(bool(reporter and reporter.paused))],
                                 dtype=torch.int32, device=par.device)
            dist.broadcast(flags, src=0)
            stop, paused = bool(flags[0].item()), bool(flags[1].item())
            if stop or not paused:
                return stop
            time.sleep(0.5)

    def run(self, args: Any) -> int:
        from ..data.datasets import build_dataloader
        from ..models import build_model
        from ..parallel.state import destroy_parallel, init_parallel
        from ..utils.seed import PiscesLxDeterminism

        PiscesLxDeterminism.seed_everything(args.seed)
        model_cfg = resolve_model_config(args.model_size, args.model_config)
        dist_cfg = dict(model_cfg.extra.get("distributed") or {})
        tp = args.tensor_parallel or int(dist_cfg.get("tensor_parallel", 1))
        ep = args.expert_parallel or int(dist_cfg.get("expert_parallel", 1))
        pp = args.pipeline_parallel or int(dist_cfg.get("pipeline_parallel", 1))
        cp = getattr(args, "context_parallel", None) or int(dist_cfg.get("context_parallel", 1))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world == 1:
            tp = ep = pp = cp = 1
        device = torch.device(args.device) if args.device else None
        par = init_parallel(tp=tp, ep=ep, pp=pp, cp=cp, device=device)
        model_cfg.context_parallel = cp
        if args.no_fused_comm:
            from ..parallel import fused
            fused.set_enabled(False)
        stage_cfg = load_stage_config(args.stage, args.train_config)
        tcfg = build_trainer_config(model_cfg, stage_cfg, args)
        seq_len = args.seq_len or int(stage_cfg.get("seq_len", 512))
        batch = args.batch_size or tcfg.micro_batch_size * int(stage_cfg.get("gradient_accumulation_steps", 1))
        dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, None: None}[args.dtype]
        if par.device.type == "cpu":
            model_cfg.use_gradient_checkpointing = False
        if args.dry_run:
            if par.rank == 0:
                print(json.dumps({"model": model_cfg.count_parameters(), "trainer": tcfg.__dict__, "seq_len": seq_len,
                                  "batch": batch, "parallel": {"tp": tp, "ep": ep, "pp": pp, "cp": cp, "world": world}},
                                 default=str))
            return 0
        model = build_model(model_cfg, par.device, dtype, parallel=par if world > 1 else None, seed=args.seed)
        attach_optional_components(model, model_cfg, par)
        tcfg.streaming_optimizer = bool(stage_cfg.get("streaming_optimizer", False))
        policy_notes = self.apply_policy(model_cfg, stage_cfg, tcfg, args, par, seq_len)
        if getattr(args, "sharding", None):
            tcfg.sharding = args.sharding
        if getattr(args, "state_dtype", None):
            tcfg.state_dtype = args.state_dtype
        if pp > 1:
            tcfg.streaming_optimizer = False
        trainer = YvTrainer(model, tcfg, parallel=par if world > 1 else None)
        store = PiscesLxRunStore(Path(args.run_dir) if args.run_dir else None)
        run_id = args.run_id or PiscesLxRunIdFactory.new("train")
        reporter = None
        if par.rank == 0:
            if not (store.run_dir(run_id) / "state.json").exists():
                store.init_run(run_id, {"command": "train", "args": {k: v for k, v in vars(args).items()},
                                        "policy": policy_notes})
            for note in policy_notes:
                print(f"[policy] {note}", flush=True)
            store.update_state(run_id, status="running", pid=os.getpid())
            reporter = PiscesLxTrainingRunReporter(store, run_id, trainer)
            trainer.callbacks.append(reporter)
        if args.resume_ckpt:
            from .checkpoint import load_checkpoint
            load_checkpoint(trainer, args.resume_ckpt, reset_lr=args.reset_lr)
        # context-parallel peers and the stages of one pipeline read the same sequences
        loader = build_dataloader(args.dataset, model_cfg.vocab_size, seq_len, batch, seed=args.seed + par.data_rank)
        status = "completed"
        try:
            for batch_t in loader:
                if trainer.global_step >= tcfg.max_steps or (reporter is not None and reporter.stop_requested):
                    break
                while reporter is not None and reporter.paused and not reporter.stop_requested and world == 1:
                    time.sleep(0.5)
                    reporter.poll_control()
                if world > 1 and trainer.global_step % self.CONTROL_SYNC_STEPS == 0:
                    # rank 0 reads the control channel; every rank must leave (or wait) at the same step, or the
                    # next collective never completes
                    if self._sync_control(reporter, par):
                        break
                res = trainer.train_step(batch_t)
                if par.rank == 0 and trainer.global_step % max(tcfg.log_steps, 1) == 0:
                    print(f"step {res['global_step']} loss {res['loss']:.4f} lr {res['learning_rate']:.3e} "
                          f"tok/s {res['token_throughput']:.0f}", flush=True)
                if tcfg.save_steps and trainer.global_step % tcfg.save_steps == 0:
                    from .checkpoint import save_checkpoint
                    save_checkpoint(trainer, f"{tcfg.output_dir}/checkpoint_step_{trainer.global_step}.pt")
        except KeyboardInterrupt:
            status = "interrupted"
        except Exception as e:
            status = "failed"
            if par.rank == 0:
                store.append_event(run_id, "error", message=str(e))
            raise
        finally:
            from .checkpoint import save_checkpoint
            if tcfg.save_steps:
                save_checkpoint(trainer, f"{tcfg.output_dir}/final_model.pt")
            if par.rank == 0:
                store.update_state(run_id, status=status, finished=time.time(), global_step=trainer.global_step)
            if world > 1:
                destroy_parallel()
        return 0


class PiscesLxInferOrchestrator:
    def __init__(self, args: Any):
        self.args = args

    def run(self, args: Any) -> int:
        from ..models.tokenizer import YvTokenizer
        if args.dry_run:
            print(json.dumps({"prompt_tokens": len(YvTokenizer.instance().encode(args.prompt)), "model_size": args.model_size}))
            return 0
        model = load_model_for_inference(args.model_size, args.ckpt, args.device, args.model_config)
        tok = YvTokenizer.for_vocab(model.cfg.vocab_size)
        ids = torch.tensor([tok.encode(args.prompt)], dtype=torch.long, device=next(model.parameters()).device)
        ids = ids.clamp_(0, model.cfg.vocab_size - 1)
        t0 = time.perf_counter()
        if args.speculative:
            from ..models.speculative import YvSpeculativeDecoder
            out, stats = YvSpeculativeDecoder(model).speculative_generate(ids, max_new_tokens=args.max_new_tokens)
        else:
            out, stats = model.generate(ids, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                                        top_k=args.top_k, top_p=args.top_p)
        dt = time.perf_counter() - t0
        text = tok.decode(out[0, ids.shape[1]:].tolist())
        print(json.dumps({"text": text, "stats": stats, "seconds": dt,
                          "tokens_per_second": stats.get("generated_tokens", 0) / max(dt, 1e-9)}))
        return 0


class PiscesLxPreferenceOrchestrator:
    """``manage.py train --rlhf`` / ``--train_mode preference`` (reference orchestrator ``_run_preference``): DPO over
    ``{"prompt", "chosen", "rejected"}`` records of ``--rlhf_dataset`` (jsonl), with a frozen reference copy of the
    policy.  Without a dataset a small synthetic preference set is used, so that the path can be exercised offline."""

    def __init__(self, args: Any):
        self.args = args

    def run(self, args: Any) -> int:
        from ..models import build_model
        from ..models.tokenizer import YvTokenizer
        from .alignment import PiscesLxDPOTrainingOperator
        from .rl import PiscesLxPreferenceDataProcessor
        model_cfg = resolve_model_config(args.model_size, args.model_config)
        model_cfg.use_gradient_checkpointing = False
        device = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
        model = build_model(model_cfg, device, torch.bfloat16 if device.type == "cuda" else torch.float32, seed=args.seed)
        if args.ckpt:
            from .checkpoint import extract_state_dict
            model.load_reference_state_dict(extract_state_dict(torch.load(args.ckpt, map_location="cpu", weights_only=False)),
                                            strict=False)
        tok = YvTokenizer.for_vocab(model_cfg.vocab_size)
        if args.rlhf_dataset:
            records = [json.loads(l) for l in open(args.rlhf_dataset, encoding="utf-8") if l.strip()]
        else:
            records = [{"prompt": f"question {i}: ", "chosen": "a careful and correct answer", "rejected": "no"} for i in range(16)]
        if args.rlhf_max_samples:
            records = records[: args.rlhf_max_samples]
        proc = PiscesLxPreferenceDataProcessor(tok, max_length=args.rlhf_max_length)
        opt = torch.optim.AdamW(model.parameters(), lr=args.rlhf_lr, weight_decay=0.0)
        op = PiscesLxDPOTrainingOperator(model, opt)
        if args.dry_run:
            print(json.dumps({"mode": "preference", "records": len(records), "batch": args.rlhf_batch_size, "epochs": args.rlhf_epochs}))
            return 0
        step, last = 0, {}
        for _ in range(args.rlhf_epochs):
            for s in range(0, len(records), args.rlhf_batch_size):
                b = proc.pairs(records[s:s + args.rlhf_batch_size])
                b = {k: v.to(device).clamp_(max=model_cfg.vocab_size - 1) if "labels" not in k else v.to(device) for k, v in b.items()}
                for k in ("chosen_labels", "rejected_labels"):
                    b[k] = torch.where(b[k] >= model_cfg.vocab_size, torch.full_like(b[k], -100), b[k])
                loss, last = op.step(b["chosen"], b["rejected"], b["chosen_labels"], b["rejected_labels"])
                step += 1
                if args.max_steps and step >= args.max_steps:
                    break
            if args.max_steps and step >= args.max_steps:
                break
        print(json.dumps({"steps": step, "loss": loss, **last}))
        if args.output_dir:
            from .checkpoint import _atomic_save
            _atomic_save({"model_state_dict": {k: v.cpu() for k, v in model.to_reference_state_dict().items()},
                          "global_step": step}, os.path.join(args.output_dir, "preference_final.pt"))
        return 0


def run_quant_export(args: Any) -> int:
    """``manage.py train --train_mode quant_export --ckpt C --quant METHOD --quant_bits N --save OUT``: post-training
    quantisation of a checkpoint through the PTQ engine and a reference-layout file of the de-quantised weights plus
    the quantisation report."""
    from ..quant.pipeline import PiscesLxQuantizationConfig, PiscesLxQuantizationEngine, PiscesLxQuantizationMethod
    model = load_model_for_inference(args.model_size, args.ckpt, args.device or "cpu", args.model_config)
    method = PiscesLxQuantizationMethod((args.quant or "rtn").lower())
    qcfg = PiscesLxQuantizationConfig(method=method, bits=int(args.quant_bits))
    if args.dry_run:
        print(json.dumps({"mode": "quant_export", "method": method.value, "bits": qcfg.bits}))
        return 0
    result = PiscesLxQuantizationEngine(qcfg).quantize(model)
    out = args.save or os.path.join(args.output_dir or ".", "quantized.pt")
    from .checkpoint import _atomic_save
    _atomic_save({"model_state_dict": {k: v.cpu() for k, v in model.to_reference_state_dict().items()},
                  "quantization": {"method": method.value, "bits": qcfg.bits}}, out)
    print(json.dumps({"saved": out, "method": method.value, "bits": qcfg.bits,
                      "layers": result.layers, "mean_bits": result.mean_bits, "seconds": result.seconds}, default=str))
    return 0
