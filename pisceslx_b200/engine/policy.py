"""Training policy layer: rules applied after model YAML, stage YAML and CLI overrides have been merged and before the
trainer is built.

Two rule sets:

* ``apply_convergence_policy`` - the guarantees of the reference's flagship policy
  (tools/train/orchestrator.py:584-721): a from-scratch stage trains every parameter (weight quantisation and LoRA
  forced off whatever the YAMLs say), an adapter stage (SFT-with-base-weight, DPO / ORPO / PPO, or any run given
  ``model_name_or_path``) gets 4-bit NF4 base weights with LoRA of a rank that grows with the model (32 / 64 / 128)
  on all attention and expert projections and 8-bit optimizer states; FP4 and GaLore optimizer modes are switched off;
  the scheduler is cosine or linear, with a warm-up that is at least one step and shorter than the run, and a floor of
  0.1 x the peak rate; gradient checkpointing stays on unless the configuration says ``false`` explicitly; bf16; and the
  cadences default to save 1000 / eval 500 / log 10.  A resume checkpoint is NOT a base weight: resuming never turns a
  from-scratch run into an adapter run.
* ``apply_memory_policy`` - what the reference decides per GPU generation with fixed thresholds
  (``:1565-1619``) is computed here from a memory model of the 180 GB part: bytes of weights, optimizer state and
  per-layer activations under the chosen layout decide the Muon momentum format (bf16 or block-quantised int8), whether
  gradients are consumed inside backward, the activation-recomputation mode, and the micro-batch size.

Both return the list of decisions they took, which the orchestrator logs and stores in the run's ``spec.json``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

ADAPTER_STAGES = ("alignment_dpo", "alignment_orpo", "alignment_ppo", "specialized")
LORA_TARGETS = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


@dataclass
class YvTrainingPlan:
    """The trainer-facing result of the merged configuration layers."""
    stage: str = "pretrain"
    optimizer: str = "muon"
    scheduler: str = "cosine"
    warmup_steps: int = 0
    warmup_type: str = "exponential"
    min_lr_ratio: float = 0.0
    max_steps: int = 0
    gradient_checkpointing: Any = None            # None = not stated; "false" / False = explicitly off
    mixed_precision: str = "bf16"
    flash_attention: bool = True
    save_steps: int = 0
    eval_steps: int = 0
    log_steps: int = 0
    quantization: Dict[str, Any] = field(default_factory=lambda: {"enable_quantization": False, "quant_method": None,
                                                                  "bits": None, "group_size": None})
    lora: Dict[str, Any] = field(default_factory=lambda: {"enabled": False, "r": 0, "lora_alpha": 0, "target_modules": []})
    use_fp4: bool = False
    use_galore: bool = False
    # memory policy outputs
    state_dtype: Optional[str] = None
    streaming_optimizer: bool = False
    recompute_policy: str = "config"
    micro_batch_size: int = 1

    @classmethod
    def from_layers(cls, model_training_cfg: Optional[Dict[str, Any]], stage_cfg: Optional[Dict[str, Any]],
                    stage: str = "pretrain") -> "YvTrainingPlan":
        """Later layers win: model YAML ``training_config`` < stage YAML."""
        plan = cls(stage=stage)
        for layer in (model_training_cfg or {}, stage_cfg or {}):
            opt, sch = layer.get("optimizer") or {}, layer.get("scheduler") or {}
            if isinstance(opt, str):
                opt = {"name": opt}
            plan.optimizer = str(opt.get("name", plan.optimizer))
            plan.use_fp4 = bool(opt.get("use_fp4", plan.use_fp4))
            plan.use_galore = bool(opt.get("use_galore", plan.use_galore))
            plan.scheduler = str(sch.get("name", sch.get("type", plan.scheduler)))
            plan.warmup_steps = int(sch.get("warmup_steps", plan.warmup_steps) or 0)
            plan.warmup_type = str(sch.get("warmup_type", plan.warmup_type))
            plan.min_lr_ratio = float(sch.get("min_lr_ratio", plan.min_lr_ratio) or 0.0)
            for k in ("max_steps", "save_steps", "eval_steps", "log_steps", "micro_batch_size"):
                if layer.get(k) is not None:
                    setattr(plan, k, int(layer[k]))
            if "gradient_checkpointing" in layer:
                plan.gradient_checkpointing = layer["gradient_checkpointing"]
            if layer.get("mixed_precision"):
                plan.mixed_precision = str(layer["mixed_precision"])
            if "flash_attention" in layer:
                plan.flash_attention = bool(layer["flash_attention"])
            if isinstance(layer.get("quantization"), dict):
                plan.quantization.update(layer["quantization"])
            if isinstance(layer.get("lora"), dict):
                plan.lora.update(layer["lora"])
        return plan


def lora_rank_for(hidden_size: int, n_layer: int) -> Dict[str, int]:
    scale = max(int(hidden_size or 0), int(n_layer or 0) * 128)
    if scale <= 1024:
        return {"r": 32, "lora_alpha": 64}
    if scale <= 2048:
        return {"r": 64, "lora_alpha": 128}
    return {"r": 128, "lora_alpha": 256}


def apply_convergence_policy(plan: YvTrainingPlan, model_cfg: Any, model_name_or_path: Optional[str] = None,
                             resume_ckpt: Optional[str] = None) -> List[str]:
    notes: List[str] = []
    base_weight = str(model_name_or_path or "").strip()
    adapter_run = plan.stage in ADAPTER_STAGES or bool(base_weight)
    if resume_ckpt and not adapter_run:
        notes.append("resume checkpoint given: continuing the same full-parameter run (not an adapter run)")
    q, l = plan.quantization, plan.lora
    if adapter_run:
        q.update(enable_quantization=True, quant_method="nf4", bits=4)
        if q.get("group_size") is None:
            q["group_size"] = 128
        want = lora_rank_for(getattr(model_cfg, "hidden_size", 0), getattr(model_cfg, "n_layer", 0))
        l["enabled"] = True
        l["r"] = max(int(l.get("r") or 0), want["r"])
        l["lora_alpha"] = max(int(l.get("lora_alpha") or 0), want["lora_alpha"])
        targets = list(l.get("target_modules") or [])
        if not targets:
            targets = list(LORA_TARGETS)
        elif "k_proj" not in targets:
            targets.append("k_proj")
        l["target_modules"] = targets
        if plan.optimizer != "adamw8bit":
            notes.append(f"adapter run: optimizer {plan.optimizer} -> adamw8bit (8-bit states)")
            plan.optimizer = "adamw8bit"
        notes.append(f"adapter run: NF4 base weights, LoRA r={l['r']} alpha={l['lora_alpha']} on {len(targets)} projections")
    else:
        if q.get("enable_quantization") or l.get("enabled"):
            notes.append("from-scratch stage: weight quantisation and LoRA switched off (nothing to adapt)")
        q["enable_quantization"] = False
        l["enabled"] = False
    if plan.use_fp4 or plan.use_galore:
        notes.append("optimizer FP4 / GaLore modes switched off")
        plan.use_fp4 = plan.use_galore = False
    if plan.scheduler.lower() not in ("cosine", "linear"):
        notes.append(f"scheduler {plan.scheduler} -> cosine")
        plan.scheduler = "cosine"
    cap = max(1, plan.max_steps // 10) if plan.max_steps > 0 else 100
    if plan.warmup_steps <= 0:
        plan.warmup_steps = min(100, cap)
    elif plan.max_steps > 0 and plan.warmup_steps >= plan.max_steps:
        notes.append(f"warm-up {plan.warmup_steps} >= run length {plan.max_steps}: -> {cap}")
        plan.warmup_steps = cap
    if plan.min_lr_ratio <= 0.0:
        plan.min_lr_ratio = 0.1
    if str(plan.gradient_checkpointing) not in ("false", "False"):
        plan.gradient_checkpointing = True
    else:
        plan.gradient_checkpointing = False
    if not plan.mixed_precision:
        plan.mixed_precision = "bf16"
    plan.save_steps = plan.save_steps if plan.save_steps > 0 else 1000
    plan.eval_steps = plan.eval_steps if plan.eval_steps > 0 else 500
    plan.log_steps = plan.log_steps if plan.log_steps > 0 else 10
    return notes


def apply_memory_policy(plan: YvTrainingPlan, model_cfg: Any, *, tp: int = 1, ep: int = 1, dp: int = 1, seq_len: int = 4096,
                        hbm_gb: float = 180.0, budget: float = 0.90) -> List[str]:
    """Decide state format, gradient intake, recomputation and micro-batch from bytes, not from GPU names."""
    notes: List[str] = []
    counts = model_cfg.count_parameters() if hasattr(model_cfg, "count_parameters") else {}
    total = float(counts.get("total", 0) or 0)
    n_moe = sum(1 for i in range(getattr(model_cfg, "n_layer", 0)) if model_cfg.is_moe_layer(i)) \
        if hasattr(model_cfg, "is_moe_layer") else 0
    expert = float(n_moe * getattr(model_cfg, "moe_num_experts", 0) * 3 * getattr(model_cfg, "hidden_size", 0)
                   * (getattr(model_cfg, "moe_expert_intermediate_size", 0) or 0))
    dense = max(total - expert, 0.0)
    # parameters resident on one rank: experts split over ep, tensor-parallel matrices over tp (embeddings replicated)
    local = expert / max(ep, 1) + dense / max(tp, 1)
    weights_gb = local * 2 / 1e9
    # ZeRO-1: the optimizer state of a tensor lives on its owner only
    state_share = 1.0 / max(dp // max(ep, 1), 1) if expert else 1.0 / max(dp, 1)
    momentum_bf16_gb = local * 2 * state_share / 1e9
    room = hbm_gb * budget
    hidden, n_layer = getattr(model_cfg, "hidden_size", 0), getattr(model_cfg, "n_layer", 0)
    top_k = getattr(model_cfg, "moe_top_k", 0) or 0
    # stored activations of one layer for one sequence: token rows (about 10 x hidden) + expert rows (top_k x FFN x 2)
    ffn = getattr(model_cfg, "moe_expert_intermediate_size", 0) or getattr(model_cfg, "intermediate_size", 0) or 0
    act_layer_gb = seq_len * (10 * hidden + top_k * 2 * ffn + 2 * hidden) * 2 / max(tp, 1) / 1e9
    grads_gb = weights_gb                                      # a full set of gradients, when they are kept
    if weights_gb + momentum_bf16_gb + grads_gb + act_layer_gb * 2 <= room:
        plan.streaming_optimizer, plan.state_dtype = False, None
        notes.append(f"weights {weights_gb:.0f} GB + states {momentum_bf16_gb:.0f} GB + gradients {grads_gb:.0f} GB fit: "
                     "plain step (gradients kept, clipping available)")
    else:
        plan.streaming_optimizer = True
        notes.append(f"weights {weights_gb:.0f} GB + states + gradients exceed {room:.0f} GB: gradients are consumed inside backward")
        if weights_gb + momentum_bf16_gb + act_layer_gb * n_layer * 0.5 > room:
            plan.state_dtype = "int8"
            notes.append("Muon momentum block-quantised to int8 so that more layers keep their activations")
        else:
            plan.state_dtype = "bf16"
    free_gb = room - weights_gb - (momentum_bf16_gb * (0.5 if plan.state_dtype == "int8" else 1.0))
    if plan.streaming_optimizer is False:
        free_gb -= grads_gb
    mb = 1
    while act_layer_gb * (mb * 2) * 2 <= free_gb and mb < 8:
        mb *= 2
    plan.micro_batch_size = max(plan.micro_batch_size, 1) if plan.micro_batch_size > 1 else mb
    if plan.gradient_checkpointing is False and act_layer_gb * plan.micro_batch_size * n_layer > free_gb:
        notes.append("gradient checkpointing was switched off explicitly but the activations do not fit: recomputation "
                     "is sized from measured memory instead")
    plan.recompute_policy = "auto" if plan.gradient_checkpointing is not False or \
        act_layer_gb * plan.micro_batch_size * n_layer > free_gb else "config"
    notes.append(f"micro-batch {plan.micro_batch_size} sequence(s); activations of one layer {act_layer_gb * plan.micro_batch_size:.2f} GB; "
                 f"recomputation: {plan.recompute_policy}")
    return notes
