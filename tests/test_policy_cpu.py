"""Training policy layer (reference tools/train/orchestrator.py:584-721 for the convergence rules)."""
from pisceslx_b200 import YvConfig
from pisceslx_b200.engine.policy import YvTrainingPlan, apply_convergence_policy, apply_memory_policy, lora_rank_for


def test_from_scratch_stage_forces_full_parameter_training():
    model_yaml = {"quantization": {"enable_quantization": True, "quant_method": "nf4", "bits": 4},
                  "lora": {"enabled": True, "r": 16}, "optimizer": {"name": "adamw", "use_galore": True}}
    stage_yaml = {"scheduler": {"name": "exponential", "warmup_steps": 5000}, "max_steps": 200,
                  "gradient_checkpointing": "false"}
    plan = YvTrainingPlan.from_layers(model_yaml, stage_yaml, stage="pretrain")
    notes = apply_convergence_policy(plan, YvConfig.tiny_text_moe(), resume_ckpt="ckpt/checkpoint_step_5.pt")
    assert not plan.quantization["enable_quantization"] and not plan.lora["enabled"]
    assert plan.optimizer == "adamw" and not plan.use_galore            # the declared optimizer survives
    assert plan.scheduler == "cosine" and plan.warmup_steps == 20 and plan.min_lr_ratio == 0.1
    assert plan.gradient_checkpointing is False                          # explicit "false" is respected
    assert (plan.save_steps, plan.eval_steps, plan.log_steps) == (1000, 500, 10)
    assert any("resume" in n for n in notes) and any("nothing to adapt" in n for n in notes)


def test_adapter_runs_get_nf4_lora_and_8bit_states():
    cfg = YvConfig.tiny_text_moe()
    cfg.hidden_size, cfg.n_layer = 4096, 32
    plan = YvTrainingPlan.from_layers({"lora": {"r": 8, "target_modules": ["q_proj", "v_proj"]}}, {"save_steps": 50},
                                      stage="alignment_dpo")
    apply_convergence_policy(plan, cfg)
    assert plan.quantization == {"enable_quantization": True, "quant_method": "nf4", "bits": 4, "group_size": 128}
    assert plan.lora["enabled"] and plan.lora["r"] == 128 and plan.lora["lora_alpha"] == 256
    assert plan.lora["target_modules"] == ["q_proj", "v_proj", "k_proj"] and plan.optimizer == "adamw8bit"
    assert plan.save_steps == 50 and plan.gradient_checkpointing is True and plan.warmup_steps == 100
    # a base weight turns any stage into an adapter run; a small model gets the small rank
    plan2 = YvTrainingPlan.from_layers(None, None, stage="sft")
    apply_convergence_policy(plan2, YvConfig.tiny_text_moe(), model_name_or_path="weights/base.pt")
    assert plan2.lora["enabled"] and plan2.lora["r"] == lora_rank_for(256, 4)["r"] == 32
    assert len(plan2.lora["target_modules"]) == 7


def test_memory_policy_follows_the_byte_count():
    big = YvConfig.yv_7b_moe(vocab_size=154856, n_layer=32)
    one = YvTrainingPlan(stage="pretrain")
    notes = apply_memory_policy(one, big, tp=1, ep=1, dp=1, seq_len=4096)
    # 80 GB of weights + 80 GB of momentum on one 180 GB GPU: no room for gradients, quantised momentum
    assert one.streaming_optimizer and one.state_dtype == "int8" and one.recompute_policy == "auto"
    assert any("consumed inside backward" in n for n in notes)
    eight = YvTrainingPlan(stage="pretrain")
    apply_memory_policy(eight, big, tp=2, ep=4, dp=4, seq_len=4096)
    assert eight.state_dtype != "int8" and eight.micro_batch_size >= 2  # sharded experts leave room
    small = YvTrainingPlan(stage="pretrain", gradient_checkpointing=False)
    apply_memory_policy(small, YvConfig.tiny_text_moe(), seq_len=256)
    assert not small.streaming_optimizer and small.state_dtype is None and small.recompute_policy == "config"
