"""Training configuration tree, pipeline operator (callbacks, checkpoints, interruption), curriculum and multi-task operators."""
import os

import pytest
import torch
import torch.nn as nn

from pisceslx_b200.engine.train_config import (PiscesLxDataConfig, PiscesLxLoRAConfig, PiscesLxOptimizerConfig, PiscesLxSchedulerConfig,
                                               PiscesLxTrainingConfig, PiscesLxTrainingEvolutionConfig, PiscesLxTrainingQuantizationConfig,
                                               PiscesLxTrainingStage)
from pisceslx_b200.engine.train_pipeline import (PiscesLxCurriculumLearningOperator, PiscesLxMultiTaskTrainingOperator, PiscesLxTrainingInterruption,
                                                 PiscesLxTrainingPipelineOperator, _InterruptState)


def test_stage_enum_and_sections():
    assert PiscesLxTrainingStage("rl_grpo").loss_type == "grpo" and PiscesLxTrainingStage.SFT.loss_type == "lm"
    assert PiscesLxTrainingStage.ALIGNMENT_DPO.needs_reference_model and not PiscesLxTrainingStage.PRETRAIN.needs_reference_model
    o = PiscesLxOptimizerConfig(betas=[0.9, 0.95], use_fused_adamw=True, use_galore=True, galore_rank=64)
    assert o.betas == (0.9, 0.95) and o.resolved_name() == "fused_adamw"
    g = o.galore_config()
    assert g.rank == 64 and g.mode == "lowrank" and g.beta2 == 0.95 and g.update_proj_gap == 200
    assert PiscesLxSchedulerConfig(warmup_steps=0, warmup_ratio=0.1).resolved_warmup(500) == 50
    assert PiscesLxSchedulerConfig(warmup_steps=1000).resolved_warmup(300) == 300
    assert PiscesLxDataConfig(datasets=[{"name": "a", "weight": 3}, {"name": "b", "weight": 1}]).normalized_weights() == {"a": 0.75, "b": 0.25}
    q = PiscesLxTrainingQuantizationConfig(quant_method="int8")
    assert q.bits == 8 and q.to_pipeline_config().bits == 8
    with pytest.raises(ValueError):
        PiscesLxTrainingQuantizationConfig(quant_method="int3")
    ev = PiscesLxTrainingEvolutionConfig()
    cfg, hidden = ev.to_pipeline_config(current_layers=6)
    assert [s.kind for s in cfg.growth] == ["depth", "experts", "depth"] and cfg.growth[0].value == [2, 3, 4, 5] and len(cfg.growth[2].value) == 8
    assert hidden == [{"hidden_size": 2048, "train_steps": 500}] and ev.total_steps() == 7500


def test_lora_config_wraps_matching_linears():
    class Blk(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj, self.v_proj, self.up = nn.Linear(8, 8), nn.Linear(8, 8, bias=False), nn.Linear(8, 16)
    m = nn.Sequential(Blk(), Blk())
    x = torch.randn(2, 8)
    before = m[0].q_proj(x)
    c = PiscesLxLoRAConfig(enabled=True, r=4, lora_alpha=8, target_modules=["q_proj", "v_proj"], lora_dropout=0.0)
    assert c.scaling == 2.0 and c.apply(m) == 4
    assert torch.allclose(m[0].q_proj(x), before, atol=1e-6)                            # B starts at zero; the bias is kept
    train = [n for n, p in m.named_parameters() if p.requires_grad]
    assert len(train) == 8 and all("lora_" in n for n in train)
    assert PiscesLxLoRAConfig().apply(m) == 0
    with pytest.raises(ValueError):
        PiscesLxLoRAConfig(r=0)
    with pytest.raises(ValueError):
        PiscesLxLoRAConfig(bias="some")


def test_training_config_round_trip_stage_file_and_overrides(tmp_path, monkeypatch):
    c = PiscesLxTrainingConfig.from_dict({"max_steps": 50, "optimizer": {"learning_rate": 3e-4, "name": "muon", "nonsense": 1}, "stage": "sft",
                                          "data": {"batch_size": 2}, "unknown": 5})
    assert c.optimizer.learning_rate == 3e-4 and c.stage is PiscesLxTrainingStage.SFT and c.data.batch_size == 2
    d = c.to_dict()
    assert d["stage"] == "sft" and PiscesLxTrainingConfig.from_dict(d).to_dict() == d
    f = tmp_path / "st.yaml"
    f.write_text("training:\n  max_steps: 77\n  packing: true\noptimizer:\n  lr: 0.001\n  weight_decay: 0.2\nscheduler:\n  type: linear\n  warmup_steps: 5\n"
                 "data:\n  sequence_length: 128\nbeta: 0.3\nmoe:\n  routing_temperature: 1.1\nlora:\n  enabled: true\n  r: 16\n")
    declared = c.load_stage_config("alignment_dpo", str(f))
    assert c.stage is PiscesLxTrainingStage.ALIGNMENT_DPO and c.loss_type == "dpo" and c.max_steps == 77 and c.packing
    assert c.optimizer.learning_rate == 0.001 and c.optimizer.weight_decay == 0.2 and c.scheduler.name == "linear" and c.scheduler.warmup_steps == 5
    assert c.data.sequence_length == 128 and c.beta == 0.3 and c.moe["routing_temperature"] == 1.1 and c.moe["temperature_max"] == 3.0 and c.lora.r == 16
    assert "optimizer.learning_rate" in declared and "max_steps" in c.stage_declared_keys
    assert c.load_stage_config("rl_memsep", str(tmp_path / "missing.yaml")) == [] and c.stage is PiscesLxTrainingStage.RL_MEMSEP
    c.apply_overrides({"optimizer.learning_rate": 5e-5, "max_steps": 9, "fsdp.cpu_offload": True})
    assert c.optimizer.learning_rate == 5e-5 and c.max_steps == 9 and c.fsdp["cpu_offload"] is True
    with pytest.raises(KeyError):
        c.apply_overrides({"optimizer.nope": 1})
    monkeypatch.setenv("PISCESLX_HOME", str(tmp_path))
    assert c.resolved_output_dir() == str(tmp_path / ".pisceslx/ckpt")
    c.output_dir = "/abs/x"
    assert c.resolved_output_dir() == "/abs/x"
    with pytest.raises(ValueError):
        PiscesLxTrainingConfig(mixed_precision="int3")


def test_validate_and_trainer_mapping(tmp_path):
    c = PiscesLxTrainingConfig(max_steps=100, output_dir=str(tmp_path), gradient_accumulation_steps=4, data={"batch_size": 2},
                               optimizer={"name": "adamw", "learning_rate": 1e-3, "max_grad_norm": 0.5}, scheduler={"warmup_steps": 0, "warmup_ratio": 0.2, "min_lr_ratio": 0.1})
    assert c.validate() == [] and c.effective_batch_size() == 8
    t = c.to_trainer_config()
    assert (t.micro_batch_size, t.optimizer, t.lr, t.warmup_steps, t.clip_grad_norm, t.min_lr_ratio, t.sharding) == (2, "adamw", 1e-3, 20, 0.5, 0.1, "zero1")
    assert t.optimizer_kwargs["betas"] == (0.9, 0.999) and t.output_dir == str(tmp_path)
    c.distributed, c.world_size = True, 8
    c.parallel_3d.update(dp_size=2, tp_size=2, pp_size=1)
    c.enable_distillation = True
    problems = c.validate()
    assert any("world_size" in p for p in problems) and any("distill_teacher_path" in p for p in problems)
    assert c.to_trainer_config().sharding == "full_shard" and c.effective_batch_size() == 16
    bad = PiscesLxTrainingConfig(max_steps=0, gradient_accumulation_steps=0)
    assert len(bad.validate()) == 2


class _Trainer:
    def __init__(self):
        self.model = nn.Linear(2, 2)
        self.global_step, self.best_metric, self.saved, self.loaded = 0, float("inf"), [], None

    def train_step(self, batch):
        self.global_step += 1
        return {"loss": 1.0 / self.global_step, "grad_norm": 0.5, "throughput": 10.0}

    def save_checkpoint(self, path, metadata=None):
        self.saved.append((os.path.basename(path), metadata))

    def load_checkpoint(self, path):
        self.loaded = path


def test_pipeline_epochs_callbacks_checkpoints_and_step_budget(tmp_path):
    cfg = PiscesLxTrainingConfig(max_steps=7, save_steps=3, eval_steps=2, output_dir=str(tmp_path))
    tr = _Trainer()
    op = PiscesLxTrainingPipelineOperator(cfg, tr, install_signal_handler=False)
    events = []
    cb = lambda stage, **kw: events.append(stage)
    op.add_callback(cb)
    op.add_callback(cb)
    op.add_callback(lambda stage, **kw: 1 / 0 if stage == "epoch_end" else None)
    hist = op.execute({"train_dataloader": [{}] * 5, "epochs": 3, "resume_from": "ck.pt"}).output
    assert tr.global_step == 7 and tr.loaded == "ck.pt" and [e["batch_count"] for e in hist["epochs"]] == [5, 2]
    assert [s[0] for s in tr.saved] == ["checkpoint_step_3.pt", "checkpoint_step_6.pt", "final_model.pt"] and tr.saved[-1][1] == {"is_final": True}
    assert events[0] == "training_start" and events[-1] == "training_end" and events.count("evaluation_start") == 3 and events.count("batch_end") == 7
    assert len(op.callback_errors) == 2 and "ZeroDivisionError" in op.callback_errors[0]
    assert abs(hist["epochs"][0]["avg_loss"] - sum(1 / i for i in range(1, 6)) / 5) < 1e-9
    op.remove_callback(cb)
    assert len(op.callbacks) == 1
    assert isinstance(PiscesLxTrainingPipelineOperator({"max_steps": 3}).train_config, PiscesLxTrainingConfig)
    with pytest.raises(TypeError):
        PiscesLxTrainingPipelineOperator(3.5)


def test_pipeline_evaluate_best_and_early_stopping(tmp_path):
    class LM(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb, self.head = nn.Embedding(16, 8), nn.Linear(8, 16)

        def forward(self, input_ids, labels=None, return_logits=False):
            lg = self.head(self.emb(input_ids))
            loss = nn.functional.cross_entropy(lg[:, :-1].reshape(-1, 16), labels[:, 1:].reshape(-1), ignore_index=-100)
            return {"loss": loss, "logits": lg}

    tr = _Trainer()
    tr.model = LM()
    cfg = PiscesLxTrainingConfig(max_steps=100, save_steps=0, eval_steps=0, output_dir=str(tmp_path), early_stopping_patience=2)
    op = PiscesLxTrainingPipelineOperator(cfg, tr, install_signal_handler=False)
    val = [{"input_ids": torch.randint(0, 16, (2, 6))} for _ in range(3)]
    ev = op.evaluate(val, metrics=["accuracy"])
    assert ev["eval_batches"] == 3 and 0.0 <= ev["eval_accuracy"] <= 1.0 and abs(ev["eval_perplexity"] - torch.exp(torch.tensor(ev["eval_loss"])).item()) < 1e-3
    hist = op.fit([{}] * 2, val, epochs=10)
    # the model never changes: the first evaluation is the best, two more without a gain stop the run
    assert hist.get("early_stopped") and len(hist["evaluations"]) == 3 and hist["best_checkpoint"].endswith("best_model.pt")
    assert [s[0] for s in tr.saved] == ["best_model.pt", "final_model.pt"]


def test_interruption_is_taken_between_steps(tmp_path):
    t = [0.0]
    st = _InterruptState(1.0, clock=lambda: t[0])
    assert st.pending() is None
    st.press()
    assert st.pending() is None                                                         # a second press may still come
    t[0] = 1.5
    assert st.pending() == "full_stop"
    st.press()
    t[0] = 1.9
    st.press()
    assert st.pending() == "skip_dataset"
    cfg = PiscesLxTrainingConfig(max_steps=100, save_steps=0, eval_steps=0, output_dir=str(tmp_path))
    tr = _Trainer()
    op = PiscesLxTrainingPipelineOperator(cfg, tr, install_signal_handler=False)
    op.interrupts = _InterruptState(0.0)

    def cb(stage, **kw):
        if stage == "batch_end" and kw["batch_idx"] == 2:
            op.interrupts.press()
    op.add_callback(cb)
    with pytest.raises(PiscesLxTrainingInterruption) as e:
        op.fit([{}] * 10)
    assert e.value.mode == "full_stop" and tr.global_step == 3 and tr.saved[-1][0] == "final_model.pt" and op.last_history["interrupted"]
    # two quick presses skip the dataset and the next one runs
    tr2 = _Trainer()
    op2 = PiscesLxTrainingPipelineOperator(cfg, tr2, install_signal_handler=False)
    op2.interrupts = _InterruptState(5.0)
    fired = []

    def cb2(stage, **kw):
        if stage == "batch_end" and not fired:
            fired.append(1)
            op2.interrupts.press()
            op2.interrupts.press()
    op2.add_callback(cb2)
    out = op2.fit_datasets({"a": [{}] * 4, "b": [{}] * 4})
    assert out["skipped"] == ["a"] and tr2.global_step == 5 and "stopped_at" not in out
    assert PiscesLxTrainingInterruption.stop_all("x").mode == "full_stop" and str(PiscesLxTrainingInterruption.skip_current_dataset()) == "Training interrupted: skip_dataset"


def test_curriculum_advances_on_plateau_not_on_progress():
    sched = [{"name": "easy", "dataloader_args": {"max_len": 64}, "min_steps": 2}, {"name": "mid", "dataloader_args": {"max_len": 256}, "target_loss": 0.5},
             {"name": "hard", "dataloader_args": {"max_len": 1024}}]
    op = PiscesLxCurriculumLearningOperator(difficulty_schedule=sched)
    assert op.get_current_dataloader(lambda **kw: kw) == {"max_len": 64}
    for loss in (3.0, 2.5, 2.0, 1.6):
        assert not op.should_advance_stage({"loss": loss})                              # still falling fast: stay
    for loss in (1.59, 1.585):
        r = op.should_advance_stage({"loss": loss})
    assert not r
    assert op.should_advance_stage({"loss": 1.584})                                     # three reports with < 2 % gain
    assert op.advance_stage() and op.current_stage == 1 and op.history[0]["name"] == "easy" and op.history[0]["steps"] == 7
    assert op.execute({"metrics": {"loss": 0.4}}).output["advanced"] and op.current_stage == 2 and op.is_last_stage
    assert not op.should_advance_stage({"loss": 0.0}) and not op.advance_stage()
    sd = op.state_dict()
    op2 = PiscesLxCurriculumLearningOperator(config={"difficulty_schedule": sched})
    op2.load_state_dict(sd)
    assert op2.current_stage == 2 and len(op2.history) == 2
    m = PiscesLxCurriculumLearningOperator(difficulty_schedule=[{"max_steps": 3}, {}])
    assert not m.should_advance_stage({"loss": 1.0, "steps": 2}) and m.should_advance_stage({"loss": 0.9, "steps": 2})


def test_multitask_weighted_loss():
    op = PiscesLxMultiTaskTrainingOperator(task_weights={"lm": 1.0, "cls": 0.5})
    a, b = torch.tensor(2.0, requires_grad=True), torch.tensor(4.0, requires_grad=True)
    loss = op.compute_multi_task_loss({"lm": {"loss": a}, "cls": {"loss": b}, "aux": {"logits": 1}})
    loss.backward()
    assert float(loss.detach()) == 4.0 and float(a.grad) == 1.0 and float(b.grad) == 0.5 and op.get_task_metrics() == {"lm": 2.0, "cls": 2.0}
    n = PiscesLxMultiTaskTrainingOperator(config={"task_weights": {"x": 3.0}}, normalize=True)
    assert float(n.execute({"task_outputs": {"x": torch.tensor(2.0), "y": {"loss": torch.tensor(6.0)}}}).output["loss"]) == 3.0
    with pytest.raises(ValueError):
        op.compute_multi_task_loss({"aux": {}})
