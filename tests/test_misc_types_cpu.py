"""Small records, enumerations, errors and the operators bound to existing components."""
import pytest
import torch
import torch.nn as nn

from pisceslx_b200.config import YvConfig
from pisceslx_b200.engine.misc_types import (
    PiscesLxAgenticRLConfig, PiscesLxBuilder, PiscesLxGPUAllocation, PiscesLxHostMemoryBudgetError, PiscesLxKnowledgeBuildCli, PiscesLxKnowledgeBuilderConfig,
    PiscesLxMuonParameterError, PiscesLxPipelineSchedule, PiscesLxPreferenceAlignmentOperator, PiscesLxProfiler, PiscesLxRecoveryState, PiscesLxRunCancelled,
    PiscesLxSelfPlayConfig, PiscesLxSubconsciousTrainingConfig, PiscesLxTensorLifetime, PiscesLxTrainingOperator, PiscesLxTrainingPhase, PiscesLxVRAMOptConfig,
    YvHostTierError, check_muon_parameters)


def test_errors_and_muon_check():
    assert PiscesLxRunCancelled("user").reason == "user" and "2.00 GB" in str(PiscesLxHostMemoryBudgetError(2.0, 1.0, "build"))
    assert issubclass(PiscesLxHostMemoryBudgetError, MemoryError) and issubclass(YvHostTierError, RuntimeError)
    m = nn.Sequential(nn.Linear(4, 4), nn.LayerNorm(4))
    assert check_muon_parameters(list(m.named_parameters()), exclude=("bias", "1.")) == ["0.weight"]
    with pytest.raises(PiscesLxMuonParameterError) as e:
        check_muon_parameters([("w", torch.zeros(3))], exclude=())
    assert e.value.shape == (3,)


def test_schedule_and_phase_configs():
    S = PiscesLxPipelineSchedule
    assert S("1f1b").bubble_fraction(4, 12) == pytest.approx(3 / 15) and S.INTERLEAVED.bubble_fraction(4, 12, 2) == pytest.approx(3 / 27)
    assert S.ZERO_BUBBLE.bubble_fraction(4, 12) == pytest.approx(1 / 15) and S.GPipe.trainer_name() == "gpipe" and S.ZERO_BUBBLE.trainer_name() == "1f1b"
    c = PiscesLxSubconsciousTrainingConfig(phase="joint_rl")
    assert c.phase is PiscesLxTrainingPhase.JOINT_RL and c.learning_rate() == 3e-6

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.router, self.film_gen, self.body = nn.Linear(2, 2), nn.Linear(2, 2), nn.Linear(2, 2)
    g = c.param_groups(M())
    assert {x["name"]: x["lr"] for x in g} == {"router": 1e-5, "film": 1e-6, "rest": 3e-6}
    assert [x["name"] for x in PiscesLxSubconsciousTrainingConfig().param_groups(M())] == ["router", "film"]


def test_rl_and_self_play_configs():
    a = PiscesLxAgenticRLConfig(max_tool_calls=3)
    assert a.episode_reward(5, 10, True, needed_steps=6) == pytest.approx(3 * 0.1 + 1.0 - 0.04) and a.episode_reward(0, 2, False) == pytest.approx(-0.02)
    s = PiscesLxSelfPlayConfig(mmr_lambda=0.5)
    sim = [[1, .9, 0], [.9, 1, 0], [0, 0, 1]]
    assert s.select_diverse([1.0, 0.95, 0.5], sim, 2) == [0, 2]                         # the near-duplicate loses to the different sample
    assert PiscesLxSelfPlayConfig(use_mmr_diversity=False).select_diverse([1.0, 0.95, 0.5], sim, 2) == [0, 1]
    with pytest.raises(ValueError):
        PiscesLxSelfPlayConfig(score_method="dice")


def test_knowledge_builder_and_cli(tmp_path):
    cfg = PiscesLxKnowledgeBuilderConfig(knowledge_dim=8, chunk_size=4, chunk_overlap=1, n_list=2, pq_subvectors=2)
    assert cfg.chunks(list(range(10))) == [[0, 1, 2, 3], [3, 4, 5, 6], [6, 7, 8, 9]]
    enc = lambda texts: torch.stack([torch.tensor([float(len(t) % 7), float(sum(map(ord, t)) % 11)] * 4) for t in texts])
    b = PiscesLxBuilder(cfg, enc).build([f"text number {i} " * (i + 1) for i in range(12)])
    assert b is not None
    with pytest.raises(ValueError):
        PiscesLxBuilder(cfg)
    (tmp_path / "in").mkdir()
    (tmp_path / "in" / "a.txt").write_text("\n\n".join(f"paragraph {i} " * (i + 2) for i in range(8)))
    out = PiscesLxKnowledgeBuildCli.main(["--input", str(tmp_path / "in"), "--output", str(tmp_path / "k.pt"), "--knowledge-dim", "8", "--n-list", "2"], encode=enc)
    assert out["texts"] == 8 and (tmp_path / "k.pt").exists()


def test_lifetime_allocation_recovery_and_vram():
    t = PiscesLxTensorLifetime("act", 0, 30, 1000, [0, 10, 30])
    assert t.lifetime == 30 and t.next_use_after(10) == 30 and t.idle_gap_at(10) == 20 and t.worth_offloading(10, 100.0) and not t.worth_offloading(10, 50.0)
    assert t.idle_gap_at(30) == 1 << 30
    assert PiscesLxGPUAllocation("t1", [2, 5]).to_env() == {"CUDA_VISIBLE_DEVICES": "2,5"}
    r = PiscesLxRecoveryState(max_restarts=2)
    assert r.record_restart("nan loss", "ck1") and r.backoff_seconds() == 5.0 and r.record_restart("oom") and r.backoff_seconds() == 10.0
    assert not r.record_restart("again") and r.restart_count == 2 and r.last_checkpoint == "ck1" and len(r.recovery_history) == 2
    big = PiscesLxVRAMOptConfig.for_device(180.0, 14.0)
    assert big.zero_stage == 1 and not big.cpu_offload_optimizer and big.recommended_seq_len == 8192
    mid, tight = PiscesLxVRAMOptConfig.for_device(180.0, 40.0), PiscesLxVRAMOptConfig.for_device(180.0, 140.0)
    assert mid.zero_stage == 3 and not mid.cpu_offload_optimizer and tight.cpu_offload_optimizer and tight.activation_quantization
    cfg = YvConfig.tiny_text_moe(vocab_size=32)
    assert PiscesLxVRAMOptConfig(use_gradient_checkpointing=False).apply(cfg).use_gradient_checkpointing is False


def test_alignment_front_profiler_and_training_operator(tmp_path):
    from pisceslx_b200.models.model import YvModelForCausalLM
    torch.manual_seed(0)
    model = YvModelForCausalLM(YvConfig.tiny_text_moe(vocab_size=64))
    ch, rj = torch.randint(4, 60, (2, 6)), torch.randint(4, 60, (2, 6))
    mask = torch.ones(2, 6, dtype=torch.long)
    op = PiscesLxPreferenceAlignmentOperator()
    res = op.execute({"method": "DPO", "model": model, "preference_data": [{"chosen_input_ids": ch, "rejected_input_ids": rj, "chosen_attention_mask": mask,
                                                                             "rejected_attention_mask": mask}]})
    assert res.is_success() and res.output["method"] == "dpo" and res.output["samples"] == 1
    assert not op.execute({"method": "rlhf", "model": model}).is_success()
    assert isinstance(PiscesLxProfiler(), PiscesLxProfiler)
    top = PiscesLxTrainingOperator({"max_steps": 3, "output_dir": str(tmp_path), "save_steps": 0, "data": {"batch_size": 2}, "gradient_accumulation_steps": 1,
                                    "optimizer": {"name": "adamw", "learning_rate": 1e-3}, "scheduler": {"warmup_steps": 1}})
    batches = [{"input_ids": torch.randint(4, 60, (2, 16))} for _ in range(5)]
    out = top.execute({"model": model, "batches": batches}).output
    assert out["steps"] == 3 and out["trainer"].global_step == 3 and out["final_loss"] > 0
    bad = PiscesLxTrainingOperator({"max_steps": 0})
    assert not bad.execute({"model": model, "batches": batches}).is_success()
