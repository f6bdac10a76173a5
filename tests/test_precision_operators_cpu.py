"""FP8 / FP4 / sharded training operators on the host."""
import pytest
import torch
import torch.nn as nn

from pisceslx_b200.config import YvConfig
from pisceslx_b200.engine.precision_operators import (PiscesLxFP4Config, PiscesLxFP4Operator, PiscesLxFP4Trainer, PiscesLxFP8Operator, PiscesLxFP8TextDataset,
                                                      PiscesLxFP8TrainingConfig, PiscesLxFP8TrainingOperator, PiscesLxFSDPTrainingConfig, PiscesLxFSDPTrainingOperator)
from pisceslx_b200.models.tokenizer import YvTokenizer
from pisceslx_b200.quant.fp4 import PiscesLxFP4Linear
from pisceslx_b200.quant.fp8 import YvFP8Linear


class _LM(nn.Module):
    def __init__(self, vocab=300, hidden=128):
        super().__init__()
        self.embed = nn.Embedding(vocab, hidden)
        self.up, self.down = nn.Linear(hidden, 256, bias=False), nn.Linear(256, hidden, bias=False)
        self.tiny = nn.Linear(hidden, 4, bias=False)
        self.lm_head = nn.Linear(hidden, vocab, bias=False)

    def forward(self, input_ids, attention_mask=None, labels=None):
        h = self.embed(input_ids)
        n = torch.arange(1, h.shape[1] + 1).view(1, -1, 1)
        h = h + self.down(torch.relu(self.up(h.cumsum(1) / n))) + 0.0 * self.tiny(h).sum(-1, keepdim=True)
        return {"logits": self.lm_head(h)}


RECS = [{"prompt": f"say {w}: ", "response": w * 3} for w in ("ab", "cd", "ef", "gh")]


def _tok():
    return YvTokenizer(use_files=False)


def test_fp8_operator_converts_and_trains(tmp_path):
    torch.manual_seed(0)
    m = _LM()
    cfg = PiscesLxFP8TrainingConfig(micro_batch_size=2, gradient_accumulation_steps=1, learning_rate=5e-3, max_steps=30, warmup_steps=2, log_interval=5,
                                    checkpoint_interval=15, checkpoint_dir=str(tmp_path), max_grad_norm="1.0", weight_decay=0.0)
    assert cfg.max_grad_norm == 1.0
    op = PiscesLxFP8Operator()
    res = op.execute({"model": m, "config": cfg, "train_records": RECS, "tokenizer": _tok()})
    assert res.is_success(), res.error
    o = res.output
    assert sorted(o["converted_layers"]) == ["down", "up"] and isinstance(m.up, YvFP8Linear) and type(m.tiny) is nn.Linear and type(m.lm_head) is nn.Linear
    assert o["recipe"]["scaling"] == "block" and o["recipe"]["backward"] == "e5m2" and o["hardware"]["cuda"] is False
    assert o["final_loss"] < 0.8 * o["first_loss"] and len(o["checkpoints"]) == 2
    m2 = _LM()
    op.convert(m2, cfg)
    assert op._load_checkpoint(o["checkpoints"][-1], m2, None) == 30 and torch.equal(m2.up.weight, m.up.weight)
    r2 = op.execute({"model": m2, "convert": False, "train_records": RECS, "tokenizer": _tok(),
                     "config": PiscesLxFP8TrainingConfig(micro_batch_size=2, gradient_accumulation_steps=1, max_steps=32, resume_from=o["checkpoints"][-1],
                                                         checkpoint_interval=0, log_interval=1)})
    assert r2.output["steps"] == 2
    with pytest.raises(ValueError):
        PiscesLxFP8TrainingConfig(scaling="fp3")
    assert not PiscesLxFP8TrainingOperator().execute({"model": _LM(), "config": PiscesLxFP8TrainingConfig(train_data=str(tmp_path / "no.jsonl"))}).is_success()


def test_fp8_text_dataset_reads_plain_text(tmp_path):
    (tmp_path / "d.txt").write_text("first paragraph\n\nsecond paragraph\n\n")
    ds = PiscesLxFP8TextDataset(str(tmp_path / "d.txt"), _tok(), 16)
    assert len(ds) == 2 and (ds[0]["labels"] != -100).all()


def test_stochastic_rounding_to_e5m2_is_on_grid_and_unbiased():
    g = torch.Generator().manual_seed(0)
    x = torch.rand(2000, generator=g) * 2 - 1
    r = PiscesLxFP4Operator._stochastic_round_to_fp8(x, g)
    s = 57344.0 / x.abs().max()
    y = r.float() * s
    assert torch.equal(y.to(torch.float8_e5m2).float(), y)                               # every value is representable
    reps = torch.stack([PiscesLxFP4Operator._stochastic_round_to_fp8(x, g) for _ in range(200)]).mean(0)
    assert (reps - x).abs().mean() < 0.01 and abs(float((reps - x).mean())) < 1e-3
    nearest = (x * s).to(torch.float8_e5m2).float() / s
    assert (nearest - x).abs().mean() > (reps - x).abs().mean()                          # averaging beats round-to-nearest


@pytest.mark.parametrize("storage", ["master", "packed"])
def test_fp4_operator_both_storages(storage, tmp_path):
    torch.manual_seed(0)
    m = _LM()
    cfg = PiscesLxFP4Config(micro_batch_size=2, gradient_accumulation_steps=1, learning_rate=5e-3 if storage == "master" else 0.05, max_steps=40, warmup_steps=2,
                            log_interval=5, checkpoint_interval=0, storage=storage, weight_decay=0.0)
    tr = PiscesLxFP4Trainer(m, cfg)
    out = tr.train(RECS, _tok(), save_dir=str(tmp_path))
    assert out["storage"] == storage and out["final_loss"] < out["first_loss"] and (tmp_path / "fp4_model.pt").exists()
    if storage == "master":
        assert isinstance(m.up, PiscesLxFP4Linear) and sorted(out["converted_layers"]) == ["down", "tiny", "up"]
    else:
        assert out["compression_ratio"] > 1.3                                           # the embedding and the head stay in fp32
    tr.load_checkpoint(str(tmp_path / "fp4_model.pt"))
    with pytest.raises(ValueError):
        PiscesLxFP4Config(block_size=7)
    with pytest.raises(ValueError):
        PiscesLxFP4Config(storage="disk")


def test_fsdp_config_and_single_process_run():
    c = PiscesLxFSDPTrainingConfig(sharding_strategy="ZERO3", backward_prefetch="BACKWARD_POST")
    assert c.get_sharding_strategy() == "full_shard" and c.get_backward_prefetch() == 0
    assert PiscesLxFSDPTrainingConfig(sharding_strategy="shard_grad_op").get_sharding_strategy() == "zero1" and PiscesLxFSDPTrainingConfig().get_backward_prefetch() == 1
    with pytest.raises(ValueError):
        PiscesLxFSDPTrainingConfig(sharding_strategy="ZERO9").get_sharding_strategy()
    with pytest.raises(ValueError):
        PiscesLxFSDPTrainingConfig(backward_prefetch="SOMETIMES").get_backward_prefetch()
    t = c.to_trainer_config()
    assert t.sharding == "full_shard" and t.recompute_policy == "auto" and t.state_dtype == "fp32"
    from pisceslx_b200.models.model import YvModelForCausalLM
    torch.manual_seed(0)
    model = YvModelForCausalLM(YvConfig.tiny_text_moe(vocab_size=300))
    cfg = PiscesLxFSDPTrainingConfig(micro_batch_size=2, gradient_accumulation_steps=1, learning_rate=3e-3, warmup_steps=1, max_steps=6, max_seq_length=32, world_size=1)
    res = PiscesLxFSDPTrainingOperator().execute({"model": model, "config": cfg, "train_records": RECS, "tokenizer": _tok()})
    assert res.is_success(), res.error
    o = res.output
    assert o["steps"] == 6 and o["final_loss"] < o["first_loss"] and o["distributed"]["world_size"] == 1
    info = o["sharding_info"]
    assert info["sharding"] == "full_shard" and info["parameters_per_rank"] == info["total_parameters"] and info["backward_prefetch_units"] == 1
    eight = PiscesLxFSDPTrainingOperator._collect_sharding_info(model, cfg, 8)
    assert eight["parameters_per_rank"] == info["total_parameters"] // 8
