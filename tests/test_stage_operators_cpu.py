"""Configured SFT / DPO stage operators, datasets, step-level DPO and PPO operators."""
import json

import pytest
import torch
import torch.nn as nn

from pisceslx_b200.engine.stage_operators import (
    PAD_MULTIPLE, PiscesLxDPOConfig, PiscesLxDPODataset, PiscesLxDPOLoggingCallback, PiscesLxDPOOperator, PiscesLxDPOOperators,
    PiscesLxDPOTrainingConfig, PiscesLxDPOTrainingOperator, PiscesLxGRMConfig, PiscesLxPPOConfig, PiscesLxPPOStepOperator,
    PiscesLxSFTDataset, PiscesLxSFTTrainingConfig, PiscesLxSFTTrainingOperator, masked_sequence_logps, preference_loss, read_records,
    split_prompt_response)
from pisceslx_b200.models.tokenizer import YvTokenizer


class _LM(nn.Module):
    """Embedding -> causal mean mixer -> head: small, but the next token depends on the context."""

    def __init__(self, vocab=300, hidden=32):
        super().__init__()
        self.emb, self.mix, self.head = nn.Embedding(vocab, hidden), nn.Linear(hidden, hidden), nn.Linear(hidden, vocab)

    def forward(self, input_ids, attention_mask=None, labels=None):
        h = self.emb(input_ids)
        n = torch.arange(1, h.shape[1] + 1, device=h.device).view(1, -1, 1)
        h = h + torch.tanh(self.mix(h.cumsum(1) / n))
        return {"logits": self.head(h)}


def _tok():
    return YvTokenizer(use_files=False)


def test_record_layouts_and_reading(tmp_path):
    assert split_prompt_response({"instruction": "Add", "input": "1 2", "output": "3"}) == ("### Instruction:\nAdd\n\n### Input:\n1 2\n\n### Response:\n", "3")
    assert split_prompt_response({"prompt": "p", "completion": "c"}) == ("p", "c")
    assert split_prompt_response({"text": "only"}) == ("", "only")
    p, r = split_prompt_response({"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}]})
    assert "hi" in p and p.endswith("<|assistant|>\n") and r == "yo"
    p, r = split_prompt_response({"conversations": [{"from": "human", "value": "q"}, {"from": "gpt", "value": "a"}]})
    assert "q" in p and r == "a"
    (tmp_path / "a.jsonl").write_text('{"prompt": "x", "response": "y"}\n\n{"text": "z"}\n')
    (tmp_path / "b.json").write_text(json.dumps({"data": [{"text": "w"}]}))
    assert len(read_records(tmp_path / "a.jsonl")) == 2 and len(read_records(tmp_path)) == 3
    with pytest.raises(FileNotFoundError):
        read_records(tmp_path / "none.jsonl")


def test_sft_dataset_masks_prompt_and_truncates_from_the_left():
    tok = _tok()
    ds = PiscesLxSFTDataset([{"prompt": "abcdefghij", "response": "XYZ"}], tok, max_seq_length=8)
    s = ds[0]
    resp = tok.encode("XYZ", add_eos=True)
    assert s["input_ids"].tolist()[-len(resp):] == resp and len(s["input_ids"]) == 8
    n_prompt = 8 - len(resp)
    assert (s["labels"][:n_prompt] == -100).all() and s["labels"][n_prompt:].tolist() == resp
    assert s["input_ids"][:n_prompt].tolist() == tok.encode("abcdefghij")[-n_prompt:]
    b = ds.collate([s, ds[0]])
    assert b["input_ids"].shape == (2, PAD_MULTIPLE) and int(b["attention_mask"].sum()) == 16 and (b["labels"][:, 8:] == -100).all()
    assert ds._format_sample({"prompt": "a", "response": "b"}) == "ab"


def test_sft_operator_learns_and_checkpoints(tmp_path):
    torch.manual_seed(0)
    tok = _tok()
    recs = [{"prompt": f"say {w}: ", "response": w * 3} for w in ("ab", "cd", "ef", "gh")]
    cfg = PiscesLxSFTTrainingConfig(output_dir=str(tmp_path), micro_batch_size=2, gradient_accumulation_steps=2, learning_rate=5e-3, warmup_steps=2,
                                    max_steps=40, checkpoint_interval=20, eval_interval=20, log_interval=5, use_bf16=False, save_total_limit=1)
    seen = []
    res = PiscesLxSFTTrainingOperator().execute({"model": _LM(), "config": cfg, "train_records": recs, "val_records": recs[:2], "tokenizer": tok,
                                                 "callback": lambda s, l: seen.append(s)})
    assert res.is_success(), res.error
    o = res.output
    assert o["final_loss"] < 0.6 * o["first_loss"] and o["eval_loss"] is not None and seen[0] == 5 and seen[-1] == 40
    assert len(o["checkpoints"]) == 2 and o["tokens"] == 40 * 2 * 2 * PAD_MULTIPLE
    files = sorted(f.name for f in tmp_path.iterdir() if f.suffix == ".pt")
    assert "sft_step_40.pt" in files and len(files) <= 2                              # retention: the last, and the best when it differs
    lrs = [h["lr"] for h in o["history"] if "lr" in h]
    assert lrs[-1] < lrs[1] and lrs[-1] >= cfg.learning_rate * cfg.min_lr_ratio - 1e-12
    assert not PiscesLxSFTTrainingOperator().execute({"model": _LM(), "config": PiscesLxSFTTrainingConfig(train_data=str(tmp_path / "no.jsonl"))}).is_success()
    with pytest.raises(ValueError):
        PiscesLxSFTTrainingConfig(micro_batch_size=0)
    assert PiscesLxSFTTrainingConfig(use_fp16=True).use_bf16 is False


def test_masked_logps_ignore_padding():
    torch.manual_seed(0)
    m = _LM()
    ids = torch.randint(5, 200, (1, 6))
    lab = ids.clone()
    lab[:, :2] = -100
    a, _, _ = masked_sequence_logps(m, ids, lab)
    ids_p = torch.cat([ids, torch.zeros(1, 10, dtype=torch.long)], 1)
    lab_p = torch.cat([lab, torch.full((1, 10), -100)], 1)
    b, per, mask = masked_sequence_logps(m, ids_p, lab_p)
    assert torch.allclose(a, b, atol=1e-5) and int(mask.sum()) == 4 and float(b.detach()) > -100      # not minus a billion per padded token


def test_preference_loss_kinds():
    pc, pr, z = torch.tensor([-1.0, -2.0]), torch.tensor([-3.0, -1.0]), torch.zeros(2)
    l, st = preference_loss(pc, pr, z, z, beta=0.5, loss_type="sigmoid")
    assert torch.allclose(l, -torch.nn.functional.logsigmoid(torch.tensor([1.0, -0.5])).mean()) and float(st["accuracy"]) == 0.5
    l, _ = preference_loss(pc, pr, z, z, beta=0.5, loss_type="hinge")
    assert torch.allclose(l, torch.tensor([0.0, 1.5]).mean())
    l, _ = preference_loss(pc, pr, z, z, beta=0.5, loss_type="ipo")
    assert torch.allclose(l, torch.tensor([1.0, 4.0]).mean())
    l0, _ = preference_loss(pc, pr, pc, pr, beta=0.5)
    assert torch.allclose(l0, torch.log(torch.tensor(2.0)))                            # policy == reference
    with pytest.raises(ValueError):
        preference_loss(pc, pr, z, z, loss_type="nope")
    with pytest.raises(ValueError):
        PiscesLxDPOTrainingConfig(loss_type="nope")


def test_dpo_dataset_and_training_operator(tmp_path):
    torch.manual_seed(0)
    tok = _tok()
    recs = [{"prompt": f"q{i}: ", "chosen": "good good", "rejected": "bad bad"} for i in range(6)]
    ds = PiscesLxDPODataset(recs, tok, max_prompt_length=3, max_response_length=5)
    s = ds[0]
    assert len(s["chosen_input_ids"]) == 8 and (s["chosen_labels"][:3] == -100).all() and s["chosen_input_ids"][:3].tolist() == tok.encode("q0: ")[-3:]
    b = ds.collate([ds[0], ds[1]])
    assert b["input_ids"].shape == (4, PAD_MULTIPLE) and torch.equal(b["input_ids"][0, :3], b["input_ids"][2, :3])
    cfg = PiscesLxDPOTrainingConfig(output_dir=str(tmp_path), micro_batch_size=3, gradient_accumulation_steps=1, learning_rate=3e-3, warmup_steps=2,
                                    max_steps=30, beta=0.5, checkpoint_interval=0, eval_interval=30, log_interval=5, use_bf16=False)
    cb = PiscesLxDPOLoggingCallback(sink=None)
    model = _LM()
    res = PiscesLxDPOTrainingOperator().execute({"model": model, "config": cfg, "train_records": recs, "val_records": recs[:3], "tokenizer": tok, "callback": cb})
    assert res.is_success(), res.error
    o = res.output
    assert o["accuracy"] == 1.0 and o["margin"] > 0.5 and o["final_loss"] < 0.5 and o["eval_accuracy"] == 1.0
    assert len(cb.records) == 6 and cb.summary()["step"] == 30
    lines = []
    PiscesLxDPOLoggingCallback(sink=lines.append)(1, {"loss": 0.5})
    assert lines == ["[dpo] step 1 loss=0.5"]
    # reference-free runs without a frozen copy
    cfg2 = PiscesLxDPOTrainingConfig(output_dir=str(tmp_path), max_steps=2, reference_free=True, checkpoint_interval=0, use_bf16=False, gradient_accumulation_steps=1)
    assert PiscesLxDPOTrainingOperator().execute({"model": _LM(), "config": cfg2, "train_dataset": ds}).is_success()
    assert isinstance(PiscesLxDPOOperators.create_training_operator(), PiscesLxDPOTrainingOperator)
    assert PiscesLxDPOOperators.create_config(beta=0.3).beta == 0.3 and len(PiscesLxDPOOperators.create_dataset(recs, tok)) == 6
    assert PiscesLxGRMConfig().grm_use_implicit_reward


def test_step_level_dpo_operator():
    torch.manual_seed(0)
    m = _LM()
    ch, rj = torch.randint(5, 200, (2, 7)), torch.randint(5, 200, (2, 7))
    mask = torch.ones(2, 7, dtype=torch.long)
    data = [{"chosen_input_ids": ch, "rejected_input_ids": rj, "chosen_attention_mask": mask, "rejected_attention_mask": mask}, {"chosen_input_ids": ch}]
    op = PiscesLxDPOOperator()
    out0 = op.execute({"model": m, "preference_data": data, "config": PiscesLxDPOConfig(reference_free=True)}).output
    assert out0["samples"] == 1 and abs(out0["loss"] - 0.6931) < 0.2
    opt = torch.optim.SGD(m.parameters(), lr=0.5)
    for _ in range(10):
        out = op.execute({"model": m, "preference_data": data, "config": PiscesLxDPOConfig(reference_free=True, beta=0.5), "optimizer": opt}).output
    assert out["loss"] < out0["loss"] and out["accuracy"] == 1.0 and out["mean_chosen_reward"] > out["mean_rejected_reward"]
    assert not op.execute({"model": m, "preference_data": []}).is_success()
    assert not op.execute({"model": m, "preference_data": [{"chosen_input_ids": ch}]}).is_success()
    loss, rc, rr = op._compute_dpo_loss(torch.tensor([0.0]), torch.tensor([-1.0]), torch.zeros(1), torch.zeros(1), PiscesLxDPOConfig())
    assert float(rc) == 0.0 and abs(float(rr) + 0.1) < 1e-6


def test_ppo_step_operator_from_config():
    from pisceslx_b200.config import YvConfig
    from pisceslx_b200.models.model import YvModelForCausalLM
    torch.manual_seed(0)
    model = YvModelForCausalLM(YvConfig.tiny_text_moe(vocab_size=64))
    prompts = torch.randint(4, 60, (2, 4))
    cfg = PiscesLxPPOConfig(ppo_epochs=1, learning_rate=1e-4, kl_target=0.05)
    op = PiscesLxPPOStepOperator()
    assert not op.validate_inputs({"model": model, "prompts": prompts})
    res = op.execute({"model": model, "prompts": prompts, "reward_fn": lambda p, r: float((r == 7).float().mean()) if r.numel() else 0.0, "config": cfg,
                      "max_new_tokens": 4, "steps": 2})
    assert res.is_success(), res.error
    o = res.output
    assert len(o["history"]) == 2 and {"policy_loss", "value_loss", "kl", "reward_mean"} <= set(o) and o["ppo"].kl.target == 0.05
