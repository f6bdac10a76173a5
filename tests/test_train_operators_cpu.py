"""CPU tests of the training operators: distillation, RLVR / DAPO, on-policy distillation, memory separation,
evolution pipeline, advanced-training coordinator."""
from __future__ import annotations

import torch
import torch.nn as nn

from pisceslx_b200 import YvConfig
from pisceslx_b200.engine import operators as O
from pisceslx_b200.models import build_model


class TinyLM(nn.Module):
    def __init__(self, vocab=32, dim=16, seed=0):
        super().__init__()
        torch.manual_seed(seed)
        self.emb, self.out = nn.Embedding(vocab, dim), nn.Linear(dim, vocab)

    def forward(self, input_ids):
        return {"logits": self.out(self.emb(input_ids))}


def test_distillation_operator_pulls_student_to_teacher():
    teacher, student = TinyLM(seed=1), TinyLM(seed=2)
    g = torch.Generator().manual_seed(0)
    batches = [torch.randint(0, 32, (4, 12), generator=g) for _ in range(40)]
    op = O.PiscesLxDistillationOperator(O.PiscesLxDistillationConfig(alpha=1.0, lr=0.02, max_steps=40))
    r = op.execute({"student": student, "teacher": teacher, "batches": batches})
    h = r.output["history"]
    assert r.is_success() and len(h) == 40 and h[-1]["soft"] < 0.5 * h[0]["soft"]
    assert not op.execute({"student": student}).is_success()
    ds = O.PiscesLxDistillationDataset(batches[:3])
    assert len(ds) == 3 and torch.equal(ds[1]["labels"], batches[1])


def _bandit():
    """A policy over 4 answers per prompt id; the right answer for every prompt is "3"."""
    pol = nn.Embedding(2, 4)
    nn.init.zeros_(pol.weight)

    def sample(p, prompt):
        a = torch.multinomial(torch.softmax(p(prompt)[0], -1), 1)
        return a, str(int(a))

    def logprob(p, prompt, resp):
        return torch.log_softmax(p(prompt)[0], -1)[resp].sum()
    return pol, sample, logprob


def test_rlvr_trainer_operator_and_dapo():
    torch.manual_seed(0)
    pol, sample, logprob = _bandit()
    tr = O.PiscesLxRLVRTrainer(pol, torch.optim.SGD(pol.parameters(), lr=1.0), sample, logprob,
                               O.PiscesLxRLVRConfig(group_size=8))
    ds = O.PiscesLxRLVRDataset([{"prompt": torch.tensor([0]), "answer": "3"}, {"prompt": torch.tensor([1]), "answer": "3"}])
    res = O.PiscesLxRLVROperator().execute({"trainer": tr, "dataset": ds, "steps": 30, "rows_per_step": 2})
    hist = res.output["history"]
    assert res.is_success() and sum(h["mean_reward"] for h in hist[-5:]) / 5 > sum(h["mean_reward"] for h in hist[:5]) / 5
    assert torch.softmax(pol.weight, -1)[:, 3].min() > 0.5
    torch.manual_seed(1)
    pol2, sample2, logprob2 = _bandit()
    dapo = O.PiscesLxDAPO(pol2, torch.optim.SGD(pol2.parameters(), lr=1.0), sample2, logprob2, group_size=8)
    assert dapo.cfg.dynamic_sampling and dapo.cfg.clip_eps_high == 0.28
    rows = [{"prompt": torch.tensor([0]), "answer": "3"}]
    for _ in range(30):
        out = dapo.step(rows)
    assert torch.softmax(pol2.weight, -1)[0, 3] > 0.5
    # a group with identical rewards carries no gradient and is dropped
    none = dapo.step([{"prompt": torch.tensor([1]), "answer": "never"}])
    assert none["kept_groups"] == 0 and none["loss"] == 0.0
    num = O.PiscesLxRLVRTrainer(pol, None, sample, logprob, O.PiscesLxRLVRConfig(verifier=O.PiscesLxRLVRVerifierType.NUMERIC))
    assert num.verifier.reward("3.0", "3") == 1.0


def test_on_policy_distillation():
    torch.manual_seed(0)
    teacher, student = TinyLM(seed=1), TinyLM(seed=2)

    def gen(model, prompt, n):
        ids = prompt
        for _ in range(n):
            nxt = model(input_ids=ids)["logits"][:, -1].argmax(-1, keepdim=True)
            ids = torch.cat([ids, nxt], 1)
        return ids
    tr = O.PiscesLxOPDTrainer(student, teacher, torch.optim.Adam(student.parameters(), lr=0.02), gen, O.PiscesLxOPDConfig(max_new_tokens=6))
    prompts = [torch.randint(0, 32, (1, 4)) for _ in range(4)]
    first = tr.step(prompts)["kl"]
    for _ in range(40):
        last = tr.step(prompts)["kl"]
    assert last < 0.5 * first and O.PiscesLxOpd is O.PiscesLxOPDTrainer


def test_memsep_phases_gate_and_alignment_loss():
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.backbone = nn.Linear(4, 4)
            self.memory_router = nn.Linear(4, 4)
            self.memory_gate = 0.0
    net = Net()
    tr = O.PiscesLxMemsep.create_memsep_trainer(net, ramp_steps=10, gate_max=0.8)
    st = tr.get_stats()
    assert st["phase"] == "core_reasoning" and st["gate"] == 0.0 and st["trainable_memory"] == 0 and st["trainable_backbone"] == 20
    assert float(tr.compute_memory_loss({"distances": torch.ones(2, 3)})) == 0.0
    tr.start_phase(O.PiscesLxMemSepPhase.MEMORY_ROUTER_TRAINING)
    gates = [tr.pre_step() for _ in range(12)]
    assert gates[0] == 0.0 and abs(gates[-1] - 0.8) < 1e-6 and all(b >= a for a, b in zip(gates, gates[1:]))
    assert abs(net.memory_gate - 0.8) < 1e-6
    st = tr.get_stats()
    assert st["trainable_backbone"] == 0 and st["trainable_memory"] == 20
    groups = tr.params.get_optimizer_param_groups(1e-3)
    assert [g["name"] for g in groups] == ["memory"]
    loss = tr.compute_memory_loss({"distances": torch.tensor([[0.2, 0.9]]), "knowledge": torch.randn(1, 5, 2, 8)})
    assert float(loss) > 0.4 * 0.5 - 1e-6                   # hinge: mean(relu([0.2, 0.9] - 0.5)) = 0.2, plus the variance term
    tr.start_phase(O.PiscesLxMemSepPhase.KNOWLEDGE_STORE_BUILD)
    assert tr.get_stats()["gate"] == 0.8 and tr.get_stats()["trainable_memory"] == 0


def test_evolution_pipeline_distils_then_grows_the_model():
    torch.manual_seed(0)
    cfg = YvConfig.tiny_text_moe(vocab_size=128)
    cfg.n_layer = 1
    model = build_model(cfg)
    teacher = build_model(cfg, seed=5)
    g = torch.Generator().manual_seed(0)
    data = [torch.randint(0, 128, (2, 10), generator=g) for _ in range(4)]
    F0 = model.model.layers[0].mlp.ffn
    n0 = sum(p.numel() for p in model.parameters())
    opt_holder = {}

    def train_step(m, ids):
        if "opt" not in opt_holder or opt_holder["n"] != sum(p.numel() for p in m.parameters()):
            opt_holder["opt"], opt_holder["n"] = torch.optim.SGD(m.parameters(), lr=1e-3), sum(p.numel() for p in m.parameters())
        loss = m(input_ids=ids, labels=ids)["loss"]
        opt_holder["opt"].zero_grad(); loss.backward(); opt_holder["opt"].step()
        return loss.detach()
    pipe = O.PiscesLxEvolutionPipeline(O.PiscesLxEvolutionConfig(
        growth=(O.PiscesLxGrowthStage("expert_width", F0 + 8, train_steps=2), O.PiscesLxGrowthStage("depth", [0], train_steps=1)),
        distill=O.PiscesLxDistillationConfig(max_steps=3, lr=1e-3)))
    res = pipe.execute({"model": model, "teacher": teacher, "batches": lambda: iter(data), "train_step": train_step})
    assert res.is_success(), res.error
    s = res.output
    assert s["stages"] == ["distillation", "growth", "done"] and s["n_logged"]["distill_loss"] == 3
    assert s["n_logged"]["growth_loss"] == 3 and s["last"]["params"] > n0 and len(model.model.layers) == 2
    assert model.model.layers[0].mlp.ffn == F0 + 8 and pipe.get_progress()["stages"][-1] == "done"
    assert torch.isfinite(model(input_ids=data[0]).logits).all()


def test_advanced_training_coordinator():
    torch.manual_seed(0)
    m = TinyLM()
    cfg = O.PiscesLxAdvancedTrainingConfig(mixed_precision="fp32", grad_clip=0.5, lr=0.1, warmup_steps=2, total_steps=10,
                                           label_smoothing=0.1, schedule="cosine")
    co = O.PiscesLxAdvancedTrainingCoordinator(m, torch.optim.SGD(m.parameters(), lr=0.0), cfg)
    ids = torch.randint(0, 32, (4, 9))
    mbs = [{"input_ids": ids[:2], "labels": ids[:2]}, {"input_ids": ids[2:], "labels": ids[2:]}]
    outs = [co.train_step(mbs) for _ in range(10)]
    assert abs(outs[0]["lr"] - 0.05) < 1e-9 and abs(outs[1]["lr"] - 0.1) < 1e-9 and outs[-1]["lr"] < 0.01
    assert outs[-1]["loss"] < outs[0]["loss"] and outs[0]["non_finite_tensors"] == 0
    assert all(o["clipped"] == (o["grad_norm"] > 0.5) for o in outs)
    sched = O.PiscesLxLearningRateSchedulerOperator(O.PiscesLxAdvancedTrainingConfig(lr=1.0, schedule="linear", total_steps=4))
    assert [round(sched.lr_at(s), 2) for s in range(5)] == [1.0, 0.75, 0.5, 0.25, 0.0]
    net = nn.Sequential(nn.Linear(2, 2), nn.Dropout(0.5))
    reg = O.PiscesLxRegularizationOperator(O.PiscesLxAdvancedTrainingConfig(dropout=0.1))
    assert reg.run({"model": net}) == {"dropout_modules": 1} and net[1].p == 0.1
    amp = O.PiscesLxMixedPrecisionTrainingOperator(O.PiscesLxAdvancedTrainingConfig(mixed_precision="bf16"))
    y = amp.run({"fn": lambda: torch.randn(4, 4) @ torch.randn(4, 4), "device_type": "cpu"})
    assert y.dtype == torch.bfloat16
