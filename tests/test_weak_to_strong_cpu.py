"""Weak-to-strong operator: labels and curriculum, the three losses, self-correction, a student that ends up better than
its supervisor, iterative amplification."""
import pytest
import torch
from torch import nn

from pisceslx_b200.engine import weak_to_strong as W

V = 6


class Tok(nn.Module):
    """Per-token classifier [B, S] ids -> [B, S, V] logits."""

    def __init__(self, width=16, seed=0):
        super().__init__()
        torch.manual_seed(seed)
        self.e = nn.Embedding(32, width)
        self.h = nn.Linear(width, V)

    def forward(self, input_ids, attention_mask=None):
        return {"logits": self.h(torch.tanh(self.e(input_ids)))}


def _task(n=256, s=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 32, (n, s), generator=g)
    return ids, ids % V                                      # the true label of a token is its id modulo V


def _supervisor(noise=0.25):
    """Right on most tokens, confidently wrong on a fixed subset of ids."""
    m = Tok(seed=1)
    with torch.no_grad():
        m.e.weight.zero_()
        m.h.weight.zero_()
        m.h.bias.zero_()
        wrong = set(range(0, 32, int(1 / noise)))
        table = torch.full((32, V), -2.0)
        for t in range(32):
            lab = (t + 1) % V if t in wrong else t % V
            table[t, lab] = 1.0 if t in wrong else 4.0       # less confident where it is wrong
        m.e = nn.Embedding.from_pretrained(table, freeze=True)
        m.h = nn.Identity()
        m.forward = lambda input_ids, attention_mask=None: {"logits": m.e(input_ids)}
    return m


def test_config_and_curriculum():
    with pytest.raises(ValueError):
        W.PiscesLxWeakToStrongConfig(confidence_threshold=0.4, final_confidence_threshold=0.6)
    with pytest.raises(ValueError):
        W.PiscesLxWeakToStrongConfig(loss_type="mse")
    c = W.PiscesLxWeakToStrongConfig(confidence_threshold=0.9, final_confidence_threshold=0.5, curriculum_steps=4)
    cur = W.PiscesLxCurriculumScheduler(c)
    ths, ws = [], []
    for _ in range(6):
        ths.append(round(cur.get_current_threshold(), 3))
        ws.append(cur.get_difficulty_weight())
        cur.step()
    assert ths == [0.9, 0.8, 0.7, 0.6, 0.5, 0.5] and ws[0] == 0.5 and ws[-1] == 1.0
    flat = W.PiscesLxCurriculumScheduler(W.PiscesLxWeakToStrongConfig(use_curriculum=False))
    assert flat.get_current_threshold() == 0.7 and flat.get_difficulty_weight() == 1.0
    cur2 = W.PiscesLxCurriculumScheduler(c)
    cur2.load_state_dict(cur.state_dict())
    assert cur2.current_step == 6


def test_label_generator_masks_and_freezes():
    sup = Tok(seed=3)
    gen = W.PiscesLxWeakLabelGenerator(sup, W.PiscesLxWeakToStrongConfig(confidence_threshold=0.3, final_confidence_threshold=0.1))
    assert not any(p.requires_grad for p in sup.parameters()) and not sup.training
    ids = torch.randint(0, 32, (3, 5))
    am = torch.ones(3, 5, dtype=torch.long)
    am[:, -2:] = 0
    lab, conf, valid = gen.generate(ids, am)
    assert lab.shape == conf.shape == valid.shape == (3, 5) and not bool(valid[:, -2:].any())
    assert bool(((conf > 0) & (conf <= 1)).all())


@pytest.mark.parametrize("loss_type", ["ce", "kl", "js"])
def test_losses_are_zero_gradient_free_when_nothing_is_valid_and_train_otherwise(loss_type):
    sup, student = _supervisor(), Tok(seed=5)
    cfg = W.PiscesLxWeakToStrongConfig(loss_type=loss_type, use_curriculum=False, confidence_threshold=0.999999, final_confidence_threshold=0.0,
                                       use_self_correction=False)
    op = W.PiscesLxWeakToStrongOperator(sup, student, cfg)
    ids, _ = _task(8)
    out = op.train_step(ids)
    assert float(out["valid_positions"]) == 0 and float(out["loss"]) == 0.0
    cfg2 = W.PiscesLxWeakToStrongConfig(loss_type=loss_type, use_curriculum=False, confidence_threshold=0.5, final_confidence_threshold=0.0)
    op2 = W.PiscesLxWeakToStrongOperator(sup, student, cfg2)
    out2 = op2.train_step(ids)
    assert float(out2["loss"]) > 0 and float(out2["valid_positions"]) > 0
    out2["loss"].backward()
    assert student.h.weight.grad is not None and float(student.h.weight.grad.abs().sum()) > 0


def test_self_correction_targets_confident_disagreements_only():
    sc = W.PiscesLxSelfCorrection(W.PiscesLxWeakToStrongConfig())
    strong = torch.tensor([[[9.0, 0, 0], [0.2, 0.1, 0.0], [0.0, 9.0, 0.0]]], requires_grad=True)
    weak_labels = torch.tensor([[1, 1, 1]])
    conf = torch.tensor([[0.6, 0.6, 0.6]])
    mask, own = sc.correction_mask(strong, weak_labels, conf)
    assert mask.tolist() == [[True, False, False]] and own.tolist() == [[0, 0, 1]]     # confident+different | unsure | agrees
    loss = sc.compute_correction_loss(strong, weak_labels, conf)
    loss.backward()
    assert float(strong.grad[0, 1].abs().sum()) == 0 and float(strong.grad[0, 2].abs().sum()) == 0 and float(strong.grad[0, 0].abs().sum()) > 0
    none = sc.compute_correction_loss(strong.detach(), torch.tensor([[0, 0, 1]]), conf)
    assert float(none) == 0.0


def test_student_generalises_past_its_supervisor():
    torch.manual_seed(0)
    ids, truth = _task(512)
    sup = _supervisor(0.25)
    weak_acc = float((sup(ids)["logits"].argmax(-1) == truth).float().mean())
    assert 0.7 < weak_acc < 0.8
    student = Tok(width=4, seed=7)                           # too small to memorise the supervisor's exceptions
    with torch.no_grad():                                    # give it the structure of the task: id mod V is linear here
        student.e = nn.Embedding.from_pretrained(torch.nn.functional.one_hot(torch.arange(32) % V, V).float() * 2 - 1, freeze=True)
        student.h = nn.Linear(V, V)
    cfg = W.PiscesLxWeakToStrongConfig(confidence_threshold=0.9, final_confidence_threshold=0.3, curriculum_steps=60, strong_model_lr=0.1)
    op = W.PiscesLxWeakToStrongOperator(sup, student, cfg)
    opt = torch.optim.Adam(student.parameters(), lr=0.1)
    stats = op.fit([(ids[i:i + 64], truth[i:i + 64]) for i in range(0, 512, 64)], opt, epochs=12)
    strong_acc = float((student(ids)["logits"].argmax(-1) == truth).float().mean())
    assert strong_acc > weak_acc + 0.05 and stats["strong_accuracy"] > stats["weak_accuracy"]
    s = op.get_statistics()
    assert s["steps"] == 96 and 0 < s["valid_positions"] <= s["total_positions"] and s["corrections"] >= 0
    r = op.execute({"input_ids": ids[:4], "labels": truth[:4]})
    assert r.is_success() and "loss" in r.output and not op.execute({"input_ids": None}).is_success()


def test_iterative_amplification_rounds():
    torch.manual_seed(0)
    ids, truth = _task(128)
    base = Tok(seed=11)
    made = []
    amp = W.PiscesLxIterativeAmplification(base, W.PiscesLxWeakToStrongConfig(confidence_threshold=0.3, final_confidence_threshold=0.1,
                                                                              curriculum_steps=4), num_iterations=2,
                                           optimizer_factory=lambda m: (made.append(m), torch.optim.SGD(m.parameters(), lr=0.05))[1])
    batches = [(ids[i:i + 32], truth[i:i + 32]) for i in range(0, 128, 32)]
    m1 = amp.step(batches)
    assert m1 is not base and amp.iteration == 1 and any(p.requires_grad for p in m1.parameters())
    final = amp.run(batches)
    assert amp.iteration == 2 and len(amp.history) == 2 and final is made[-1] and amp.step(batches) is final
    big = W.PiscesLxIterativeAmplification(base, num_iterations=1, student_factory=lambda cur, it: Tok(width=32, seed=it))
    assert big._new_student().e.embedding_dim == 32
