"""CPU tests of self-play fine-tuning, weak-to-strong training and expert width growth."""
from __future__ import annotations

import torch
import torch.nn as nn

from pisceslx_b200 import YvConfig
from pisceslx_b200.models import build_model


def test_spin_loss_and_self_play_round():
    from pisceslx_b200.engine.alignment import PiscesLxSelfPlayTrainer, spin_loss
    z = torch.zeros(3)
    assert abs(float(spin_loss(z, z, z, z)) - 0.6931) < 1e-3
    assert spin_loss(z + 5, z - 5, z, z, beta=1.0) < 0.01 < spin_loss(z - 5, z + 5, z, z, beta=1.0)
    torch.manual_seed(0)
    # a toy "policy": logits over 5 answers from a prompt id; the data always answers 3
    pol = nn.Embedding(4, 5)
    opt = torch.optim.SGD(pol.parameters(), lr=0.5)
    gen = lambda m, p: m(p).argmax(-1)
    lp = lambda m, p, r: torch.log_softmax(m(p), -1).gather(-1, r.view(-1, 1)).sum()
    tr = PiscesLxSelfPlayTrainer(pol, opt, gen, lp, beta=1.0)
    prompts = [torch.tensor([i]) for i in range(4)]
    real = [torch.tensor([3]) for _ in range(4)]
    for _ in range(3):
        tr.start_round()
        for _ in range(10):
            out = tr.step(prompts, real)
    assert tr.round == 3 and out["round"] == 3
    assert all(int(gen(pol, p)) == 3 for p in prompts)
    assert not any(p.requires_grad for p in tr.opponent.parameters())


def test_weak_to_strong_trainer_overrules_label_noise():
    from pisceslx_b200.engine.alignment import PiscesLxWeakToStrongTrainer
    torch.manual_seed(1)
    x = torch.randn(400, 8)
    true = (x[:, 0] > 0).long()
    weak = true.clone()
    flip = torch.rand(400) < 0.2
    weak[flip] = 1 - weak[flip]
    student = nn.Linear(8, 2)
    tr = PiscesLxWeakToStrongTrainer(student, torch.optim.Adam(student.parameters(), lr=0.05), alpha_max=0.5, warmup_steps=20)
    for _ in range(150):
        st = tr.step(x, weak)
    assert st["alpha"] == 0.5
    acc_true = float((student(x).argmax(-1) == true).float().mean())
    assert acc_true > 0.93 and acc_true > st["agreement_with_weak"]      # closer to the truth than to its supervisor


def test_expert_width_growth_preserves_function():
    from pisceslx_b200.engine.alignment import grow_expert_width
    torch.manual_seed(2)
    cfg = YvConfig.tiny_text_moe(vocab_size=256)
    cfg.n_layer = 1
    m = build_model(cfg)
    m.eval()
    ids = torch.randint(0, 256, (1, 12))
    before = m(input_ids=ids).logits
    layer = m.model.layers[0].mlp
    F = layer.ffn
    grow_expert_width(layer, F + 16)
    assert layer.experts_w13.shape[1] == 2 * (F + 16) and layer.experts_w2.shape[2] == F + 16
    after = m(input_ids=ids).logits
    assert torch.allclose(before, after, atol=1e-5)
    m.train()
    m(input_ids=ids, labels=ids)["loss"].backward()
    assert layer.experts_w2.grad[..., F:].abs().sum() > 0              # the new columns receive gradient
