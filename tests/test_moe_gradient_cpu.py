"""MoE gradient operator: classification, per-expert clipping on stacked tensors, adaptive threshold, normalisation,
auxiliary losses that train the router."""
import inspect

import pytest
import torch
from torch import nn

from pisceslx_b200.config import YvConfig
from pisceslx_b200.models.model import YvModelForCausalLM
from pisceslx_b200.optim import moe_gradient as M


def _model():
    torch.manual_seed(0)
    cfg = YvConfig.tiny_text_moe(vocab_size=128)
    cfg.n_layer = 1
    return YvModelForCausalLM(cfg)


def test_classification_of_the_framework_model():
    m = _model()
    op = M.PiscesLxMoEGradientOperator()
    c = op.classify(m)
    assert set(c["expert"]["ffn"]) == {"model.layers.0.mlp.experts_w13", "model.layers.0.mlp.experts_w2"}
    assert "model.layers.0.mlp.router.gate.weight" in c["gating"] and "model.layers.0.mlp.shared_w13" in c["non_expert"]
    assert "lm_head" in c["non_expert"] and "model.layers.0.norm_mlp.weight" in c["non_expert"]
    assert op._detect_expert_parameter("blocks.3.moe.experts.7.attn.q_proj") == (True, M.PiscesLxMoEExpertType.ATTENTION)
    assert op._detect_expert_parameter("blocks.3.attention.q_proj")[0] is False


def test_each_expert_is_clipped_on_its_own():
    m = _model()
    op = M.PiscesLxMoEGradientOperator(M.PiscesLxMoEGradientConfig(expert_clip_threshold=1.0, enable_adaptive_clip=False))
    op.classify(m)
    for p in m.parameters():
        p.grad = torch.zeros_like(p)
    w = m.model.layers[0].mlp.experts_w13
    w.grad[0] = 10.0                                            # one spiking expert
    w.grad[1] = 1e-3                                            # an ordinary one
    m.lm_head.grad.fill_(0.5)
    keep = w.grad[1].clone()
    out = op.process(m)
    norms = w.grad.flatten(1).norm(dim=1)
    assert float(norms[0]) == pytest.approx(1.0, rel=1e-4) and torch.equal(w.grad[1], keep)
    assert float(out["num_clipped"]) == 1 and float(out["non_expert_grad_norm"]) == pytest.approx(0.5 * m.lm_head.numel() ** 0.5, rel=1e-4)
    assert float(m.lm_head.grad[0, 0]) == 0.5                   # dense parameters are left alone
    src = inspect.getsource(M.PiscesLxMoEGradientOperator.process)
    assert ".item()" not in src and ".tolist()" not in src and " float(" not in src


def test_adaptive_threshold_follows_the_recent_norms():
    m = _model()
    cfg = M.PiscesLxMoEGradientConfig(expert_clip_threshold=5.0, warmup_steps=0, min_history=4, clip_percentile=50.0, clip_history_window=8)
    op = M.PiscesLxMoEGradientOperator(cfg)
    op.classify(m)
    w = m.model.layers[0].mlp.experts_w13
    thr = []
    for step in range(8):
        for p in m.parameters():
            p.grad = torch.zeros_like(p)
        w.grad[0] = 0.01 if step < 6 else 3.0                   # quiet history, then a spike
        out = op.process(m)
        thr.append(float(out["clip_threshold"]))
    assert thr[0] == 5.0 and thr[3] == 5.0                      # not enough history yet
    quiet = 0.01 * w.grad[0].numel() ** 0.5
    assert thr[5] == pytest.approx(1.2 * quiet, rel=1e-3)       # the median of the quiet steps
    assert float(w.grad[0].norm()) <= thr[7] * 1.001 and thr[7] < 5.0   # the spike (norm ~1000) was cut to the adaptive bound
    assert op.get_gradient_statistics()["history"] == 8.0
    op.reset()
    assert op.steps == 0 and op._history is None


def test_normalisation_sets_the_ratio_to_the_dense_norm():
    m = _model()
    op = M.PiscesLxMoEGradientOperator(M.PiscesLxMoEGradientConfig(expert_clip_threshold=1e9, enable_adaptive_clip=False,
                                                                   enable_gradient_normalization=True, expert_norm_factor=0.5))
    op.classify(m)
    for p in m.parameters():
        p.grad = torch.randn_like(p) * 1e-4
    m.lm_head.grad = torch.randn_like(m.lm_head)
    out = op.process(m)
    assert float(out["expert_grad_norm_after"]) == pytest.approx(0.5 * float(out["non_expert_grad_norm"]), rel=1e-3)
    assert float(out["scale_gap"]) > 100


def test_auxiliary_losses_are_zero_when_balanced_and_train_the_router():
    op = M.PiscesLxMoEGradientOperator(M.PiscesLxMoEGradientConfig(load_balancing_weight=1.0, importance_weight=1.0, utilization_weight=1.0))
    T, E = 64, 4
    uniform = torch.full((T, E), 0.25)
    idx = torch.arange(T).unsqueeze(1) % E
    a = op.auxiliary_losses(uniform, idx)
    assert float(a["load_balancing"]) == pytest.approx(0.0, abs=1e-6) and float(a["importance"]) == pytest.approx(0.0, abs=1e-6)
    logits = nn.Parameter(torch.zeros(T, E))
    with torch.no_grad():
        logits[:, 0] += 3.0                                     # collapsed onto expert 0
    opt = torch.optim.SGD([logits], lr=5.0)
    first = None
    for _ in range(50):
        probs = torch.softmax(logits, -1)
        loss = op.auxiliary_losses(probs, probs.argmax(-1, keepdim=True))["total"]
        first = first if first is not None else float(loss)
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert float(loss) < 0.3 * first and float(torch.softmax(logits, -1).mean(0).max()) < 0.5
    only_idx = op.auxiliary_losses(None, torch.zeros(10, 1, dtype=torch.long), num_experts=4)
    assert float(only_idx["load_balancing"]) > 0 and float(only_idx["importance"]) == 0
    assert float(op.auxiliary_losses()["total"]) == 0


def test_facade_and_clipper_on_a_training_step():
    m = _model().train()
    f = M.PiscesLxMoEGradientFacade(m, expert_clip_threshold=0.05, warmup_steps=0)
    ids = torch.randint(0, 128, (2, 16))
    m(ids, labels=ids)["loss"].backward()
    out = f.process()
    assert float(out["expert_grad_norm"]) > 0 and float(out["max_expert_norm"]) >= 0
    w = m.model.layers[0].mlp.experts_w13
    assert float(w.grad.flatten(1).norm(dim=1).max()) <= 0.05 * 1.001
    assert set(f.get_statistics()) >= {"expert_grad_norm", "num_clipped", "steps"}
    r = f.operator.execute({"model": m, "router_probs": torch.softmax(torch.randn(8, 8), -1)})
    assert r.is_success() and "auxiliary" in r.output and not f.operator.execute({"model": 1}).is_success()
    ps = [nn.Parameter(torch.ones(10)), nn.Parameter(torch.ones(10))]
    for p in ps:
        p.grad = torch.full_like(p, 3.0)
    total = M.PiscesLxExpertGradientClipper(max_norm=1.0).clip(ps)
    assert float(total) == pytest.approx(3.0 * 20 ** 0.5) and float(torch.cat([p.grad for p in ps]).norm()) == pytest.approx(1.0, rel=1e-4)
    with pytest.raises(ValueError):
        M.PiscesLxMoEGradientConfig(clip_percentile=0)
