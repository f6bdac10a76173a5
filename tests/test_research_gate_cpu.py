"""Research router and the sparsity objective: routing contract (shapes, distribution, capacity by zeroing), the phases,
the sparse gates' route into the loss, pruning, the stage cache, and the device-side adaptation."""
import inspect

import pytest
import torch
from torch import nn

from pisceslx_b200.config import YvConfig
from pisceslx_b200.models.model import YvModel, YvModelForCausalLM
from pisceslx_b200.models.moe_gate_research import HEADS, YvResearchMoEGate, straight_through_gate


def _cfg(**kw):
    extra = {"moe_random_to_gradient_steps": 2, "moe_routing_head_warmup_min": 2, "moe_gate_warmup_steps": 3}
    extra.update(kw.pop("extra", {}))
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    cfg.moe_gate_type = "research"
    cfg.extra.update(extra)
    for k, v in kw.items():
        setattr(cfg, k, v)
    return cfg


def _gate(**kw):
    torch.manual_seed(0)
    cfg = _cfg(**kw)
    return YvResearchMoEGate(cfg), cfg


def test_shapes_and_distribution():
    g, cfg = _gate()
    g.eval()
    x = torch.randn(24, cfg.hidden_size)
    w, idx, aux = g(x)
    assert w.shape == (24, g.slots) and idx.shape == (24, g.slots)
    assert torch.allclose(w.sum(-1), torch.ones(24), atol=1e-5)
    assert int(idx.min()) >= 0 and int(idx.max()) < cfg.moe_num_experts
    assert aux.ndim == 0 and torch.isfinite(aux)
    # an expert appears once per token
    assert all(len(set(r.tolist())) == g.slots for r in idx)


def test_random_phase_then_learned_phase():
    g, cfg = _gate()
    g.train()
    x = torch.randn(32, cfg.hidden_size)
    w, _, _ = g(x)                                      # step 1: random routing, uniform weights
    assert torch.allclose(w, torch.full_like(w, 1.0 / g.slots))
    g(x)
    w3, _, _ = g(x)                                     # step 3: learned routing
    assert not torch.allclose(w3, torch.full_like(w3, 1.0 / g.slots))
    assert float(g.total_routed) == 96.0 and float(g.expert_usage.sum()) == 32 * g.slots


def test_straight_through_gate_is_value_neutral():
    p = nn.Parameter(torch.tensor(0.3))
    f = straight_through_gate(p)
    assert float(f.detach()) == 1.0
    f.backward()
    s = torch.sigmoid(torch.tensor(0.3))
    assert torch.allclose(p.grad, s * (1 - s))


def test_sparse_gates_receive_gradient_from_the_route_and_the_regulariser():
    g, cfg = _gate()
    g.train()
    x = torch.randn(16, cfg.hidden_size)
    for _ in range(3):
        w, idx, aux = g(x)
    (w * torch.randn_like(w)).sum().backward()
    for n in HEADS:
        assert getattr(g, "sparse_gate_" + n).grad is not None, n
    g.zero_grad()
    g.sparsity_loss().backward()
    for n in HEADS:
        gr = getattr(g, "sparse_gate_" + n).grad
        assert gr is not None and float(gr) > 0


def test_prune_removes_closed_heads_only():
    g, cfg = _gate()
    with torch.no_grad():
        g.sparse_gate_got.fill_(-6.0)
        g.sparse_gate_soft_moe.fill_(-6.0)
    done = g.prune_routing_heads(0.05)
    assert done == {"got", "soft_moe"}
    assert not hasattr(g, "got_cluster_proj") and not hasattr(g, "gate_k") and hasattr(g, "hicl_prototypes")
    g.eval()
    w, idx, _ = g(torch.randn(8, cfg.hidden_size))
    assert torch.allclose(w.sum(-1), torch.ones(8), atol=1e-5)
    assert float(g.sparsity_loss()) == pytest.approx(2 * g.sparsity_reg_weight * float(torch.sigmoid(torch.tensor(5.0))), rel=1e-5)
    st = g.get_extra_state()
    assert st["pruned"] == ["got", "soft_moe"]
    g2, _ = _gate()
    g2.set_extra_state(st)
    g2.load_state_dict(g.state_dict())                  # same keys once the same heads are dropped


def test_route_of_a_token_ignores_later_tokens():
    g, cfg = _gate()
    g.eval()
    x = torch.randn(20, cfg.hidden_size)
    y = x.clone()
    y[12:] = torch.randn(8, cfg.hidden_size)
    w1, i1, _ = g(x)
    w2, i2, _ = g(y)
    assert torch.equal(i1[:12], i2[:12]) and torch.allclose(w1[:12], w2[:12], atol=1e-6)


def test_modal_affinity_moves_the_route():
    g, cfg = _gate()
    g.eval()
    with torch.no_grad():
        g.expert_modal_affinity[3, 1] = 50.0
    x = torch.randn(10, cfg.hidden_size)
    _, idx, _ = g(x, modal_id=torch.ones(10, dtype=torch.long))
    assert bool((idx == 3).any(-1).all())
    _, idx0, _ = g(x, modal_id=torch.zeros(2, dtype=torch.long))     # one id per sequence of 5 tokens
    assert idx0.shape == idx.shape


def test_capacity_drops_by_zeroing():
    g, cfg = _gate(moe_drop_tokens=True, moe_capacity_factor=0.25, moe_min_capacity=1)
    g.eval()
    with torch.no_grad():
        g.expert_bias[0] = 2.0                          # crowd one expert
    x = torch.randn(64, cfg.hidden_size)
    w, idx, _ = g(x)
    cap = g.capacity(64)
    kept = ((idx == 0) & (w > 0)).sum()
    assert int(kept) <= cap and int((idx == 0).sum()) > cap
    live = w.sum(-1) > 0
    assert torch.allclose(w.sum(-1)[live], torch.ones(int(live.sum())), atol=1e-5)


def test_importance_tiers_mask_trailing_slots_and_train_the_projection():
    g, cfg = _gate(extra={"ultra_sparse_tier1_threshold": 2.0, "ultra_sparse_tier2_threshold": 3.0})
    g.eval()                                            # thresholds above 1: every token is in the lowest tier
    w, _, _ = g(torch.randn(12, cfg.hidden_size))
    assert bool((w[:, 1:] == 0).all()) and torch.allclose(w[:, 0], torch.ones(12))
    g2, cfg = _gate()
    g2.eval()
    x = torch.randn(12, cfg.hidden_size)
    w, _, _ = g2(x)
    (w * torch.randn_like(w)).sum().backward()
    assert g2.importance_proj[0].weight.grad is not None
    assert float(g2.importance_proj[0].weight.grad.abs().sum()) > 0


def test_stage_cache_reuses_the_route_and_follows_the_batch():
    g, cfg = _gate(extra={"path_moe_stage_size": 3})
    g.eval()
    a, b = torch.randn(8, cfg.hidden_size), torch.randn(8, cfg.hidden_size)
    w1, i1, _ = g(a)
    w2, i2, _ = g(b)                                    # second call of the stage: the cached route
    assert torch.equal(i1, i2) and torch.equal(w1, w2) and not w2.requires_grad
    c = torch.randn(11, cfg.hidden_size)                # other row count: must route anew
    w3, i3, _ = g(c)
    assert i3.shape[0] == 11
    g(c), g(c)
    w4, i4, _ = g(b)                                    # stage over (3 calls): routed from b itself
    g2, _ = _gate()
    g2.eval()
    assert torch.equal(i4, g2(b)[1])


def test_adaptation_stays_on_the_device_and_reacts_to_imbalance():
    g, cfg = _gate(moe_noise_std=0.0)
    g.train()
    E = cfg.moe_num_experts
    with torch.no_grad():                               # a history in which one expert took nearly everything
        g.expert_usage.copy_(torch.full((E,), 1.0))
        g.expert_usage[0] = 5000.0
        g.total_routed.fill_(float(g.expert_usage.sum()) / g.slots)
    g.current_step = 10
    t0, b0 = float(g.temperature), g.expert_bias.clone()
    g._calls = g.bias_update_freq - 1
    x = torch.randn(256, cfg.hidden_size)
    g(x)
    assert float(g.temperature) != t0
    assert float(g.expert_bias[0]) < float(b0[0]) and float(g.expert_bias[1]) > float(b0[1])
    assert float(g._effective_k()) in (float(g.k_min), float(g.top_k), float(g.k_max))
    src = inspect.getsource(YvResearchMoEGate._adapt) + inspect.getsource(YvResearchMoEGate._rebalance)
    assert ".item()" not in src and ".tolist()" not in src and "float(self." not in src


def test_rebalance_moves_assignments_off_an_overloaded_expert():
    g, cfg = _gate(moe_noise_std=0.0)
    g.train()
    E = cfg.moe_num_experts
    with torch.no_grad():
        g.expert_usage.copy_(torch.full((E,), 20000.0))    # a fair share: neither over- nor underloaded
        g.expert_usage[0] = 100000.0
        g.expert_usage[1] = 1.0
        g.total_routed.fill_(float(g.expert_usage.sum()) / g.slots)
    g.current_step = 50
    T = 2000
    idx = torch.zeros(T, g.slots, dtype=torch.long)
    idx[:, 1] = 2
    if g.slots > 2:
        idx[:, 2:] = torch.arange(3, 1 + g.slots)[None, :]
    probs = torch.softmax(torch.randn(T, E), -1)
    out = g._rebalance(idx, probs)
    moved = int((out[:, 0] != 0).sum())
    assert 0.2 * T < moved < 0.4 * T                    # rate is capped at 30 %
    assert bool((out[out[:, 0] != 0, 0] == 1).all())    # only the underloaded expert receives
    assert all(len(set(r.tolist())) == g.slots for r in out[:50])


# ---- the sparsity objective -------------------------------------------------------------------------------------------
def _stub():
    outer = nn.Module()
    outer.w = nn.Parameter(torch.tensor(1.0))
    outer.attn = nn.Module()
    outer.attn.w = nn.Parameter(torch.tensor(2.0))
    outer.sparsity_loss = (lambda _s: _s.w * 0.25).__get__(outer, nn.Module)
    outer.attn.sparsity_loss = (lambda _s: _s.w * 0.5).__get__(outer.attn, nn.Module)
    return outer


def test_walk_sums_disjoint_contributors_and_reaches_every_gate():
    m = _stub()
    total = YvModel.sparsity_objective(m)
    assert float(total) == pytest.approx(0.25 * 1.0 + 0.5 * 2.0)
    assert total.requires_grad
    total.backward()
    assert float(m.w.grad) == 0.25 and float(m.attn.w.grad) == 0.5


def test_fold_is_not_gated_on_the_balancing_mode():
    lines = inspect.getsource(YvModelForCausalLM.forward).splitlines()
    at = next(i for i, l in enumerate(lines) if "self.sparsity_objective()" in l)
    window = "\n".join(lines[at:at + 3])
    assert "loss = loss + sparsity_loss" in window and "moe_aux_loss_free" not in window


def test_model_trains_the_sparse_gates_with_aux_loss_free_balancing():
    torch.manual_seed(0)
    cfg = _cfg(n_layer=2, extra={"sparsity_reg_weight": 1.0})
    assert cfg.moe_aux_loss_free
    model = YvModelForCausalLM(cfg)
    model.train()
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    out = model(ids, labels=ids)
    gates = [(n, p) for n, p in model.named_parameters() if "sparse_gate_" in n]
    assert len(gates) >= 4
    assert float(out["loss"]) > float(out["lm_loss"])
    out["loss"].backward()
    for n, p in gates:
        assert p.grad is not None and float(p.grad.abs()) > 0, n
