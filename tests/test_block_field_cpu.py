"""Contracts of the Subconscious Block Field (bounded modulation, dwell floor, residency and commit-back, addresser
gradient through the straight-through gate, paired initialisation, capacity accounting)."""
import torch

from pisceslx_b200.models.block_field import (YvKnowledgeBlockModule, YvResidentBlockPool, YvResonantTraceAddresser,
                                              YvSubconsciousBlockField)


def _field(**kw):
    args = dict(hidden=32, block_count=6, memory_rows=16, rank=8, pool_slots=2, min_dwell=4, trace_dim=8, seed=3)
    args.update(kw)
    return YvSubconsciousBlockField(**args)


def test_modulation_is_bounded_for_any_block_and_any_weights():
    torch.manual_seed(0)
    f = _field()
    kappa = f.relative_perturbation_bound()
    assert abs(kappa - 0.1 * (0.5 + 0.25)) < 1e-9
    for scale in (1.0, 1e3):                                     # a block with absurd weights still cannot blow h up
        blk = f.load_block(0)
        with torch.no_grad():
            for p in blk.parameters():
                p.mul_(scale)
        h = torch.randn(50, 32) * torch.logspace(-3, 3, 50).unsqueeze(1)
        gamma, beta = blk(h)
        assert float(gamma.abs().max()) <= 0.5 + 1e-6
        assert bool((beta.norm(dim=-1) <= 0.25 * h.norm(dim=-1) * (1 + 1e-5)).all())
        delta = f.alpha * (gamma * h + beta)
        assert bool((delta.norm(dim=-1) <= kappa * h.norm(dim=-1) * (1 + 1e-5)).all())
    z = torch.zeros(3, 32, requires_grad=True)                   # smooth at zero: no NaN gradient
    g, b = f.load_block(1)(z)
    (g.sum() + b.sum()).backward()
    assert torch.isfinite(z.grad).all()
    y, _ = f.read_and_modulate(torch.randn(2, 30, 32))
    assert torch.isfinite(y).all()


def test_dwell_floor_is_enforced_and_looks_at_the_past_only():
    raw = torch.tensor([[0, 0, 1, 0, 0, 0, 2, 2, 2, 2, 2, 1, 1, 1, 1, 3, 3],
                        [5, 4, 4, 4, 4, 4, 4, 3, 3, 3, 3, 3, 3, 3, 2, 2, 2]])
    out = YvResonantTraceAddresser.apply_dwell_constraint(raw, 4)
    for row in out.tolist():
        runs, prev = [], None
        for v in row:
            if v == prev:
                runs[-1] += 1
            else:
                runs.append(1)
                prev = v
        assert all(r >= 4 for r in runs[:-1]), (row, runs)      # only the run that ends the sequence may be short
    assert out[0, 2] == 0                                        # the one-token excursion to block 1 is refused
    for t in (5, 9, 13):                                         # prefix property: later tokens never change earlier choices
        assert torch.equal(YvResonantTraceAddresser.apply_dwell_constraint(raw[:, :t], 4), out[:, :t])
    assert torch.equal(YvResonantTraceAddresser.apply_dwell_constraint(raw, 1), raw)
    a = YvResonantTraceAddresser(32, 6, trace_dim=8, min_dwell=4, seed=1)
    ids, scores = a.select_sequence(torch.randn(2, 64, 32))
    assert ids.shape == (2, 64) and scores.shape == (2, 64, 6) and a.stats.mean_dwell() >= 4.0
    # decode form: hysteresis keeps the block unless the challenger wins by the margin
    a.reset()
    h = torch.randn(32)
    first, s = a.select(h)
    second_best = int(s.topk(2).indices[1])
    with torch.no_grad():
        a.traces[second_best] = a.traces[first] * 1.0 + 1e-4 * torch.randn(8)        # a near tie
    assert a.select(h)[0] == first


def test_only_served_blocks_take_part_and_eviction_commits_back():
    torch.manual_seed(1)
    f = _field(pool_slots=2).train()
    h = torch.randn(2, 40, 32, requires_grad=True)
    y, diag = f.read_and_modulate(h)
    assert len(diag["served_blocks"]) <= 2 and set(diag["resident_blocks"]) == set(diag["served_blocks"])
    y.sum().backward()
    for bid in diag["served_blocks"]:
        assert f.pool.slot_module(bid).memory.grad is not None
    assert all(p.grad is not None for p in f.addresser.parameters())
    # the call never uses more different blocks than the pool holds, so every token is served by a resident block
    assert set(torch.unique(diag["selected"]).tolist()) == set(diag["served_blocks"])
    assert not torch.equal(y, h)
    # update a resident block, push it out, bring it back: the update survived
    bid = diag["served_blocks"][0]
    with torch.no_grad():
        f.pool.slot_module(bid).memory.add_(1.0)
    marker = f.pool.slot_module(bid).memory.detach().clone()
    others = [b for b in range(f.block_count) if b not in diag["served_blocks"]][:2]
    for o in others:
        f._ensure_resident(o, torch.device("cpu"))
    assert bid not in f.pool.resident_block_ids() and bid in f._host and f.pool.stats["evictions"] >= 2
    assert torch.equal(f._ensure_resident(bid, torch.device("cpu")).memory, marker)
    pool = YvResidentBlockPool(1)
    seen = []
    pool.install(7, YvKnowledgeBlockModule(8, 4, 2), lambda i, m: seen.append(i))
    assert pool.install(9, YvKnowledgeBlockModule(8, 4, 2), lambda i, m: seen.append(i)) == 7 and seen == [7]


def test_straight_through_gate_keeps_the_forward_and_trains_the_traces():
    torch.manual_seed(2)
    f = _field()
    h = torch.randn(2, 24, 32)
    f.eval()
    with torch.no_grad():
        y_eval, d_eval = f.read_and_modulate(h)
    f.train()
    hg = h.clone().requires_grad_(True)
    y_train, d_train = f.read_and_modulate(hg)
    assert torch.equal(d_eval["selected"], d_train["selected"])
    assert torch.equal(y_eval, y_train.detach())                  # the gate's value is exactly one
    assert f._straight_through_gate(torch.randn(2, 3, 6), torch.zeros(2, 3, dtype=torch.long)) is None   # no grad: no gate
    loss = (y_train * torch.randn_like(y_train)).sum()
    loss.backward()
    g = f.addresser.traces.grad
    assert g is not None and float(g.abs().sum()) > 0
    before = f.addresser.traces.detach().clone()
    torch.optim.SGD(f.addresser.parameters(), lr=0.1).step()
    assert not torch.equal(before, f.addresser.traces.detach())


def test_paired_initialisation_routes_a_block_direction_to_that_block_and_capacity_is_accounted():
    f1, f2 = _field(seed=5), _field(seed=5)
    f1.paired_initialize()
    f2.paired_initialize()
    assert torch.equal(f1.addresser.traces, f2.addresser.traces)                      # deterministic
    hits = 0
    for i in range(f1.block_count):
        direction = torch.linalg.svd(f1.load_block(i).query.float(), full_matrices=False).Vh[0]
        hits += int(f1.addresser.scores(direction).argmax()) == i
    assert hits == f1.block_count
    cap = f1.measurable_capacity()
    assert cap["params_per_block"] == float(f1.load_block(0).param_count)
    assert cap["nominal_capacity"] == cap["params_per_block"] * 6 and cap["resident_params"] == 0.0
    f1.read_and_modulate(torch.randn(1, 8, 32))
    assert f1.measurable_capacity()["resident_params"] > 0


def test_block_field_in_the_trunk_trains_the_addresser_and_stays_causal():
    from pisceslx_b200 import YvConfig
    from pisceslx_b200.engine.loader import attach_optional_components
    from pisceslx_b200.models import build_model
    cfg = YvConfig.tiny_text_moe(vocab_size=256)
    cfg.n_layer, cfg.use_subconscious_blocks, cfg.block_count = 2, True, 5
    cfg.block_memory_rows, cfg.block_min_dwell_tokens = 8, 4
    m = build_model(cfg, "cpu", torch.float32, seed=0)
    attach_optional_components(m, cfg)
    ids = torch.randint(0, 256, (2, 24), generator=torch.Generator().manual_seed(0))
    out = m(input_ids=ids, labels=ids)
    out["loss"].backward()
    diag = m.model.block_field_diagnostics
    assert len(diag["served_blocks"]) <= cfg.block_pool_slots and "selected" not in diag       # values only, no graph nodes
    assert float(m.model.block_field.addresser.traces.grad.abs().sum()) > 0
    m.eval()
    with torch.no_grad():
        y = m(input_ids=ids).logits
        ids2 = ids.clone()
        ids2[-1, 17] = (ids2[-1, 17] + 3) % 256               # the last row: earlier rows' block budget is unaffected
        y2 = m(input_ids=ids2).logits
    assert torch.allclose(y[:, :17], y2[:, :17], atol=1e-5) and not torch.allclose(y[-1, 17:], y2[-1, 17:], atol=1e-5)
