"""MoE runtime operator: routing, adaptive temperature, capacity, routing cache, request sharing, brownout, layout switch."""
import json

import torch
import torch.nn as nn

from pisceslx_b200.serve.moe_runtime import (
    PiscesLxBatchExpertSharing, PiscesLxBrownoutExpertGroup, PiscesLxExpertCacheManager, PiscesLxExpertStats,
    PiscesLxMoebiusParallelismMode, PiscesLxMoebiusParallelismSwitch, PiscesLxMoERoutingStrategy, PiscesLxMoERuntimeConfig,
    PiscesLxMoERuntimeOperator, PiscesLxMoeRuntime)


class _Gate(nn.Module):
    def __init__(self, hidden=16, experts=8, skew=0.0):
        super().__init__()
        self.num_experts = experts
        self.gate = nn.Linear(hidden, experts, bias=False)
        self.register_buffer("expert_bias", torch.zeros(experts))
        if skew:
            with torch.no_grad():
                self.expert_bias[0] = skew


class _Model(nn.Module):
    def __init__(self, layers=2, **kw):
        super().__init__()
        self.layers = nn.ModuleList([_Gate(**kw) for _ in range(layers)])


def test_config_round_trip(tmp_path):
    c = PiscesLxMoERuntimeConfig(top_k=3, routing_strategy=PiscesLxMoERoutingStrategy.CAPACITY)
    p = tmp_path / "c.json"
    p.write_text(json.dumps({**c.to_dict(), "unknown": 1}))
    c2 = PiscesLxMoERuntimeConfig.from_json(str(p))
    assert c2.top_k == 3 and c2.routing_strategy == "capacity"
    c3 = PiscesLxMoERuntimeConfig.from_model_config({"moe_top_k": 4, "routing_temp": 1.0})
    assert c3.top_k == 4 and c3.routing_temp == 1.0


def test_route_matches_plain_softmax_topk():
    torch.manual_seed(0)
    m = _Model()
    op = PiscesLxMoeRuntime.create_moe_runtime_operator(PiscesLxMoERuntimeConfig(routing_strategy="top_k", top_k=2), m)
    assert op.num_experts == 8 and len(op._gates) == 2
    x = torch.randn(32, 16)
    r = op.route(x, layer=1)
    probs = torch.softmax(m.layers[1].gate(x), -1)
    p, i = probs.topk(2, -1)
    assert torch.equal(r["expert_indices"], i)
    assert torch.allclose(r["routing_probs"], p / p.sum(-1, keepdim=True), atol=1e-6)
    assert not r["cache_hit"]


def test_adaptive_temperature_rises_under_skew_and_is_capped():
    torch.manual_seed(0)
    m = _Model(layers=1, skew=8.0)
    cfg = PiscesLxMoERuntimeConfig(adaptive_temp_interval=2, top_k=1)
    op = PiscesLxMoeRuntime.create_moe_runtime_operator(cfg, m)
    t0 = op._adaptive_temp
    for _ in range(40):
        op.route(torch.randn(64, 16))
    assert op._adaptive_temp > t0
    assert op._adaptive_temp <= cfg.adaptive_temp_cap + 1e-9
    s = op.get_stats()
    assert 0 in s["overutilized"] and s["utilization_max"] > 1.5
    assert s["capacity_scale"] > 1.0


def test_balanced_routing_keeps_temperature():
    torch.manual_seed(0)
    m = _Model(layers=1, hidden=64, experts=4)
    with torch.no_grad():
        m.layers[0].gate.weight.mul_(0.01)
    op = PiscesLxMoeRuntime.create_moe_runtime_operator(PiscesLxMoERuntimeConfig(adaptive_temp_interval=2), m)
    for _ in range(20):
        op.route(torch.randn(512, 64))
    assert abs(op._adaptive_temp - op.config.routing_temp) < 1e-9


def test_capacity_drops_overflow_and_priority_serves_weighted_tokens_first():
    torch.manual_seed(0)
    m = _Model(layers=1, skew=20.0)
    cfg = PiscesLxMoERuntimeConfig(routing_strategy="capacity", top_k=1, dynamic_capacity=False, enable_adaptive_temp=False, min_capacity=1)
    op = PiscesLxMoeRuntime.create_moe_runtime_operator(cfg, m)
    x = torch.randn(64, 16)
    r = op.route(x)
    cap = r["capacity"]
    kept = (r["routing_probs"] > 0).sum()
    assert (r["expert_indices"] == 0).all()
    assert int(kept) == cap and int(r["dropped"]) == 64 - cap
    op2 = PiscesLxMoeRuntime.create_moe_runtime_operator(PiscesLxMoERuntimeConfig(**{**cfg.to_dict(), "routing_strategy": "priority"}), m)
    w = torch.zeros(64)
    w[-cap:] = 1.0
    r2 = op2.route(x, token_weights=w)
    assert (r2["routing_probs"][-cap:] > 0).all() and int((r2["routing_probs"] > 0).sum()) == cap


def test_routing_cache_hits_on_same_tokens():
    m = _Model(layers=1)
    op = PiscesLxMoeRuntime.create_moe_runtime_operator(None, m)
    x = torch.randn(5, 16)
    ids = [3, 1, 4, 1, 5]
    a = op.route(x, token_ids=ids)
    b = op.route(x, token_ids=ids)
    assert not a["cache_hit"] and b["cache_hit"] and torch.equal(a["expert_indices"], b["expert_indices"])
    assert not op.route(x, token_ids=[3, 1, 4, 1, 6])["cache_hit"]
    assert op.cache.get_hit_rate() > 0
    mgr = PiscesLxExpertCacheManager(max_entries=2)
    for i in range(3):
        mgr.insert(str(i), torch.zeros(1, 1), torch.zeros(1, 1))
    assert mgr.get("0") is None and mgr.get("2") is not None and mgr.evictions == 1


def test_aux_loss_is_one_alpha_when_uniform():
    m = _Model(layers=1, experts=4)
    with torch.no_grad():
        m.layers[0].gate.weight.zero_()
    op = PiscesLxMoeRuntime.create_moe_runtime_operator(PiscesLxMoERuntimeConfig(top_k=4), m)
    r = op.route(torch.randn(8, 16), return_aux_loss=True)
    assert abs(float(r["load_balance_loss"]) - op.config.load_balance_alpha) < 1e-6


def test_batch_sharing_prefix():
    s = PiscesLxBatchExpertSharing(similarity_threshold=0.75)
    s.register("a", [1, 2, 3, 4, 5, 6, 7, 8])
    s.register("b", [9, 9, 9])
    out = s.share_prefix_kv([1, 2, 3, 4, 5, 6, 0, 0])
    assert out == {"source_request": "a", "shared_tokens": 6, "similarity": 0.75, "remaining_tokens": 2}
    assert s.share_prefix_kv([7, 7]) is None
    assert s.compute_similarity([1, 2], [1, 3]) == 0.5
    g = s.group_by_experts([{0, 1}, {5}, {1, 2}])
    assert sorted(map(sorted, g)) == [[0, 2], [1]]


def test_brownout_masks_inactive_groups():
    torch.manual_seed(0)
    m = _Model(layers=1)
    op = PiscesLxMoeRuntime.create_moe_runtime_operator(PiscesLxMoERuntimeConfig(routing_strategy="top_k"), m)
    op.brownout.importance = [1.5, 0.1]
    groups = op.brownout_groups(load_factor=1.0)
    assert isinstance(groups[0], PiscesLxBrownoutExpertGroup) and groups[0].active and not groups[1].active
    r = op.route(torch.randn(64, 16))
    assert set(r["expert_indices"].flatten().tolist()) <= set(groups[0].expert_ids)
    op.reset()
    assert op._mask is None


def test_moebius_switch_with_hysteresis():
    calls = []
    sw = PiscesLxMoebiusParallelismSwitch(world_size=8, hidden=4096, ffn=1408, top_k=2, switcher=calls.append)
    assert sw.mode is PiscesLxMoebiusParallelismMode.EXPERT_PARALLEL
    modes = {n: sw.preferred(n, 64)[0] for n in (1, 8, 64, 4096, 65536)}
    assert len(set(modes.values())) >= 1
    target = PiscesLxMoebiusParallelismMode.TENSOR_PARALLEL
    sw.switch(target)
    assert sw.mode is target and sw.switch_count == 1 and calls == [target]
    sw.switch(target)
    assert sw.switch_count == 1
    single = PiscesLxMoebiusParallelismSwitch(world_size=1)
    assert not single.should_switch(1, 64)
    assert sw.step(4096, 64) in tuple(PiscesLxMoebiusParallelismMode)


def test_operator_front_and_stats():
    m = _Model(layers=1)
    op = PiscesLxMoeRuntime.from_model(m)
    assert op.validate_inputs({"action": "route"}) and not op.validate_inputs({"action": "nope"})
    out = op.run({"action": "route", "hidden_states": torch.randn(2, 3, 16)})
    assert out["expert_indices"].shape == (6, 2)
    op.record_execution([3, 0, 1, 0, 0, 0, 0, 2], latency_ms=1.5)
    st = op.run({"action": "stats"})
    assert st["experts"][0]["tokens"] == 3 and st["calls"] == 1
    assert op.run({"action": "share", "input_ids": [1, 2, 3], "request_id": "r"})["shared"] is None
    assert op.run({"action": "share", "input_ids": [1, 2, 3, 4]})["shared"]["shared_tokens"] == 3
    e = PiscesLxExpertStats(0)
    e.update(10, 2.0)
    e.update(20, 4.0)
    assert e.avg_tokens == 15 and e.avg_latency_ms == 3.0
