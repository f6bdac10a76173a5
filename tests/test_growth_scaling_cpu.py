"""Growth classes (depth / width / expert / hybrid), function-preserving hidden growth, the scaling-law operator."""
import math

import pytest
import torch

from pisceslx_b200.config import YvConfig
from pisceslx_b200.engine import growth as G
from pisceslx_b200.models.model import YvModelForCausalLM


def _model(n_layer=2):
    torch.manual_seed(0)
    cfg = YvConfig.tiny_text_moe(vocab_size=256)
    cfg.n_layer = n_layer
    return YvModelForCausalLM(cfg).eval(), cfg


def _logits(m, ids):
    with torch.no_grad():
        return m(ids)["logits"].float()


def test_hidden_growth_preserves_the_function_and_stays_trainable():
    m, cfg = _model()
    ids = torch.randint(0, 256, (2, 12))
    before = _logits(m, ids)
    n0 = sum(p.numel() for p in m.parameters())
    G.grow_hidden(m, 320)
    assert cfg.hidden_size == 320 and m.model.embed.weight.shape == (256, 320) and m.lm_head.shape == (256, 320)
    assert m.model.layers[0].attention.qkv_proj.shape[1] == 320 and m.model.layers[0].attention.o_proj.shape[0] == 320
    assert m.model.layers[0].mlp.experts_w2.shape[1] == 320 and m.model.layers[0].mlp.router.gate.in_features == 320
    after = _logits(m, ids)
    assert torch.allclose(before, after, atol=2e-4), float((before - after).abs().max())
    assert sum(p.numel() for p in m.parameters()) > n0
    m.train()
    out = m(ids, labels=ids)
    out["loss"].backward()
    g = m.model.layers[0].attention.o_proj.grad
    assert g is not None and float(g[256:].abs().sum()) > 0          # the new channels receive gradient
    with pytest.raises(ValueError):
        G.grow_hidden(m, 320)


def test_depth_grower_strategies_and_preservation():
    m, cfg = _model(2)
    ids = torch.randint(0, 256, (1, 10))
    before = _logits(m, ids)
    g = G.PiscesLxDepthGrower(G.PiscesLxModelGrowthConfig("depth", num_new_layers=2, layer_copy_strategy="uniform"))
    assert g.positions(4) == [1, 3] and G.PiscesLxDepthGrower(G.PiscesLxModelGrowthConfig(num_new_layers=3)).positions(5) == [4, 4, 4]
    g.grow(m)
    assert len(m.model.layers) == 4 and cfg.n_layer == 4 and [b.layer_idx for b in m.model.layers] == [0, 1, 2, 3]
    assert torch.allclose(before, _logits(m, ids), atol=1e-5)
    m2, _ = _model(2)
    b2 = _logits(m2, ids)
    G.PiscesLxDepthGrower(G.PiscesLxModelGrowthConfig(num_new_layers=1, preserve_knowledge=False, init_noise_scale=0.01)).grow(m2)
    assert len(m2.model.layers) == 3 and not torch.allclose(b2, _logits(m2, ids), atol=1e-5)
    with pytest.raises(ValueError):
        G.PiscesLxModelGrowthConfig(layer_copy_strategy="random")


def test_width_and_expert_growers():
    m, cfg = _model(1)
    ids = torch.randint(0, 256, (1, 10))
    before = _logits(m, ids)
    G.PiscesLxWidthGrower(G.PiscesLxModelGrowthConfig("width", new_expert_ffn=384)).grow(m)
    assert m.model.layers[0].mlp.experts_w13.shape[1] == 768 and cfg.moe_expert_intermediate_size == 384
    assert torch.allclose(before, _logits(m, ids), atol=1e-5)
    G.PiscesLxExpertGrower(G.PiscesLxModelGrowthConfig("expert", num_new_experts=4)).grow(m)
    assert m.model.layers[0].mlp.experts_w13.shape[0] == 12 and cfg.moe_num_experts == 12
    after = _logits(m, ids)                                              # twins displace second choices: close, not equal
    assert bool(torch.isfinite(after).all()) and 0 < float((before - after).abs().max()) < 1.0
    with pytest.raises(ValueError):
        G.PiscesLxWidthGrower(G.PiscesLxModelGrowthConfig("width")).grow(m)


def test_growth_operator_hybrid():
    m, cfg = _model(1)
    op = G.PiscesLxModelGrowthOperator()
    r = op.execute({"model": m, "config": {"growth_type": "hybrid", "num_new_layers": 1, "num_new_experts": 2, "new_hidden_size": 288}})
    assert r.is_success(), r.error
    o = r.output
    assert o["applied"] == ["PiscesLxDepthGrower", "PiscesLxExpertGrower", "PiscesLxWidthGrower"]
    assert o["layers"] == 2 and o["hidden_size"] == 288 and o["parameters_after"] > o["parameters_before"]
    ids = torch.randint(0, 256, (1, 6))
    assert bool(torch.isfinite(_logits(m, ids)).all())
    assert not op.execute({"model": "nope"}).is_success()
    assert isinstance(op.grow(_model(1)[0], G.PiscesLxModelGrowthConfig("depth", num_new_layers=1)), torch.nn.Module)


def test_chinchilla_scaler_and_operator():
    sc = G.PiscesLxChinchillaScaler(G.PiscesLxScalingConfig(tokens_per_parameter=20.0, sustained_flops_per_gpu=1e15, model_flops_utilization=0.5))
    n, d = sc.optimal_nd(6 * 20 * 1e18)
    assert n == pytest.approx(1e9) and d == pytest.approx(2e10)
    assert sc.to_flops(1.0, "gpu_hours") == pytest.approx(3600 * 5e14)
    cfg = YvConfig.tiny_text_moe(vocab_size=256)
    cnt = sc.estimate_params(cfg)
    assert cnt["total"] > cnt["active"] > 0
    name, preset, counts = sc.get_config_for_params(cnt["active"], {"tiny": cfg, "other": YvConfig.yv_7b_moe()})
    assert name == "tiny" and counts == cnt
    assert sc.chinchilla_memory_correction(100.0, True, 5e8, 1e9) == 50.0 and sc.chinchilla_memory_correction(100.0, False, 5e8, 1e9) == 100.0
    assert sc.chinchilla_memory_correction(100.0, True, 1e6, 1e9) == 10.0
    op = G.PiscesLxScalingOperator()
    r = op.execute({"operation": "optimal", "compute_budget": 1e22})
    assert r.is_success(), r.error
    assert r.output["optimal_tokens"] == pytest.approx(20 * r.output["optimal_parameters"]) and 0 < r.output["compute_efficiency"] <= 1
    assert r.output["recommended_config"]["active_params"] > 0 and r.output["gpu_hours"] > 0
    assert op.execute({"operation": "estimate", "config": cfg}).output == cnt
    assert op.execute({"operation": "memory", "base_memory": 10, "optimal_params": 1, "original_params": 2}).output["memory_correction"] == 5.0
    assert not op.execute({"operation": "nope"}).is_success()
