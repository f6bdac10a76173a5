"""Hessian collection, low-rank KV compression, sensitivity-driven mixed precision, quantisation benchmark operator, configs."""
import pytest
import torch
import torch.nn as nn

from pisceslx_b200.quant.advanced import (PiscesLxAdvancedQuantizationConfig, PiscesLxAdvancedQuantizer, PiscesLxBenchmarkConfig, PiscesLxGPTQHessianComputer,
                                          PiscesLxHyperQuantizer, PiscesLxQuantizationBenchmarkOperator, PiscesLxQuantizationEngineConfig,
                                          PiscesLxQuantizationPipelineConfig, PiscesLxSTARKVCompression, YvQuantizationType)


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a, self.b, self.lm_head = nn.Linear(16, 32), nn.Linear(32, 16), nn.Linear(16, 10)

    def forward(self, x, labels=None):
        y = self.lm_head(self.b(torch.relu(self.a(x))))
        return {"logits": y, "loss": nn.functional.cross_entropy(y.reshape(-1, 10), labels.reshape(-1))} if labels is not None else y


def test_hessian_is_two_over_n_xtx_and_factor_inverts_it():
    torch.manual_seed(0)
    net = _Net()
    data = [torch.randn(4, 5, 16) for _ in range(3)]
    hc = PiscesLxGPTQHessianComputer(damp_percent=0.01)
    hs = hc.compute_hessian(net, data)
    assert set(hs) == {"a", "b"} and hc.samples["a"] == 60
    x = torch.cat([d.reshape(-1, 16) for d in data])
    assert torch.allclose(hs["a"], 2.0 / 60 * x.t() @ x, atol=1e-4)
    hb = torch.cat([torch.relu(net.a(d)).reshape(-1, 32) for d in data]).detach()
    assert torch.allclose(hs["b"], 2.0 / 60 * hb.t() @ hb, atol=1e-4)
    assert len(hc.compute_hessian(net, data, num_samples=1, layers=["a"])) == 1 and hc.samples["a"] == 20
    assert not net.a._forward_pre_hooks                                                  # the hooks are gone
    d = hc.damped(hs["b"])
    assert (d.diagonal() > 0).all() and torch.allclose(d - torch.diag(d.diagonal()), hs["b"] - torch.diag(hs["b"].diagonal()))
    U = hc.inverse_cholesky(hs["a"])
    assert torch.allclose(U.t() @ U, torch.linalg.inv(hc.damped(hs["a"]).double()).float(), atol=1e-3) and torch.equal(U, U.triu())


def test_kv_compression_reconstructs_low_rank_heads_and_attends_without_rebuilding():
    torch.manual_seed(0)
    B, H, T, D, r = 2, 3, 40, 16, 3
    k = torch.randn(B, H, T, r) @ torch.randn(B, H, r, D)
    v = torch.randn(B, H, T, r) @ torch.randn(B, H, r, D)
    c = PiscesLxSTARKVCompression(D, compression_target=0.75, energy=0.999)
    pk, pv, rank = c.compress(k, v)
    assert c.max_rank == 4 and pk["coeff"].shape == (B, H, T, 4) and pk["basis"].shape == (B, H, D, 4) and (rank == r).all()
    k2, v2 = c.decompress(pk, pv)
    assert (k2 - k).norm() / k.norm() < 1e-3 and (v2 - v).norm() / v.norm() < 1e-3
    assert c.bytes_ratio(pk, T, D) == pytest.approx((T * 3 + D * 3) / (T * D))
    q = torch.randn(B, H, 5, D)
    ref = torch.softmax(q @ k.transpose(-1, -2) / D ** 0.5, -1) @ v
    assert torch.allclose(c.attend(q, pk, pv), ref, atol=1e-3)
    causal = c.attend(torch.randn(B, H, T, D), pk, pv, causal=True)
    assert causal.shape == (B, H, T, D) and torch.isfinite(causal).all()
    full = torch.randn(B, H, T, D)
    pf, _, rf = c.compress(full, full)
    assert (rf == 4).all() and 0.4 < (c.decompress(pf, pf)[0] - full).norm() / full.norm() < 1.0     # full-rank noise cannot be kept at rank 4


def test_advanced_quantizer_gives_sensitive_layers_more_bits():
    torch.manual_seed(0)
    net = _Net()
    with torch.no_grad():
        net.a.weight.mul_(1.0)
        net.b.weight[:, :2] *= 40.0                                                     # outlier columns: hard to quantise coarsely
    calib = [torch.randn(8, 16) for _ in range(4)]
    q = PiscesLxAdvancedQuantizer(PiscesLxAdvancedQuantizationConfig(target_compression_ratio=0.35, group_size=0, candidate_bits=(2, 4, 8)))
    sens = q.analyze_sensitivity(net, calib)
    assert set(sens) == {"a", "b"} and sens["b"] > sens["a"] > 0
    before = {n: m.weight.clone() for n, m in (("a", net.a), ("b", net.b))}
    out = PiscesLxAdvancedQuantizer.advanced_quantize(net, calib, q.config)
    assert out["allocation"]["b"] >= out["allocation"]["a"] and out["mean_bits"] <= 0.35 * 16 + 1e-9 and out["layers"] == 2
    assert not torch.equal(net.a.weight, before["a"]) and torch.equal(net.lm_head.weight, net.lm_head.weight)
    assert len(torch.unique(net.a.weight[0])) <= 2 ** out["allocation"]["a"]
    flat = PiscesLxAdvancedQuantizer(PiscesLxAdvancedQuantizationConfig(adaptive_bit_allocation=False, sensitivity_analysis=False)).quantize(_Net())
    assert set(flat["allocation"].values()) == {4}


def test_benchmark_operator_against_a_baseline(tmp_path):
    torch.manual_seed(0)
    net = _Net()
    cfg = PiscesLxBenchmarkConfig(batch_size=2, sequence_length=4, num_warmup_iterations=1, num_benchmark_iterations=5, vocab_size=16)
    op = PiscesLxQuantizationBenchmarkOperator(cfg)
    op.generate_test_inputs = lambda m: torch.randn(2, 4, 16)
    held = [{"x": torch.randn(3, 16), "labels": torch.randint(0, 10, (3,))} for _ in range(2)]
    base = op.execute({"model": net, "model_name": "fp", "heldout": held, "as_baseline": True}).output
    assert base["timing"] == "host" and base["latency"]["p95_ms"] >= base["latency"]["p50_ms"] and base["passes_quality_threshold"] and "perplexity" in base["accuracy"]
    with torch.no_grad():
        for p in net.parameters():
            p.add_(torch.randn_like(p))
    r = op.run_full_benchmark(net, "broken", "rtn", 2, held)
    assert "loss_increase" in r["comparison_with_baseline"] and r["comparison_with_baseline"]["memory_ratio"] == pytest.approx(1.0) and not r["passes_quality_threshold"]
    assert op.get_stats() == {"runs": 2, "has_baseline": True} and op.export_results(str(tmp_path / "b.json")).endswith("b.json")


def test_configs_and_names():
    e = PiscesLxQuantizationEngineConfig(method="awq", bits=3, mixed_precision=True, sensitive_layers=["layers.0.q"], preserve_accuracy_layers=["vision"])
    qc = e.to_quantization_config()
    assert qc.method.value == "awq" and qc.bits == 3 and "vision" in qc.skip and qc.per_layer_bits == {"layers.0.q": 8}
    p = PiscesLxQuantizationPipelineConfig(bits=4)
    assert p.resolved_method(True) == "gptq" and p.resolved_method(False) == "rtn" and PiscesLxQuantizationPipelineConfig(bits=6).resolved_method(True) == "awq"
    assert PiscesLxQuantizationPipelineConfig(method="smoothquant").resolved_method(False) == "smoothquant"
    assert YvQuantizationType("mx") is YvQuantizationType.MX and PiscesLxHyperQuantizer is not None
