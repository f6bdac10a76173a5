"""Hybrid gate family, long-convolution and flash SSM forms, unified residual, mHC layer replacement."""
import inspect

import pytest
import torch
from torch import nn

from pisceslx_b200.models import hybrid_gates as hg
from pisceslx_b200.models.ssm import selective_scan_reference

H = 32


def test_progressive_gate_moves_from_fixed_to_learned_weights():
    torch.manual_seed(0)
    g = hg.YvProgressiveHybridGate(H, total_steps=4, sequence_threshold=16).eval()
    a, s, x = torch.randn(2, 8, H), torch.randn(2, 8, H), torch.randn(2, 8, H)
    out = g(a, s, x)
    assert torch.allclose(out["attention_weight"], torch.full((2,), 0.7)) and float(out["hybrid_ratio"]) == 0.0
    assert torch.allclose(out["fused_output"], 0.7 * a + 0.3 * s, atol=1e-6)
    long = g(torch.randn(2, 20, H), torch.randn(2, 20, H), torch.randn(2, 20, H))
    assert torch.allclose(long["ssm_weight"], torch.full((2,), 0.7))
    g.train()
    for _ in range(6):
        out = g(a, s, x)
    assert float(g.current_step) == 6.0 and float(out["hybrid_ratio"]) == pytest.approx(0.5)     # sigmoid(0) * min(1, 6/4)
    assert torch.allclose(out["attention_weight"] + out["ssm_weight"], torch.ones(2), atol=1e-6)
    assert not torch.allclose(out["attention_weight"], torch.full((2,), 0.7))
    out["fused_output"].sum().backward()
    assert g.hybrid_ratio.grad is not None and g.gate_proj[0].weight.grad is not None
    assert ".item()" not in inspect.getsource(hg._ScheduledWeights.blend)


def test_scheduled_fusion_takes_one_branch_when_sure():
    torch.manual_seed(0)
    f = hg.YvScheduledUnifiedFusion(H, total_steps=1).eval()
    a, s, x = torch.randn(3, 5, H), torch.randn(3, 5, H), torch.randn(3, 5, H)
    assert torch.allclose(f(a, s, x), 0.7 * a + 0.3 * s, atol=1e-6)
    with torch.no_grad():
        f.current_step.fill_(10.0)
        f.hybrid_ratio.fill_(20.0)                        # ratio -> 1: the learned weights alone
        f.gate[2].weight.zero_()
        f.gate[2].weight[0] = 50.0 * torch.sign(f.gate[0](f.content_encoder(x.mean(1))).mean(0).sign() + 0.5)
    out = f(a, s, x)
    w = torch.softmax(f.gate(f.content_encoder(x.mean(1))), -1)
    for b in range(3):
        if float(w[b, 0]) > 0.95:
            assert torch.equal(out[b], a[b])
        elif float(w[b, 1]) > 0.95:
            assert torch.equal(out[b], s[b])


def test_adaptive_router_routes_and_trains():
    torch.manual_seed(0)
    r = hg.YvAdaptiveRouter(H, 4, capacity_factor=1.0)
    x = torch.randn(2, 10, H)
    out, loss = r(x, lambda t: t * 2.0, lambda t: t * -1.0)
    ma, ms = r.last_masks
    assert tuple(out.shape) == (2, 10, H) and loss.ndim == 0 and float(loss) >= 0
    assert bool((ma | ms).all())                          # nothing passes through unprocessed
    assert int(ma.sum(-1).min()) >= r.capacity(10) and r.capacity(10) == 5
    assert not bool((ma & ms).all())                      # with factor 1 the branches share only some tokens
    (out.sum() + loss).backward()
    assert r.router.weight.grad is not None and float(r.router.weight.grad.abs().sum()) > 0
    both = hg.YvAdaptiveRouter(H, 4, capacity_factor=2.0)
    both(x, lambda t: t, lambda t: t)
    assert bool(both.last_masks[0].all()) and bool(both.last_masks[1].all())


def test_hierarchical_fusion_and_config():
    torch.manual_seed(0)
    f = hg.YvHierarchicalFusion(H, 3)
    a, s = torch.randn(2, 6, H), torch.randn(2, 6, H)
    assert tuple(f(a, s).shape) == (2, 6, H)
    cfg = hg.YvHybridConfig(hidden_size=H, fusion="progressive")
    assert isinstance(cfg.build_fusion(), hg.YvProgressiveHybridGate)
    assert isinstance(hg.YvHybridConfig(hidden_size=H, fusion="hierarchical").build_fusion(), hg.YvHierarchicalFusion)
    assert isinstance(hg.YvHybridConfig(hidden_size=H).build_fusion(), hg.YvScheduledUnifiedFusion)
    assert hg.YvHybridMode("routed") is hg.YvHybridMode.ROUTED


def test_vkernel_convolution_equals_its_recurrence():
    torch.manual_seed(0)
    v = hg.YvVKernel(H, 8).eval()
    x = torch.randn(2, 50, H)
    with torch.no_grad():
        conv, rec = v(x), v.recurrent_reference(x)
    assert torch.allclose(conv, rec, atol=1e-4)
    assert bool((v.decays() > 0).all() and (v.decays() < 1).all())
    k = v.kernel(50, x.device)
    assert v.kernel(20, x.device).data_ptr() == k.data_ptr()              # cached in evaluation
    y = x.clone()
    y[:, 30:] = 0
    assert torch.allclose(v(y)[:, :30], conv[:, :30], atol=1e-5)          # causal
    v.train()
    v(x).sum().backward()
    assert v.A_log.grad is not None and v.B.grad is not None and v._kernel_cache is None


def test_flash_ssm_matches_the_scan_oracle_and_its_own_decode_steps():
    torch.manual_seed(0)
    m = hg.YvFlashSSM(H, d_state=16).eval()
    x = torch.randn(2, 12, H)
    with torch.no_grad():
        full = m(x)
        u, delta, Bm, Cm = m._split(x)
        u = torch.nn.functional.conv1d(torch.nn.functional.pad(u.transpose(1, 2), (3, 0)), m.conv_weight.unsqueeze(1),
                                       m.conv_bias, groups=H).transpose(1, 2)
        ref = m.out_proj(selective_scan_reference(u, delta, -torch.exp(m.A_log), Bm, Cm, m.D)[0])
        cache = hg.YvStateCache(2, 16, H)
        steps = torch.cat([m.step(x[:, t:t + 1], cache) for t in range(12)], 1)
    assert torch.allclose(full, ref, atol=1e-5) and torch.allclose(steps, full, atol=1e-4)
    snap = cache.clone()
    cache.reset(torch.tensor([0]))
    assert float(cache.state[0].abs().sum()) == 0 and float(cache.state[1].abs().sum()) > 0
    assert torch.equal(snap.state[1], cache.state[1])
    m.train()
    m(x).sum().backward()
    assert m.A_log.grad is not None and m.conv_weight.grad is not None


def test_duality_layer_switches_form_by_length():
    torch.manual_seed(0)
    d = hg.YvSSDualityLayer(H, 16, threshold=8).eval()
    short, long_ = torch.randn(1, 8, H), torch.randn(1, 9, H)
    with torch.no_grad():
        assert torch.allclose(d(short), d.recurrent_mode(short)) and torch.allclose(d(long_), d.conv_mode(long_))


def test_unified_residual_parts():
    import types
    torch.manual_seed(0)
    cfg = types.SimpleNamespace(n_layer=8, extra={"residual_dropout": 0.0})
    r = hg.YvUnifiedResidual(H, 2, cfg)
    assert float(r.residual_scales[0]) == pytest.approx(16 ** -0.5)
    h, o = torch.randn(2, 4, H), torch.randn(2, 4, H)
    std = 0.25 * o
    want = h + std + (0.13 * std + 0.87 * h)
    assert torch.allclose(r(h, o, 0), want, atol=1e-6)                    # the mixing gate starts closed
    assert torch.allclose(r.forward_deepnorm(h, o, 1), 0.13 * std + 0.87 * h, atol=1e-6)
    with torch.no_grad():
        r.mhc_scale.fill_(1.0)
    mixed = r(h, o, 0)
    assert not torch.allclose(mixed, want)
    # a doubly stochastic mixing keeps the sum over the channel groups
    upd = h + std
    delta = (mixed - want).view(2, 4, r.n_hc, -1).sum(2)
    assert torch.allclose(delta, torch.zeros_like(delta), atol=1e-4)
    r(h, o, 0).sum().backward()
    assert r.mhc_mix.logits.grad is not None
    assert torch.allclose(r.forward_combined(h, o), r(h, o, 0))


def test_mhc_layer_replacement_keeps_the_sub_modules():
    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm1, self.attn = nn.LayerNorm(H), nn.Linear(H, H)
            self.norm2, self.mlp = nn.LayerNorm(H), nn.Sequential(nn.Linear(H, 2 * H), nn.GELU(), nn.Linear(2 * H, H))

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Block(), Block(), nn.Linear(H, H)])

    torch.manual_seed(0)
    m = Model()
    attn0 = m.layers[0].attn
    m, done = hg.YvMHCLayerReplacement.upgrade_transformer(m, n_streams=4)
    assert done == 2 and isinstance(m.layers[2], nn.Linear)              # a module without both parts is left alone
    assert m.layers[0].f[1] is attn0 and isinstance(m.layers[0].f[0], nn.LayerNorm)
    net = hg.YvMHCLayerReplacement.wrap(m.layers[:2], 4)
    x = torch.randn(2, 5, H)
    y = net(x)
    assert tuple(y.shape) == (2, 5, H)
    y.sum().backward()
    assert attn0.weight.grad is not None
