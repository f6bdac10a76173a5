"""ROOT optimizer / operator / scheduler and GaLore operator / adapter."""
import math

import pytest
import torch
import torch.nn as nn

from pisceslx_b200.optim import build_optimizer
from pisceslx_b200.optim.galore import (PiscesLxGaLoreConfig, PiscesLxGaLoreOperator, PiscesLxGaLoreOptimizerAdapter, basis_bytes,
                                        dequantize_basis, quantize_basis)
from pisceslx_b200.optim.root import (PiscesLxROOTConfig, PiscesLxROOTOperator, PiscesLxROOTOptimizer, PiscesLxROOTScheduler,
                                      compute_spectral_norm, orthogonalize_momentum, soft_threshold_denoise)


def test_root_config_validation():
    with pytest.raises(ValueError):
        PiscesLxROOTConfig(lr=-1)
    with pytest.raises(ValueError):
        PiscesLxROOTConfig(beta1=1.0)
    assert PiscesLxROOTConfig().to_dict()["orthogonalization_steps"] == 5


def test_orthogonalize_batched_and_spectral_norm():
    torch.manual_seed(0)
    x = torch.randn(3, 32, 48)
    o = orthogonalize_momentum(x, 8)
    s = torch.linalg.svdvals(o)
    assert s.max() < 1.3 and s.min() > 0.5
    assert torch.allclose(orthogonalize_momentum(x[1], 8), o[1], atol=1e-5)          # the stack is per matrix
    v = torch.randn(7)
    assert orthogonalize_momentum(v) is v
    m = torch.randn(2, 20, 30)
    sig, u = compute_spectral_norm(m, 60)
    assert torch.allclose(sig, torch.linalg.svdvals(m)[:, 0], rtol=1e-3)
    sig2, _ = compute_spectral_norm(m, 2, u)                                         # warm start holds the answer
    assert torch.allclose(sig2, sig, rtol=1e-4)


def test_soft_threshold_is_relative():
    x = torch.tensor([[3.0, -0.01, 0.02, -4.0]])
    y, kept = soft_threshold_denoise(x, 0.1)
    t = 0.1 * x.pow(2).mean().sqrt()
    assert torch.allclose(y, torch.tensor([[3.0 - t, 0.0, 0.0, -4.0 + t]]), atol=1e-6) and abs(float(kept) - 0.5) < 1e-6
    y2, _ = soft_threshold_denoise(x * 1e-3, 0.1)
    assert torch.allclose(y2, y * 1e-3, atol=1e-9)                                   # scale free


def test_root_optimizer_minimises_and_matches_single_matrix_path():
    torch.manual_seed(0)
    target = torch.randn(24, 32)
    ws = [nn.Parameter(torch.zeros(24, 32)) for _ in range(3)]
    b = nn.Parameter(torch.zeros(32))
    opt = PiscesLxROOTOptimizer(ws + [b], lr=0.02, min_dim_for_ortho=8)
    first = None
    for _ in range(150):
        opt.zero_grad()
        loss = sum(((w - target) ** 2).mean() for w in ws) + ((b - 1.0) ** 2).mean()
        loss.backward()
        opt.step()
        first = first or float(loss.detach())
    assert float(loss.detach()) < 0.1 * first
    assert torch.allclose(ws[0], ws[1], atol=1e-5)                                    # identical problems, identical trajectories in the stack
    assert set(opt.last_stats) >= {"kept", "spectral_norm", "orthogonalized"} and float(opt.last_stats["orthogonalized"]) == 3
    assert float(opt.last_stats["spectral_norm"]) <= 1.3
    # state round trip
    sd = opt.state_dict()
    opt2 = PiscesLxROOTOptimizer(ws + [b], lr=0.02, min_dim_for_ortho=8)
    opt2.load_state_dict(sd)
    assert opt2.state[ws[0]]["step"] == 150
    assert opt.get_config()["betas"] == (0.9, 0.999)


def test_root_flags_and_maximize():
    w = nn.Parameter(torch.ones(4, 4))
    opt = PiscesLxROOTOptimizer([w], lr=0.1, use_orthogonalization=False, use_soft_threshold=False, spectral_norm_clip=0.0, maximize=True, amsgrad=True)
    (w.sum()).backward()
    opt.step()
    assert (w > 1.0).all() and "max_exp_avg_sq" in opt.state[w]                       # plain Adam, ascending
    m = nn.Linear(8, 8)
    o = build_optimizer(m, "root", lr=1e-3)
    assert isinstance(o, PiscesLxROOTOptimizer)


def test_root_operator_functional_step():
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(16, 32), nn.Tanh(), nn.Linear(32, 4))
    x, y = torch.randn(64, 16), torch.randn(64, 4)
    op, state, cfg = PiscesLxROOTOperator(), {}, PiscesLxROOTConfig(lr=3e-3, min_dim_for_ortho=4)
    losses = []
    for _ in range(60):
        m.zero_grad()
        loss = ((m(x) - y) ** 2).mean()
        loss.backward()
        res = op.execute({"model": m, "config": cfg, "optimizer_state": state})
        assert res.is_success()
        state = res.output["optimizer_state"]
        losses.append(float(loss))
    assert losses[-1] < losses[0]
    st = res.output["statistics"]
    assert st["orthogonalized_params"] == 2 and st["total_params"] == 4 and res.output["orthogonalized_ratio"] == 0.5
    assert not op.execute({"model": None}).is_success()
    assert op._should_orthogonalize(torch.zeros(16, 16), cfg) and not op._should_orthogonalize(torch.zeros(16), cfg)
    g = {"0.weight": torch.zeros_like(m[0].weight)}
    op.execute({"model": m, "gradients": g, "config": cfg, "optimizer_state": state})
    assert m[0].weight.grad is g["0.weight"]


def test_root_scheduler_shapes_and_state():
    w = nn.Parameter(torch.zeros(2))
    opt = torch.optim.SGD([{"params": [w], "lr": 1.0}, {"params": [nn.Parameter(torch.zeros(1))], "lr": 0.5}])
    s = PiscesLxROOTScheduler(opt, warmup_steps=10, total_steps=110, min_lr=0.1, decay_type="cosine")
    lrs = [s.step() for _ in range(110)]
    assert abs(lrs[4] - 0.5) < 1e-9 and abs(lrs[9] - 1.0) < 1e-9 and abs(lrs[-1] - 0.1) < 1e-9
    assert abs(lrs[59] - (0.1 + 0.45 * (1 + math.cos(math.pi * 0.5)))) < 1e-9
    assert abs(opt.param_groups[1]["lr"] - 0.1) < 1e-9
    sd = s.state_dict()
    s2 = PiscesLxROOTScheduler(opt, decay_type="linear")
    s2.load_state_dict(sd)
    assert s2.current_step == 110 and s2.decay_type == "cosine" and s2.base_lrs == [1.0, 0.5]
    for kind, mid in (("linear", 0.55), ("exponential", 10 ** -0.5), ("constant", 1.0)):
        o = torch.optim.SGD([w], lr=1.0)
        k = PiscesLxROOTScheduler(o, warmup_steps=0, total_steps=100, min_lr=0.1, decay_type=kind)
        k.current_step = 49
        assert abs(k.step() - mid) < 1e-9
    with pytest.raises(ValueError):
        PiscesLxROOTScheduler(opt, decay_type="step")


def test_basis_quantisation_round_trip():
    torch.manual_seed(0)
    p = torch.linalg.qr(torch.randn(63, 5)).Q
    for bits, tol in ((8, 0.01), (4, 0.12)):
        q = quantize_basis(p, bits)
        d = dequantize_basis(q)
        assert d.shape == p.shape and (d - p).abs().max() < tol * p.abs().max() * 1.01 + 1e-6
    assert basis_bytes(quantize_basis(p, 4)) < basis_bytes(quantize_basis(p, 8)) < basis_bytes(p)


@pytest.mark.parametrize("proj_type", ["rand", "std"])
def test_projection_captures_low_rank_gradient(proj_type):
    torch.manual_seed(0)
    g = torch.randn(40, 4) @ torch.randn(4, 64) + 0.01 * torch.randn(40, 64)
    op = PiscesLxGaLoreOperator()
    cfg = PiscesLxGaLoreConfig(rank=4, proj_type=proj_type, quantization_bits=0)
    p = op._compute_projection_matrix(g, 4, cfg)
    assert p.shape == (64, 4) and torch.allclose(p.t() @ p, torch.eye(4), atol=1e-4)
    f = op._apply_galore_transform(g, p, cfg)
    assert (f - g).norm() / g.norm() < 0.05
    ref = torch.linalg.svd(g, full_matrices=False)[2][:4].t()
    assert torch.allclose(p @ p.t(), ref @ ref.t(), atol=2e-2)                       # the same subspace


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(32, 48), nn.Tanh(), nn.Linear(48, 8))


def test_galore_filter_mode_feeds_an_optimizer():
    m = _model()
    x, y = torch.randn(128, 32), torch.randn(128, 8)
    ad = PiscesLxGaLoreOptimizerAdapter(PiscesLxGaLoreConfig(rank=8, update_proj_gap=5, quantization_bits=8))
    opt = torch.optim.Adam(m.parameters(), lr=3e-3)
    losses = []
    for i in range(40):
        opt.zero_grad()
        loss = ((m(x) - y) ** 2).mean()
        loss.backward()
        raw = m[0].weight.grad.clone()
        _, st = ad.step(m)
        if i == 0:
            assert torch.linalg.matrix_rank(m[0].weight.grad) <= 8 and not torch.equal(raw, m[0].weight.grad)
            assert st["active_projections"] == 1 and st["refreshed_this_step"] == 1     # 48 x 8 has a short side of 8: left alone
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0] and st["step"] == 40
    assert ad.state["last_update_steps"]["0.weight"] == 36


def test_galore_lowrank_mode_trains_with_small_state_and_adapts_rank():
    m = _model()
    x, y = torch.randn(128, 32), torch.randn(128, 8)
    cfg = PiscesLxGaLoreConfig(rank=8, update_proj_gap=10, mode="lowrank", lr=1e-2, quantization_bits=4, rank_adapt_interval=20,
                               rank_adapt_threshold=0.05, min_rank=4, max_rank=16)
    ad = PiscesLxGaLoreOptimizerAdapter(cfg)
    rest = torch.optim.Adam(m.parameters(), lr=1e-2)
    losses, ranks = [], []
    for _ in range(60):
        rest.zero_grad()
        loss = ((m(x) - y) ** 2).mean()
        loss.backward()
        _, st = ad.step(m)
        assert m[0].weight.grad is None and m[2].weight.grad is not None
        rest.step()
        losses.append(float(loss))
        ranks.append(st["rank"])
    assert losses[-1] < 0.7 * losses[0]
    assert st["state_bytes_lowrank"] < st["state_bytes_full_adam"]
    assert ranks[-1] != 8 and 4 <= ranks[-1] <= 16 and "captured_energy" in ad.state
    sd = ad.state_dict()
    ad2 = PiscesLxGaLoreOptimizerAdapter(cfg)
    ad2.load_state_dict(sd, m)
    assert ad2.state["step"] == 60


def test_galore_config_and_expert_only():
    with pytest.raises(ValueError):
        PiscesLxGaLoreConfig(rank=0)
    with pytest.raises(ValueError):
        PiscesLxGaLoreConfig(mode="x")
    assert PiscesLxGaLoreConfig(use_int4_projection=True).quantization_bits == 4
    op = PiscesLxGaLoreOperator()
    assert op.validate_config(PiscesLxGaLoreConfig()) and not op.validate_config({})
    cfg = PiscesLxGaLoreConfig(rank=4, moe_expert_only=True)
    assert op._eligible("layers.0.experts.w1", torch.zeros(16, 16), cfg, 4) and not op._eligible("layers.0.attn.q", torch.zeros(16, 16), cfg, 4)
    assert not op.execute({"model": 3}).is_success()
