"""CPU tests of the state-space variants and the manifold-constrained hyper-connections."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from pisceslx_b200.models.ssm_family import (YvAdaptiveDiscretization, YvBidirectionalSSM, YvComplexStateSpace,
                                             YvGatedSSM, YvHierarchicalSSM, YvMHC, YvMHCBlock, YvMHCLoss,
                                             YvMHCTransformer, YvMIMOStateSpace, YvMamba3Config, YvMamba3Decoder,
                                             YvMamba3Encoder, YvMamba3Integration, YvMamba3Stack,
                                             YvManifoldConstraint, YvMultiHeadSSM, YvSinkhornKnopp, YvSSDuality,
                                             YvSSMType, YvTrapezoidalDiscretization)


def _causal(mod, x, atol=1e-5):
    y = mod(x)
    x2 = x.clone(); x2[:, -1] += 1.0
    return torch.allclose(mod(x2)[:, :-1], y[:, :-1], atol=atol)


def test_discretisation_rules():
    a, b, dt = torch.tensor(-2.0), torch.tensor(1.0), torch.tensor(0.01)
    ab, bb = YvTrapezoidalDiscretization.discretize(a, b, dt)
    assert abs(float(ab) - math.exp(-0.02)) < 1e-6 and abs(float(bb) - 0.01 / 1.01) < 1e-9     # second-order match of exp
    assert abs(float(YvTrapezoidalDiscretization.discretize(torch.tensor(-1e4), b, torch.tensor(1.0))[0])) < 1.0   # stable
    ad = YvAdaptiveDiscretization(8, 1e-3, 0.1)
    dt = ad(torch.randn(2, 5, 8))
    assert dt.shape == (2, 5, 8) and dt.min() >= 1e-3 and dt.max() <= 0.1


def test_ssm_variants_shapes_and_causality():
    torch.manual_seed(0)
    x = torch.randn(2, 16, 32)
    kw = dict(state_dim=8)
    assert _causal(YvGatedSSM(32, **kw), x) and _causal(YvMultiHeadSSM(32, 4, **kw), x)
    assert _causal(YvHierarchicalSSM(32, (1, 4), **kw), x) and _causal(YvMamba3Integration(32, **kw), x)
    bi = YvBidirectionalSSM(32, **kw)
    assert bi(x).shape == x.shape and not _causal(bi, x)               # the reversed scan sees the future by design
    for t in YvSSMType:
        st = YvMamba3Stack(YvMamba3Config(hidden_size=32, state_dim=8, n_layers=2, ssm_type=t))
        assert st(x).shape == x.shape and torch.isfinite(st(x)).all()
    cfg = YvMamba3Config(hidden_size=32, state_dim=8, n_layers=1)
    assert isinstance(YvMamba3Encoder(cfg).layers[0], YvBidirectionalSSM) and isinstance(YvMamba3Decoder(cfg).layers[0], YvGatedSSM)
    assert _causal(YvMamba3Decoder(cfg), x)
    hs = YvHierarchicalSSM(32, (8,), **kw)
    assert float(hs(x)[:, :7].abs().sum()) == 0.0                      # no pooled block is complete before position 7


def test_complex_and_mimo_state_spaces_match_their_recurrences():
    torch.manual_seed(1)
    u = torch.randn(2, 24, 6)
    css = YvComplexStateSpace(6, state_dim=4)
    assert torch.allclose(css(u), css.recurrent(u), atol=1e-4) and _causal(css, u, 1e-4)
    mimo = YvMIMOStateSpace(6, 5, state_dim=3)
    y = mimo(u)
    decay = torch.sigmoid(mimo.a)
    h = torch.zeros(2, 3)
    ref = []
    for t in range(24):
        h = decay * h + u[:, t] @ mimo.B.t()
        ref.append(h @ mimo.C.t() + u[:, t] @ mimo.D.t())
    assert y.shape == (2, 24, 5) and torch.allclose(y, torch.stack(ref, 1), atol=1e-4)


def test_state_space_duality():
    torch.manual_seed(2)
    L, N = 12, 4
    a, b, c, u = torch.rand(L) * 0.8 + 0.1, torch.randn(L, N), torch.randn(L, N), torch.randn(L)
    assert torch.allclose(YvSSDuality.attention_form(a, b, c, u), YvSSDuality.recurrent_form(a, b, c, u), atol=1e-4)


def test_sinkhorn_manifold_and_hyper_connections():
    torch.manual_seed(3)
    P = YvSinkhornKnopp.project(torch.randn(5, 5), iters=50)
    assert torch.allclose(P.sum(0), torch.ones(5), atol=1e-4) and torch.allclose(P.sum(1), torch.ones(5), atol=1e-4) and P.min() > 0
    mc = YvManifoldConstraint(4)
    assert mc().diagonal().min() > 0.8                                  # starts near the identity
    hc = YvMHC(4)
    s = torch.randn(4, 2, 3, 8)
    out = hc(s, lambda t: torch.zeros_like(t))
    assert torch.allclose(out.sum(0), s.sum(0), atol=1e-4)              # doubly stochastic mixing conserves the stream sum
    blk = YvMHCBlock(nn.Linear(8, 8), nn.Linear(8, 8), 4)
    net = YvMHCTransformer([blk, YvMHCBlock(nn.Linear(8, 8), nn.Linear(8, 8), 4)], 4)
    x = torch.randn(2, 3, 8)
    y = net(x)
    assert y.shape == x.shape
    loss = YvMHCLoss()(net) + y.sum()
    loss.backward()
    assert blk.hc_f.mix.logits.grad is not None and torch.isfinite(loss)
