"""K-FAC operator: exact Kronecker inverse in the eigenbasis, bias handling, functional capture, damping, selection."""
import pytest
import torch
from torch import nn

from pisceslx_b200.ops import functional as F_
from pisceslx_b200.optim.kfac import (PiscesLxKFacConfig, PiscesLxKFacFacade, PiscesLxKFacLayerType, PiscesLxKFacOperator)


def _net():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(6, 5), nn.Tanh(), nn.Linear(5, 3))


def test_preconditioned_gradient_is_the_damped_kronecker_inverse():
    net = _net()
    op = PiscesLxKFacOperator(PiscesLxKFacConfig(damping=1e-2, momentum=0.0, warmup_steps=0, update_freq=1, include_bias=True,
                                                 adaptive_damping=False, clip_gradients=False, keep_gradient_norm=False))
    assert len(op.register_hooks(net)) == 4 and op.layer_info["0"]["type"] is PiscesLxKFacLayerType.LINEAR
    x, y = torch.randn(32, 6), torch.randn(32, 3)
    nn.functional.mse_loss(net(x), y).backward()
    raw_w, raw_b = net[0].weight.grad.clone(), net[0].bias.grad.clone()
    nb, na = op.precondition_gradients()
    cov = op.get_covariance_matrices()["0"]
    A, G = cov["A"], cov["G"]
    assert A.shape == (7, 7) and G.shape == (5, 5)                                 # the bias adds a homogeneous coordinate
    K = torch.kron(G.double(), A.double()) + 1e-2 * torch.eye(35, dtype=torch.double)
    full = torch.cat([raw_w, raw_b[:, None]], 1).double().reshape(-1)              # row-major vec pairs with kron(G, A)
    want = torch.linalg.solve(K, full).reshape(5, 7).float()
    assert torch.allclose(net[0].weight.grad, want[:, :6], atol=1e-4, rtol=1e-3)
    assert torch.allclose(net[0].bias.grad, want[:, 6], atol=1e-4, rtol=1e-3)
    assert float(nb) > 0 and float(na) > 0 and 0 < op.get_statistics()["curvature_factor"] < 1


def test_warmup_norm_keeping_and_adaptive_damping():
    net = _net()
    op = PiscesLxKFacOperator(PiscesLxKFacConfig(damping=1e-3, warmup_steps=2, update_freq=1, clip_gradients=False))
    op.register_hooks(net)
    x, y = torch.randn(16, 6), torch.randn(16, 3)
    for step in range(4):
        net.zero_grad()
        nn.functional.mse_loss(net(x), y).backward()
        raw = net[2].weight.grad.clone()
        nb, na = op.precondition_gradients()
        if step < 2:
            assert torch.equal(net[2].weight.grad, raw) and float(nb) == 0          # statistics only
        else:
            assert not torch.allclose(net[2].weight.grad, raw)
            assert float(net[2].weight.grad.norm()) == pytest.approx(float(raw.norm()), rel=1e-4)
    assert op.damping > 1e-3                                                       # the raw natural gradient was far larger
    low = PiscesLxKFacOperator(PiscesLxKFacConfig(damping=0.5, damping_upper_bound=1.0))
    low._update_adaptive_damping(torch.tensor(1.0), torch.tensor(0.1))
    assert low.damping == pytest.approx(0.5 * 0.95)
    with pytest.raises(ValueError):
        PiscesLxKFacConfig(momentum=1.0)
    with pytest.raises(ValueError):
        PiscesLxKFacConfig(damping=2.0)


def test_selection_exclusion_diag_and_embedding():
    torch.manual_seed(0)

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(11, 6)
            self.enc, self.head, self.skip = nn.Linear(6, 6), nn.Linear(6, 4), nn.Linear(6, 6)

        def forward(self, ids):
            h = self.emb(ids)
            return self.head(torch.tanh(self.enc(h)) + 0 * self.skip(h))

    m = M()
    op = PiscesLxKFacOperator(PiscesLxKFacConfig(layer_exclusion=["skip"], include_embedding=True, diag_first=True, warmup_steps=0,
                                                 update_freq=1, momentum=0.0, clip_gradients=False))
    op.register_hooks(m)
    assert set(op.layer_info) == {"emb", "enc", "head"} and op.layer_info["emb"]["type"] is PiscesLxKFacLayerType.EMBEDDING
    ids = torch.randint(0, 11, (8, 5))
    m(ids).pow(2).mean().backward()
    raw = m.emb.weight.grad.clone()
    op.precondition_gradients()
    assert op.cov_a["enc"].dim() == 1 and op.cov_a["emb"].shape == (11,) and bool(torch.isfinite(m.emb.weight.grad).all())
    unseen = (torch.bincount(ids.reshape(-1), minlength=11) == 0)
    assert float(m.emb.weight.grad[unseen].abs().sum()) == 0 and not torch.allclose(m.emb.weight.grad, raw)
    only = PiscesLxKFacOperator(PiscesLxKFacConfig(layer_selection=["he*"]))
    only.register_hooks(M())
    assert set(only.layer_info) == {"head"}


def test_functional_capture_sees_bare_parameters():
    torch.manual_seed(0)
    w1, w2 = nn.Parameter(torch.randn(5, 6) * 0.3), nn.Parameter(torch.randn(3, 5) * 0.3)
    op = PiscesLxKFacOperator(PiscesLxKFacConfig(warmup_steps=0, update_freq=1, momentum=0.0, clip_gradients=False, keep_gradient_norm=False,
                                                 damping=1e-2, adaptive_damping=False))
    assert op.register_functional({"w1": w1, "w2": w2, "vec": nn.Parameter(torch.randn(4))}) == 2
    x, y = torch.randn(20, 6), torch.randn(20, 3)
    orig = F_.linear
    with op.capture():
        loss = nn.functional.mse_loss(F_.linear(torch.tanh(F_.linear(x, w1)), w2), y)
    assert F_.linear is orig                                                       # restored on exit
    loss.backward()
    raw = w1.grad.clone()
    op.precondition_gradients()
    cov = op.get_covariance_matrices()
    assert set(cov) == {"w1", "w2"} and cov["w1"]["A"].shape == (6, 6) and cov["w1"]["G"].shape == (5, 5)
    K = torch.kron(cov["w1"]["G"].double(), cov["w1"]["A"].double()) + 1e-2 * torch.eye(30, dtype=torch.double)
    want = torch.linalg.solve(K, raw.double().reshape(-1)).reshape(5, 6).float()
    assert torch.allclose(w1.grad, want, atol=1e-4, rtol=1e-3)


def test_natural_gradient_beats_plain_descent_on_a_badly_conditioned_problem():
    def run(use_kfac):
        torch.manual_seed(0)
        lin = nn.Linear(8, 1, bias=False)
        scale = torch.logspace(0, 2, 8)                                            # input scales from 1 to 100
        X = torch.randn(256, 8) * scale
        target = X @ torch.ones(8, 1) / scale.mean()
        opt = torch.optim.SGD(lin.parameters(), lr=1e-4 if not use_kfac else 0.2)
        k = PiscesLxKFacFacade(lin, warmup_steps=0, update_freq=1, momentum=0.5, damping=1e-4, adaptive_damping=False,
                               clip_gradients=False, keep_gradient_norm=False) if use_kfac else None
        for _ in range(60):
            opt.zero_grad()
            loss = nn.functional.mse_loss(lin(X), target)
            loss.backward()
            if k:
                k.precondition_gradients()
            opt.step()
        if k:
            st = k.get_statistics()
            assert st["updates"] == 60 and st["observed"] == 1
            k.cleanup()
        return float(nn.functional.mse_loss(lin(X), target))
    assert run(True) < 0.05 * run(False)


def test_operator_front():
    net = _net()
    op = PiscesLxKFacOperator(PiscesLxKFacConfig(warmup_steps=0, update_freq=5))
    assert op.execute({"action": "register", "model": net}).output == {"hooks": 4, "layers": 2}
    nn.functional.mse_loss(net(torch.randn(8, 6)), torch.randn(8, 3)).backward()
    r = op.execute({"action": "precondition"})
    assert r.is_success() and r.output["step"] == 1 and float(r.output["norm_before"]) > 0
    assert op.execute({"action": "update"}).output == {"refreshed": 2}
    assert op.execute({"action": "statistics"}).output["layers"] == 2
    op.execute({"action": "reset"})
    assert op.steps == 0 and not op.cov_a and not op.execute({"action": "dance"}).is_success()
    op.remove_hooks()
