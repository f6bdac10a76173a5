"""Ink package around the optimizer: configuration, gradient compression with error feedback, checkpoint selection,
KV cache quantisation, expert residency, integrator transforms and the operator front."""
import pytest
import torch
from torch import nn

from pisceslx_b200.optim import ink_extras as ix


def test_config_validation_and_estimate():
    c = ix.PiscesLxInkConfig(momentum_bits=8, variance_bits=4, momentum_block_size=128, variance_block_size=256)
    assert c.get_memory_savings_ratio() == pytest.approx(1 - ((1 + 4 / 128) + (0.5 + 4 / 256)) / 8)
    for bad in ({"lr": -1}, {"betas": (1.0, 0.9)}, {"momentum_bits": 3}, {"sparse_ratio": 0.0}, {"gradient_block_size": 0}):
        with pytest.raises(ValueError):
            ix.PiscesLxInkConfig(**bad)
    d = ix.PiscesLxInkConfig.from_optimizer_config({"lr": 3e-4, "use_galore": True, "unknown": 1})
    assert d.lr == 3e-4 and d.use_galore and d.to_dict()["betas"] == [0.9, 0.999]


def test_nibble_packing_round_trip():
    q = torch.randint(-8, 8, (5, 12), dtype=torch.int8)
    p = ix.pack_nibbles(q)
    assert p.dtype == torch.uint8 and p.shape == (5, 6) and torch.equal(ix.unpack_nibbles(p), q)


@pytest.mark.parametrize("bits", [8, 4])
def test_gradient_compressor_dense_and_error_feedback(bits):
    g = torch.Generator().manual_seed(0)
    comp = ix.PiscesLxInkGradientCompressor(bits, 64, stochastic_rounding=True, generator=g)
    grad = torch.randn(37, 50)
    pay = comp.compress(grad)
    rec = comp.decompress(pay)
    assert rec.shape == grad.shape and float((rec - grad).abs().max()) <= float(grad.abs().max()) / (127 if bits == 8 else 7) * 1.01
    ratio = grad.numel() * 4 / comp.payload_bytes(pay)
    assert ratio > (3.5 if bits == 8 else 6.5)
    # with a key, the sum of what is sent over many rounds tracks the sum of the gradients
    sent, true = torch.zeros_like(grad), torch.zeros_like(grad)
    for _ in range(30):
        gi = torch.randn(37, 50) * 0.1 + 0.02
        true += gi
        sent += comp.decompress(comp.compress(gi, key="w"))
    assert float((sent - true).abs().max()) <= comp.residual_norm("w") + 1e-4
    assert float((sent - true).norm() / true.norm()) < 0.05
    st = comp.get_statistics()
    assert st["total_compressions"] == 31 and st["avg_compression_ratio"] > 3
    other = ix.PiscesLxInkGradientCompressor()
    other.load_state_dict(comp.state_dict())
    assert other.gradient_bits == bits and other.residual_norm("w") == pytest.approx(comp.residual_norm("w"))


def test_gradient_compressor_sparse_keeps_the_largest_and_remembers_the_rest():
    comp = ix.PiscesLxInkGradientCompressor(8, 32, stochastic_rounding=False)
    grad = torch.zeros(1000)
    grad[[3, 500, 900]] = torch.tensor([5.0, -7.0, 6.0])
    grad += torch.randn(1000) * 0.01
    pay = comp.compress_sparse(grad, 0.003, key="g")
    rec = comp.decompress(pay)
    assert pay["count"] == 3 and set(rec.nonzero().flatten().tolist()) == {3, 500, 900}
    assert torch.allclose(rec[[3, 500, 900]], grad[[3, 500, 900]], atol=0.06)
    assert comp.residual_norm("g") > 0
    # the remembered small entries come back once they accumulate
    total = rec.clone()
    for _ in range(200):
        total += comp.decompress(comp.compress_sparse(torch.zeros(1000), 0.05, key="g"))
    assert float((total - grad).norm()) < 0.25 * float((rec - grad).norm())


class Block(nn.Module):
    def __init__(self, h, f):
        super().__init__()
        self.a, self.b = nn.Linear(h, f), nn.Linear(f, h)

    def forward(self, x):
        return x + self.b(torch.relu(self.a(x)))


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = nn.Linear(8, 32)
        self.layers = nn.ModuleList([Block(32, 64), Block(32, 256), Block(32, 64), Block(32, 256)])
        self.head = nn.Linear(32, 4)

    def forward(self, x):
        x = self.embed(x)
        for l in self.layers:
            x = l(x)
        return self.head(x)


def test_checkpoint_selector_picks_by_cost_and_keeps_the_numbers():
    torch.manual_seed(0)
    net = Net()
    sel = ix.PiscesLxInkCheckpointSelector(checkpoint_ratio=0.5, activation_size_threshold=0)
    info = sel.analyze_model(net, tokens=128)
    assert info["total_layers"] == 4 and set(info["layer_info"]) == {"layers.0", "layers.1", "layers.2", "layers.3"}
    chosen = sel.get_checkpoint_layers()
    assert chosen == {"layers.0", "layers.2"}                    # same activation width, a quarter of the recomputation
    x = torch.randn(16, 8)
    net(x).sum().backward()
    ref = [p.grad.clone() for p in net.parameters()]
    net.zero_grad()
    calls = {"n": 0}
    assert sel.apply_checkpoint(net, lambda f, *a, **k: (calls.__setitem__("n", calls["n"] + 1), torch.utils.checkpoint.checkpoint(f, *a, use_reentrant=False, **k))[1]) == 2
    assert sel.apply_checkpoint(net) == 2                         # idempotent
    net(x).sum().backward()
    assert calls["n"] == 2 and all(torch.allclose(a, p.grad, atol=1e-6) for a, p in zip(ref, net.parameters()))
    net.eval()
    net(x)
    assert calls["n"] == 2                                        # no recomputation outside training
    est = sel.estimate_memory_savings(net, 4, 32)
    assert est["checkpoint_layers"] == 2 and 0 < est["savings_percent"] < 100 and est["extra_flops"] > 0
    assert sel.remove_checkpoint(net) == 2
    big_only = ix.PiscesLxInkCheckpointSelector(1.0, activation_size_threshold=1 << 40)
    big_only.analyze_model(net)
    assert big_only.get_checkpoint_layers() == set()
    act = torch.randn(3, 100)
    c = sel.compress_activation(act)
    assert float((sel.recompute_activation(c) - act).abs().max()) < float(act.abs().max()) / 127 + 1e-6
    s2 = ix.PiscesLxInkCheckpointSelector()
    s2.load_state_dict(sel.state_dict())
    assert s2.checkpoint_ratio == 0.5


@pytest.mark.parametrize("bits,tol,ratio", [(8, 0.02, 1.5), (4, 0.25, 2.7)])
def test_kv_cache_quantizer(bits, tol, ratio):
    torch.manual_seed(0)
    q = ix.PiscesLxInkKVCacheQuantizer(bits, block_size=16)
    k = torch.randn(2, 4, 50, 32, dtype=torch.bfloat16)
    k[..., 5] *= 20                                               # an outlier channel must not hurt the others
    v = torch.randn(2, 4, 50, 32, dtype=torch.bfloat16)
    ck, cv = q.quantize_k(k), q.quantize_v(v)
    dk, dv = q.dequantize_k(ck), q.dequantize_v(cv)
    assert dk.shape == k.shape and dv.dtype == torch.bfloat16
    others = [c for c in range(32) if c != 5]
    rel = lambda a, b: float((a.float() - b.float()).norm() / b.float().norm())
    assert rel(dk[..., others], k[..., others]) < tol and rel(dv, v) < tol
    q.store("l0", k, v)
    s = q.get_memory_savings()
    assert s["compression_ratio"] > ratio and q.get_cache_size("l0")["stored_bytes"] == s["stored_bytes"]
    a, b = q.load("l0")
    assert torch.equal(a, dk) and torch.equal(b, dv)
    q.clear_cache()
    assert q.get_cache_size()["stored_bytes"] == 0


def test_moe_manager_keeps_the_hot_experts_resident():
    moves = []
    m = ix.PiscesLxInkMoEManager(max_experts_on_gpu=2, device="gpu", host="cpu", mover=lambda mod, d: moves.append((mod.tag, d)))
    for e in range(4):
        mod = nn.Linear(4, 4)
        mod.tag = e
        m.register_expert(e, mod)
    for e in (0, 1, 0, 2):
        m.record_access(e)
        m.load_expert(e)
    assert m.get_active_experts() == {0, 2} and moves == [(0, "gpu"), (1, "gpu"), (1, "cpu"), (2, "gpu")]
    assert m.should_offload(0) and not m.should_offload(2) and not m.load_expert(99)
    st = m.get_statistics()
    assert (st["hits"], st["misses"], st["loads"], st["offloads"]) == (1, 3, 3, 1)
    for _ in range(10):
        m.record_access(3)
    assert m.get_overutilized_experts() == [3] and 1 in m.get_underutilized_experts()
    ch = m.dynamic_manage()
    assert 3 in m.get_active_experts() and 3 in ch["loaded"] and len(m.get_active_experts()) <= 2
    fp = m.get_memory_footprint()
    assert fp["resident_experts"] == len(m.get_active_experts()) and fp["total_mb"] > fp["gpu_mb"] > 0
    m2 = ix.PiscesLxInkMoEManager(2, device="gpu", mover=lambda mod, d: None)
    for e in range(4):
        m2.register_expert(e, nn.Linear(4, 4))
    m2.load_state_dict(m.state_dict())
    assert m2.get_active_experts() == m.get_active_experts()


def test_integrator_transforms_are_switchable():
    torch.manual_seed(0)
    off = ix.PiscesLxInkIntegrator(ix.PiscesLxInkConfig())
    g = torch.randn(64, 48)
    assert off.apply_galore("w", g)[1] is None and off.apply_root_ortho(g) is g and off.apply_fp4_forward("w", g) is g
    on = ix.PiscesLxInkIntegrator(ix.PiscesLxInkConfig(use_galore=True, galore_rank=8, use_fp4=True, use_root_ortho=True,
                                                       root_spectral_norm_clip=0.5, fp4_stochastic_rounding=False))
    on.initialize()
    low, back = on.apply_galore("w", g)
    assert low.shape == (64, 8) and back(low).shape == g.shape           # the short side is projected
    assert on.apply_galore("bias", torch.randn(48))[1] is None
    w = nn.Parameter(torch.randn(32, 32))
    wq = on.apply_fp4_forward("w", w)
    assert not torch.equal(wq, w) and 0 < on.get_fp4_state("w")["error"] < 0.2
    wq.sum().backward()
    assert torch.equal(w.grad, torch.ones_like(w))                # straight through
    o = on.apply_root_ortho(g)
    sv = torch.linalg.svdvals(o.float())
    assert float(sv.max()) < 1.6 and float(sv.min()) > 0.3
    spiky = torch.randn(32, 32) * 0.01
    spiky[3, 4] = 50.0
    den = on.apply_root_denoise(spiky)
    assert float(den[3, 4]) < 50.0 and torch.equal(den[0], spiky[0])
    clipped = on.apply_root_spectral_clip(g)
    assert float(torch.linalg.svdvals(clipped.float()).max()) <= 0.5 * 1.05
    st = on.get_statistics()["calls"]
    assert st["galore"] == 1 and st["ortho"] == 1 and st["clip"] == 1 and on.get_component_status()["initialized"]
    fresh = ix.PiscesLxInkIntegrator(on.config)
    fresh.load_state_dict(on.state_dict())
    assert torch.equal(fresh.get_galore_state("w")["P"], on.get_galore_state("w")["P"])


def test_operator_trains_a_model_with_small_state():
    torch.manual_seed(0)
    net = Net()
    op = ix.PiscesLxInkOperator(ix.PiscesLxInkConfig(lr=1e-2, weight_decay=0.0, max_grad_norm=1.0, variance_bits=8))
    assert not op.execute({"action": "step"})["success"]          # not initialised yet
    op.initialize(net, apply_checkpoint=True)
    x, y = torch.randn(64, 8), torch.randint(0, 4, (64,))
    losses = []
    for _ in range(40):
        op.execute({"action": "zero_grad"})
        loss = nn.functional.cross_entropy(net(x), y)
        loss.backward()
        losses.append(float(loss))
        r = op.execute({"action": "step"})
        assert r["success"]
    assert losses[-1] < 0.7 * losses[0]
    mem = op.execute({"action": "memory"})["output"]
    assert mem["state_bytes"] < 0.45 * mem["fp32_adam_state_bytes"]
    st = op.execute({"action": "statistics"})["output"]
    assert st["steps"] == 40 and st["checkpoint"]["checkpoint_layers"] == 2 and st["last_grad_norm"] > 0
    assert not op.execute({"action": "dance"})["success"]
    sd = op.state_dict()
    op2 = ix.PiscesLxInkOperator(op.config)
    op2.initialize(Net())
    op2.load_state_dict(sd)
    assert op2.get_statistics()["steps"] == 40
