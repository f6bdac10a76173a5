"""CPU tests of the modules offered under the reference's names (fronts of this package's kernels and modules)."""
from __future__ import annotations

import torch
import torch.nn as nn

from pisceslx_b200 import YvConfig
from pisceslx_b200.models.compat import (YvCrossAttention, YvExpertChoiceMLP, YvFlashAttention, YvGateInitializer,
                                         YvLayerRouter, YvLoRALayer, YvModelForMaskedLM, YvMoELayer, YvPagedAttention,
                                         YvRingAttention, YvSelectiveScan, YvStateCache, YvSwiGLU)


def test_swiglu_flash_and_cross_attention():
    torch.manual_seed(0)
    x = torch.randn(2, 9, 32)
    ff = YvSwiGLU(32, 48)
    h = x @ ff.w13.t()
    assert torch.allclose(ff(x), (torch.nn.functional.silu(h[..., :48]) * h[..., 48:]) @ ff.w2.t(), atol=1e-5)
    fa = YvFlashAttention(32, 4, 2, causal=True)
    y = fa(x)
    x2 = x.clone(); x2[:, -1] += 1
    assert y.shape == x.shape and torch.allclose(fa(x2)[:, :-1], y[:, :-1], atol=1e-5)
    # against an explicit softmax with grouped KV heads
    qkv = x.reshape(18, 32) @ fa.qkv.t()
    q, k, v = qkv[:, :32].view(2, 9, 4, 8), qkv[:, 32:48].view(2, 9, 2, 8), qkv[:, 48:].view(2, 9, 2, 8)
    k, v = k.repeat_interleave(2, 2), v.repeat_interleave(2, 2)
    s = torch.einsum("bshd,bthd->bhst", q, k) * 8 ** -0.5
    s = s.masked_fill(~torch.tril(torch.ones(9, 9, dtype=torch.bool)), float("-inf"))
    ref = torch.einsum("bhst,bthd->bshd", torch.softmax(s, -1), v).reshape(2, 9, 32) @ fa.o.t()
    assert torch.allclose(y, ref, atol=1e-4)
    ca = YvCrossAttention(32, 20, 4)
    assert ca(x, torch.randn(2, 5, 20)).shape == x.shape


def test_paged_and_ring_attention_fronts():
    torch.manual_seed(1)
    hq, hk, d, bs = 4, 2, 8, 4
    pa = YvPagedAttention(hq, hk, d)
    kc, vc = torch.zeros(6, bs, hk, d), torch.zeros(6, bs, hk, d)
    ks, vs = torch.randn(5, hk * d), torch.randn(5, hk * d)
    table = torch.tensor([[2, 4]], dtype=torch.int32)
    for t in range(5):                                            # one sequence growing token by token over two blocks
        slot = torch.tensor([table[0, t // bs] * bs + t % bs], dtype=torch.int32)
        q = torch.randn(1, hq * d)
        o = pa(q, ks[t:t + 1], vs[t:t + 1], kc, vc, slot, table, torch.tensor([t + 1], dtype=torch.int32))
    kk = ks.view(5, hk, d).repeat_interleave(2, 1)
    vv = vs.view(5, hk, d).repeat_interleave(2, 1)
    p = torch.softmax(torch.einsum("hd,thd->ht", q.view(hq, d), kk) * d ** -0.5, -1)
    assert torch.allclose(o.view(hq, d), torch.einsum("ht,thd->hd", p, vv), atol=1e-5)
    ra = YvRingAttention(hq, hk, d)                               # no process group: plain attention over the shard
    qq, k2, v2 = torch.randn(7, hq * d), torch.randn(7, hk * d), torch.randn(7, hk * d)
    assert ra(qq, k2, v2).shape == (7, hq * d)


def test_expert_choice_mlp_layer_router_and_masked_lm():
    torch.manual_seed(2)
    ec = YvExpertChoiceMLP(16, 24, n_experts=4, capacity_factor=1.0)
    x = torch.randn(2, 8, 16)
    y = ec(x)
    assert y.shape == x.shape and torch.isfinite(y).all()
    y.sum().backward()
    assert ec.w13.grad is not None and ec.router.grad is not None
    lr = YvLayerRouter(16, n_layers=3)
    w = lr(x)
    assert w.shape == (2, 3) and (w > 0.9).all()                  # starts with every layer on
    upd = torch.ones_like(x)
    assert torch.allclose(lr.apply(x, upd, torch.zeros(2, 3), 1), x) and float(lr.budget_loss(w)) > 0
    hard = YvLayerRouter(16, 3, hard=True).eval()
    assert set(hard(x).unique().tolist()) <= {0.0, 1.0}
    cfg = YvConfig.tiny_text_moe(vocab_size=128)
    cfg.n_layer = 1
    mlm = YvModelForMaskedLM(cfg)
    ids = torch.randint(0, 128, (2, 10))
    labels = torch.full_like(ids, -100); labels[:, 3] = ids[:, 3]
    out = mlm(ids, labels=labels)
    assert out["logits"].shape == (2, 10, 128) and torch.isfinite(out["loss"])
    assert YvLoRALayer.__name__ == "YvLoRA" and YvMoELayer.__name__ == "YvDynamicMoELayer"


def test_selective_scan_front_state_cache_and_gate_initialisers():
    torch.manual_seed(3)
    b, l, dch, n = 2, 6, 4, 3
    u, dl = torch.randn(b, l, dch), torch.rand(b, l, dch) * 0.1
    A, B, C, D = -torch.rand(dch, n), torch.randn(b, l, n), torch.randn(b, l, n), torch.randn(dch)
    scan = YvSelectiveScan()
    full = scan(u, dl, A, B, C, D)
    cache = YvStateCache()
    st = cache.get(0, b, dch, n)
    steps = [scan.step(u[:, t:t + 1], dl[:, t:t + 1], A, B[:, t:t + 1], C[:, t:t + 1], D, st) for t in range(l)]
    assert torch.allclose(torch.cat(steps, 1), full, atol=1e-5) and cache.get(0, b, dch, n) is st
    before = st.clone()
    cache.reorder(torch.tensor([1, 0]))
    assert torch.equal(cache.states[0][0], before[1])
    cache.reset(row=0)
    assert float(cache.states[0][0].abs().sum()) == 0 and float(cache.states[0][1].abs().sum()) > 0
    w = nn.Parameter(torch.empty(4, 16))
    YvGateInitializer.orthogonal_(w, gain=1.0)
    assert torch.allclose(w.data @ w.data.t(), torch.eye(4), atol=1e-5)
    centers = torch.randn(4, 16) * 5
    samples = (centers[:, None, :] + 0.05 * torch.randn(4, 30, 16)).reshape(-1, 16)
    YvGateInitializer.kmeans_(w, samples, iters=15)
    assign = (torch.nn.functional.normalize(samples, dim=-1) @ torch.nn.functional.normalize(w.data, dim=-1).t()).argmax(-1).view(4, 30)
    assert all(assign[i].unique().numel() == 1 for i in range(4))        # every sample cluster is served by one gate row
