"""CPU tests of the alternative MoE routers and the auxiliary KV-cache components."""
from __future__ import annotations

import math

import torch
import torch.nn as nn


def test_expert_choice_and_fine_grained_routers():
    from pisceslx_b200.models.routers import YvExpertChoiceRouter, YvFineGrainedRouter
    torch.manual_seed(0)
    x = torch.randn(64, 32)
    ec = YvExpertChoiceRouter(32, 8, capacity_factor=1.0, max_k=4)
    w, idx, aux = ec(x)
    assert w.shape == (64, 4) and (aux["tokens_per_expert"] == aux["tokens_per_expert"][0]).all()   # equal load
    assert ((w > 0).sum(-1) <= 4).all()
    fg = YvFineGrainedRouter(32, n_groups=4, n_sub=3, top_k=2)
    w, idx, aux = fg(x)
    assert idx.shape == (64, 2) and int(idx.max()) < 12 and torch.allclose(w.sum(-1), torch.ones(64))
    assert (idx[:, 0] // 3 != idx[:, 1] // 3).all()          # one sub-expert per chosen group
    assert float(aux["load_balance"]) > 0


def test_expert_oriented_path_gate_and_phi_balancing():
    from pisceslx_b200.models.routers import YvExpertOrientedRouter, YvPathMoEGate, YvPhiBalancing
    torch.manual_seed(1)
    x = torch.randn(128, 32)
    eo = YvExpertOrientedRouter(32, 8, top_k=2)
    eo.train()
    w, idx, aux = eo(x)
    assert aux["similarity"].abs().max() <= 1 + 1e-5 and abs(float(eo.load.sum()) - 1) < 1e-5
    calls = []

    class Inner(nn.Module):
        def forward(self, t):
            calls.append(1)
            return torch.ones(t.shape[0], 2), torch.zeros(t.shape[0], 2, dtype=torch.long), {}
    pg = YvPathMoEGate(Inner(), stage_size=3)
    for _ in range(7):
        pg(x)
    assert len(calls) == 3                                    # calls 1, 4, 7 route; the others reuse
    phi = YvPhiBalancing(4, lr=0.1, ema=0.5)
    skew = torch.tensor([0.7, 0.1, 0.1, 0.1])
    for _ in range(20):
        b = phi.update(skew)
    assert b[0] < 0 and (b[1:] > 0).all() and b.abs().max() <= 2.0
    logits = torch.log(skew) + b
    assert torch.softmax(logits, -1)[0] < 0.7                 # the bias pushes load off the hot expert


def test_modal_aware_and_ultra_sparse_gates():
    from pisceslx_b200.models.routers import YvModalAwareRouter, YvUltraSparseGate
    torch.manual_seed(2)
    x = torch.randn(40, 32)
    ma = YvModalAwareRouter(32, 8, top_k=2, n_modalities=3, n_cross=1)
    modal = torch.randint(0, 3, (40,))
    w, idx, _ = ma(x, modal)
    cross = modal == 2
    assert (idx[cross] == 7).any(-1).all()                    # the dedicated expert is always selected
    assert torch.allclose(w.sum(-1), torch.ones(40), atol=1e-5)
    w0, idx0, _ = ma(x)
    assert idx0.shape == (40, 2)
    us = YvUltraSparseGate(32, 8, tiers=(1, 2, 4), q1=0.5, q2=0.9)
    xs = torch.randn(200, 32)
    force = torch.zeros(200, dtype=torch.bool); force[:3] = True
    w, idx, aux = us(xs, force)
    live = (w.detach() > 0).sum(-1)
    assert torch.equal(live, aux["tier_k"]) and (aux["tier_k"][:3] == 4).all()
    assert 1.0 < float(aux["mean_k"]) < 2.5
    w.sum().backward()
    assert us.scorer[0].weight.grad is not None


def test_hicl_prototype_router_and_graph_of_tokens_router():
    from pisceslx_b200.models.routers import (YvDGEncoder, YvGraphOfTokensRouter, YvHiClRouter, YvRoMARegularizer,
                                              YvTokenGraphBuilder)
    torch.manual_seed(6)
    enc = YvDGEncoder(16, expansion=4, sparsity_k=5)
    c = enc(torch.randn(7, 16))
    assert c.shape == (7, 64) and ((c != 0).sum(-1) <= 5).all() and torch.allclose(c.norm(dim=-1), torch.ones(7), atol=1e-5)
    r = YvHiClRouter(16, 4, top_k=2, dg_sparsity_k=8, momentum=0.5)
    # two well separated token populations end up on different prototypes after a few EMA updates
    a, b = torch.randn(1, 16) + torch.zeros(40, 16), -(torch.randn(1, 16) + torch.zeros(40, 16))
    a, b = a + 0.05 * torch.randn_like(a), b + 0.05 * torch.randn_like(b)
    r.train()
    p0 = r.prototypes.clone()
    for _ in range(10):
        w, idx, aux = r(torch.cat([a, b]))
    assert not torch.equal(p0, r.prototypes) and torch.allclose(w.sum(-1), torch.ones(80), atol=1e-5)
    top = idx[:, 0]
    assert len(set(top[:40].tolist())) == 1 and len(set(top[40:].tolist())) == 1 and top[0] != top[40]
    assert aux["similarity"].abs().max() <= 1 + 1e-5
    # graph clustering: two constant phrases -> two clusters, each routed as a unit
    g = YvTokenGraphBuilder(16, max_clusters=4)
    x = torch.cat([torch.randn(1, 16).expand(5, -1), torch.randn(1, 16).expand(6, -1)])
    cid = g.clusters(x)
    assert cid[:5].unique().numel() == 1 and cid[5:].unique().numel() == 1 and cid[0] != cid[5]
    got = YvGraphOfTokensRouter(16, 8, top_k=2, max_clusters=4)
    w, idx, aux = got(x)
    assert aux["n_clusters"] == 2 and (idx[:5] == idx[0]).all() and (idx[5:] == idx[5]).all()
    assert torch.allclose(w.sum(-1), torch.ones(11), atol=1e-5)
    roma = YvRoMARegularizer(16, n_neighbors=2)
    probs = torch.softmax(torch.randn(6, 8), -1)
    assert float(roma(torch.randn(6, 16), probs)) > 0 and float(roma(torch.randn(6, 16), probs[:1].expand(6, -1))) < 1e-12


def test_triroute_and_brownout_grouper():
    from pisceslx_b200.serve.runtime import PiscesLxBrownoutMoEGrouper, PiscesLxTriRouteDecision
    torch.manual_seed(5)
    tr = PiscesLxTriRouteDecision(32, n_head=4, n_experts=8)
    out = tr(torch.randn(6, 32))
    assert out["attention_mode"].shape == (6, 4) and int(out["attention_mode"].max()) < 3
    assert set(out["kv_bits"].tolist()) <= {2, 4, 8, 16} and float(out["expert_logit_delta"].abs().max()) == 0.0
    c = tr.cost(out)
    c.backward()
    assert tr.mode_head.weight.grad is not None and 0 < float(c) < 2
    g = PiscesLxBrownoutMoEGrouper(8, group_size=2, threshold=0.5)
    # experts (0, 5), (1, 4), (2, 7), (3, 6) always fire together
    pairs = torch.tensor([[0, 5], [1, 4], [2, 7], [3, 6]])
    idx = pairs[torch.randint(0, 4, (200,))]
    g.fit(idx)
    assert sorted(map(tuple, g.groups)) == [(0, 5), (1, 4), (2, 7), (3, 6)]
    hot = pairs[torch.tensor([0] * 150 + [1] * 45 + [2] * 5)]          # pair (3, 6) never used, (2, 7) rarely
    for _ in range(40):
        g.observe(torch.full((200, 2), 0.5), hot)
    off = g.brownout(load_factor=1.0)
    off_groups = sorted(tuple(g.groups[i]) for i in off)
    assert off_groups == [(2, 7), (3, 6)]
    m = g.logit_mask()
    assert torch.isinf(m[[2, 7, 3, 6]]).all() and (m[[0, 5, 1, 4]] == 0).all()
    assert g.brownout(load_factor=0.0) == []                            # no load: everything stays on
    assert len(g.brownout(load_factor=100.0)) == 3                      # the most important group always stays


def test_kv_ring_and_lynx_quantizer():
    from pisceslx_b200.models.cache_extras import YvKVCacheRing, YvLynxKVQuantizer
    torch.manual_seed(3)
    ring = YvKVCacheRing(initial=4)
    ks = [torch.randn(2, 3, 8) for _ in range(6)]
    for k in ks:
        kk, vv = ring.append(k, k * 2)
    assert torch.equal(kk, torch.cat(ks, -2)) and torch.equal(vv, torch.cat(ks, -2) * 2)
    assert ring.reallocations <= 4                            # geometric growth: far fewer than one per append
    wrap = YvKVCacheRing(max_seq_len=8, initial=4)
    for k in ks:
        kk, _ = wrap.append(k, k)
    assert kk.shape[-2] == 8 and torch.equal(kk, torch.cat(ks, -2)[..., -8:, :])
    lq = YvLynxKVQuantizer(4, 4)
    kv = torch.randn(32, 64)
    c = lq.encode(kv)
    e_anchor = (lq.decode(c, refine=False) - kv).norm() / kv.norm()
    e_full = (lq.decode(c, refine=True) - kv).norm() / kv.norm()
    assert e_full < e_anchor / 4 and e_full < 0.02


def test_predictive_delta_coder_and_star_adapter():
    from pisceslx_b200.models.cache_extras import YvPredictiveDeltaCoder, YvSTARKVAdapter
    torch.manual_seed(4)
    W = torch.randn(8, 32) * 0.3
    h = torch.randn(256, 32)
    kv = h @ W.t() + 0.01 * torch.randn(256, 8)
    pdc = YvPredictiveDeltaCoder(32, 8, bits=4)
    q0, s0 = pdc.encode(kv, h)
    opt = torch.optim.Adam(pdc.parameters(), lr=0.05)
    for _ in range(150):
        opt.zero_grad()
        pdc.training_loss(kv, h).backward()
        opt.step()
    q1, s1 = pdc.encode(kv, h)
    assert float(s1.mean()) < float(s0.mean()) * 0.3          # a trained predictor leaves a much smaller residual
    rec = pdc.decode(q1, s1, h)
    assert float((rec - kv).abs().max()) < float(s1.max()) * 0.51 + 1e-6
    warm = YvPredictiveDeltaCoder(32, 8, warmup=True)
    assert torch.equal(warm.predict(h, kv), kv)
    ad = YvSTARKVAdapter(bits=8, keep=4, activate_after=16)
    assert not ad.update(0, torch.randn(8, 2, 4)) and ad.read(0) is None
    big = torch.randn(32, 2, 4)
    assert ad.update(0, big) and float((ad.read(0) - big).abs().max()) < 0.05


def test_plt_trie_and_multimodal_cache():
    from pisceslx_b200.models.cache_extras import YvMultimodalCacheManager, YvPLTTrieIndex
    trie = YvPLTTrieIndex(distance_threshold_bits=0.0, block_size=2)
    trie.insert([1, 2, 3, 4, 5], [-0.1] * 5, block_ids=[10, 11])
    m = trie.find_longest_match([1, 2, 3, 4, 9])
    assert m["block_ids"] == [10, 11] and m["matched_tokens"] == 4 and m["distance_bits"] == 0
    assert trie.find_longest_match([1, 2, 7, 4])["block_ids"] == [10]
    assert trie.find_longest_match([7, 7]) is None
    soft = YvPLTTrieIndex(distance_threshold_bits=8.0, block_size=2)
    soft.insert([1, 2, 3, 4], [-0.1] * 4, block_ids=[20, 21])
    lp = [-0.1, -0.1, math.log(0.05), -0.1]                   # the differing token costs about 4.3 bits
    assert soft.find_longest_match([1, 2, 9, 4], lp)["block_ids"] == [20, 21]
    lp[2] = math.log(0.001)                                   # about 10 bits: too far
    assert soft.find_longest_match([1, 2, 9, 4], lp)["block_ids"] == [20]
    trie.insert([6, 7], [-0.1, -0.1], block_ids=[30])
    trie.acquire([6, 7], 2)
    freed = trie.evict(1)
    assert freed == [] and trie.find_longest_match([1, 2, 3, 4]) is not None    # leaf 5 carried no block
    mm = YvMultimodalCacheManager({"image": 0.001})
    enc_calls = []

    def enc(t):
        enc_calls.append(1)
        return t.float().mean(0, keepdim=True).expand(64, -1).contiguous()
    img = torch.rand(4, 3)
    a = mm.get_or_encode("image", img, enc)
    b = mm.get_or_encode("image", img.clone(), enc)
    assert a is b and len(enc_calls) == 1 and mm.hits == 1
    mm.get_or_encode("image", torch.rand(4, 3), enc)
    assert len(mm.store["image"]) == 1                        # the 1 KB budget holds one 768-byte entry
