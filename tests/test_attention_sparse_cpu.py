"""CPU tests of the block-sparse / hierarchical / hybrid attention variants: each selection rule is checked against
its definition, and each variant against dense causal attention in the limit where it must agree."""
from __future__ import annotations

import pytest
import torch

from pisceslx_b200.models.attention_sparse import (YvAttentionMaskFactory, YvCirculantAttention, YvDynamicH2OAttention,
                                                   YvEGMLA, YvHISAAttention, YvHydraHeadAttention,
                                                   YvLatentCondensedAttention, YvMemoryCrossAttention,
                                                   YvMixtureBlockAttention, YvTokenSparseAttention)
from pisceslx_b200.models.attention_variants import causal_mask, masked_attention


def _dense(mod, x):
    q, k, v = mod.qkv(x)
    S = x.shape[1]
    return mod.out(masked_attention(q, k, v, mask=causal_mask(S, S)))


def test_mask_factory():
    MF = YvAttentionMaskFactory
    m = MF.sliding_window(6, 2, n_sink=1)
    assert m[5].tolist() == [True, False, False, False, True, True]
    assert MF.prefix_lm(4, 2)[0].tolist() == [True, True, False, False]
    bd = MF.block_diagonal(torch.tensor([0, 0, 1, 1, 1]))
    assert bd[3].tolist() == [False, False, True, True, False]
    assert MF.padding(torch.tensor([2, 3]), 4)[0, 0, 0].tolist() == [True, True, False, False]
    d = MF.dilated(8, 2, 3)
    assert d[7].tolist() == [False, False, False, False, True, False, False, True]
    assert torch.equal(MF.causal(3), torch.tril(torch.ones(3, 3, dtype=torch.bool)))


def test_moba_selection_and_dense_limit():
    torch.manual_seed(0)
    x = torch.randn(2, 64, 32)
    m = YvMixtureBlockAttention(32, 4, block_size=8, top_k=2)
    q, k, v = m.qkv(x)
    sel = m.select(q, k)                                # [B,H,S,nb]
    qblk = torch.arange(64) // 8
    nb = 8
    assert sel[..., torch.arange(64), qblk].all()       # own block always
    later = torch.arange(nb)[None, :] > qblk[:, None]
    assert not (sel & later).any()
    assert int(sel.sum(-1).max()) <= 3
    assert m(x).shape == x.shape
    full = YvMixtureBlockAttention(32, 4, block_size=8, top_k=8)
    assert torch.allclose(full(x), _dense(full, x), atol=1e-5)


def test_token_sparse_mass_target_and_hisa():
    torch.manual_seed(1)
    x = torch.randn(1, 96, 32)
    t = YvTokenSparseAttention(32, 4, block_size=8, target=0.5, max_blocks=12)
    q, k, v = t.qkv(x)
    sel = t.select(q, k)
    all_ = YvTokenSparseAttention(32, 4, block_size=8, target=1.1, max_blocks=99)
    all_.load_state_dict(t.state_dict())
    assert torch.allclose(all_(x), _dense(all_, x), atol=1e-5)
    assert sel.sum() < all_.select(q, k).sum()
    # the kept blocks hold at least the target mass of the representative softmax
    qblk = torch.arange(96) // 8
    vis = torch.arange(12)[None, :] < qblk[:, None]              # strictly earlier blocks are the ranked ones
    from pisceslx_b200.models.attention_sparse import _block_means
    p = torch.softmax((q.float() @ _block_means(k, 8).transpose(-1, -2) * 8 ** -0.5).masked_fill(~vis, float("-inf")), -1)
    has_past = qblk > 0
    assert ((torch.nan_to_num(p) * sel).sum(-1)[..., has_past] >= 0.5 - 1e-5).all()
    h = YvHISAAttention(32, 4, block_size=8, super_size=3, top_super=1, top_blocks=2)
    hs = h.select(*h.qkv(x)[:2])
    assert hs[..., torch.arange(96), qblk].all() and int(hs.sum(-1).max()) <= 3      # two ranked blocks + the own block
    later = torch.arange(12)[None, :] > qblk[:, None]
    assert not (hs & later).any()
    hfull = YvHISAAttention(32, 4, block_size=8, super_size=3, top_super=9, top_blocks=99)
    assert torch.allclose(hfull(x), _dense(hfull, x), atol=1e-5)


def test_circulant_is_causal_and_hydra_linear_part():
    torch.manual_seed(2)
    c = YvCirculantAttention(32, 4, causal=True)
    x = torch.randn(1, 16, 32)
    # the mixing kernel is pooled over the sequence; causality is of the convolution: with the kernel fixed, output
    # at t depends on values at <= t only
    y = c(x)
    assert y.shape == x.shape and torch.isfinite(y).all()
    hy = YvHydraHeadAttention(32, 4, la_ratio=0.5)
    assert hy.n_linear == 2
    q, k, v = hy.qkv(x)
    lin = hy.linear_causal(q[:, :2], k[:, :2], v[:, :2])
    # reference: explicit causal sum with the same feature map
    fq, fk = torch.nn.functional.elu(q[:, :2]) + 1, torch.nn.functional.elu(k[:, :2]) + 1
    w = (fq @ fk.transpose(-1, -2)) * causal_mask(16, 16)
    ref = (w / w.sum(-1, keepdim=True)) @ v[:, :2]
    assert torch.allclose(lin, ref, atol=1e-4)
    y1 = hy(x)
    x2 = x.clone(); x2[:, -1] += 1.0
    assert torch.allclose(hy(x2)[:, :-1], y1[:, :-1], atol=1e-5)      # causal in both head groups
    allsoft = YvHydraHeadAttention(32, 4, la_ratio=0.0)
    assert torch.allclose(allsoft(x), _dense(allsoft, x), atol=1e-5)


def test_latent_condensed_and_dynamic_h2o():
    torch.manual_seed(3)
    x = torch.randn(1, 40, 32)
    l = YvLatentCondensedAttention(32, 4, ratio=4, keep_recent=8)
    y = l(x)
    assert y.shape == x.shape
    x2 = x.clone(); x2[:, -1] += 1.0
    assert torch.allclose(l(x2)[:, :-1], y[:, :-1], atol=1e-5)
    short = YvLatentCondensedAttention(32, 4, ratio=4, keep_recent=64)
    assert torch.allclose(short(x), _dense(short, x), atol=1e-5)
    h = YvDynamicH2OAttention(32, 4, recent=8, heavy=4, archive_block=4)
    k, v = torch.randn(4, 40, 8), torch.randn(4, 40, 8)
    mass = torch.rand(4, 40)
    tiers = h.compress(k, v, mass)
    assert tiers["recent_k"].shape == (4, 8, 8) and tiers["heavy_k"].shape == (4, 4, 8) and tiers["archive_k"].shape == (4, 8, 8)
    assert float(tiers["archive_count"].sum()) == 4 * (32 - 4)
    assert torch.equal(tiers["heavy_idx"], mass[:, :32].topk(4, -1).indices.sort(-1).values)
    o = h.decode_step(torch.randn(4, 1, 8), tiers)
    assert o.shape == (4, 1, 8) and torch.isfinite(o).all()
    # when every old key is identical the archive (with its log-count bias) reproduces exact attention
    k2 = torch.cat([torch.ones(1, 32, 8).expand(4, -1, -1), torch.randn(4, 8, 8)], 1)
    v2 = torch.cat([torch.full((4, 32, 8), 0.5), torch.randn(4, 8, 8)], 1)
    q = torch.randn(4, 1, 8)
    exact = torch.softmax((q @ k2.transpose(-1, -2)) * 8 ** -0.5, -1) @ v2
    assert torch.allclose(h.decode_step(q, h.compress(k2, v2, torch.rand(4, 40))), exact, atol=1e-5)


def test_egmla_cache_and_memory_cross_attention():
    torch.manual_seed(4)
    m = YvEGMLA(64, 4, kv_lora_rank=8, q_lora_rank=16)
    x = torch.randn(2, 10, 64)
    full, lat = m(x)
    assert lat.shape == (2, 10, 8) and abs(m.cache_reduction() - (1 - 8 / 128)) < 1e-9
    a, la = m(x[:, :7])
    b, lb = m(x[:, 7:], past_latent=la)
    assert torch.allclose(torch.cat([a, b], 1), full, atol=1e-5) and torch.allclose(lb, lat, atol=1e-6)
    mc = YvMemoryCrossAttention(64, 24, n_head=4)
    mem = torch.randn(2, 5, 24)
    y = mc(x, mem)
    assert y.shape == x.shape
    mask = torch.tensor([[True] * 5, [True, True, False, False, False]])
    y2 = mc(x, mem, mask)
    mem2 = mem.clone(); mem2[1, 2:] = 9.0
    assert torch.allclose(mc(x, mem2, mask), y2, atol=1e-5)


@pytest.mark.parametrize("cls,kw", [("YvTokenSparseAttention", dict(block_size=8, target=0.5, max_blocks=3)),
                                    ("YvMixtureBlockAttention", dict(block_size=8, top_k=2)),
                                    ("YvHISAAttention", dict(block_size=8, super_size=2, top_super=1, top_blocks=2))])
def test_block_sparse_attention_is_structurally_causal(cls, kw):
    """Perturbing one token leaves every EARLIER output bit-identical, selection map included: block representatives
    that contain future tokens must never take part in a ranking (the reference states the same contract for its
    token-sparse layer, tools/test/test_block_sparse_attn_contract.py:103)."""
    import pisceslx_b200.models.attention_sparse as A
    torch.manual_seed(0)
    m = getattr(A, cls)(64, 4, **kw)
    x = torch.randn(2, 64, 64)
    y = m(x)
    q, k, _ = m.qkv(x)
    sel = m.select(q, k)
    for j in (5, 21, 43, 62):
        x2 = x.clone()
        x2[:, j] += torch.randn(64)
        y2 = m(x2)
        q2, k2, _ = m.qkv(x2)
        assert torch.equal(y[:, :j], y2[:, :j]), (cls, j)
        assert torch.equal(sel[:, :, :j], m.select(q2, k2)[:, :, :j]), (cls, j)
        assert not torch.equal(y[:, j:], y2[:, j:])
