"""CPU tests of the vision-side extras and the remaining norm / rotary variants."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from pisceslx_b200.models.multimodal.vision_extras import (YvAdaptiveLayerNorm, YvDiffusionImageEnhancer,
                                                          YvDynamicResolutionProcessor, YvGroupNorm, YvImageDecoder,
                                                          YvLinearScalingRoPE, YvMoVEVisionEncoder,
                                                          YvMrRoPERotaryEmbedding, YvSigLIPVisionEncoder,
                                                          YvSparseCutRouter)


def test_norm_and_rotary_variants():
    torch.manual_seed(0)
    x = torch.randn(2, 5, 16)
    aln = YvAdaptiveLayerNorm(16, 8)
    assert torch.allclose(aln(x, torch.randn(2, 8)), torch.nn.functional.layer_norm(x, (16,), eps=1e-6), atol=1e-6)
    aln.mod.bias.data[:16] = 1.0
    assert torch.allclose(aln(x, torch.zeros(2, 8)), 2 * torch.nn.functional.layer_norm(x, (16,), eps=1e-6), atol=1e-5)
    gn = YvGroupNorm(4, 16)
    y = gn(x)
    assert y.shape == x.shape and abs(float(y[0].reshape(5, 4, 4)[:, 0].mean())) < 1e-5
    pos = torch.arange(32)
    lin = YvLinearScalingRoPE(8, scale=4.0)
    base = YvLinearScalingRoPE(8, scale=1.0)
    assert torch.allclose(lin(pos * 4)[0], base(pos)[0], atol=1e-6)
    pro = YvMrRoPERotaryEmbedding(16, 1e4, 1e6, "pro")
    uni = YvMrRoPERotaryEmbedding(16, 1e4, 1e6, "uni")
    assert pro(pos)[0].shape == (32, 16)
    # progressive radix: frequencies fall monotonically and end slower than a pure small-base ladder
    assert (pro.inv_freq[1:] < pro.inv_freq[:-1]).all()
    d = torch.arange(8).float() / 8
    assert pro.inv_freq[-1] < (1e4 ** -d)[-1] and torch.isclose(uni.inv_freq[2], torch.tensor(1e4) ** -d[2])
    c, s = pro(pos)
    assert torch.allclose(c ** 2 + s ** 2, torch.ones_like(c), atol=1e-6)


def test_dynamic_resolution_and_sparse_cut():
    proc = YvDynamicResolutionProcessor(patch=14, min_patches=4, max_patches=64)
    r = proc(torch.rand(3, 300, 500))
    gh, gw = r["grid"]
    assert r["image"].shape == (3, gh * 14, gw * 14) and gh * gw <= 64
    assert abs(gw / gh - 500 / 300) < 0.45                  # aspect ratio kept up to patch rounding
    small = proc(torch.rand(3, 10, 10))
    assert small["grid"][0] * small["grid"][1] >= 4
    torch.manual_seed(1)
    sc = YvSparseCutRouter(16, ratio=0.25)
    t = torch.randn(2, 12, 16)
    kept, idx = sc(t)
    assert kept.shape == (2, 3, 16) and (idx[:, 1:] > idx[:, :-1]).all()
    assert torch.allclose(kept, torch.gather(t, 1, idx[..., None].expand(-1, -1, 16)), atol=1e-6)
    kept.sum().backward()
    assert sc.score.weight.grad is not None and sc.score.weight.grad.abs().sum() > 0


class _ToyTrunk(nn.Module):
    def __init__(self, dim, scale=1.0):
        super().__init__()
        self.proj, self.scale = nn.Linear(3 * 4 * 4, dim), scale

    def forward(self, img):
        B = img.shape[0]
        p = img.unfold(2, 4, 4).unfold(3, 4, 4).permute(0, 2, 3, 1, 4, 5).reshape(B, -1, 48)
        return self.proj(p) * self.scale


def test_move_and_siglip():
    torch.manual_seed(2)
    img = torch.rand(3, 3, 8, 8)
    a, b = _ToyTrunk(16), _ToyTrunk(16, 2.0)
    one = YvMoVEVisionEncoder({"a": a}, 16)
    assert torch.equal(one(img), a(img))
    two = YvMoVEVisionEncoder({"a": a, "b": b}, 16, top_k=1)
    out = two(img)
    pa, pb = a(img), b(img)
    pick_a = (out - pa).abs().amax(-1) < 1e-6
    pick_b = (out - pb).abs().amax(-1) < 1e-6
    assert (pick_a | pick_b).all()                           # top-1: each token comes from exactly one encoder
    both = YvMoVEVisionEncoder({"a": a, "b": b}, 16, top_k=2)
    assert both(img).shape == (3, 4, 16)
    sig = YvSigLIPVisionEncoder(_ToyTrunk(16), 16, embed_dim=8, n_head=4)
    e = sig(img)
    assert e.shape == (3, 8) and torch.allclose(e.norm(dim=-1), torch.ones(3), atol=1e-5)
    txt = torch.nn.functional.normalize(torch.randn(3, 8), dim=-1)
    l_match = sig.sigmoid_loss(txt, txt)
    l_rand = sig.sigmoid_loss(e, txt)
    assert torch.isfinite(l_rand) and l_match < sig.sigmoid_loss(txt, -txt)
    l_rand.backward()
    assert sig.logit_bias.grad is not None


def test_image_decoder_and_diffusion_enhancer():
    torch.manual_seed(3)
    dec = YvImageDecoder(32, base=4, stages=2, channels=32)
    img = dec(torch.randn(2, 32))
    assert img.shape == (2, 3, 16, 16) and img.abs().max() <= 1
    enh = YvDiffusionImageEnhancer(channels=16, steps=100)
    loss = enh.training_loss(img.detach())
    assert torch.isfinite(loss)
    loss.backward()
    assert enh.out.weight.grad is not None
    te = enh.time_embedding(torch.tensor([0, 50]))
    assert te.shape == (2, 16) and torch.allclose(te[0, :8], torch.zeros(8)) and torch.allclose(te[0, 8:], torch.ones(8))
    # with the zero-initialised output layer the predicted noise is 0, so the deterministic sampler returns
    # x0 = x_t / sqrt(abar_t) clipped: enhancing from t_start = 0 is the identity
    same = enh.enhance(img.detach(), t_start=0, n_steps=1)
    assert torch.allclose(same, (enh.abar[0].sqrt() * img.detach() + (1 - enh.abar[0]).sqrt() * 0).clamp(-1, 1) / 1.0, atol=0.05)
    out = enh.enhance(img.detach(), t_start=50, n_steps=5)
    assert out.shape == img.shape and torch.isfinite(out).all()
