"""SigLIP blocks: attention against a plain reference, layer, multi-scale mix, GRN, cross-modal attention, tower."""
import math

import pytest
import torch
import torch.nn.functional as F

from pisceslx_b200.models.multimodal.siglip import (YvSigLIPAttention, YvSigLIPCrossModalAttention, YvSigLIPGRN, YvSigLIPMLP, YvSigLIPMultiScaleFeatureExtractor,
                                                    YvSigLIPTower, YvSigLIPTransformerLayer)


def test_attention_matches_plain_softmax():
    torch.manual_seed(0)
    a = YvSigLIPAttention(32, 4).eval()
    x = torch.randn(2, 7, 32)
    q, k, v = a.qkv(x).view(2, 7, 3, 4, 8).permute(2, 0, 3, 1, 4)
    ref = (torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(8), -1) @ v).transpose(1, 2).reshape(2, 7, 32)
    assert torch.allclose(a(x), a.out_proj(ref), atol=1e-5)
    with pytest.raises(ValueError):
        YvSigLIPAttention(30, 4)
    assert YvSigLIPMLP(32)(x).shape == x.shape and YvSigLIPMLP(32, 48).fc1.out_features == 48


def test_layer_scale_zero_is_identity_and_grads_flow():
    torch.manual_seed(0)
    x = torch.randn(2, 5, 16, requires_grad=True)
    assert torch.equal(YvSigLIPTransformerLayer(16, 4, layer_scale=0.0)(x), x)
    y = YvSigLIPTransformerLayer(16, 4)(x)
    y.sum().backward()
    assert x.grad is not None and not torch.allclose(y, x)


def test_grn_definition():
    torch.manual_seed(0)
    g = YvSigLIPGRN(6)
    x = torch.randn(2, 9, 6)
    assert torch.equal(g(x), x)                                                          # gamma = beta = 0
    with torch.no_grad():
        g.gamma.fill_(0.5)
        g.beta.fill_(0.1)
    n = x.norm(dim=1, keepdim=True)
    ref = x + 0.5 * x * (n / n.mean(-1, keepdim=True)) + 0.1
    assert torch.allclose(g(x), ref, atol=1e-6)


def test_multi_scale_matches_per_scale_layers():
    torch.manual_seed(0)
    m = YvSigLIPMultiScaleFeatureExtractor(8, 12)
    assert m.scale_indices == [2, 5, 8, 11] and YvSigLIPMultiScaleFeatureExtractor(8, 2).scale_indices == [0, 0, 0, 1]
    with torch.no_grad():
        m.scale_weights.copy_(torch.tensor([0.1, 0.5, -0.3, 1.0]))
        m.norm_weight.normal_(1.0, 0.1)
        m.proj_bias.normal_()
    hs = [torch.randn(2, 5, 8) for _ in range(12)]
    w = torch.softmax(m.scale_weights, 0)
    ref = 0
    for s, i in enumerate(m.scale_indices):
        h = F.layer_norm(hs[i], (8,)) * m.norm_weight[s, 0, 0] + m.norm_bias[s, 0, 0]
        ref = ref + w[s] * F.gelu(h @ m.proj_weight[s].t() + m.proj_bias[s, 0])
    assert torch.allclose(m(hs), ref, atol=1e-5)


def test_cross_modal_attention_respects_the_text_mask():
    torch.manual_seed(0)
    c = YvSigLIPCrossModalAttention(16, 4).eval()
    v, t = torch.randn(2, 6, 16), torch.randn(2, 5, 16)
    mask = torch.tensor([[1, 1, 1, 0, 0], [1, 1, 1, 1, 1]])
    out = c(v, t, mask)
    t2 = t.clone()
    t2[0, 3:] = 99.0                                                                     # padded text must not matter
    assert torch.allclose(c(v, t2, mask)[0], out[0], atol=1e-5) and not torch.allclose(c(v, t2)[0], out[0], atol=1e-3)
    assert out.shape == v.shape


def test_tower_embeds_and_trains():
    torch.manual_seed(0)
    tw = YvSigLIPTower(image_size=16, patch_size=8, hidden_size=32, num_layers=4, num_heads=4, embed_dim=12)
    imgs = torch.randn(4, 3, 16, 16)
    emb, tok = tw(imgs)
    assert emb.shape == (4, 12) and tok.shape == (4, 4, 32) and torch.allclose(emb.norm(dim=-1), torch.ones(4), atol=1e-5)
    txt = F.normalize(torch.randn(4, 12), dim=-1)
    opt = torch.optim.Adam(tw.parameters(), lr=3e-3)
    first = None
    for _ in range(30):
        loss = tw.sigmoid_loss(tw(imgs)[0], txt)
        opt.zero_grad()
        loss.backward()
        opt.step()
        first = first if first is not None else float(loss.detach())
    assert float(loss.detach()) < first
    with pytest.raises(ValueError):
        YvSigLIPTower(image_size=15, patch_size=8)
