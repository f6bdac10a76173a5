"""Fused MLA projections and latent-space (weight-absorbed) decoding against the explicit keys / values."""
import math

import pytest
import torch

from pisceslx_b200.config import YvConfig
from pisceslx_b200.models.attention import YvAttention
from pisceslx_b200.models.mla_fused import PiscesLxFusedMLAProjector
from pisceslx_b200.ops import reference as ref


def _attention(enhanced, q_lora):
    torch.manual_seed(0)
    cfg = YvConfig.tiny_text_moe(vocab_size=128)
    cfg.use_mla, cfg.kv_lora_rank, cfg.mla_q_lora_rank = True, 32, (48 if q_lora else 0)
    cfg.use_enhanced_mla, cfg.mla_rope_dim = enhanced, 16
    return YvAttention(cfg, 0, 1, None).eval(), cfg


@pytest.mark.parametrize("enhanced,q_lora", [(False, False), (True, False), (True, True)])
def test_fused_projection_matches_the_separate_tensors(enhanced, q_lora):
    att, cfg = _attention(enhanced, q_lora)
    proj = PiscesLxFusedMLAProjector.from_attention(att)
    x = torch.randn(11, cfg.hidden_size)
    with torch.no_grad():
        a, b = att._qkv_mla(x), proj.qkv(x)
    assert a.shape == b.shape and torch.allclose(a, b, atol=1e-5)
    assert proj.in_fused.shape == (2 * 32 + cfg.n_head * cfg.head_dim, cfg.hidden_size)
    assert proj.kv_decompress_fused.shape[0] == 2 * cfg.n_kv_head * cfg.head_dim + (16 if enhanced else 0)
    bt = proj.bytes_per_token()
    assert bt["ratio"] == pytest.approx(2 * cfg.n_kv_head * cfg.head_dim / (32 + (16 if enhanced else 0)))


@pytest.mark.parametrize("enhanced", [False, True])
def test_latent_space_decode_equals_attention_over_explicit_keys_and_values(enhanced):
    att, cfg = _attention(enhanced, False)
    proj = PiscesLxFusedMLAProjector.from_attention(att)
    hq, hk, d, S = cfg.n_head, cfg.n_kv_head, cfg.head_dim, 23
    rot = proj.mla_rope_dim
    half = max(rot // 2, 1)
    inv = 1.0 / (1e4 ** (torch.arange(half).float() / half))
    ang = torch.arange(64).float()[:, None] * inv[None]
    cos, sin = ang.cos(), ang.sin()
    x = torch.randn(2, S, cfg.hidden_size)
    lengths = torch.tensor([S, S - 5])
    with torch.no_grad():
        outs, caches, qs = [], [], []
        for b in range(2):
            L = int(lengths[b])
            q, latent = proj.compress(x[b, :L])
            k, v, _ = proj.decompress_kv(latent)
            pos = torch.arange(L)
            if enhanced:
                qr, kr = ref.apply_rope(q, cos, sin, pos, rot), ref.apply_rope(k, cos, sin, pos, rot)
            else:
                qr, kr = q, k
            g = hq // hk
            kk, vv = kr.repeat_interleave(g, 1), v.repeat_interleave(g, 1)          # [L, hq, d]
            s = torch.einsum("hd,shd->hs", qr[-1].float(), kk.float()) / math.sqrt(d)
            outs.append(torch.einsum("hs,shd->hd", torch.softmax(s, -1), vv.float()))
            entry = proj.cache_entry(latent, pos, cos, sin)
            caches.append(torch.cat([entry, entry.new_zeros(S - L, entry.shape[1])], 0))
            qs.append(q[-1])
        want = torch.stack(outs)
        got = proj.decode_absorbed(torch.stack(qs), torch.stack(caches), lengths, lengths - 1, cos, sin)
    assert got.shape == (2, hq, d) and torch.allclose(got.float(), want, atol=2e-5), float((got.float() - want).abs().max())
    assert torch.stack(caches).shape[-1] == 32 + (16 if enhanced else 0)


def test_from_attention_requires_the_latent_path():
    cfg = YvConfig.tiny_text_moe(vocab_size=128)
    with pytest.raises(ValueError):
        PiscesLxFusedMLAProjector.from_attention(YvAttention(cfg, 0, 1, None))
