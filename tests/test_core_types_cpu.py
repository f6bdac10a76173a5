"""Typed configuration views and the memory fusion / separation layers."""
import pytest
import torch

from pisceslx_b200.config import YvConfig
from pisceslx_b200.models.core_types import (YvAttentionBackend, YvAttentionConfig, YvBlockConfig, YvBlockType, YvCacheBlock, YvCacheType, YvLayerConfig, YvLayerType,
                                             YvMemoryFusionGate, YvMemorySeparationLayer, YvModality, YvModelType, YvNorms, YvRegularizationConfig, YvSpecialTokenType)


def test_records_read_the_flat_configuration():
    cfg = YvConfig.tiny_text_moe(vocab_size=64)
    a = YvAttentionConfig.from_config(cfg)
    assert a.hidden_size == cfg.hidden_size and a.n_head == cfg.n_head and a.head_dim == (cfg.head_dim or cfg.hidden_size // cfg.n_head)
    assert a.backend() in tuple(YvAttentionBackend) and a.scale == a.head_dim ** -0.5 and a.kv_bytes_per_token() > 0
    assert YvAttentionConfig(use_ring_attention=True).backend() is YvAttentionBackend.RING and YvAttentionConfig(sliding_window=128).backend() is YvAttentionBackend.SLIDING_WINDOW
    assert YvAttentionConfig(use_mla=False, n_kv_head=8, hidden_size=1024, n_head=8).kv_bytes_per_token() == 2 * 8 * 128 * 2
    with pytest.raises(ValueError):
        YvAttentionConfig(n_head=6, n_kv_head=4)
    b = YvBlockConfig.from_config(cfg)
    assert b.n_layer == cfg.n_layer and b.resolved_type() is YvBlockType.STANDARD and YvBlockConfig(use_parallel=True).resolved_type() is YvBlockType.PARALLEL
    al, be = YvBlockConfig(n_layer=32).deepnorm_constants()
    assert abs(al - 64 ** 0.25) < 1e-9 and abs(be - 256 ** -0.25) < 1e-9
    with pytest.raises(ValueError):
        YvBlockConfig(block_type="weird")
    l = YvLayerConfig.from_config(cfg, 1)
    assert l.layer_idx == 1 and l.num_experts == cfg.moe_num_experts and isinstance(l.layer_type, YvLayerType)
    assert YvModelType("hybrid") and YvCacheType("paged") and YvModality("video") and YvSpecialTokenType("tool")


def test_cache_block_and_regularisation_and_norms():
    blk = YvCacheBlock(3, block_size=4)
    assert blk.append(3) == 0 and not blk.is_full and blk.append(3) == 2 and blk.is_full and blk.free_slots == 0
    blk.share()
    assert not blk.release() and blk.release() and blk.ref_count == 0
    r = YvRegularizationConfig(diversity_weight=0.1, warmup_steps=10)
    assert r.weight_at("diversity", 0) == pytest.approx(0.01) and r.weight_at("diversity", 100) == 0.1 and YvRegularizationConfig().weight_at("z_loss", 0) == 1e-3
    x = torch.randn(2, 8)
    assert YvNorms.create("rmsnorm", 8)(x).shape == x.shape and isinstance(YvNorms.create("ln", 8), torch.nn.LayerNorm) and YvNorms.create("none", 8)(x) is x
    with pytest.raises(ValueError):
        YvNorms.create("batch", 8)


def test_fusion_gate_starts_closed_and_learns_to_open():
    torch.manual_seed(0)
    g = YvMemoryFusionGate(hidden_size=16, memory_size=8)
    h, m = torch.randn(2, 5, 16), torch.randn(2, 5, 8)
    out = g(h, m)
    assert (out - h).abs().max() < 0.1 * g.proj(m).abs().max() and float(g.last_gate_mean) < 0.03 and g(h, None) is h
    masked = g(h, m[:, 0], memory_mask=torch.tensor([1, 0]))
    assert torch.equal(masked[1], h[1]) and not torch.equal(masked[0], h[0])
    target = h + g.proj(m).detach() * 0 + m @ torch.randn(8, 16)
    opt = torch.optim.Adam(g.parameters(), lr=0.05)
    first = None
    for _ in range(150):
        loss = (g(h, m) - target).pow(2).mean()
        opt.zero_grad(); loss.backward(); opt.step()
        first = first if first is not None else float(loss.detach())
    assert float(loss.detach()) < 0.2 * first and float(g.last_gate_mean) > 0.2


def test_separation_layer_is_identity_at_start_and_separates():
    torch.manual_seed(0)
    s = YvMemorySeparationLayer(hidden_size=16, query_size=16)
    h = torch.randn(2, 4, 16)
    r, q = s(h)
    assert torch.allclose(r, h, atol=1e-5) and q.shape == (2, 4, 16) and 0.0 <= float(s.separation_loss.detach()) <= 1.0
    opt = torch.optim.Adam(s.parameters(), lr=0.02)
    first = float(s.separation_loss.detach())
    for _ in range(100):
        s(h)
        opt.zero_grad(); s.separation_loss.backward(); opt.step()
    s(h)
    assert float(s.separation_loss.detach()) < 0.3 * first + 1e-4
    assert YvMemorySeparationLayer(hidden_size=16, query_size=8)(h)[1].shape == (2, 4, 8)
