"""YvUnifiedCacheManager: exact by default, every lossy policy opt-in (reference model/core/cache.py:1760-2430)."""
import torch

from pisceslx_b200.models.cache_unified import YvUnifiedCacheConfig, YvUnifiedCacheManager


def _kv(t, seed, B=1, hk=2, d=16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(B, hk, t, d, generator=g), torch.randn(B, hk, t, d, generator=g)


def test_default_configuration_is_exact_and_blocked():
    m = YvUnifiedCacheManager(YvUnifiedCacheConfig(n_layer=2, block_tokens=8, max_cache_size=1000))
    assert m.get_kv_cache(0) is None
    ks, vs = [], []
    for step, t in enumerate([5, 1, 1, 9, 1]):                      # prefill, decode steps, a chunk that spans blocks
        k, v = _kv(t, step)
        ks.append(k); vs.append(v)
        out_k, out_v = m.update_kv_cache(0, k, v)
    assert torch.equal(out_k, torch.cat(ks, 2)) and torch.equal(out_v, torch.cat(vs, 2))
    st = m.get_cache_stats()
    assert st["tokens_per_layer"][0] == 17 and st["evicted_tokens"] == 0 and st["hit_rate"] > 0
    ck = m.create_checkpoint()
    m2 = YvUnifiedCacheManager(YvUnifiedCacheConfig(n_layer=2, block_tokens=8))
    m2.restore_checkpoint(ck)
    assert torch.equal(m2.get_kv_cache(0)[0], out_k)
    m.clear_cache()
    assert m.get_kv_cache(0) is None


def test_cold_block_quantisation_and_eviction_are_opt_in_and_bounded():
    m = YvUnifiedCacheManager(YvUnifiedCacheConfig(block_tokens=8, quantize_cold_blocks=True, max_cache_size=1000))
    k, v = _kv(20, 1)
    out_k, out_v = m.update_kv_cache(0, k, v)
    assert m.stats["quantized_blocks"] == 2                          # two closed blocks of 8, the open one stays dense
    assert torch.equal(out_k[:, :, 16:], k[:, :, 16:])
    err = (out_k[:, :, :16] - k[:, :, :16]).abs().max() / k.abs().max()
    assert 0 < err < 1e-2                                            # int8 with a scale per row
    # eviction from the front once 1.5 x max_cache_size is exceeded, down to max_cache_size, whole blocks
    e = YvUnifiedCacheManager(YvUnifiedCacheConfig(block_tokens=8, max_cache_size=32))
    for i in range(7):
        ek, ev = _kv(8, 10 + i)
        out_k, _ = e.update_kv_cache(0, ek, ev)
    assert out_k.shape[2] == 32 and e.stats["evicted_tokens"] == 24
    assert torch.equal(out_k[:, :, -8:], ek)


def test_h2o_keeps_recent_and_heavy_hitters():
    m = YvUnifiedCacheManager(YvUnifiedCacheConfig(block_tokens=16, h2o=True, h2o_recent=4, h2o_heavy=3, max_cache_size=1000))
    k, v = _kv(12, 3)
    attn = torch.zeros(1, 2, 1, 12)
    attn[..., [1, 5, 6]] = 1.0                                       # the heavy hitters among the older tokens
    out_k, _ = m.update_kv_cache(0, k, v, attention_scores=attn)
    assert out_k.shape[2] == 7 and m.stats["h2o_dropped_tokens"] == 5
    assert torch.equal(out_k, k[:, :, [1, 5, 6, 8, 9, 10, 11]])


def test_compaction_keeps_the_important_half_of_old_blocks():
    m = YvUnifiedCacheManager(YvUnifiedCacheConfig(block_tokens=8, compact=True, max_cache_size=24, evict_factor=1.0))
    k, v = _kv(32, 4)
    k[:, :, [0, 3, 4, 7]] *= 10                                      # large-norm keys in the first block
    out_k, _ = m.update_kv_cache(0, k, v)
    assert m.stats["compacted_tokens"] == 8                          # two old blocks, half of each
    assert torch.equal(out_k[:, :, :4], k[:, :, [0, 3, 4, 7]])


def test_paged_ssm_speculative_multimodal_and_prefix_stores():
    m = YvUnifiedCacheManager(YvUnifiedCacheConfig(n_layer=2, n_kv_head=2, head_dim=16, paged_blocks=4, paged_block_size=4))
    assert m.allocate_paged_sequence(7)
    g = torch.Generator().manual_seed(5)
    k0, v0 = torch.randn(6, 2, 16, generator=g), torch.randn(6, 2, 16, generator=g)
    k1, v1 = torch.randn(6, 2, 16, generator=g), torch.randn(6, 2, 16, generator=g)
    assert m.append_paged(7, 0, k0, v0) and m.append_paged(7, 1, k1, v1)
    rk, rv = m.read_paged(7, 1)
    assert torch.equal(rk, k1) and torch.equal(rv, v1) and torch.equal(m.read_paged(7, 0)[0], k0)
    assert not m.append_paged(7, 0, torch.zeros(20, 2, 16), torch.zeros(20, 2, 16))     # more than the pool holds
    m.free_paged_sequence(7)
    assert m.get_cache_stats()["paged_free_blocks"] == 4
    m.update_ssm_state(1, torch.ones(3), seq_id=2)
    assert torch.equal(m.get_ssm_state(1, seq_id=2), torch.ones(3)) and m.get_ssm_state(0, seq_id=2) is None
    mid = m.get_optimal_draft_length()
    for _ in range(8):
        m.store_speculative_draft(4, torch.arange(4), accepted=4)
    assert m.get_optimal_draft_length() == 8 > mid and torch.equal(m.get_speculative_draft(4)["tokens"], torch.arange(4))
    for _ in range(64):
        m.store_speculative_draft(4, torch.arange(4), accepted=0)
    assert m.get_optimal_draft_length() == 2
    m.store_multimodal_cache("image", "abc", torch.ones(2))
    assert torch.equal(m.get_multimodal_cache("image", "abc"), torch.ones(2)) and m.get_multimodal_cache("image", "x") is None
    m.set_generation_cache("audio", torch.zeros(1))
    assert m.get_generation_cache("audio") is not None
    m.insert_plt_prefix(list(range(8)), [-0.1] * 8, [0, 1])
    assert m.find_plt_prefix_match(list(range(8)) + [99]) is not None
