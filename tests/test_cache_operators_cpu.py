"""Multi-LoRA slot-stacked serving, tensor-level prefix cache, chunked-prefill planner and operator."""
import json

import pytest
import torch

from pisceslx_b200.serve.cache_operators import (
    PiscesLxChunkedPrefillOperator, PiscesLxChunkedPrefillPlanner, PiscesLxMultiLoRAConfig, PiscesLxMultiLoRAOperator,
    PiscesLxPrefixCacheManager, PiscesLxPrefixCachingOperator)


def _adapter(r, i, o, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(r, i, generator=g) * 0.1, torch.randn(o, r, generator=g) * 0.1


def test_multi_lora_mixed_batch_matches_per_row_reference():
    op = PiscesLxMultiLoRAOperator(32, 24, PiscesLxMultiLoRAConfig(max_lora_adapters=4, max_lora_rank=8))
    ads = {"a": _adapter(8, 32, 24, 1), "b": _adapter(4, 32, 24, 2), "c": _adapter(2, 32, 24, 3)}
    alphas = {"a": 16.0, "b": None, "c": 4.0}
    for n, (a, b) in ads.items():
        op.load_adapter(n, a, b, alpha=alphas[n])
    x, base = torch.randn(6, 32), torch.randn(6, 24)
    names = ["a", None, "b", "c", "a", None]
    y = op.apply(x, base, op.slots_for(names))
    for t, n in enumerate(names):
        ref = base[t]
        if n is not None:
            a, b = ads[n]
            s = alphas[n] / a.shape[0] if alphas[n] is not None else 1.0
            ref = ref + s * (x[t] @ a.t()) @ b.t()
        assert torch.allclose(y[t], ref, atol=1e-5), (t, n)


def test_multi_lora_eviction_priority_and_reuse():
    op = PiscesLxMultiLoRAOperator(8, 8, PiscesLxMultiLoRAConfig(max_lora_adapters=2, max_lora_rank=2))
    a, b = _adapter(2, 8, 8, 0)
    r1 = op.run({"adapter_name": "keep", "lora_a": a, "lora_b": b, "priority": 5})
    op.run({"adapter_name": "x", "lora_a": a, "lora_b": b})
    assert not r1["cached"] and op.run({"adapter_name": "keep"})["cached"]
    op.run({"adapter_name": "y", "lora_a": a, "lora_b": b})           # evicts x (lower priority), not keep
    assert sorted(op.get_loaded_adapters()) == ["keep", "y"]
    st = op.get_stats()
    assert st["evictions"] == 1 and st["cache_hits"] == 1 and st["free_slots"] == 0
    with pytest.raises(KeyError):
        op.slots_for(["x"])
    # an evicted slot contributes nothing
    z = op.apply(torch.randn(2, 8), torch.zeros(2, 8), torch.tensor([-1, -1]))
    assert torch.count_nonzero(z) == 0
    with pytest.raises(ValueError):
        op.load_adapter("big", torch.zeros(3, 8), torch.zeros(8, 3))
    op.cleanup()
    assert op.get_loaded_adapters() == [] and float(op.A.abs().sum()) == 0


def test_multi_lora_from_path(tmp_path):
    a, b = _adapter(2, 8, 8, 0)
    d = tmp_path / "ad"
    d.mkdir()
    torch.save({"lora_A": a, "lora_B": b, "alpha": 4.0}, d / "adapter_model.pt")
    (d / "adapter_config.json").write_text(json.dumps({"r": 2}))
    cfg = PiscesLxMultiLoRAConfig.from_adapter_path(str(d))
    assert cfg.max_lora_rank == 2
    op = PiscesLxMultiLoRAOperator(8, 8, cfg)
    res = op.execute({"adapter_name": "p", "adapter_path": str(d)})
    assert res.is_success() and res.output["adapter_info"]["rank"] == 2
    x = torch.randn(1, 8)
    assert torch.allclose(op.apply(x, torch.zeros(1, 8), op.slots_for(["p"])), 2.0 * (x @ a.t()) @ b.t(), atol=1e-5)


def _kv(n):
    return (torch.arange(n * 4, dtype=torch.float32).view(1, 1, n, 4), torch.ones(1, 1, n, 4))


def test_prefix_cache_longest_prefix_and_partial():
    m = PiscesLxPrefixCacheManager(block=4)
    p1 = list(range(10))
    m.insert(p1, _kv(10))
    e, n = m.match(p1)
    assert n == 10 and e.hit_count == 1
    e, n = m.match(p1 + [99, 98])                       # the entry is a whole prefix of the query
    assert n == 10
    e, n = m.match(p1[:6] + [77, 76, 75])               # shares 6 tokens: one whole block, then the tail is compared too
    assert n == 6
    kv = m.get(p1[:6] + [77])
    assert kv[0].shape[-2] == 6 and torch.equal(kv[0], _kv(10)[0][..., :6, :])
    assert m.match([5, 5, 5, 5, 5])[0] is None
    s = m.get_stats()
    assert s["hits"] == 2 and s["partial_hits"] == 2 and s["misses"] == 1 and abs(s["hit_rate"] - 0.8) < 1e-9
    off = PiscesLxPrefixCacheManager(block=4, enable_substring_matching=False)
    off.insert(p1, _kv(10))
    assert off.match(p1 + [1])[0] is None and off.match(p1)[1] == 10


def test_prefix_cache_memory_budget_and_policies():
    one = sum(t.numel() * 4 for t in _kv(8))
    m = PiscesLxPrefixCacheManager(max_memory_bytes=2 * one, block=4)
    for i in range(3):
        m.insert([i] * 8, _kv(8))
    assert len(m.cache) == 2 and m.stats["evictions"] == 1 and m.match([0] * 8)[0] is None
    assert m.get_memory_usage()["used_bytes"] == 2 * one
    lfu = PiscesLxPrefixCacheManager(max_memory_bytes=2 * one, eviction_policy="lfu", block=4)
    lfu.insert([1] * 8, _kv(8))
    lfu.insert([2] * 8, _kv(8))
    lfu.match([1] * 8)
    lfu.insert([3] * 8, _kv(8))
    assert lfu.match([2] * 8)[0] is None and lfu.match([1] * 8)[0] is not None
    # a dropped entry hands its blocks to another holder of the same prefix
    sh = PiscesLxPrefixCacheManager(block=4)
    sh.insert([1, 2, 3, 4, 5], _kv(5))
    sh.insert([1, 2, 3, 4, 6], _kv(5))
    sh.invalidate(sh._compute_prompt_hash([1, 2, 3, 4, 6]))
    assert sh.match([1, 2, 3, 4, 9])[1] == 4
    with pytest.raises(ValueError):
        PiscesLxPrefixCacheManager(eviction_policy="random")


def test_prefix_caching_operator_actions():
    op = PiscesLxPrefixCachingOperator(block=2)
    ids = [1, 2, 3, 4]
    assert op.execute({"action": "insert", "token_ids": ids, "kv_cache": _kv(4)}).output["inserted"]
    out = op.execute({"token_ids": ids + [5]}).output
    assert out["cache_hit"] and out["matched_tokens"] == 4 and out["remaining_tokens"] == 1
    assert not op.execute({"action": "insert", "token_ids": ids}).is_success()
    assert op.execute({"action": "invalidate"}).output["invalidated_count"] == 1
    assert not op.execute({"token_ids": ids}).output["cache_hit"]
    assert op.execute({"action": "clear"}).output["cleared"]
    assert not op.execute({"action": "bogus", "token_ids": ids}).is_success()


def test_chunk_planner_alignment_budget_and_cached_skip():
    p = PiscesLxChunkedPrefillPlanner(max_chunk_size=1000, min_chunk_size=100, align=128)
    assert p.compute_optimal_chunk_size(500) == 500
    assert p.compute_optimal_chunk_size(5000) == 896                 # largest multiple of 128 under 1000
    assert p.compute_optimal_chunk_size(5000, current_memory_usage=0.9) == 384
    ch = p.split_into_chunks(list(range(2000)))
    assert ch == [(0, 896, 0), (896, 1792, 896), (1792, 2000, 1792)]
    ch = p.split_into_chunks(list(range(2000)), cached_tokens=1500)
    assert ch == [(1500, 2000, 1500)]
    b = PiscesLxChunkedPrefillPlanner(max_chunk_size=4096, min_chunk_size=128, memory_budget_bytes=1 << 20, bytes_per_token=1024)
    assert b.compute_optimal_chunk_size(10000) == 1024
    assert b.compute_optimal_chunk_size(10000, current_memory_usage=0.5) == 512
    assert b.compute_optimal_chunk_size(10000, current_memory_usage=1.0) == 128
    o = PiscesLxChunkedPrefillPlanner(max_chunk_size=256, min_chunk_size=128, overlap_chunks=True, overlap_size=32)
    ch = o.split_into_chunks(list(range(600)))
    assert ch[1] == (256, 512, 224) and ch[-1][1] == 600
    assert o.get_stats()["total_chunks"] == 3
    with pytest.raises(ValueError):
        PiscesLxChunkedPrefillPlanner(max_chunk_size=10, min_chunk_size=20)


def test_chunked_prefill_operator_drives_a_cache():
    op = PiscesLxChunkedPrefillOperator(max_chunk_size=256, min_chunk_size=128)
    ids = list(range(700))
    seen = []

    def step(chunk, start, state):
        seen.append((start, len(chunk)))
        return (state or 0) + sum(chunk)

    out = op.execute({"action": "prefill", "token_ids": ids, "step_fn": step}).output
    assert out["state"] == sum(ids) and out["chunk_count"] == 3 and seen == [(0, 256), (256, 256), (512, 188)]
    assert op.execute({"action": "stats"}).output["total_requests"] == 1
    assert not op.execute({"action": "prefill", "token_ids": ids}).is_success()
