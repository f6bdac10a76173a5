"""GPU tests of the engine layer: memory-sized recomputation, prefetch loader, step profiler, serving engine."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from pisceslx_b200 import YvConfig
from pisceslx_b200.models import build_model


def _tiny():
    cfg = YvConfig.tiny_text_moe(vocab_size=2048)
    cfg.n_layer = 4
    cfg.use_gradient_checkpointing = True
    return cfg


def _losses(policy: str, steps: int = 4):
    from pisceslx_b200.engine.trainer import YvTrainer, YvTrainerConfig
    torch.manual_seed(0)
    m = build_model(_tiny(), "cuda", torch.bfloat16, seed=3)
    tr = YvTrainer(m, YvTrainerConfig(micro_batch_size=2, optimizer="adamw", lr=1e-3, max_steps=100, clip_grad_norm=0.0,
                                      recompute_policy=policy))
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 2048, (4, 256), generator=g)
    out = [tr.train_step({"input_ids": ids, "labels": ids})["loss"] for _ in range(steps)]
    return out, tr


def test_auto_recompute_plan_keeps_activations_when_memory_allows_and_matches_full_recompute():
    ref, _ = _losses("config")
    got, tr = _losses("auto")
    pl = tr.recompute_planner
    assert pl.stage == 3 and pl.stored_layers == 4 and pl.layer_bytes and pl.layer_bytes > 0
    assert [l.use_recompute for l in tr.model.model.layers] == [False] * 4
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (ref, got)
    assert got[-1] < got[0]


def test_prefetch_loader_overlaps_copy_and_delivers_in_order():
    from pisceslx_b200.data.prefetch import PiscesLxPrefetchLoader
    src = [{"input_ids": torch.full((2, 8), i, dtype=torch.long), "meta": i} for i in range(6)]
    got = list(PiscesLxPrefetchLoader(src, depth=2))
    assert [int(b["input_ids"][0, 0]) for b in got] == list(range(6))
    assert all(b["input_ids"].is_cuda for b in got) and [b["meta"] for b in got] == list(range(6))


def test_step_profiler_records_device_time_and_phases():
    from pisceslx_b200.engine.profiler import PiscesLxProfilingConfig, PiscesLxProfilingOperator
    prof = PiscesLxProfilingOperator(PiscesLxProfilingConfig(warmup_steps=0))
    x = torch.randn(2048, 2048, device="cuda")
    for _ in range(2):
        prof.start_step()
        with prof.phase("matmul"):
            y = x @ x
        with prof.phase("reduce"):
            y.sum().item()
        rec = prof.end_step(tokens=1000)
    assert rec["step_ms"] > 0 and set(rec["phases_ms"]) == {"matmul", "reduce"} and rec["tokens_per_s"] > 0
    s = prof.summary()
    assert s["steps"] == 2 and s["bottleneck"] in ("matmul", "reduce")


def test_serving_engine_on_gpu_matches_generate():
    from pisceslx_b200.serve.engine import YvEngineConfig, YvInferenceEngine
    torch.manual_seed(1)
    m = build_model(_tiny(), "cuda", torch.bfloat16, seed=4).eval()
    eng = YvInferenceEngine(m, cfg=YvEngineConfig(max_num_seqs=4, num_blocks=64, block_size=64, eos_token_id=-1))
    prompts = [[5, 6, 7, 8], [9, 10, 11], [12] * 70]
    reqs = [eng.add_request(p, max_new_tokens=5) for p in prompts]
    eng.run_until_done()
    for p, r in zip(prompts, reqs):
        ref, _ = m.generate(torch.tensor([p], device="cuda"), max_new_tokens=5, eos_token_id=-1)
        assert r.output_ids == ref[0, len(p):].tolist()
    g = eng.get_stats()["decode_graphs"]
    assert g["disabled_reason"] is None and g["graph_replays"] >= 4 and g["eager_steps"] == 0 and g["buckets"] == [4]


def test_graph_decode_equals_eager_decode_across_buckets_and_block_boundaries():
    from pisceslx_b200.serve.engine import YvEngineConfig, YvInferenceEngine
    m = build_model(_tiny(), "cuda", torch.bfloat16, seed=5).eval()
    outs = []
    for graphs in (True, False):
        eng = YvInferenceEngine(m, cfg=YvEngineConfig(max_num_seqs=8, num_blocks=64, block_size=64, eos_token_id=-1,
                                                      use_cuda_graphs=graphs, graph_max_seq_len=256))
        # different lengths: requests finish at different steps, so the batch shrinks through buckets 8 -> 4 -> 2 -> 1;
        # the 60-token prompt crosses a cache-block boundary while decoding
        reqs = [eng.add_request([3 + i] * n, max_new_tokens=k) for i, (n, k) in
                enumerate([(60, 12), (5, 3), (9, 7), (17, 9), (2, 2)])]
        eng.run_until_done()
        outs.append([r.output_ids for r in reqs])
        st = eng.get_stats()["decode_graphs"]
        if graphs:
            assert st["disabled_reason"] is None and st["graph_replays"] > 0 and len(st["buckets"]) >= 3
        else:
            assert st["graph_replays"] == 0 and st["eager_steps"] > 0
    assert outs[0] == outs[1]
    # a sequence longer than the graph's table width falls back to the eager step
    eng = YvInferenceEngine(m, cfg=YvEngineConfig(max_num_seqs=2, num_blocks=64, block_size=64, eos_token_id=-1,
                                                  graph_max_seq_len=256))
    r = eng.add_request([7] * 300, max_new_tokens=3)
    eng.run_until_done()
    assert len(r.output_ids) == 3 and eng.get_stats()["decode_graphs"]["eager_steps"] > 0
