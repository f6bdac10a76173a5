"""CPU tests of the model-family and tooling breadth: attention variants, task heads, block variants, cache policies,
expert variants, reasoning / agent scaffolding, operator runtime, extra optimizers, knowledge index, serving runtime,
benchmark harness, export, watermark, host tiers."""
import json
import math

import pytest
import torch

from pisceslx_b200 import YvConfig
from pisceslx_b200.models import build_model


def tiny():
    cfg = YvConfig.tiny_text_moe(vocab_size=300)
    cfg.n_layer = 2
    return cfg


# ------------------------------------------------------------------------------------------- attention variants
def test_attention_variants_masks_and_equivalences():
    from pisceslx_b200.models import attention_variants as av
    torch.manual_seed(0)
    x = torch.randn(2, 12, 32)
    # sliding window with window >= S equals plain causal attention with the same weights
    sw = av.YvSlidingWindowAttention(32, 4, window=64)
    q, k, v = sw.qkv(x)
    ref = sw.out(av.masked_attention(q, k, v, av.causal_mask(12, 12)))
    assert torch.allclose(sw(x), ref, atol=1e-6)
    m = av.YvSlidingWindowAttention(32, 4, window=3, n_sink=1).mask(8, x.device)
    assert m[7].tolist() == [True, False, False, False, False, True, True, True]
    # top-k sparse attention with k >= S equals dense causal attention
    sp = av.YvSparseAttention(32, 4, top_k=12)
    q, k, v = sp.qkv(x)
    assert torch.allclose(sp(x), sp.out(av.masked_attention(q, k, v, av.causal_mask(12, 12))), atol=1e-5)
    assert av.YvSparseAttention(32, 4, top_k=2)(x).shape == x.shape
    # ALiBi slopes: geometric, bias zero on the diagonal and decreasing with distance
    al = av.YvALiBi(8)
    b = al(5, 5)
    assert b.shape == (8, 5, 5) and float(b[:, 2, 2].abs().max()) == 0 and bool((b[:, 4, 0] < b[:, 4, 3]).all())
    assert abs(float(al.slopes[0]) - 2 ** -1) < 1e-6 and al.get_slopes(6).numel() == 6
    # linear attention is causal: changing a later token leaves earlier outputs untouched
    la = av.YvLinearAttention(32, 4)
    y1 = la(x)
    x2 = x.clone(); x2[:, -1] += 1.0
    assert torch.allclose(la(x2)[:, :-1], y1[:, :-1], atol=1e-5)
    o, acc, keep = av.YvH2OAttention(32, 4, recent=4, heavy=2)(x)
    assert o.shape == x.shape and acc.shape == (2, 4, 12) and int(keep[0, 0].sum()) == 6
    for mod in (av.YvMultiQueryAttention(32, 4), av.YvLocalGlobalAttention(32, 4, window=3, global_every=4),
                av.YvAttentionSink(32, 4, window=4), av.YvLatentKVAttention(32, 4, kv_lora_rank=8, rope_dim=4, q_lora_rank=8)):
        assert mod(x).shape == x.shape
    lat = av.YvLatentKVAttention(32, 4, kv_lora_rank=8, rope_dim=4)
    assert lat.latent(x).shape == (2, 12, 12)                       # what a cache keeps per token
    qn, kn = av.YvQKNormalizer(8)(torch.randn(2, 4, 5, 8) * 7, torch.randn(2, 4, 5, 8) * 3)
    assert abs(float(qn.pow(2).mean(-1).sqrt().mean()) - 1.0) < 0.05


# ------------------------------------------------------------------------------------------- heads / blocks
def test_task_heads_and_draft_heads():
    from pisceslx_b200.models.heads import (YvDSparkHead, YvMedusaHead, YvModelForQuestionAnswering,
                                            YvModelForSequenceClassification, YvModelForTokenClassification)
    cfg = tiny()
    ids = torch.randint(0, 300, (2, 9))
    mask = torch.ones(2, 9, dtype=torch.long); mask[1, 6:] = 0
    sc = YvModelForSequenceClassification(cfg, 3)
    out = sc(ids, mask, labels=torch.tensor([0, 2]))
    assert out["logits"].shape == (2, 3) and torch.isfinite(out["loss"])
    out["loss"].backward()
    assert sc.score.grad is not None
    tc = YvModelForTokenClassification(cfg, 5)(ids, mask, labels=torch.randint(0, 5, (2, 9)))
    assert tc["logits"].shape == (2, 9, 5) and torch.isfinite(tc["loss"])
    qa = YvModelForQuestionAnswering(cfg)(ids, mask, torch.tensor([1, 2]), torch.tensor([3, 4]))
    assert qa["start_logits"].shape == (2, 9) and torch.isfinite(qa["loss"])
    med = YvMedusaHead(16, 50, n_heads=3)
    assert med.propose(torch.randn(2, 16)).shape == (2, 3)
    ds = YvDSparkHead(16, 50, rank=8)
    emb = torch.nn.Embedding(50, 16)
    assert ds.draft(torch.randn(2, 16), torch.tensor([1, 2]), emb, 4).shape == (2, 4)


def test_block_variants():
    from pisceslx_b200.models import block_variants as bv
    torch.manual_seed(1)
    w = torch.randn(12, 16) * 0.1
    x = torch.randn(3, 16)
    lora = bv.YvLoRA(w, rank=4)
    assert torch.allclose(lora(x), x @ w.t(), atol=1e-6)             # B starts at zero: identity adapter
    lora.lora_b.data.normal_()
    assert torch.allclose(lora(x), x @ lora.merged_weight().t(), atol=1e-5)
    dora = bv.YvDoRA(w, rank=4)
    assert torch.allclose(dora(x), x @ w.t(), atol=1e-5)             # magnitude starts at the row norms
    blk = torch.nn.Linear(16, 16)
    mod = bv.YvMixtureOfDepths(16, capacity=0.5)
    h = torch.randn(2, 8, 16)
    out, idx = mod(h, blk)
    assert idx.shape == (2, 4)
    untouched = torch.ones(2, 8, dtype=torch.bool); untouched.scatter_(1, idx, False)
    assert torch.equal(out[untouched], h[untouched])
    act_out, ponder = bv.YvAdaptiveComputationTime(16, max_steps=3)(h, blk)
    assert act_out.shape == h.shape and 1.0 <= float(ponder) <= 3.0
    dn = bv.YvDeepNorm(16, n_layers=8)
    assert abs(dn.alpha - 16 ** 0.25) < 1e-9 and dn(h, blk(h)).shape == h.shape
    pb = bv.YvParallelBlock(16, blk, bv.YvGeGLU(16, 32))
    assert pb(h).shape == h.shape
    assert bv.YvDeepNormBlock(16, 4, blk, bv.YvGeGLU(16, 32))(h).shape == h.shape
    ca = bv.YvCrossAttentionBlock(16, 4)
    mem, mm = torch.randn(2, 5, 16), torch.tensor([[1, 1, 1, 0, 0], [1, 1, 1, 1, 1]])
    y = ca(h, mem, mm)
    mem2 = mem.clone(); mem2[0, 3:] += 10.0                           # masked memory rows do not matter
    assert torch.allclose(ca(h, mem2, mm)[0], y[0], atol=1e-5)
    assert torch.allclose(bv.YvLayerScale(16, 0.5)(h), 0.5 * h)


# ------------------------------------------------------------------------------------------- cache policies
def test_cache_policies_and_prefix_sharing():
    from pisceslx_b200.models.cache import YvCacheConfig, YvPagedKVCache
    from pisceslx_b200.models import cache_policies as cp
    cache = YvPagedKVCache(1, 1, 8, YvCacheConfig(block_size=4, num_blocks=6), torch.device("cpu"))
    mgr = cp.YvPagedCacheManager(cache, cp.YvEvictionPolicy("lru"))
    assert mgr.reserve(1, 8) and cache.append_slots(1, 8)
    assert mgr.reserve(2, 8) and cache.append_slots(2, 8)
    mgr.policy.touch(1)                                               # sequence 2 is now the least recently used
    assert mgr.reserve(3, 12) and mgr.evicted == [2]
    pol = cp.YvEvictionPolicy("importance")
    pol.touch(1, importance=0.9); pol.touch(2, importance=0.1)
    assert pol.victim() == 2 and pol.victim(protect=[2]) == 1
    keep = cp.YvH2OSelector(recent=2, heavy=2).select(torch.tensor([0.1, 5.0, 0.2, 4.0, 0.3, 0.0, 0.0]))
    assert keep.tolist() == [1, 3, 5, 6]
    rows = torch.randn(5, 64)
    for mode, tol in (("int8", 0.02), ("fp8", 0.08)):
        c = cp.YvCacheCompressor(mode)
        q, s = c.compress(rows)
        assert float((c.decompress(q, s, torch.float32) - rows).abs().max() / rows.abs().max()) < tol
    # speculative rollback returns whole blocks
    cache2 = YvPagedKVCache(1, 1, 8, YvCacheConfig(block_size=4, num_blocks=8), torch.device("cpu"))
    cache2.add_sequence(7); cache2.append_slots(7, 5)
    spec = cp.YvSpeculativeCacheManager(cache2)
    spec.mark(7); cache2.append_slots(7, 6)
    free_before = cache2.alloc.available()
    spec.rollback(7, accepted=1)
    assert cache2.lengths[7] == 6 and cache2.alloc.available() == free_before + 1
    # prefix cache: the second request re-uses the first one's full blocks
    cache3 = YvPagedKVCache(1, 1, 8, YvCacheConfig(block_size=4, num_blocks=8), torch.device("cpu"))
    pc = cp.YvPrefixCache(cache3)
    toks = list(range(10))
    assert pc.match(1, toks) == 0
    cache3.append_slots(1, 10)
    pc.publish(1, toks)
    assert pc.match(2, toks[:8] + [99, 98]) == 8 and cache3.tables[2] == cache3.tables[1][:2]
    ssm = cp.YvSSMCacheManager()
    st = ssm.get(1, 0, lambda: {"h": torch.zeros(2)})
    st["h"] += 1
    ssm.fork(1, 2)
    assert float(ssm.get(2, 0, dict)["h"].sum()) == 2.0
    ssm.free(1)
    assert (1, 0) not in ssm.states


# ------------------------------------------------------------------------------------------- experts
def test_expert_variants_and_training_aids():
    from pisceslx_b200.models import moe_extras as me
    torch.manual_seed(2)
    x = torch.randn(10, 16)
    for kind in ("swiglu", "standard", "geglu", "multilayer"):
        assert me.YvExpertFactory.create(kind, 16, 32)(x).shape == x.shape
    frozen = me.YvExpertFactory.create("swiglu", 16, 32, pure_lookup=True)
    assert not any(p.requires_grad for p in frozen.parameters())
    layer = me.YvDynamicMoELayer(16, 32, num_experts=4, top_k=2, kind="geglu", num_shared=1)
    y, aux = layer(x.view(2, 5, 16))
    assert y.shape == (2, 5, 16) and float(aux) > 0
    (y.sum() + aux).backward()
    assert layer.gate.grad is not None
    reg = me.YvExpertDiversityRegularizer(1.0)
    same = torch.randn(1, 8, 8).repeat(4, 1, 1)
    assert float(reg(same)) > float(reg(torch.randn(4, 8, 8)))
    feats = torch.cat([torch.randn(20, 8) + 5, torch.randn(20, 8) - 5])
    cent, assign = me.YvGradientClusterInitializer(2).cluster(feats)
    assert len(set(assign[:20].tolist())) == 1 and assign[0] != assign[-1]
    w = [torch.randn(4, 6, 6)]
    moved = me.YvExpertEvolution(noise=0.0).step(w, torch.tensor([100, 90, 80, 0]))
    assert moved == (3, 0) and torch.equal(w[0][3], w[0][0])


# ------------------------------------------------------------------------------------------- reasoning / agent
def test_reasoning_and_agent_loop():
    from pisceslx_b200.models import reasoning as rs
    script = iter(["Step 1: 2 + 3 = 5.\nStep 2: 5 * 4 = 20.\nFinal answer: 20",
                   "Step 1: 2 + 3 = 6.\nFinal answer: 24", "Step 1: 2 + 3 = 5.\nFinal answer: 20"])
    gen = lambda prompt, n: next(script)
    t = rs.YvMultiPathReasoner(gen, n_paths=3).reason("(2+3)*4?")
    assert t.answer == "20" and t.votes == {"20": 2, "24": 1}
    v = rs.YvVeriCoTVerifier()
    assert v.verify(rs.YvReasoningTrace(steps=["2 + 3 = 5", "5 * 4 = 20"])) and not v.verify(rs.YvReasoningTrace(steps=["2 + 3 = 6"]))
    tools = rs.YvToolRegistry()

    @tools.register("add", "adds two numbers", {"a": "number", "b": "number"})
    def add(a, b):
        return a + b

    turns = iter(['I will add. <tool_call><name>add</name><arguments>{"a": 2, "b": 5}</arguments></tool_call>', "The sum is 7."])
    res = rs.YvAgentic(lambda p, n: next(turns), tools).run("what is 2+5?")
    assert res["answer"] == "The sum is 7." and res["trajectory"][0]["observation"] == 7
    bridge = rs.YvMCPToolBridge(tools)
    r = json.loads(bridge.handle(rs.YvMCPMessage("tools/call", {"name": "add", "arguments": {"a": 1, "b": 2}}, 5).to_json()))
    assert r["result"] == 3 and r["id"] == 5
    assert "error" in json.loads(bridge.handle(rs.YvMCPMessage("nope", {}, 1).to_json()))
    from pisceslx_b200.third_party.mcp_service import MCPPlaza, MCPRegistry
    reg = MCPRegistry(); reg.register_server("math", tools)
    plaza = MCPPlaza(reg)
    sid = plaza.open_session("math", max_calls=1)
    assert json.loads(plaza.request(sid, rs.YvMCPMessage("tools/list", {}, 1).to_json()))["result"][0]["name"] == "add"
    assert "budget" in plaza.request(sid, rs.YvMCPMessage("tools/list", {}, 2).to_json())


# ------------------------------------------------------------------------------------------- operators / optim
def test_operator_runtime_timeout_retry_parallel():
    import time
    from pisceslx_b200.utils.opsc import (PiscesLxFunctionOperator, PiscesLxOperatorExecutor, PiscesLxOperatorRegistry,
                                          PiscesLxOperatorStatus, PiscesLxStreamPool)
    reg = PiscesLxOperatorRegistry()
    calls = {"n": 0}

    def flaky(inp):
        calls["n"] += 1
        if calls["n"] < 3:
            raise ValueError("not yet")
        return inp["x"] * 2

    reg.register("flaky", lambda: PiscesLxFunctionOperator("flaky", flaky))
    ex = PiscesLxOperatorExecutor(reg)
    r = ex.execute("flaky", {"x": 4}, retries=3, backoff=0.001)
    assert r.status == PiscesLxOperatorStatus.SUCCESS and r.output == 8 and r.metadata["attempt"] == 3
    slow = PiscesLxFunctionOperator("slow", lambda i: time.sleep(0.5))
    assert ex.execute(slow, {}, timeout=0.05).status == PiscesLxOperatorStatus.CANCELLED
    outs = ex.execute_parallel([(PiscesLxFunctionOperator("sq", lambda i: i["v"] ** 2), {"v": k}) for k in range(4)])
    assert [o.output for o in outs] == [0, 1, 4, 9]
    assert reg.names() == ["flaky"] and PiscesLxStreamPool(torch.device("cpu")).fork_join([lambda: 1, lambda: 2]) == [1, 2]
    ex.shutdown()


def test_extra_optimizers_and_training_aids():
    from pisceslx_b200.optim import extras as ox
    torch.manual_seed(3)
    w = torch.nn.Parameter(torch.randn(32, 48))
    target = torch.randn(32, 48)
    opt = ox.PiscesLxGaLoreAdamW([w], lr=0.05, rank=4, update_gap=5, scale=1.0)
    l0 = float((w - target).pow(2).mean())
    for _ in range(60):
        opt.zero_grad(); (w - target).pow(2).mean().backward(); opt.step()
    assert float((w - target).pow(2).mean()) < l0
    assert opt.state[w]["m"].shape == (4, 48)                        # moments live in the projected space
    w2 = torch.nn.Parameter(torch.randn(16, 24))
    ro = ox.PiscesLxROOTOptimizer([w2], lr=0.02)
    l0 = float(w2.pow(2).sum())
    for _ in range(30):
        ro.zero_grad(); w2.pow(2).sum().backward(); ro.step()
    assert float(w2.pow(2).sum()) < l0
    plan = ox.PiscesLxTERAIOManager(100).plan({"a": (60, 1), "b": (60, 9), "c": (30, 5)})
    assert plan == {"a": "gpu", "b": "host", "c": "gpu"}
    g = torch.randn(4, 8, 8); g[2] *= 100
    norms = ox.PiscesLxMoEGradientOperator(max_norm=1.0).apply(g)
    assert float(g[2].norm()) <= 1.0 + 1e-4 and float(norms[2]) > 100
    mt = ox.PiscesLxMultiTaskUncertainty(2)
    assert abs(float(mt([torch.tensor(2.0), torch.tensor(3.0)])) - 5.0) < 1e-6
    m = build_model(tiny())
    base = torch.optim.SGD([{"params": [p]} for _, p in m.named_parameters()], lr=1.0)
    sch = ox.PiscesLxModalityLRScheduler(base, m.named_parameters(), {"embed": 0.1})
    sch.apply(1.0)
    lrs = {n: g["lr"] for (n, _), g in zip(m.named_parameters(), base.param_groups)}
    assert lrs["model.embed.weight"] == 0.1 and lrs["model.norm.weight"] == 1.0
    c = ox.chinchilla_optimal(6 * 20 * 1e9 * 1e9)
    assert abs(c["params"] - 1e9) / 1e9 < 1e-6


# ------------------------------------------------------------------------------------------- knowledge / serving
def test_ivfpq_index_and_knowledge_builder(tmp_path):
    from pisceslx_b200.engine.knowledge import PiscesLxKnowledgeBuilder, nt_xent
    torch.manual_seed(4)
    z = torch.randn(8, 16)
    assert float(nt_xent(z, z + 0.01 * torch.randn(8, 16))) < float(nt_xent(z, torch.randn(8, 16)))
    vocab = {}

    def encode(texts):
        out = torch.zeros(len(texts), 64)
        for i, t in enumerate(texts):
            for w in t.lower().split():
                out[i, vocab.setdefault(w, len(vocab)) % 64] += 1.0
        return out

    docs = [f"topic{k} " * 4 + f"detail{k}" for k in range(24)]
    kb = PiscesLxKnowledgeBuilder(encode, 64, n_list=4, m=4)
    kb.build(docs)
    assert kb.query("topic7 topic7 detail7", k=1)[0][0] == docs[7]
    kb.save(str(tmp_path))
    assert kb.load_vectors(str(tmp_path)).shape == (24, 64)
    books, codes = kb.to_pq_field()
    assert books.shape[0] == 4 and codes.shape == (24, 4)


def test_subconscious_trainer_phases():
    from pisceslx_b200.engine.knowledge import PiscesLxSubconsciousTrainer
    from pisceslx_b200.models.subconscious import YvKnowledgeRouter
    torch.manual_seed(5)
    m = build_model(tiny())
    router = YvKnowledgeRouter(m.cfg.hidden_size, 6)
    tr = PiscesLxSubconsciousTrainer(m, router, lr=0.05)
    ids = torch.randint(0, 300, (4, 8))
    labels = torch.tensor([0, 1, 2, 3])
    first = float(torch.nn.functional.cross_entropy(tr._router_logits(ids), labels))
    assert tr.phase1_router_pretrain(ids, labels, steps=30) < first
    tr.phase2_policy(ids, steps=2)
    tr.phase3_self_play(ids, rounds=1, new_tokens=2)
    assert [p["phase"] for p in tr.phase_log] == [1, 2, 2, 3]


def test_serving_runtime_helpers():
    from pisceslx_b200.serve import runtime as rt
    loads = []
    cache = rt.PiscesLxExpertCache(2, lambda e: loads.append(e) or f"w{e}")
    for e in (0, 1, 0, 2, 1):
        cache.get(e)
    assert loads == [0, 1, 2, 1] and cache.hits == 1
    lb = rt.PiscesLxExpertLoadBalancer(8, decay=0.0)
    lb.observe(torch.tensor([100, 1, 1, 1, 90, 1, 1, 1]))
    place = lb.placement(2)
    assert (0 in place[0]) != (4 in place[0]) and lb.imbalance() > 3
    groups = rt.PiscesLxBatchSharing.group([{1, 2}, {7, 8}, {2, 3}, {8, 9}])
    assert sorted(sorted(g) for g in groups) == [[0, 2], [1, 3]]
    assert rt.moebius_choose_layout(64, 4096, 1408, 64, 6, 8)["layout"] in ("ep", "tp")
    sch = rt.PiscesLxChunkedPrefillScheduler(token_budget=10, chunk=6)
    sch.add(1, list(range(9)))
    s1 = sch.step(); s2 = sch.step()
    assert s1["prefill_chunks"] == [(1, 0, 6)] and s2["prefill_chunks"] == [(1, 6, 9)] and sch.step()["decode"] == [1]
    reg = rt.PiscesLxMultiLoRARegistry()
    reg.register("a", torch.ones(2, 4), torch.ones(3, 2), 0.5)
    x, base = torch.ones(2, 4), torch.zeros(2, 3)
    out = reg.apply(x, base, ["a", None])
    assert torch.allclose(out[0], torch.full((3,), 4.0)) and float(out[1].abs().sum()) == 0
    cands = iter(["bad", "ok", "good", "best", "x", "y", "z", "w"])
    tpo = rt.PiscesLxTPO(lambda p, n: next(cands), lambda p, c: {"best": 3, "good": 2, "ok": 1}.get(c, 0), n=4, rounds=2)
    assert tpo.run("q")["answer"] == "best"


# ------------------------------------------------------------------------------------------- tools / third party
def test_benchmark_harness_export_watermark_and_tiers(tmp_path):
    from pisceslx_b200.tools import benchmark as bm, publish as pub
    from pisceslx_b200.third_party.watermark import POPSSTextWatermark, POPSSWatermarkConfig, POPSSWeightWatermark
    from pisceslx_b200.utils.host_tier import PiscesLxVramController, YvHostTierResolver, YvNumericalGuard
    from pisceslx_b200.models.tokenizer import YvTokenizer
    torch.manual_seed(6)
    cfg = tiny()
    m = build_model(cfg).eval()
    rep = bm.PiscesLxPerformanceBenchmark(m).run([torch.randint(0, 300, (1, 6))], max_new_tokens=4)
    s = rep.summary()
    assert s["ttft_p50_ms"] > 0 and s["tokens_per_s"] > 0 and len(rep.inter_token_ms) == 3
    assert bm.model_flops_per_token(cfg, 128, True) == 3 * bm.model_flops_per_token(cfg, 128, False)
    gh = bm.PiscesLxGenerativeHarness(lambda p, n: " 42 \nnoise")
    assert gh.evaluate([{"prompt": "q", "answer": "42"}, {"prompt": "q", "answer": "7"}])["exact_match"] == 0.5
    tok = YvTokenizer.instance()
    rows = bm.needle_in_haystack_rows(tok, 64, depths=(0.5,))
    assert "7319" in rows[0]["prompt"] and rows[0]["answer"] == "7319"
    idx = pub.export_safetensors(m, str(tmp_path / "export"), max_shard_bytes=200_000)
    assert len(set(idx["weight_map"].values())) > 1
    m2 = build_model(cfg, seed=99)
    pub.load_safetensors(m2, str(tmp_path / "export"))
    ids = torch.randint(0, 300, (1, 5))
    assert torch.allclose(m(input_ids=ids, return_logits=True)["logits"], m2(input_ids=ids, return_logits=True)["logits"], atol=1e-5)
    assert "FROM" in open(pub.write_docker_context(str(tmp_path / "docker"))).read() and "parameters" in pub.model_card(m)
    cm = pub.PiscesLxCacheManager(str(tmp_path / "cache"), max_bytes=100)
    cm.register("a", 80); cm.register("b", 80); cm.touch("a")
    assert cm.cleanup() == ["b"]
    wm = POPSSTextWatermark(300, POPSSWatermarkConfig(gamma=0.25, delta=8.0))
    toks = [5]
    for _ in range(60):
        toks.append(int(wm.process_logits(torch.zeros(1, 300), torch.tensor([toks[-1]])).argmax()))
    assert wm.detect(toks).detected and not wm.detect(torch.randint(0, 300, (60,)).tolist()).detected
    w = torch.randn(64, 64) * 0.02
    ww = POPSSWeightWatermark(eps=5e-3)
    assert not ww.verify(w)["detected"]
    ww.embed(w)
    assert ww.verify(w)["detected"]

    class P:
        major, total_memory = 10, 180 * 2 ** 30
    assert YvHostTierResolver.resolve(props=P()).tcgen05 and YvHostTierResolver.resolve(None).name == "cpu"
    P.major = 8
    with pytest.raises(RuntimeError):
        YvHostTierResolver.enforce(cfg, props=P())
    s = torch.zeros(3, requires_grad=True)
    g = YvNumericalGuard.straight_through_gate(s)
    g.sum().backward()
    assert torch.allclose(g, torch.ones(3)) and torch.allclose(s.grad, torch.full((3,), 0.5))
    assert PiscesLxVramController(reserve_gb=0, reader=lambda: (10 * 2 ** 30, 0)).fit_micro_batch(3 * 2 ** 30, 8) == 3
