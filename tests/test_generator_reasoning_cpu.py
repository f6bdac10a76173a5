"""Content generator (image / audio / video heads over a Yv trunk) and the hidden-state VeriCoT pair, agentic
evolution and the verification factory, on CPU."""
import torch
import torch.nn as nn


def _gen_cfg():
    from pisceslx_b200.models.multimodal import YvGenerationConfig
    return YvGenerationConfig(hidden_size=64, num_heads=4, num_layers=1, max_sequence_length=64, image_size=32,
                              num_inference_steps=4, audio_gen_duration=0.05, audio_gen_num_codebooks=2,
                              audio_gen_codebook_size=32, video_gen_num_frames=3, latent_dim=16)


def test_generator_registry_produces_every_modality_deterministically():
    from pisceslx_b200.models.multimodal import YvGenerationModality, YvGeneratorFactory
    g = YvGeneratorFactory.create_generator(_gen_cfg())
    assert g.get_available_modalities() == ["image", "audio", "video"]
    a = g.generate_from_text("a red square", "image", seed=1)
    b = g.generate_from_text("a red square", YvGenerationModality.IMAGE, seed=1)
    assert a.success and a.data.shape == (1, 3, 32, 32) and torch.equal(a.data, b.data)
    assert float(a.data.abs().max()) <= 1.0 and a.metadata["backend"] == "yv-text-to-image"
    assert not torch.equal(a.data, g.generate_from_text("a blue circle", "image", seed=1).data)       # conditioned
    w = g.generate_from_text("beep", "audio")
    assert w.success and w.data.shape == (1, 800) and w.metadata["sample_rate"] == 16000
    v = g.generate_from_text("waves", "video", seed=2)
    assert v.success and v.data.shape == (1, 3, 3, 32, 32)
    bad = g.generate_from_text("x", "smell")
    assert not bad.success and "no backend" in bad.error
    assert set(g.get_capabilities()["backends"]) == {"image", "audio", "video"}


def test_latent_denoiser_learns_a_prompt_conditioned_target():
    from pisceslx_b200.models.multimodal import YvSelfDevelopedGenerator
    torch.manual_seed(0)
    m = YvSelfDevelopedGenerator(_gen_cfg())
    params = list(m.denoiser.parameters()) + list(m.cond_proj.parameters())
    opt = torch.optim.Adam(params, lr=3e-3)
    target = torch.randn(2, 16)
    first = None
    for i in range(60):
        torch.manual_seed(i % 4)                                 # a few fixed (t, noise) draws: the loss must go down
        loss = m.diffusion_training_loss(["alpha", "beta"], target)
        opt.zero_grad()
        loss.backward()
        opt.step()
        first = first if first is not None else float(loss)
    assert float(loss) < 0.7 * first


def test_vericot_step_verifier_reflector_and_factory():
    from pisceslx_b200.models.reasoning_verify import (YvVeriCoTReflector, YvVeriCoTStepVerifier,
                                                       YvVerificationFactory)
    torch.manual_seed(0)
    ver = YvVeriCoTStepVerifier(32)
    h, ctx = torch.randn(3, 5, 32), torch.randn(3, 7, 32)
    assert torch.allclose(ver(h)["validity_score"], torch.full((3,), 0.5))          # no context: neutral
    r = ver(h, ctx, step_text="2 + 2 = 5")
    assert r["symbolic_score"] == 0.0 and float(r["combined_score"].max()) < 0.51    # the wrong sum pulls it down
    assert ver(h, ctx, step_text="2 + 2 = 4")["symbolic_score"] == 1.0
    chain = ver.verify_chain([torch.randn(1, 32) for _ in range(4)], ["1 + 1 = 2", "so", "3 * 3 = 9", "4 - 1 = 2"])
    assert len(chain["steps"]) == 4 and chain["first_invalid"] is not None and not chain["all_valid"]
    with torch.no_grad():                                       # force "invalid" so that the reflector has to act
        ver.quality_estimator[2].bias.fill_(-10.0)
        ver.quality_estimator[2].weight.zero_()
    out, info = YvVeriCoTReflector(ver, max_reflections=2)(h, ctx)
    assert info["reflections"] == 2 and not bool(info["final_valid"].any()) and not torch.equal(out, h)
    assert torch.allclose(out, h * 1.1 ** 2, atol=1e-3)
    modes = dict(YvVerificationFactory.detect_cot_failure_modes(["x = 1", "x = 1 again"], "the answer is definitely one hundred"))
    assert "premature_conclusion" in modes and "circular_reasoning" in modes
    assert "arithmetic_error" in dict(YvVerificationFactory.detect_cot_failure_modes(["2 * 3 = 7"], "7"))
    assert isinstance(YvVerificationFactory.create("vericot_reflector", 16), YvVeriCoTReflector)


def test_agentic_evolution_selects_and_mutates():
    from pisceslx_b200.models.reasoning_verify import YvAgenticEvolution
    torch.manual_seed(0)
    base = nn.Linear(4, 3)
    evo = YvAgenticEvolution(base, num_agents=4, mutation_rate=0.5, selection_pressure=0.5)
    g = torch.Generator().manual_seed(1)
    for a in list(evo.agents)[1:]:                              # spread the population out
        for p in a.parameters():
            p.data.add_(torch.randn(p.shape, generator=g))
    x = torch.randn(64, 4)
    y = (x @ torch.randn(4, 3)).argmax(-1)
    best0 = float(evo.evaluate_agents(x, y).max())
    for _ in range(15):
        evo.evaluate_agents(x, y)
        top = evo.evolve_population(g)
        assert len(top) == 2
    assert float(evo.evaluate_agents(x, y).max()) >= best0 and evo.generation == 15
    assert evo.best() is evo.agents[int(evo.agent_scores.argmax())]


def test_server_media_routes_schemas_and_rate_limit():
    import base64
    from fastapi.testclient import TestClient
    from pisceslx_b200 import YvConfig
    from pisceslx_b200.models import build_model
    from pisceslx_b200.models.multimodal import YvGenerator
    from pisceslx_b200.serve import schemas as S
    from pisceslx_b200.serve.engine import YvEngineConfig, YvInferenceEngine
    from pisceslx_b200.serve.server import PiscesLxInferService, PiscesLxRateLimiter
    t = [0.0]
    lim = PiscesLxRateLimiter(rate=1.0, burst=2, clock=lambda: t[0])
    assert lim.allow() and lim.allow() and not lim.allow()
    t[0] = 1.5
    assert lim.allow() and not lim.allow()
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    eng = YvInferenceEngine(build_model(cfg, "cpu", torch.float32, seed=0),
                            cfg=YvEngineConfig(num_blocks=64, block_size=16, eos_token_id=-1))
    svc = PiscesLxInferService(eng, rate_limiter=PiscesLxRateLimiter(rate=0.0, burst=2))
    svc.attach_generator(YvGenerator(_gen_cfg()))
    with TestClient(svc.build_app()) as c:
        r = S.PiscesLxChatCompletionResponse.model_validate(
            c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3}).json())
        assert r.usage.completion_tokens == 3 and r.choices[0].message.role == "assistant"
        S.PiscesLxCompletionResponse.model_validate(c.post("/v1/completions", json={"prompt": "ab", "max_tokens": 2}).json())
        third = c.post("/v1/completions", json={"prompt": "ab", "max_tokens": 2})        # the bucket held two requests
        assert third.status_code == 429 and S.PiscesLxErrorResponse.model_validate(third.json()).code == 429
        S.PiscesLxModelListResponse.model_validate(c.get("/v1/models").json())
        img = S.PiscesLxImageGenerationResponse.model_validate(
            c.post("/v1/images/generations", json={"prompt": "a red square", "seed": 3, "n": 2}).json())
        assert len(img.data) == 2 and len(base64.b64decode(img.data[0].b64_json)) == 32 * 32 * 3
        aud = c.post("/v1/audio/speech", json={"input": "beep"}).json()["data"]
        assert S.PiscesLxAudioSpeechResponse.model_validate(aud).samples == 800
        vid = S.PiscesLxVideoGenerationResponse.model_validate(c.post("/v1/videos/generations", json={"prompt": "w", "num_frames": 2}).json())
        assert vid.data[0].frames == 2
    svc.stop()


def test_thought_tree_memory_reasoner_semantic_cache_and_reward_tools():
    from pisceslx_b200.engine.rl import PiscesLxGenerativeRewardModel, PiscesLxRewardNormalizer
    from pisceslx_b200.models.reasoning import YvCoTMemoryReasoner, YvThoughtTreeReasoner, YvUnifiedReasoner
    from pisceslx_b200.serve.runtime import PiscesLxSemanticCache
    # a scripted "model": proposes a bad and a good step at depth 0, then answers; rates chains containing "good" higher
    calls = {"n": 0}

    def gen(prompt: str, n: int) -> str:
        if "Rate from 1 to 10" in prompt:
            return " 9" if "good" in prompt else " 2"
        calls["n"] += 1
        if "(none)" in prompt:
            return "bad idea" if calls["n"] % 2 else "good idea"
        return "Answer: 42" if "good" in prompt else "Answer: 7"
    t = YvThoughtTreeReasoner(gen, branch=2, beam=1, max_depth=3).reason("what?")
    assert t.answer == "42" and t.steps[0] == "good idea"
    assert YvUnifiedReasoner(gen, strategy="tree", branch=2, beam=1).reason("what?").answer == "42"
    seen = []

    def cot(prompt: str, n: int) -> str:
        seen.append(prompt)
        return "step one\nAnswer: 5"
    mem = YvCoTMemoryReasoner(cot, shots=1)
    mem.reason("how many apples are in the red box")
    mem.reason("how many apples are in the blue box")
    assert "Q: how many apples are in the red box" in seen[-1] and len(mem.memory) == 2
    # semantic cache: near-duplicate prompts hit, different ones miss, LRU eviction
    vocab = {"hello": 0, "world": 1, "there": 2, "bye": 3}

    def embed(text):
        v = torch.zeros(4)
        for w in text.split():
            v[vocab.get(w, 3)] += 1
        return v
    c = PiscesLxSemanticCache(embed, capacity=2, threshold=0.9)
    c.put("hello world", "A")
    assert c.get("world hello") == "A" and c.get("bye") is None
    c.put("bye", "B")
    c.get("hello world")
    c.put("there there", "C")                                   # evicts "bye" (least recently used)
    assert c.get("bye") is None and c.get("hello world") == "A" and c.stats()["entries"] == 2
    # reward normaliser: batched Welford equals the plain statistics
    norm = PiscesLxRewardNormalizer(clip=3.0)
    data = torch.randn(3, 50) * 4 + 2
    for row in data:
        norm.update(row)
    assert abs(norm.mean - float(data.mean())) < 1e-5 and abs(norm.std - float(data.flatten().std())) < 1e-4
    assert float(norm(torch.tensor([1000.0]), update=False)) == 3.0
    grm = PiscesLxGenerativeRewardModel(lambda p, n: "fine. Score: 7/10" if "right" in p else "no score here")
    assert torch.allclose(grm.score("q", ["right answer", "wrong"]), torch.tensor([0.7, 0.0]))


def test_distillation_loss_family():
    from pisceslx_b200.engine.distill_losses import (PiscesLxAttentionDistillationLoss, PiscesLxDistillationLoss,
                                                     PiscesLxDistillationLossConfig, PiscesLxLayerWiseDistillationLoss,
                                                     PiscesLxLogitsDistillationLoss, PiscesLxOptimalTransportAligner)
    torch.manual_seed(0)
    t_logits = torch.randn(2, 5, 11)
    kd = PiscesLxLogitsDistillationLoss(2.0)
    assert float(kd(t_logits, t_logits)) < 1e-6 and float(kd(torch.randn(2, 5, 11), t_logits)) > 0.01
    s_logits = torch.zeros(2, 5, 11, requires_grad=True)
    opt = torch.optim.SGD([s_logits], lr=5.0)
    first = float(kd(s_logits, t_logits))
    for _ in range(100):
        opt.zero_grad()
        kd(s_logits, t_logits).backward()
        opt.step()
    assert float(kd(s_logits, t_logits)) < 0.05 * first                         # the student matches the teacher's distribution
    a = torch.softmax(torch.randn(2, 4, 6, 6), -1)
    assert float(PiscesLxAttentionDistillationLoss()(a, a)) < 1e-6
    assert float(PiscesLxAttentionDistillationLoss()(torch.softmax(torch.randn(2, 2, 6, 6), -1), a)) > 0        # 2 vs 4 heads
    ss, ts = [torch.randn(2, 5, 8) for _ in range(2)], [torch.randn(2, 5, 16) for _ in range(4)]
    lw = PiscesLxLayerWiseDistillationLoss(8, 16)
    assert float(lw(ss, ts)) > 0 and lw.loss.proj.weight.shape == (16, 8)
    plan = PiscesLxOptimalTransportAligner().plan(ss, ts)
    assert plan.shape == (2, 4) and torch.allclose(plan.sum(1), torch.full((2,), 0.5), atol=1e-3)
    assert float(plan[0, 0]) > float(plan[0, 3]) and float(plan[1, 3]) > float(plan[1, 0])      # early to early, late to late
    full = PiscesLxDistillationLoss(PiscesLxDistillationLossConfig(hidden_weight=0.5, contrastive_weight=0.1, hard_label_weight=0.2), 8, 16)
    total, parts = full({"logits": torch.randn(2, 5, 11), "hidden_states": ss}, {"logits": t_logits, "hidden_states": ts},
                        labels=torch.randint(0, 11, (2, 5)))
    assert set(parts) == {"logits", "hidden", "contrastive", "hard"} and abs(float(total) - sum(parts.values())) < 1e-4


def test_numerical_shape_device_guards_and_rope_front():
    import pytest
    from pisceslx_b200.models.safety import (YvDeviceGuard, YvDeviceResolver, YvNumericalGuard, YvRope, YvShapeGuard)
    G = YvNumericalGuard
    assert G.get_eps(torch.bfloat16) > G.get_eps(torch.float32)
    d = G.safe_div(torch.ones(3), torch.tensor([0.0, -0.0, 2.0]))
    assert torch.isfinite(d).all() and float(d[2]) == 0.5
    assert torch.isfinite(G.safe_log(torch.zeros(2))).all()
    s = torch.tensor([0.3, 0.8], requires_grad=True)
    g = G.straight_through_gate(s)
    g.sum().backward()
    assert g.tolist() == [0.0, 1.0] and s.grad.tolist() == [1.0, 1.0]
    YvShapeGuard.check_matmul(torch.zeros(2, 3), torch.zeros(3, 4))
    with pytest.raises(ValueError, match=r"\(2, 3\) @ \(5, 4\)"):
        YvShapeGuard.check_matmul(torch.zeros(2, 3), torch.zeros(5, 4), "in q_proj")
    with pytest.raises(ValueError):
        YvShapeGuard.check_cat([torch.zeros(2, 3), torch.zeros(2, 4)], 0)
    YvShapeGuard.check_cat([torch.zeros(2, 3), torch.zeros(5, 3)], 0)
    a, b = YvDeviceGuard.align(torch.zeros(2, dtype=torch.float64), torch.ones(2, dtype=torch.float32))
    assert b.dtype == torch.float64
    with pytest.raises(ValueError):
        YvDeviceGuard.assert_same_dtype(torch.zeros(1), torch.zeros(1, dtype=torch.float64))
    dev = YvDeviceResolver.resolve("auto")
    assert YvDeviceResolver.compute_dtype(torch.device("cpu")) == torch.float32 and dev.type in ("cpu", "cuda")
    cos, sin = YvRope.precompute_freqs_cis(8, 16)
    q, k = torch.randn(16, 2, 8), torch.randn(16, 1, 8)
    qr, kr = YvRope.apply_rotary_emb(q, k, cos, sin)
    assert torch.allclose(qr.norm(dim=-1), q.norm(dim=-1), atol=1e-5) and torch.allclose(qr[0], q[0], atol=1e-6)
    # relative property: the score of (q at i, k at j) depends on i - j only
    q1, k1 = YvRope.apply_rotary_emb(q[:1].expand(16, 2, 8), k[:1].expand(16, 1, 8), cos, sin)
    sc = (q1[:, 0] @ k1[:, 0].t())
    assert torch.allclose(sc[3, 1], sc[10, 8], atol=1e-4)
