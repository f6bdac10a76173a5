"""Latent reasoning engines: geometry of every branch, convex collapse, chunked / fused cross-entropy against the plain
mean, the load-bearing hash, a real loss with gradients, and causality of the thinking logits."""
import types

import pytest
import torch
import torch.nn.functional as F

from pisceslx_b200.models.reasoning_engine import (YvAdaptiveReasoningController, YvLatentCoTReasoner,
                                                   YvLatentUnifiedReasoner, YvMultiDimensionalFactVerifier,
                                                   YvMultiPathReasoningEngine, YvRLDrivenMetacognition, prefix_mean)

HIDDEN, HEADS, VOCAB = 64, 8, 256


def _cfg(**kw):
    c = types.SimpleNamespace(hidden_size=HIDDEN, vocab_size=VOCAB, n_head=4, n_layer=2, extra={})
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def _engine(**kw):
    torch.manual_seed(0)
    e = YvMultiPathReasoningEngine(_cfg(**kw))
    assert e.reasoning_heads == HEADS
    return e


def test_head_count_snaps_to_a_divisor():
    # 64 is not divisible by 7, 6 or 5: the largest divisor not above 7 is 4
    assert YvMultiPathReasoningEngine(_cfg(reasoning_heads=7)).reasoning_heads == 4
    with pytest.raises(ValueError):
        YvMultiPathReasoningEngine(_cfg(reasoning_heads=0))


def test_pruning_branch_keeps_the_geometry():
    e = _engine().eval()
    out = e(torch.randn(2, 40, HIDDEN), input_ids=torch.randint(0, VOCAB, (2, 40)))
    assert tuple(out["thinking_logits"].shape) == (2, 40, VOCAB)
    assert out["collapse_rule"] == "path_partition"
    pw = out["path_weights"]
    assert tuple(pw.shape) == (2, 40, HEADS)
    assert torch.allclose(pw.sum(-1), torch.ones(2, 40), atol=1e-5)
    assert int((pw > 0).sum(-1).max()) == 4                     # half of the paths are kept
    assert tuple(out["fact_consistency"].shape) == (2, 40, 1) and tuple(out["uncertainty_scores"].shape) == (2, 1, 1)
    assert tuple(out["reflection_logits"].shape) == (2, 3)


def test_stream_collapse_is_convex():
    e = _engine()
    pw = F.softmax(torch.randn(4, e.reasoning_heads), -1)
    unc = torch.rand(4, 1, 1)
    w, rule = e._stream_weights(pw, unc, 3)
    assert tuple(w.shape) == (4, 3) and bool((w >= 0).all()) and rule == "path_partition"
    assert torch.allclose(w.sum(-1), torch.ones(4), atol=1e-5)
    fb, rule = e._stream_weights(None, unc, 3)
    assert rule == "uniform_confidence_scaled" and bool((fb >= 0).all()) and bool((fb.sum(-1) <= 1 + 1e-6).all())
    # per-position weights keep their leading dimensions
    w3, _ = e._stream_weights(F.softmax(torch.randn(2, 5, e.reasoning_heads), -1), unc, 3)
    assert tuple(w3.shape) == (2, 5, 3) and torch.allclose(w3.sum(-1), torch.ones(2, 5), atol=1e-5)
    # every head belongs to exactly one stream, groups differ by at most one head
    g = e._head_group_indices(8, 3, "cpu")
    counts = torch.bincount(g, minlength=3)
    assert int(counts.max() - counts.min()) <= 1 and bool((g[1:] >= g[:-1]).all())


def test_chunked_and_fused_cross_entropy_equal_the_plain_mean():
    e = _engine()
    seq = 96
    logits = torch.randn(2, seq, VOCAB)
    labels = torch.randint(0, VOCAB, (2, seq))
    labels[:, :8] = -100
    unc = torch.rand(2, 1, 1)
    streams = {n: torch.randn(2, seq, HIDDEN) for n in ("hypothesis", "evidence", "conclusion")}
    total = e._compute_reasoning_loss(streams, logits, unc, labels, None, None)
    sl, tl = logits[:, :-1].reshape(-1, VOCAB), labels[:, 1:].reshape(-1)
    plain = F.cross_entropy(sl[tl != -100], tl[tl != -100]) + 0.1 * unc.mean()
    assert torch.allclose(total, plain, atol=1e-5)
    collapsed = torch.randn(2, seq, HIDDEN)
    fused = e._compute_reasoning_loss(streams, None, unc, labels, None, None, collapsed=collapsed)
    lg = collapsed @ e.thinking_head.weight.t()
    plain = F.cross_entropy(lg[:, :-1].reshape(-1, VOCAB)[tl != -100], tl[tl != -100]) + 0.1 * unc.mean()
    assert torch.allclose(fused, plain, atol=1e-4)


def test_span_losses_use_the_marked_regions():
    e = _engine()
    e.initialize_reasoning_tokens(None)
    t = e.reasoning_tokens
    ids = torch.randint(0, VOCAB - 8, (1, 30))
    ids[0, 2], ids[0, 10], ids[0, 18], ids[0, 26] = t["start_hypothesis"], t["start_evidence"], t["start_conclusion"], t["hypothesis_merge"]
    m = e._create_reasoning_masks(ids)
    assert m["hypothesis"][0].nonzero().flatten().tolist() == list(range(2, 10))
    assert m["evidence"][0].nonzero().flatten().tolist() == list(range(10, 18))
    assert m["conclusion"][0].nonzero().flatten().tolist() == list(range(18, 26))
    streams = {n: torch.randn(1, 30, HIDDEN) for n in ("hypothesis", "evidence", "conclusion")}
    unc = torch.zeros(1, 1, 1)
    with_spans = e._compute_reasoning_loss(streams, None, unc, ids, ids, None, collapsed=torch.randn(1, 30, HIDDEN))
    torch.manual_seed(1)
    assert float(with_spans) > 0
    no_marks = torch.randint(0, VOCAB - 8, (1, 30))
    base = e._compute_reasoning_loss(streams, None, unc, no_marks, None, None, collapsed=streams["hypothesis"])
    same = e._compute_reasoning_loss(streams, None, unc, no_marks, no_marks, None, collapsed=streams["hypothesis"])
    assert torch.allclose(base, same)                           # no marker: no span term


def test_long_sequence_branch_keeps_the_geometry():
    e = _engine().eval()
    seq = e.long_sequence_tokens + 40
    out = e(torch.randn(1, seq, HIDDEN), input_ids=torch.randint(0, VOCAB, (1, seq)))
    assert tuple(out["thinking_logits"].shape) == (1, seq, VOCAB)
    assert out["collapse_rule"] == "uniform_confidence_scaled" and out["path_weights"] is None
    assert bool(torch.isfinite(out["thinking_logits"]).all())
    assert float(out["abstraction_depth"].max()) <= e.long_sequence_layer_cap


def test_lsh_hash_is_load_bearing_and_reversible():
    e = _engine().eval()
    x = torch.randn(1, 300, HIDDEN)
    with torch.no_grad():
        base = e._lsh_chunked_attention(x)
        lsh = e.chunked_attention["lsh_proj"]
        saved = lsh.weight.detach().clone()
        lsh.weight.copy_(torch.randn_like(saved))
        moved = e._lsh_chunked_attention(x)
        lsh.weight.copy_(saved)
        back = e._lsh_chunked_attention(x)
    assert bool(torch.isfinite(base).all()) and float((base - moved).abs().max()) > 0
    assert torch.allclose(back, base, atol=1e-6)


def test_training_step_produces_a_real_loss_and_gradients():
    e = _engine().train()
    labels = torch.randint(0, VOCAB, (2, 40))
    out = e(torch.randn(2, 40, HIDDEN), input_ids=labels, labels=labels)
    assert out["thinking_logits"] is None                       # the loss path does not build [B, S, V]
    loss = out["loss"]
    assert torch.isfinite(loss) and float(loss) > 0
    loss.backward()
    graded = [n for n, p in e.named_parameters() if p.grad is not None and float(p.grad.abs().sum()) > 0]
    assert any(n.startswith("thinking_head") for n in graded) and any("abstraction_layers" in n for n in graded)
    assert any("path_pruning_controller" in n for n in graded) and any("fact_verifier" in n for n in graded)


@pytest.mark.parametrize("seq", [48, 600])
def test_thinking_logits_do_not_see_the_future(seq):
    e = _engine().eval()
    x = torch.randn(1, seq, HIDDEN)
    y = x.clone()
    cut = seq - 9
    y[:, cut:] = torch.randn(1, seq - cut, HIDDEN)
    with torch.no_grad():
        a, b = e(x)["thinking_logits"], e(y)["thinking_logits"]
    assert torch.allclose(a[:, :cut], b[:, :cut], atol=1e-4)
    assert float((a[:, cut:] - b[:, cut:]).abs().max()) > 1e-3


def test_depth_is_decided_per_position_without_read_back():
    import inspect
    e = _engine().eval()
    out = e(torch.randn(2, 32, HIDDEN))
    d = out["abstraction_depth"]
    assert tuple(d.shape) == (2, 32) and float(d.min()) >= 1 and float(d.max()) <= len(e.abstraction_layers)
    src = inspect.getsource(YvMultiPathReasoningEngine._abstract) + inspect.getsource(YvMultiPathReasoningEngine.forward)
    assert ".item()" not in src and ".tolist()" not in src
    x = torch.randn(1, 6, HIDDEN)
    assert torch.allclose(prefix_mean(x)[0, 3], x[0, :4].mean(0), atol=1e-6)


def test_resize_vocab_keeps_shared_rows():
    e = _engine()
    w = e.thinking_head.weight.detach().clone()
    e.resize_vocab(VOCAB + 16)
    assert e.thinking_head.weight.shape == (VOCAB + 16, HIDDEN) and torch.equal(e.thinking_head.weight[:VOCAB], w)
    assert tuple(e.eval()(torch.randn(1, 8, HIDDEN))["thinking_logits"].shape) == (1, 8, VOCAB + 16)


def test_disabled_engine_raises_instead_of_faking():
    e = _engine(enable_dynamic_fusion=False)
    with pytest.raises(ValueError):
        e(torch.randn(1, 8, HIDDEN))


def test_fact_verifier_scores():
    torch.manual_seed(0)
    v = YvMultiDimensionalFactVerifier(HIDDEN)
    h, ev, c = (torch.randn(3, 10, HIDDEN) for _ in range(3))
    out = v(h, ev, c)
    for k in ("logical_consistency", "knowledge_accuracy", "coherence", "overall_verification"):
        assert tuple(out[k].shape) == (3, 1) and bool(((out[k] >= 0) & (out[k] <= 1)).all())
    assert out["is_valid"].dtype == torch.bool
    assert torch.allclose(v(h, ev)["coherence"], torch.full((3, 1), 0.8))


def test_metacognition_acts_learns_and_evolves_per_sample():
    torch.manual_seed(0)
    m = YvRLDrivenMetacognition(HIDDEN, memory_size=16)
    hs = torch.randn(3, 12, HIDDEN)
    out = m(hs, enable_evolution=True, layer_index=0, total_layers=4)
    assert tuple(out["action_probs"].shape) == (3, 4) and torch.allclose(out["action_probs"].sum(-1), torch.ones(3), atol=1e-5)
    assert len(out["action_name"]) == 3 and set(out["action_name"]) <= set(m.ACTIONS)
    assert out["evolved"].dtype == torch.bool and tuple(out["evolved"].shape) == (3,)
    assert tuple(out["metacognitive_feedback"].shape) == (3, HIDDEN)
    before = [p.detach().clone() for p in m.critic_network.parameters()]
    for i in range(20):                                         # wraps around the 16-slot memory
        stats = m.update(hs.mean(1), out["selected_action"], reward=1.0, next_state=hs.mean(1) * 0.9)
    assert m.memory_count == 60 and torch.isfinite(stats["critic_loss"])
    assert any(not torch.equal(a, b) for a, b in zip(before, m.critic_network.parameters()))
    assert float(m.critic_network(hs.mean(1)).mean()) > 0.2     # learned that the reward is positive
    sc = m._implicit_verify(torch.randn(3, HIDDEN), torch.randn(3, HIDDEN))
    assert bool(((sc > 0) & (sc < 1)).all())
    early, late = m._layer_entropy_control(torch.ones(1, HIDDEN), 0, 10), m._layer_entropy_control(torch.ones(1, HIDDEN), 9, 10)
    assert float(early.mean()) > 1.0 > float(late.mean())


def test_adaptive_controller_respects_the_budget():
    torch.manual_seed(0)
    c = YvAdaptiveReasoningController(HIDDEN, max_depth=12)
    hs = torch.randn(4, 20, HIDDEN)
    free = c(hs, budget_constraint=1.0)
    tight = c(hs, budget_constraint=0.05)
    assert tuple(free["optimal_depth"].shape) == (4,) and int(free["optimal_depth"].min()) >= 1
    assert int(free["optimal_depth"].max()) <= 12 and bool(free["budget_compliance"].all())
    assert bool((tight["optimal_depth"] <= free["optimal_depth"]).all()) and not bool(tight["budget_compliance"].any())
    assert len(free["strategy_name"]) == 4 and set(free["strategy_name"]) <= set(c.STRATEGIES)


def test_latent_cot_reasoner_with_memory_and_loss():
    torch.manual_seed(0)
    r = YvLatentCoTReasoner(_cfg()).eval()
    hs = torch.randn(2, 16, HIDDEN)
    out = r(hs)
    assert tuple(out["thinking_logits"].shape) == (2, VOCAB) and tuple(out["difficulty_logits"].shape) == (2, 5)
    assert tuple(out["reflection_logits"].shape) == (2, 4) and tuple(out["confidence_score"].shape) == (2, 1)
    assert tuple(out["correction_logits"].shape) == (2, HIDDEN) and tuple(out["reasoning_states"].shape) == (2, 16, HIDDEN)
    mem = [torch.randn(HIDDEN) for _ in range(5)]
    with_mem = r(hs, memory_context=mem)
    assert not torch.allclose(with_mem["thinking_logits"], out["thinking_logits"])
    with pytest.raises(ValueError):
        r(torch.randint(0, VOCAB, (2, 16)))
    labels = torch.randint(0, VOCAB, (2, 16))
    r.train()
    loss = r(hs, labels=labels)["loss"]
    assert float(loss) > 0
    loss.backward()
    assert r.thinking_head.weight.grad is not None


def test_unified_reasoner_routes_and_keeps_one_format():
    torch.manual_seed(0)
    u = YvLatentUnifiedReasoner(_cfg(mpr_seq_len_threshold=24)).eval()
    short, long_ = torch.randn(2, 12, HIDDEN), torch.randn(2, 40, HIDDEN)
    a, b = u(hidden_states=short), u(long_)
    assert a["route"] == "cot" and b["route"] == "multi_path"
    for o in (a, b):
        assert tuple(o["thinking_logits"].shape) == (2, VOCAB) and tuple(o["confidence_score"].shape) == (2, 1)
        assert tuple(o["thinking_depth"].shape) == (2,) and set(o["thinking_depth"].tolist()) <= {1, 3, 5, 10}
        assert "loss" in o and tuple(o["difficulty_logits"].shape) == (2, 5)
    with pytest.raises(ValueError):
        u(torch.randint(0, VOCAB, (2, 12)))
    u.routing = "blend"
    c = u(short)
    assert c["route"] == "blend" and tuple(c["thinking_logits"].shape) == (2, VOCAB)
    u.train()
    labels = torch.randint(0, VOCAB, (2, 40))
    out = u(long_, labels, labels=labels)                        # integer second argument: the token ids
    out["loss"].backward()
    assert u.multi_path_core.thinking_head.weight.grad is not None
    assert not u._should_use_multi_path(short) or u.routing != "length"


def test_latent_refinement_and_sampling():
    torch.manual_seed(0)
    u = YvLatentUnifiedReasoner(_cfg()).eval()
    r = u.reason_latent(torch.randn(3, 10, HIDDEN), max_depth=4)
    assert tuple(r["refined_hidden"].shape) == (3, HIDDEN) and tuple(r["reasoning_trace"].shape) == (3, 4)
    assert bool((r["num_iterations"] <= r["thinking_budget"].clamp_max(4)).all()) and int(r["num_iterations"].min()) >= 1
    lg = torch.full((2, 50), -10.0)
    lg[0, 7], lg[1, 9] = 10.0, 10.0
    assert u._sample_next_token(lg, temperature=0.0).tolist() == [7, 9]
    assert u._sample_next_token(lg, temperature=0.7, top_p=0.9, top_k=5).tolist() == [7, 9]


def test_generate_with_thinking_closes_the_span():
    torch.manual_seed(0)
    cfg = _cfg(vocab_size=300)
    u = YvLatentUnifiedReasoner(cfg).eval()
    emb = torch.nn.Embedding(300, HIDDEN)

    class Tok:
        eos_token_id = 0

        def encode(self, s):
            return [1 + (b % 250) for b in s.encode()]

        def decode(self, ids):
            return "".join(chr((i - 1) % 250) if 32 <= (i - 1) % 250 < 127 else "?" for i in ids)

    text = u.generate_with_thinking("2+2", Tok(), emb, max_new_tokens=24, max_think_tokens=6, temperature=0.0)
    assert text.startswith("<|think|>") and "</|think|>" in text
