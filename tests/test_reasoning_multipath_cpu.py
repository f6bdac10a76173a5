"""Multi-modal reasoning enhancer, prompt-level multi-path inference and its meta learner."""
import types

import pytest
import torch

from pisceslx_b200.models.reasoning_multipath import (YvMultiModalReasoningEnhancer, YvMultiPathInferenceEngine,
                                                      YvMultiPathMetaLearner)

H = 32


def _cfg(**kw):
    return types.SimpleNamespace(hidden_size=H, n_head=8, extra=kw)


def test_enhancer_modalities_move_the_state():
    torch.manual_seed(0)
    e = YvMultiModalReasoningEnhancer(_cfg()).eval()
    text, vis, aud, tmp = torch.randn(2, 10, H), torch.randn(2, 6, H), torch.randn(2, 4, H), torch.randn(2, 5, H)
    s0, c0 = e(text)
    assert tuple(s0.shape) == (2, 1, H) and tuple(c0.shape) == (2, 1) and bool(((c0 > 0) & (c0 < 1)).all())
    s1, _ = e(text, visual_features=vis)
    s2, _ = e(text, visual_features=vis, audio_features=aud)
    s3, _, inter = e(text, vis, aud, tmp, return_intermediates=True)
    assert not torch.allclose(s0, s1) and not torch.allclose(s1, s2) and not torch.allclose(s2, s3)
    assert inter["modal_contributions"] == {"visual": 0.3, "audio": 0.2} and len(inter["step_outputs"]) == 4
    assert tuple(inter["step_outputs"][0]["state_change"].shape) == (2,) and inter["used_linear_attention"] is False


def test_enhancer_long_branch_still_uses_the_modality():
    torch.manual_seed(0)
    e = YvMultiModalReasoningEnhancer(_cfg(enhancer_linear_attention_tokens=8)).eval()
    text = torch.randn(1, 12, H)
    a, _, inter = e(text, visual_features=torch.randn(1, 3, H), return_intermediates=True)
    b, _ = e(text, visual_features=torch.randn(1, 3, H))
    assert inter["used_linear_attention"] is True and not torch.allclose(a, b)
    e.train()
    s, c = e(text, torch.randn(1, 3, H), torch.randn(1, 3, H), torch.randn(1, 2, H))
    (s.sum() + c.sum()).backward()
    assert e.cross_modal_reasoner["efficient_gate"].weight.grad is not None


GOOD = ("First we note the tank holds ten litres. Because the pump adds two litres per minute, the tank fills in five "
        "minutes. Therefore the tank is full after five minutes. Finally we check that two times five is ten.")
BAD = "The tank is full. The tank is not full."


def test_inference_engine_scores_and_stops():
    calls = []

    def gen(prompt, temperature=0.7):
        calls.append((prompt, temperature))
        return GOOD if "Reason again" in prompt or temperature < 0.4 else BAD

    eng = YvMultiPathInferenceEngine(gen, max_depth=3, confidence_threshold=0.8)
    assert eng._check_self_consistency(BAD) < eng._check_self_consistency(GOOD) == 1.0
    assert eng._check_causal_consistency(GOOD) > eng._check_causal_consistency(BAD)
    assert eng._check_temporal_consistency("Finally we start. First we end.") == 0.3
    assert 0 <= eng._check_logical_validity("If it rains then the road is wet.") <= 1
    meta = eng.multi_path_reason("How long until the tank is full?", return_metadata=True)
    assert meta["answer"] == GOOD and meta["confidence"] >= 0.8 and meta["reasoning_depth"] == 1
    assert len(meta["uncertainty_evolution"]) == 1 and len(calls) == 3         # three temperatures in round 0
    n = len(calls)
    assert eng.multi_path_reason("How long until the tank is full?") == GOOD and len(calls) == n   # cached


def test_inference_engine_deepens_when_unsure_and_uses_the_callables():
    def gen(prompt, temperature=0.7):
        return GOOD if "Reason again" in prompt else BAD

    emb = lambda s: torch.tensor([float(len(s)), float(s.count("tank")), 1.0])
    lp = lambda prompt, text: torch.log_softmax(torch.tensor([[4.0, 0.0, 0.0]] * 5), -1)
    eng = YvMultiPathInferenceEngine(gen, max_depth=4, confidence_threshold=0.8, embed=emb, token_logprobs=lp)
    meta = eng.multi_path_reason("q", return_metadata=True)
    assert meta["reasoning_depth"] == 2 and meta["answer"] == GOOD
    assert meta["uncertainty_evolution"][0] > meta["uncertainty_evolution"][1]
    assert 0.5 < eng._measure_uncertainty_reduction("q", "x") <= 1.0
    assert 0.0 <= eng._estimate_logical_consistency(GOOD) <= 1.0


def test_meta_learner_patterns_parameters_and_priors():
    ml = YvMultiPathMetaLearner(hidden_size=64, min_support=6)
    assert ml.extract_reasoning_patterns() is None and ml.create_reasoning_prior("anything") is None
    with pytest.raises(ValueError):
        ml.adapt_reasoning_parameters(None)
    for i in range(8):
        deco = i % 2 == 0
        ml.record_reasoning(f"how long does tank {i} take to fill", ["Let us break down the problem" if deco else "The answer is"],
                            "5", {"reasoning_depth": 4 if deco else 2, "confidence": 0.9 if deco else 0.6,
                                  "uncertainty_evolution": [0.6, 0.3, 0.1] if deco else [0.5, 0.4]})
    pat = ml.extract_reasoning_patterns()
    assert pat["optimal_depth_distribution"]["mean_depth"] == 3.0 and pat["support"] == 8
    assert pat["confidence_indicators"]["confidence_growth"] == pytest.approx((0.5 + 0.1) / 2)
    rates = pat["reasoning_strategies"]["strategy_success_rates"]
    assert rates["decomposition"] == pytest.approx(0.9) and rates["direct"] == pytest.approx(0.6)
    params = ml.adapt_reasoning_parameters(pat)
    assert params["max_depth"] == 3 and params["confidence_threshold"] >= 0.7
    assert params["preferred_strategies"][0] == "decomposition"
    eng = YvMultiPathInferenceEngine(lambda p, temperature=0.7: "x")
    assert ml.apply_to(eng) == params and eng.max_depth == 3
    prior = ml.create_reasoning_prior("how long does tank 3 take to fill")
    assert prior["num_similar"] >= 1 and 2 <= prior["expected_depth"] <= 4
    assert len(prior["uncertainty_pattern"]["typical_pattern"]) == 3
    assert ml.create_reasoning_prior("zzzz qqqq xxxx", min_similarity=0.9) is None
    assert torch.allclose(ml._embed_query("abc"), ml._embed_query("abc")) and float(ml._embed_query("abc").norm()) == pytest.approx(1.0)
