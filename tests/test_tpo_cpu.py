"""Test-time preference optimisation: reward parsing, the iterative loop with its feedback kinds, best-of-n, batching."""
import pytest

from pisceslx_b200.serve import tpo as T


def test_reward_parsing():
    p = T.parse_reward
    assert p("0.7") == 0.7 and p("Score: .25 because") == 0.25 and p("7/10") == pytest.approx(0.7) and p("85%") == pytest.approx(0.85)
    assert p("8") == pytest.approx(0.8) and p("90") == pytest.approx(0.9) and p("1") == 1.0 and p(0.3) == 0.3 and p(7) == 1.0
    assert p("The answer is good and correct, though one part is wrong.") == pytest.approx(2 / 3)
    assert p("no idea") == 0.0 and p("hmm") == 0.5 and p("version v2.x") == 0.5


class Script:
    """A scripted policy / critic / judge: answers get better when the prompt carries feedback."""

    def __init__(self):
        self.prompts = []

    def __call__(self, prompt, temperature=0.7, **kw):
        self.prompts.append((prompt, temperature))
        if "Rate how well" in prompt:
            if "v3" in prompt:
                return "0.95"
            return "0.6" if "v2" in prompt else "0.2"
        if "Evaluate the following response" in prompt:
            return "Be shorter."
        n = prompt.count("needs improvement")
        return ["answer v1", "answer v2", "answer v3"][min(n + ("Be shorter" in prompt) - (n > 0), 2)] if n else "answer v1"


def test_iterative_alignment_improves_and_stops_early():
    s = Script()
    calls = {"n": 0}

    def policy(prompt, **kw):
        calls["n"] += 1
        if "Rate how well" in prompt or "Evaluate the following" in prompt:
            return s(prompt, **kw)
        return f"answer v{calls['n']}"

    calls["n"] = 0
    gen_only = {"k": 0}

    def gen(prompt, **kw):
        gen_only["k"] += 1
        return f"answer v{gen_only['k']}"
    op = T.PiscesLxTPOOperator(T.PiscesLxTPOConfig(max_iterations=5, reward_threshold=0.9))
    resp, st = op.align_at_inference(gen, "Explain X.", T.PiscesLxTPOPreferenceLibrary.RESPONSE_CONCISE, feedback=s, reward=s)
    assert resp == "answer v3" and st["iterations"] == 3 and st["early_stopped"] and st["reward_history"] == [0.2, 0.6, 0.95]
    assert st["feedback"] == ["Be shorter.", "Be shorter."] and st["final_reward"] == 0.95
    assert op.calls == {"generate": 3, "feedback": 2, "reward": 3}
    judge_temps = [t for p, t in s.prompts if "Rate how well" in p]
    assert judge_temps and all(t == 0.0 for t in judge_temps)                      # the judge and the critic are greedy
    seen = []
    T.PiscesLxTPOOperator().align_at_inference(lambda p, **kw: (seen.append(p), "x")[1], "Q", "pref", T.PiscesLxTPOConfig(max_iterations=2),
                                               feedback=lambda p, **kw: "FB", reward=lambda p, **kw: "0.1")
    assert seen[0] == "Q" and seen[1].startswith("Q\n\n") and "Feedback: FB" in seen[1] and "Original response: x" in seen[1]


def test_feedback_kinds_scalar_and_comparative():
    outs = iter(["bad answer", "better answer", "best answer"])
    rewards = iter(["0.3", "0.1", "0.5"])
    seen = []

    def gen(prompt, **kw):
        seen.append(prompt)
        return next(outs)
    op = T.PiscesLxTPOOperator(T.PiscesLxTPOConfig(max_iterations=3, feedback_type="comparative", early_stopping=False))
    resp, st = op.align_at_inference(gen, "Q", "pref", reward=lambda p, **kw: next(rewards), feedback=lambda p, **kw: 1 / 0)
    assert resp == "best answer" and st["final_reward"] == 0.5 and op.calls["feedback"] == 0
    assert "scored 0.30" in seen[1] and "A weaker response was:\nbetter answer" in seen[2] and "A stronger response was:\nbad answer" in seen[2]
    op2 = T.PiscesLxTPOOperator(T.PiscesLxTPOConfig(max_iterations=2, feedback_type="scalar"))
    seen2 = []
    op2.align_at_inference(lambda p, **kw: (seen2.append(p), "r")[1], "Q", "pref", reward=lambda p, **kw: "0.4")
    assert "scored 0.40 out of 1" in seen2[1]
    with pytest.raises(ValueError):
        T.PiscesLxTPOConfig(feedback_type="vibes")
    with pytest.raises(ValueError):
        T.PiscesLxTPOConfig(max_iterations=0)


class Batched:
    def __init__(self):
        self.batches = []

    def __call__(self, prompt, **kw):
        return "single"

    def generate_batch(self, prompts, **kw):
        self.batches.append(list(prompts))
        return [f"{p}#{i}" for i, p in enumerate(prompts)]


def test_best_of_n_and_batching():
    g = Batched()
    judge = lambda p, **kw: "0.9" if "#2" in p or "#5" in p else "0.1"
    al = T.PiscesLxTPOAligner(g, T.PiscesLxTPOConfig(use_best_of_n=True, n_candidates=4), reward=judge)
    resp, st = al.align("P", "pref")
    assert resp == "P#2" and st["mode"] == "best_of_n" and len(st["responses"]) == 4 and g.batches == [["P"] * 4]
    al.set_preference_templates({"short": T.PiscesLxTPOPreferenceLibrary.RESPONSE_CONCISE})
    outs = al.align_batch(["A", "B"], "short")
    assert len(g.batches) == 2 and g.batches[1] == ["A"] * 4 + ["B"] * 4                # one call for every candidate of every prompt
    assert [o[0] for o in outs] == ["A#2", "B#5"] and outs[1][1]["final_reward"] == 0.9
    resp2, st2 = al.align("P", "pref", use_best_of_n=False, max_iterations=1)
    assert resp2 == "single" and st2["iterations"] == 1
    with pytest.raises(TypeError):
        al.align("P", "pref", beam=3)
    it = al.align_batch(["A", "B"], "pref", use_best_of_n=False, max_iterations=1)
    assert [o[0] for o in it] == ["single", "single"]


def test_operator_front_and_library():
    op = T.PiscesLxTPOOperator()
    r = op.execute({"generate": lambda p, **kw: "0.9" if "Rate" in p else "ok", "prompt": "Q", "preference": "pref", "config": {"max_iterations": 2}})
    assert r.is_success() and r.output["response"] == "ok" and r.output["early_stopped"] and r.output["iterations"] == 1
    assert not op.execute({"generate": None, "prompt": "Q", "preference": "p"}).is_success()
    L = T.PiscesLxTPOPreferenceLibrary
    assert L.combine(L.RESPONSE_CONCISE, L.RESPONSE_SAFE) == "Response should be concise and to the point and Response should be safe and not contain harmful content"
    assert L.custom("x") == "x" and "MATH_STEP_BY_STEP" in L.names() and len(L.names()) == 10
