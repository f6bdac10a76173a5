"""CPU tests of the named evaluation suites with scripted generators (no model weights needed)."""
from __future__ import annotations

import math

from pisceslx_b200.tools.benchmark_suites import (PiscesLxAgentBenchmark, PiscesLxAIMEBenchmark, PiscesLxGSM8KBenchmark,
                                                  PiscesLxHumanEvalBenchmark, PiscesLxLongContextBenchmark,
                                                  PiscesLxSWEBenchFormatChecker, PiscesLxVQABenchmark, last_number,
                                                  pass_at_k)


def test_pass_at_k_and_number_extraction():
    assert pass_at_k(10, 0, 1) == 0.0 and pass_at_k(10, 10, 1) == 1.0
    assert abs(pass_at_k(10, 3, 1) - 0.3) < 1e-12
    assert abs(pass_at_k(5, 2, 2) - (1 - math.comb(3, 2) / math.comb(5, 2))) < 1e-12
    assert pass_at_k(4, 3, 2) == 1.0
    assert last_number("so 1,250 apples cost $3.50.") == "3.50" and last_number("none") is None
    assert last_number("The total is 1,234.") == "1234"


def test_gsm8k_and_aime():
    gen = lambda p, n: "6 * 7 = 42. The answer is 42." if "six" in p else "I think 13"
    rows = [{"question": "six times seven?", "answer": "blah #### 42"}, {"question": "two plus two?", "answer": "#### 4"}]
    assert PiscesLxGSM8KBenchmark(gen).evaluate(rows) == {"exact_match": 0.5, "n": 2}
    votes = iter(["answer 17", "answer 204", "so 204.0", "204"])
    aime = PiscesLxAIMEBenchmark(lambda p, n: next(votes), samples=4)
    assert aime.evaluate([{"problem": "p", "answer": 204}]) == {"accuracy": 1.0, "n": 1}


def test_humaneval_runs_candidates_in_a_child_interpreter():
    rows = [{"task_id": "t/0", "prompt": "def add(a, b):\n", "entry_point": "add",
             "test": "def check(f):\n    assert f(2, 3) == 5\n    assert f(-1, 1) == 0\n"}]
    good = PiscesLxHumanEvalBenchmark(lambda p, n: "    return a + b\n\nprint('trailing text the model added')\n", n_samples=2)
    assert good.evaluate(rows, ks=(1, 2)) == {"n": 1, "pass@1": 1.0, "pass@2": 1.0}
    bad = PiscesLxHumanEvalBenchmark(lambda p, n: "    return a - b\n")
    assert bad.evaluate(rows)["pass@1"] == 0.0
    hang = PiscesLxHumanEvalBenchmark(lambda p, n: "    while True:\n        pass\n", timeout_s=1.0)
    assert hang.evaluate(rows)["pass@1"] == 0.0
    assert good.truncate("    return 1\nclass X:\n    pass") == "    return 1"


def test_swe_format_long_context_agent_and_vqa():
    chk = PiscesLxSWEBenchFormatChecker()
    patch = "--- a/pkg/mod.py\n+++ b/pkg/mod.py\n@@ -1,2 +1,2 @@\n-x = 1\n+x = 2\n"
    assert chk.check(patch, ["pkg/mod.py"]) == {"is_diff": True, "files": ["pkg/mod.py"], "unknown_files": []}
    assert chk.check(patch, ["other.py"])["unknown_files"] == ["pkg/mod.py"]
    assert not chk.check("just prose", [])["is_diff"]
    r = chk.evaluate([{"problem_statement": "fix", "repo_files": ["pkg/mod.py"]}], lambda p, n: patch)
    assert r["well_formed_patch_rate"] == 1.0

    class Tok:
        def encode(self, s):
            return s.split()
    lc = PiscesLxLongContextBenchmark(lambda p, n: "7319" if "pass code is 7319" in p else "0", Tok())
    out = lc.evaluate(lengths=(64, 256), depths=(0.5,))
    assert out["mean"] == 1.0 and set(out["retrieval"]) == {"64@0.5", "256@0.5"}

    class Agent:
        def run(self, task):
            return {"answer": "It is 4.", "steps": [{"tool": "calc"}, {"tool": None}]}
    ab = PiscesLxAgentBenchmark(Agent).evaluate([{"task": "2+2", "expect_tool": "calc", "expect_in_answer": "4"},
                                                 {"task": "x", "expect_tool": "search", "expect_in_answer": "4"}])
    assert ab == {"tool_selection": 0.5, "answer_rate": 1.0, "mean_turns": 2.0, "n": 2}
    vqa = PiscesLxVQABenchmark(lambda img, q: "Red")
    assert abs(vqa.evaluate([{"image": None, "question": "colour?", "answers": ["red", "red", "crimson"]}])["vqa_accuracy"] - 2 / 3) < 1e-9
