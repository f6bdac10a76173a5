"""Named evaluation suites on top of the two generic harnesses (reference tools/benchmark/*: MMLU, GSM8K, AIME,
HumanEval, SWE-bench, long-context, agent and multimodal harnesses).  Data sets are read from local JSONL files (there
is no network at run time); every suite documents the row format it expects and returns a plain dict of metrics."""
from __future__ import annotations

import math
import os
import re
import subprocess
import sys
import tempfile
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence

from .benchmark import PiscesLxGenerativeHarness, PiscesLxMultipleChoiceHarness, needle_in_haystack_rows, read_jsonl

GenerateFn = Callable[[str, int], str]


def pass_at_k(n: int, c: int, k: int) -> float:
    """Unbiased pass@k estimator: 1 - C(n-c, k) / C(n, k) for n samples of which c passed."""
    if n - c < k:
        return 1.0
    return 1.0 - math.prod(1.0 - k / i for i in range(n - c + 1, n + 1))


def last_number(text: str) -> Optional[str]:
    m = re.findall(r"-?\d[\d,]*\.?\d*", text.replace("$", ""))
    return m[-1].replace(",", "").rstrip(".") if m else None


class PiscesLxMMLUBenchmark:
    """Rows: {"question", "choices": [4 strings], "answer": index, "subject"}.  Few-shot examples (same format) are
    prepended to every question; accuracy is reported overall and per subject."""

    LETTERS = "ABCD"

    def __init__(self, model: Any, tokenizer: Any, shots: Sequence[Dict[str, Any]] = ()):
        self.h, self.shots = PiscesLxMultipleChoiceHarness(model, tokenizer), list(shots)

    def format(self, r: Dict[str, Any], with_answer: bool) -> str:
        s = r["question"] + "\n" + "\n".join(f"{self.LETTERS[i]}. {c}" for i, c in enumerate(r["choices"]))
        return s + (f"\nAnswer: {self.LETTERS[int(r['answer'])]}\n\n" if with_answer else "")

    def evaluate(self, rows: Iterable[Dict[str, Any]]) -> Dict[str, Any]:
        prefix = "".join(self.format(s, True) for s in self.shots)
        per: Dict[str, List[int]] = {}
        for r in rows:
            q = {"question": prefix + self.format(r, False), "choices": [f"{l}" for l in self.LETTERS[: len(r["choices"])]],
                 "answer": r["answer"]}
            ok = self.h.evaluate([q])["accuracy"] == 1.0
            per.setdefault(r.get("subject", "all"), []).append(int(ok))
        flat = [x for v in per.values() for x in v]
        return {"accuracy": sum(flat) / max(len(flat), 1), "n": len(flat),
                "by_subject": {k: sum(v) / len(v) for k, v in per.items()}}


class PiscesLxGSM8KBenchmark:
    """Rows: {"question", "answer"} where the reference answer ends in ``#### <number>``; the model's last number counts."""

    def __init__(self, generate: GenerateFn, shots: str = ""):
        self.h = PiscesLxGenerativeHarness(generate, extract=lambda s: last_number(s) or "")
        self.shots = shots

    def evaluate(self, rows: Iterable[Dict[str, Any]], max_new_tokens: int = 256) -> Dict[str, float]:
        prepared = [{"prompt": f"{self.shots}Question: {r['question']}\nLet's think step by step.\n",
                     "answer": str(r["answer"]).split("####")[-1].strip().replace(",", "")} for r in rows]
        return self.h.evaluate(prepared, max_new_tokens)


class PiscesLxAIMEBenchmark(PiscesLxGSM8KBenchmark):
    """Rows: {"problem", "answer"} with integer answers 0..999; majority vote over ``samples`` generations."""

    def __init__(self, generate: GenerateFn, samples: int = 1):
        super().__init__(generate)
        self.samples, self.generate = samples, generate

    def evaluate(self, rows: Iterable[Dict[str, Any]], max_new_tokens: int = 1024) -> Dict[str, float]:
        n = correct = 0
        for r in rows:
            votes: Dict[str, int] = {}
            for _ in range(self.samples):
                a = last_number(self.generate(f"Problem: {r['problem']}\nSolve it and give the final integer.\n", max_new_tokens))
                if a is not None:
                    a = str(int(float(a))) if re.fullmatch(r"-?\d+\.?0*", a) else a
                    votes[a] = votes.get(a, 0) + 1
            pick = max(votes.items(), key=lambda kv: kv[1])[0] if votes else ""
            correct += int(pick == str(int(r["answer"])))
            n += 1
        return {"accuracy": correct / max(n, 1), "n": n}


class PiscesLxHumanEvalBenchmark:
    """Rows: {"task_id", "prompt", "test", "entry_point"}.  Each completion is appended to the prompt and run with the
    task's tests in a child interpreter with a time limit and an empty environment; pass@k from ``n_samples``."""

    def __init__(self, generate: GenerateFn, n_samples: int = 1, timeout_s: float = 10.0):
        self.generate, self.n, self.timeout = generate, n_samples, timeout_s

    def run_candidate(self, program: str) -> bool:
        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, "candidate.py")
            with open(path, "w") as f:
                f.write(program)
            try:
                r = subprocess.run([sys.executable, "-I", path], cwd=d, env={}, capture_output=True, timeout=self.timeout)
                return r.returncode == 0
            except subprocess.TimeoutExpired:
                return False

    @staticmethod
    def truncate(completion: str) -> str:
        """Keep the function body: stop at the first top-level statement after it."""
        out = []
        for line in completion.splitlines():
            if out and line and not line[0].isspace() and not line.startswith(("#", ")")):
                break
            out.append(line)
        return "\n".join(out)

    def evaluate(self, rows: Iterable[Dict[str, Any]], ks: Sequence[int] = (1,), max_new_tokens: int = 512) -> Dict[str, float]:
        per_task = []
        for r in rows:
            c = 0
            for _ in range(self.n):
                body = self.truncate(self.generate(r["prompt"], max_new_tokens))
                prog = f"{r['prompt']}{body}\n\n{r['test']}\n\ncheck({r['entry_point']})\n"
                c += int(self.run_candidate(prog))
            per_task.append(c)
        out = {"n": len(per_task)}
        for k in ks:
            if k <= self.n:
                out[f"pass@{k}"] = sum(pass_at_k(self.n, c, k) for c in per_task) / max(len(per_task), 1)
        return out


class PiscesLxSWEBenchFormatChecker:
    """Offline part of a SWE-bench run: checks that a generation is a well-formed unified diff touching files that
    exist in the task's repository snapshot (applying and testing the patch needs the task's container, which an
    offline box does not have)."""

    HUNK = re.compile(r"^@@ -\d+(,\d+)? \+\d+(,\d+)? @@", re.M)

    def check(self, patch: str, repo_files: Iterable[str]) -> Dict[str, Any]:
        files = re.findall(r"^\+\+\+ b/(.+)$", patch, re.M)
        known = set(repo_files)
        return {"is_diff": bool(files) and bool(self.HUNK.search(patch)), "files": files,
                "unknown_files": [f for f in files if f not in known]}

    def evaluate(self, rows: Iterable[Dict[str, Any]], generate: GenerateFn, max_new_tokens: int = 1024) -> Dict[str, float]:
        n = ok = 0
        for r in rows:
            res = self.check(generate(r["problem_statement"], max_new_tokens), r.get("repo_files", []))
            ok += int(res["is_diff"] and not res["unknown_files"])
            n += 1
        return {"well_formed_patch_rate": ok / max(n, 1), "n": n}


class PiscesLxLongContextBenchmark:
    """Needle-in-a-haystack retrieval at several context lengths and depths."""

    def __init__(self, generate: GenerateFn, tokenizer: Any):
        self.generate, self.tok = generate, tokenizer

    def evaluate(self, lengths: Sequence[int] = (1024, 8192, 32768), depths: Sequence[float] = (0.1, 0.5, 0.9)) -> Dict[str, Any]:
        grid = {}
        h = PiscesLxGenerativeHarness(self.generate, extract=lambda s: last_number(s) or "")
        for L in lengths:
            for row in needle_in_haystack_rows(self.tok, L, depths):
                grid[f"{L}@{row['depth']}"] = h.evaluate([row], 16)["exact_match"]
        return {"retrieval": grid, "mean": sum(grid.values()) / max(len(grid), 1)}


class PiscesLxAgentBenchmark:
    """Rows: {"task", "expect_tool": name, "expect_in_answer": text}.  Runs the agent (anything with ``run(task) ->
    {"answer", "steps"}``) and scores tool selection and the final answer."""

    def __init__(self, agent_factory: Callable[[], Any]):
        self.agent_factory = agent_factory

    def evaluate(self, rows: Iterable[Dict[str, Any]]) -> Dict[str, float]:
        n = tool_ok = ans_ok = 0
        turns = 0
        for r in rows:
            out = self.agent_factory().run(r["task"])
            used = [s.get("tool") for s in out.get("steps", []) if isinstance(s, dict)]
            tool_ok += int(r.get("expect_tool") in used) if r.get("expect_tool") else 1
            ans_ok += int(str(r.get("expect_in_answer", "")).lower() in str(out.get("answer", "")).lower())
            turns += len(out.get("steps", []))
            n += 1
        return {"tool_selection": tool_ok / max(n, 1), "answer_rate": ans_ok / max(n, 1), "mean_turns": turns / max(n, 1), "n": n}


class PiscesLxVQABenchmark:
    """Rows: {"image": tensor or path, "question", "answers": [strings]}; ``answer_fn(image, question) -> str``.  VQA
    accuracy: min(1, matches / 3) over the annotator answers."""

    def __init__(self, answer_fn: Callable[[Any, str], str]):
        self.answer_fn = answer_fn

    def evaluate(self, rows: Iterable[Dict[str, Any]]) -> Dict[str, float]:
        n, score = 0, 0.0
        for r in rows:
            a = self.answer_fn(r["image"], r["question"]).strip().lower()
            score += min(1.0, sum(1 for x in r["answers"] if x.strip().lower() == a) / 3.0)
            n += 1
        return {"vqa_accuracy": score / max(n, 1), "n": n}


def load_suite_rows(path: str, limit: Optional[int] = None) -> List[Dict[str, Any]]:
    rows = read_jsonl(path)
    return rows[:limit] if limit else rows


# --------------------------------------------------------------------------------------------------
# suite registry used by ``manage.py benchmark --benchmark NAME | --list | --selftest``
# --------------------------------------------------------------------------------------------------
_SELFTEST_ROWS = {
    "mmlu": [{"question": "2 + 2 = ?", "choices": ["3", "4", "5", "6"], "answer": 1, "subject": "arithmetic"},
             {"question": "The capital of France is", "choices": ["Paris", "Rome", "Oslo", "Bern"], "answer": 0, "subject": "geography"}],
    "gsm8k": [{"question": "Tom has 3 apples and buys 4 more. How many apples does he have?", "answer": "3 + 4 = 7 #### 7"}],
    "aime": [{"question": "Find 10 * 12.", "answer": "120"}],
}


def available_suites() -> List[str]:
    return ["mmlu", "gsm8k", "aime", "humaneval", "needle"]


def _generate_fn(model: Any, tokenizer: Any) -> GenerateFn:
    import torch

    def gen(prompt: str, max_new_tokens: int = 64) -> str:
        dev = next(model.parameters()).device
        ids = torch.tensor([tokenizer.encode(prompt)], dtype=torch.long, device=dev).clamp_(0, model.cfg.vocab_size - 1)
        out, _ = model.generate(ids, max_new_tokens=max_new_tokens)
        return tokenizer.decode(out[0, ids.shape[1]:].tolist())
    return gen


def run_suite(name: str, model: Any, tokenizer: Any = None, data_path: Optional[str] = None,
              max_samples: Optional[int] = None) -> Dict[str, Any]:
    """Evaluate ``model`` on suite ``name``.  Rows come from ``data_path`` (jsonl in the suite's row format) or, without
    one, from the built-in smoke rows: enough to exercise the harness end to end, not a score to report."""
    from ..models.tokenizer import YvTokenizer
    vocab = int(getattr(getattr(model, "cfg", None), "vocab_size", 0) or 0)
    tok = tokenizer or (YvTokenizer.for_vocab(vocab) if vocab else YvTokenizer.instance())
    name = name.lower()
    if name not in available_suites():
        raise ValueError(f"unknown suite {name!r}; available: {', '.join(available_suites())}")
    rows = load_suite_rows(data_path, max_samples) if data_path else list(_SELFTEST_ROWS.get(name, []))[: max_samples or None]
    gen = _generate_fn(model, tok)
    if name == "mmlu":
        res = PiscesLxMMLUBenchmark(model, tok).evaluate(rows)
    elif name == "gsm8k":
        res = PiscesLxGSM8KBenchmark(gen).evaluate(rows, 32)
    elif name == "aime":
        res = PiscesLxAIMEBenchmark(gen).evaluate(rows, 32)
    elif name == "humaneval":
        res = PiscesLxHumanEvalBenchmark(gen).evaluate(rows) if rows else {"pass@1": 0.0, "n": 0}
    else:
        res = PiscesLxLongContextBenchmark(gen, tok).evaluate(lengths=(256,), depths=(0.5,))
    return {"suite": name, "rows": len(rows), "source": data_path or "built-in smoke rows", "result": res}


def selftest() -> Dict[str, Any]:
    """Exercise the scoring code without a model: answer extraction, pass@k, the patch-format checker."""
    checks = {
        "last_number": last_number("so the total is 1,234 apples") in ("1234", "1,234"),
        "pass_at_k": abs(pass_at_k(10, 3, 1) - 0.3) < 1e-9 and pass_at_k(5, 5, 2) == 1.0,
        "gsm8k_scoring": PiscesLxGSM8KBenchmark(lambda p, n=0: "the answer is 7").evaluate(_SELFTEST_ROWS["gsm8k"])["exact_match"] == 1.0,
    }
    return {"ok": all(checks.values()), "checks": checks}
