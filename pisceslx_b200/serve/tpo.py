"""Test-time preference optimisation in full (reference opss/infer/tpo.py:76-777): align an answer with a stated
preference at inference time, without touching the weights, by iterating generate -> score -> critique -> refine, or by
best-of-n.

``serve/runtime.py::PiscesLxTPO`` is the minimal loop; this module is the configured operator with prompts, reward
parsing, early stopping, statistics, batch alignment and the preference library.  The models are callables:

  * ``generate(prompt, temperature=..., max_new_tokens=..., top_p=..., top_k=...) -> str`` - the policy;
  * optional ``feedback(prompt, ...) -> str`` and ``reward(prompt, ...) -> str | float`` - a critic and a judge
    (the policy itself when not given, as in the reference).

With a batch-capable generator (``generate_batch(prompts, ...) -> list[str]``, e.g. the serving engine, which runs the
candidates in one continuous batch) best-of-n and ``align_batch`` issue ONE call per phase instead of one per
candidate; the reference generates candidates one after another (tpo.py:385-399)."""
from __future__ import annotations

import re
from dataclasses import dataclass, field, replace
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

from ..utils.opsc import PiscesLxOperatorInterface

TextFn = Callable[..., Any]


class PiscesLxTPOFeedbackType(str, Enum):
    TEXTUAL = "textual"          # a written critique goes into the refined prompt
    SCALAR = "scalar"            # only the score does ("the answer scored 0.4 of 1")
    COMPARATIVE = "comparative"  # the best and the worst answer so far are shown side by side


@dataclass
class PiscesLxTPOConfig:
    name: str = "tpo"
    max_iterations: int = 3
    temperature: float = 0.7
    reward_threshold: float = 0.8
    feedback_type: str = "textual"
    use_best_of_n: bool = False
    n_candidates: int = 4
    early_stopping: bool = True
    max_new_tokens: int = 512
    top_p: float = 0.95
    top_k: int = 50
    improvement_prompt: str = ("The following response needs improvement based on the preference: {preference}\n\n"
                               "Original response: {response}\n\nFeedback: {feedback}\n\n"
                               "Please provide an improved response that better aligns with the preference:")
    feedback_prompt: str = ("Evaluate the following response based on the given preference.\n\nPreference: {preference}\n\n"
                            "Response: {response}\n\nProvide specific feedback on how to improve the response to better match the "
                            "preference. Focus on concrete, actionable suggestions.")
    reward_prompt: str = ("Rate how well the following response matches the given preference on a scale of 0 to 1.\n\n"
                          "Preference: {preference}\n\nResponse: {response}\n\nOutput only a single number between 0 and 1:")

    def __post_init__(self) -> None:
        self.feedback_type = PiscesLxTPOFeedbackType(getattr(self.feedback_type, "value", self.feedback_type)).value
        if self.max_iterations < 1:
            raise ValueError("max_iterations must be at least 1")
        if self.n_candidates < 1:
            raise ValueError("n_candidates must be at least 1")
        if not 0.0 <= self.reward_threshold <= 1.0:
            raise ValueError("reward_threshold must be in [0, 1]")


_POSITIVE = ("good", "great", "excellent", "perfect", "well", "correct", "yes")
_NEGATIVE = ("bad", "poor", "wrong", "incorrect", "missing", "lacks", "no")
_NUMBER = re.compile(r"(?<![\w.])(?:\d+\.\d+|\.\d+|\d+)(?:\s*/\s*(\d+(?:\.\d+)?))?(\s*%)?")


def parse_reward(text: Any) -> float:
    """A judge's answer -> a score in [0, 1].  Understands "0.7", ".7", "7/10", "70%", "Score: 0.7"; a bare number above
    1 is read on a ten- or hundred-point scale; without a number the balance of approving and disapproving words
    decides; nothing recognisable gives 0.5."""
    if isinstance(text, (int, float)):
        return max(0.0, min(1.0, float(text)))
    s = str(text)
    m = _NUMBER.search(s)
    if m:
        raw = m.group(0)
        num = float(re.match(r"\s*(\d+\.\d+|\.\d+|\d+)", raw).group(1))
        if m.group(1):
            num = num / max(float(m.group(1)), 1e-9)
        elif m.group(2):
            num = num / 100.0
        elif num > 10.0:
            num = num / 100.0
        elif num > 1.0:
            num = num / 10.0
        return max(0.0, min(1.0, num))
    words = re.findall(r"[a-z]+", s.lower())
    pos, neg = sum(w in _POSITIVE for w in words), sum(w in _NEGATIVE for w in words)
    return pos / (pos + neg) if pos + neg else 0.5


class PiscesLxTPOOperator(PiscesLxOperatorInterface):
    name = "tpo"

    def __init__(self, config: Optional[PiscesLxTPOConfig] = None):
        self.config = config or PiscesLxTPOConfig()
        self.calls = {"generate": 0, "feedback": 0, "reward": 0}

    # -- the three model calls ------------------------------------------------------------------------------------------------
    def _sampling(self, c: PiscesLxTPOConfig) -> Dict[str, Any]:
        return {"temperature": c.temperature, "max_new_tokens": c.max_new_tokens, "top_p": c.top_p, "top_k": c.top_k}

    @staticmethod
    def _call(fn: TextFn, prompt: str, kw: Dict[str, Any]) -> Any:
        try:
            return fn(prompt, **kw)
        except TypeError:
            return fn(prompt)                                   # a callable that takes the prompt only

    def generate_response(self, generate: TextFn, prompt: str, config: Optional[PiscesLxTPOConfig] = None) -> str:
        self.calls["generate"] += 1
        return str(self._call(generate, prompt, self._sampling(config or self.config)))

    def generate_many(self, generate: TextFn, prompts: Sequence[str], config: Optional[PiscesLxTPOConfig] = None) -> List[str]:
        batch = getattr(generate, "generate_batch", None)
        if callable(batch):
            self.calls["generate"] += 1
            return [str(x) for x in batch(list(prompts), **self._sampling(config or self.config))]
        return [self.generate_response(generate, p, config) for p in prompts]

    def get_textual_feedback(self, feedback: TextFn, response: str, preference: str, config: Optional[PiscesLxTPOConfig] = None) -> str:
        c = config or self.config
        self.calls["feedback"] += 1
        return str(self._call(feedback, c.feedback_prompt.format(preference=preference, response=response), self._sampling(replace(c, temperature=0.0))))

    def compute_reward(self, reward: TextFn, response: str, preference: str, config: Optional[PiscesLxTPOConfig] = None) -> float:
        c = config or self.config
        self.calls["reward"] += 1
        return parse_reward(self._call(reward, c.reward_prompt.format(preference=preference, response=response),
                                       self._sampling(replace(c, temperature=0.0, max_new_tokens=16))))

    @staticmethod
    def refine_prompt(original_prompt: str, response: str, feedback: str, preference: str, config: PiscesLxTPOConfig) -> str:
        return f"{original_prompt}\n\n" + config.improvement_prompt.format(preference=preference, response=response, feedback=feedback)

    # -- alignment --------------------------------------------------------------------------------------------------------------
    def _best_of_n_align(self, generate: TextFn, prompt: str, preference: str, c: PiscesLxTPOConfig, reward: TextFn) -> Tuple[str, Dict[str, Any]]:
        cands = self.generate_many(generate, [prompt] * c.n_candidates, c)
        rewards = [self.compute_reward(reward, r, preference, c) for r in cands]
        best = max(range(len(cands)), key=lambda i: (rewards[i], -i))
        return cands[best], {"iterations": 1, "final_reward": rewards[best], "reward_history": rewards, "early_stopped": False,
                             "responses": cands, "mode": "best_of_n"}

    def align_at_inference(self, generate: TextFn, prompt: str, preference: str, config: Optional[PiscesLxTPOConfig] = None,
                           feedback: Optional[TextFn] = None, reward: Optional[TextFn] = None) -> Tuple[str, Dict[str, Any]]:
        c = config or self.config
        feedback, reward = feedback or generate, reward or generate
        if c.use_best_of_n:
            return self._best_of_n_align(generate, prompt, preference, c, reward)
        stats: Dict[str, Any] = {"iterations": 0, "final_reward": 0.0, "reward_history": [], "early_stopped": False, "responses": [],
                                 "feedback": [], "mode": c.feedback_type}
        cur, best, best_r, worst, worst_r = prompt, None, float("-inf"), None, float("inf")
        for it in range(c.max_iterations):
            stats["iterations"] = it + 1
            resp = self.generate_response(generate, cur, c)
            r = self.compute_reward(reward, resp, preference, c)
            stats["responses"].append(resp)
            stats["reward_history"].append(r)
            if r > best_r:
                best, best_r = resp, r
            if r < worst_r:
                worst, worst_r = resp, r
            if c.early_stopping and r >= c.reward_threshold:
                stats["early_stopped"] = True
                break
            if it < c.max_iterations - 1:
                if c.feedback_type == "comparative" and worst is not best:
                    fb = f"A weaker response was:\n{worst}\n\nA stronger response was:\n{best}\n\nGo beyond the stronger one."
                elif c.feedback_type in ("scalar", "comparative"):          # nothing to compare with yet: the score alone
                    fb = f"The response scored {r:.2f} out of 1 against the preference."
                else:
                    fb = self.get_textual_feedback(feedback, resp, preference, c)
                stats["feedback"].append(fb)
                cur = self.refine_prompt(prompt, best if c.feedback_type == "comparative" else resp, fb, preference, c)
        stats["final_reward"] = best_r
        return best if best is not None else "", stats

    # -- operator front -----------------------------------------------------------------------------------------------------------
    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return callable(inputs.get("generate")) and isinstance(inputs.get("prompt"), str) and isinstance(inputs.get("preference"), str)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        c = inputs.get("config", self.config)
        if isinstance(c, dict):
            c = replace(self.config, **c)
        resp, stats = self.align_at_inference(inputs["generate"], inputs["prompt"], inputs["preference"], c,
                                              inputs.get("feedback"), inputs.get("reward"))
        return {"response": resp, **stats}


class PiscesLxTPOAligner:
    """A policy (and optionally a critic and a judge) bound once: ``aligner.align(prompt, preference, **overrides)``,
    ``align_batch(prompts, preference)``, and named preference templates."""

    def __init__(self, generate: TextFn, config: Optional[PiscesLxTPOConfig] = None, feedback: Optional[TextFn] = None,
                 reward: Optional[TextFn] = None):
        self.generate, self.feedback, self.reward = generate, feedback, reward
        self.config = config or PiscesLxTPOConfig()
        self.operator = PiscesLxTPOOperator(self.config)
        self._templates: Dict[str, str] = {}

    def _merge_config(self, kwargs: Dict[str, Any]) -> PiscesLxTPOConfig:
        known = {k: v for k, v in kwargs.items() if k in PiscesLxTPOConfig.__dataclass_fields__}
        unknown = set(kwargs) - set(known)
        if unknown:
            raise TypeError(f"unknown TPO options: {sorted(unknown)}")
        return replace(self.config, **known) if known else self.config

    def set_preference_templates(self, templates: Dict[str, str]) -> None:
        self._templates.update(templates)

    def _preference(self, preference: str) -> str:
        return self._templates.get(preference, preference)

    def align(self, prompt: str, preference: str, **kwargs: Any) -> Tuple[str, Dict[str, Any]]:
        return self.operator.align_at_inference(self.generate, prompt, self._preference(preference), self._merge_config(kwargs),
                                                self.feedback, self.reward)

    def align_batch(self, prompts: Sequence[str], preference: str, **kwargs: Any) -> List[Tuple[str, Dict[str, Any]]]:
        """Best-of-n over a batch issues one generation call for all prompts x candidates when the policy can batch;
        the iterative mode aligns the prompts one by one (their refinement histories differ)."""
        c, pref = self._merge_config(kwargs), self._preference(preference)
        if not c.use_best_of_n:
            return [self.operator.align_at_inference(self.generate, p, pref, c, self.feedback, self.reward) for p in prompts]
        n = c.n_candidates
        flat = self.operator.generate_many(self.generate, [p for p in prompts for _ in range(n)], c)
        judge = self.reward or self.generate
        out = []
        for i, _ in enumerate(prompts):
            cands = flat[i * n:(i + 1) * n]
            rewards = [self.operator.compute_reward(judge, r, pref, c) for r in cands]
            b = max(range(n), key=lambda j: (rewards[j], -j))
            out.append((cands[b], {"iterations": 1, "final_reward": rewards[b], "reward_history": rewards, "early_stopped": False,
                                   "responses": cands, "mode": "best_of_n"}))
        return out


class PiscesLxTPOPreferenceLibrary:
    CODE_QUALITY = "Code should be efficient, well-documented, and follow best practices"
    CODE_SECURITY = "Code should be secure, handle edge cases, and not have vulnerabilities"
    CODE_READABLE = "Code should be readable, with clear variable names and structure"
    RESPONSE_CONCISE = "Response should be concise and to the point"
    RESPONSE_DETAILED = "Response should be detailed and comprehensive"
    RESPONSE_FRIENDLY = "Response should be friendly and helpful"
    RESPONSE_PROFESSIONAL = "Response should be professional and formal"
    RESPONSE_ACCURATE = "Response should be factually accurate and precise"
    RESPONSE_SAFE = "Response should be safe and not contain harmful content"
    MATH_STEP_BY_STEP = "Solution should show step-by-step reasoning"

    @staticmethod
    def custom(description: str) -> str:
        return description

    @staticmethod
    def combine(*preferences: str) -> str:
        return " and ".join(p.rstrip(". ") for p in preferences if p)

    @classmethod
    def names(cls) -> List[str]:
        return sorted(k for k, v in vars(cls).items() if k.isupper() and isinstance(v, str))
