"""The full ReAct agent (reference model/multimodal/react_agentic.py:57-1400) and the text-to-feature encoders used by
the agentic stack (reference model/multimodal/semantic_encoder.py:85-527).

``models/agentic_tools.py`` has the tools, the executor, the memory and a lean policy-driven loop; this module adds what
the reference's orchestrator does around such a loop:

  * goal understanding (a structured goal parsed from the model's JSON answer, plus neural heads that classify intent,
    domain and complexity from hidden states - batched tensors, no ``.item()``);
  * task decomposition into a plan whose steps may depend on one another;
  * the think -> act -> observe -> reflect cycle with error analysis, eight retry strategies, back-off, alternates,
    escalation and statistics that learn which resolution works for which kind of error;
  * persistence: checkpoints of the execution state (in memory, and as JSON files when a directory is given), resume,
    interruption, progress and a completion estimate.

The agent talks to the language model through ``generate(prompt) -> str`` and to the world through a
``YvToolExecutor`` (or a plain ``{name: callable}`` dictionary), so it runs offline and is scriptable in tests.  The
clock and the sleep function are injectable; nothing sleeps unless asked to."""
from __future__ import annotations

import json
import os
import random
import re
import time
from dataclasses import asdict, dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from .agentic_tools import YvSEERToolBase, YvToolExecutor, YvToolResult, YvToolType


# ---------------------------------------------------------------------------------------------------------------- structures
class YvReActAgenticState(str, Enum):
    IDLE = "idle"
    UNDERSTANDING = "understanding"
    PLANNING = "planning"
    EXECUTING = "executing"
    OBSERVING = "observing"
    REFLECTING = "reflecting"
    COMPLETED = "completed"
    FAILED = "failed"
    WAITING = "waiting"


class YvReActStepType(str, Enum):
    ANSWER = "answer"
    SEARCH = "search"
    TOOL_CALL = "tool_call"
    CODE_EXEC = "code_exec"
    WRITE_FILE = "write_file"
    READ_FILE = "read_file"
    ASK_HUMAN = "ask_human"
    PLAN_TASK = "plan_task"
    REFLECT = "reflect"
    FINISH = "finish"


class YvReActRetryKind(str, Enum):
    IMMEDIATE = "immediate"
    BACKOFF = "backoff"
    ALTERNATE = "alternate"
    DEGRADE = "degrade"
    SKIP = "skip"
    ABORT = "abort"
    ESCALATE = "escalate"
    CHECKPOINT_RESTORE = "checkpoint_restore"


_STEP_ALIASES = {"search": YvReActStepType.SEARCH, "code": YvReActStepType.CODE_EXEC, "code_exec": YvReActStepType.CODE_EXEC,
                 "write": YvReActStepType.WRITE_FILE, "write_file": YvReActStepType.WRITE_FILE,
                 "read": YvReActStepType.READ_FILE, "read_file": YvReActStepType.READ_FILE,
                 "answer": YvReActStepType.ANSWER, "ask": YvReActStepType.ASK_HUMAN, "ask_human": YvReActStepType.ASK_HUMAN,
                 "tool": YvReActStepType.TOOL_CALL, "tool_call": YvReActStepType.TOOL_CALL,
                 "finish": YvReActStepType.FINISH, "reflect": YvReActStepType.REFLECT, "plan": YvReActStepType.PLAN_TASK}


@dataclass
class YvReActGoal:
    original_text: str
    intent: str = ""
    constraints: List[str] = field(default_factory=list)
    success_criteria: List[str] = field(default_factory=list)
    domain: str = "general"
    complexity: int = 1

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


@dataclass
class YvReActStep:
    step_id: int
    description: str
    action_type: YvReActStepType
    params: Dict[str, Any] = field(default_factory=dict)
    depends_on: List[int] = field(default_factory=list)
    status: str = "pending"                    # pending | executing | completed | failed | skipped
    result: Optional[str] = None
    reflection: Optional[str] = None
    attempts: int = 0


@dataclass
class YvReActTaskPlan:
    goal: YvReActGoal
    steps: List[YvReActStep] = field(default_factory=list)
    current_step: int = 0
    status: str = "created"

    def add_step(self, description: str, action_type: YvReActStepType, params: Optional[Dict[str, Any]] = None,
                 depends_on: Optional[Sequence[int]] = None) -> int:
        sid = len(self.steps)
        self.steps.append(YvReActStep(sid, description, action_type, dict(params or {}), list(depends_on or [])))
        return sid

    def get_next_step(self) -> Optional[YvReActStep]:
        """The first pending step whose dependencies are all completed or skipped; None when nothing can run."""
        for s in self.steps:
            if s.status in ("pending", "executing") and \
                    all(self.steps[d].status in ("completed", "skipped") for d in s.depends_on if 0 <= d < len(self.steps)):
                return s
        return None

    def update_step(self, step_id: int, status: str, result: Optional[str] = None) -> None:
        if 0 <= step_id < len(self.steps):
            self.steps[step_id].status = status
            if result is not None:
                self.steps[step_id].result = result

    def counts(self) -> Dict[str, int]:
        out = {k: 0 for k in ("pending", "executing", "completed", "failed", "skipped")}
        for s in self.steps:
            out[s.status] = out.get(s.status, 0) + 1
        return out

    def blocked(self) -> bool:
        """Pending steps exist but none can run (a dependency failed)."""
        return self.get_next_step() is None and any(s.status == "pending" for s in self.steps)

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        for s in d["steps"]:
            s["action_type"] = YvReActStepType(s["action_type"]).value
        return d

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "YvReActTaskPlan":
        plan = cls(YvReActGoal(**d["goal"]), [], int(d.get("current_step", 0)), d.get("status", "created"))
        for s in d["steps"]:
            plan.steps.append(YvReActStep(**{**s, "action_type": YvReActStepType(s["action_type"])}))
        return plan


@dataclass
class YvReActStepAction:
    action_type: YvReActStepType
    params: Dict[str, Any] = field(default_factory=dict)
    thought: str = ""
    confidence: float = 1.0


@dataclass
class YvReActStepObservation:
    action: YvReActStepAction
    result: Any
    success: bool
    error: Optional[str] = None
    execution_time: float = 0.0


def _first_json(text: str, opener: str, closer: str) -> Any:
    """The outermost ``opener ... closer`` span of ``text`` parsed as JSON; raises ValueError if there is none."""
    a, b = text.find(opener), text.rfind(closer)
    if a < 0 or b <= a:
        raise ValueError("no JSON span")
    return json.loads(text[a:b + 1])


# ---------------------------------------------------------------------------------------------------------------- understanding
class YvGoalUnderstanding(nn.Module):
    """Two ways to read a goal: ``forward(hidden_states [B, S, H])`` classifies intent (10 classes), domain (8) and a
    complexity in [0, 1] from the last position - all per-sample tensors; ``understand(text, generate)`` asks the model
    for a JSON description and parses it into a ``YvReActGoal`` (falling back to the text itself)."""

    PROMPT = ("Analyse the request and answer with one JSON object with the keys intent (string), constraints (list of "
              "strings), success_criteria (list of strings), domain (string) and complexity (integer 1-5).\n\nRequest: {text}\n\nJSON:")

    def __init__(self, hidden_size: int = 4096):
        super().__init__()
        H = hidden_size
        self.hidden_size = H
        self.intent_classifier = nn.Sequential(nn.Linear(H, max(H // 2, 1)), nn.ReLU(), nn.Linear(max(H // 2, 1), 10))
        self.complexity_estimator = nn.Sequential(nn.Linear(H, max(H // 4, 1)), nn.ReLU(), nn.Linear(max(H // 4, 1), 1), nn.Sigmoid())
        self.domain_classifier = nn.Sequential(nn.Linear(H, max(H // 2, 1)), nn.ReLU(), nn.Linear(max(H // 2, 1), 8))

    def forward(self, hidden_states: torch.Tensor) -> Dict[str, torch.Tensor]:
        last = hidden_states[:, -1]
        il, dl = self.intent_classifier(last), self.domain_classifier(last)
        return {"intent_logits": il, "intent_class": il.argmax(-1), "domain_logits": dl, "domain_class": dl.argmax(-1),
                "complexity_score": self.complexity_estimator(last).squeeze(-1)}

    def understand(self, text: str, generate: Callable[[str], str]) -> YvReActGoal:
        try:
            p = _first_json(generate(self.PROMPT.format(text=text)), "{", "}")
            if not isinstance(p, dict):
                raise ValueError("not an object")
            as_list = lambda v: [str(x) for x in v] if isinstance(v, (list, tuple)) else ([str(v)] if v else [])
            return YvReActGoal(text, str(p.get("intent", "") or text[:100]), as_list(p.get("constraints")),
                               as_list(p.get("success_criteria")), str(p.get("domain", "general") or "general"),
                               max(1, min(5, int(p.get("complexity", 1)))))
        except (ValueError, TypeError):
            return YvReActGoal(text, text[:100], [], [], "general", 1)


class YvTaskDecomposition(nn.Module):
    """``decompose(goal, generate)`` asks for a JSON list of steps (description, action_type, params, depends_on) and
    builds the plan; an unparsable answer gives a single answer step.  The neural part scores, for a matrix of step
    embeddings [N, H] and the goal embedding [H], how strongly each step depends on each other one (``dependencies``),
    which ``order`` turns into an execution order."""

    PROMPT = ("Break the goal into at most {max_steps} steps.  Answer with one JSON list; every item has the keys description, "
              "action_type (one of search, code_exec, write_file, read_file, tool_call, answer, ask_human, finish), params "
              "(object) and depends_on (list of earlier step numbers, starting at 0).\n\nGoal: {intent}\nConstraints: "
              "{constraints}\n\nJSON:")

    def __init__(self, hidden_size: int = 4096, max_steps: int = 12):
        super().__init__()
        H = hidden_size
        self.hidden_size, self.max_steps = H, max_steps
        self.step_generator = nn.Sequential(nn.Linear(2 * H, H), nn.ReLU(), nn.Linear(H, H))
        self.dependency_analyzer = nn.Sequential(nn.Linear(H, max(H // 2, 1)), nn.ReLU(), nn.Linear(max(H // 2, 1), 1), nn.Sigmoid())

    def dependencies(self, step_embeddings: torch.Tensor, goal_embedding: torch.Tensor) -> torch.Tensor:
        """[N, N] in (0, 1), strictly lower triangular: entry (i, j) scores 'step i needs step j' for j < i."""
        N = step_embeddings.shape[0]
        g = goal_embedding.expand(N, -1)
        h = self.step_generator(torch.cat([step_embeddings, g], -1))
        pair = h.unsqueeze(1) * h.unsqueeze(0)                                     # [N, N, H]
        return self.dependency_analyzer(pair).squeeze(-1).tril(-1)

    @staticmethod
    def order(dependencies: torch.Tensor, threshold: float = 0.5) -> List[int]:
        """A topological order of the steps under the dependencies above the threshold (ties by index)."""
        need = (dependencies > threshold).tolist()
        done: List[int] = []
        left = list(range(len(need)))
        while left:
            ready = [i for i in left if all((not need[i][j]) or j in done for j in range(len(need)))]
            nxt = ready[0] if ready else left[0]
            done.append(nxt)
            left.remove(nxt)
        return done

    def decompose(self, goal: YvReActGoal, generate: Callable[[str], str]) -> YvReActTaskPlan:
        plan = YvReActTaskPlan(goal)
        try:
            items = _first_json(generate(self.PROMPT.format(max_steps=self.max_steps, intent=goal.intent,
                                                            constraints="; ".join(goal.constraints) or "none")), "[", "]")
            if not isinstance(items, list) or not items:
                raise ValueError("no steps")
            for i, it in enumerate(items[: self.max_steps]):
                if not isinstance(it, dict):
                    continue
                kind = _STEP_ALIASES.get(str(it.get("action_type", "answer")).lower(), YvReActStepType.ANSWER)
                deps = [int(d) for d in it.get("depends_on", []) if isinstance(d, (int, float)) and 0 <= int(d) < len(plan.steps)]
                plan.add_step(str(it.get("description", f"Step {i + 1}")), kind,
                              it.get("params") if isinstance(it.get("params"), dict) else {}, deps)
            if not plan.steps:
                raise ValueError("no usable step")
        except (ValueError, TypeError):
            plan.steps.clear()
            plan.add_step(f"Complete the goal: {goal.intent}", YvReActStepType.ANSWER)
        plan.status = "ready"
        return plan


# ---------------------------------------------------------------------------------------------------------------- correction
class YvReActSelfCorrection(nn.Module):
    """Error analysis and the choice of what to do next.  ``analyze_error`` sorts an error text into seven kinds,
    ``determine_retry_strategy`` maps (kind, attempts so far) to one of the eight strategies, ``learn_from_error`` keeps
    per-kind statistics of which resolution succeeded, and ``should_escalate`` reads them.  The two small networks embed
    an error context and propose a corrected state (``propose``)."""

    KINDS = ("timeout", "resource_not_found", "permission_denied", "invalid_input", "network_error", "rate_limit", "unknown")
    CRITICAL = ("permission_denied", "security_violation", "data_corruption")

    def __init__(self, hidden_size: int = 4096, max_retry_attempts: int = 5, base_backoff_delay: float = 1.0,
                 max_backoff_delay: float = 60.0, rng: Optional[random.Random] = None):
        super().__init__()
        H = hidden_size
        self.error_analyzer = nn.Sequential(nn.Linear(H, max(H // 2, 1)), nn.ReLU(), nn.Linear(max(H // 2, 1), len(self.KINDS)))
        self.correction_generator = nn.Sequential(nn.Linear(2 * H, H), nn.ReLU(), nn.Linear(H, H))
        self._max_retry_attempts, self._base_backoff_delay, self._max_backoff_delay = max_retry_attempts, base_backoff_delay, max_backoff_delay
        self._retry_history: Dict[str, List[Dict[str, Any]]] = {}
        self._error_patterns: Dict[str, Dict[str, Any]] = {}
        self._rng = rng or random.Random(0)

    def propose(self, state: torch.Tensor, error_embedding: torch.Tensor) -> Dict[str, torch.Tensor]:
        """state, error_embedding [B, H] -> kind logits [B, 7] and a corrected state [B, H]."""
        return {"error_logits": self.error_analyzer(error_embedding),
                "corrected_state": state + self.correction_generator(torch.cat([state, error_embedding], -1))}

    @staticmethod
    def classify(error: str) -> str:
        e = error.lower()
        if "timeout" in e or "timed out" in e or "timeoutexpired" in e:
            return "timeout"
        if "not found" in e or "missing" in e or "unknown tool" in e or "no such file" in e:
            return "resource_not_found"
        if "permission" in e or "access" in e or "outside the tool's root" in e:
            return "permission_denied"
        if "invalid" in e or "wrong" in e or "typeerror" in e or "valueerror" in e:
            return "invalid_input"
        if "connection" in e or "network" in e or "offline" in e:
            return "network_error"
        if "rate" in e or "limit" in e:
            return "rate_limit"
        return "unknown"

    def analyze_error(self, error: str, action_type: Union[YvReActStepType, str] = YvReActStepType.TOOL_CALL) -> Dict[str, Any]:
        kind = self.classify(error)
        return {"error_type": kind, "action_type": getattr(action_type, "value", str(action_type)),
                "should_retry": kind in ("timeout", "resource_not_found", "network_error", "rate_limit"),
                "should_alternate": kind in ("permission_denied", "invalid_input"),
                "should_abort": kind == "unknown" and len(error) > 100}

    @staticmethod
    def generate_correction(error_info: Dict[str, Any]) -> Dict[str, Any]:
        if error_info["should_retry"]:
            return {"strategy": "retry", "message": "retrying with the same parameters", "changes": []}
        if error_info["should_alternate"]:
            return {"strategy": "alternate", "message": "trying another approach",
                    "changes": ["use different parameters", "simplify the task"]}
        return {"strategy": "skip", "message": "skipping this step", "changes": ["mark the step optional", "continue"]}

    def determine_retry_strategy(self, error: str, attempt_count: int, context: Optional[Dict[str, Any]] = None) -> YvReActRetryKind:
        kind = self.classify(error)
        K = YvReActRetryKind
        if attempt_count >= self._max_retry_attempts:
            return K.ESCALATE
        if kind in ("timeout", "network_error", "rate_limit"):
            return K.IMMEDIATE if attempt_count == 0 else (K.BACKOFF if attempt_count < 3 else K.ALTERNATE)
        if kind == "permission_denied":
            return K.ESCALATE
        if kind in ("invalid_input", "resource_not_found"):
            return K.ALTERNATE if attempt_count < 2 else K.SKIP
        if context and context.get("has_checkpoint") and attempt_count >= 2:
            return K.CHECKPOINT_RESTORE
        return K.BACKOFF if attempt_count < 2 else (K.ALTERNATE if attempt_count < 4 else K.ESCALATE)

    def calculate_backoff_time(self, attempt_count: int, base_delay: Optional[float] = None,
                               max_delay: Optional[float] = None) -> float:
        base, top = base_delay or self._base_backoff_delay, max_delay or self._max_backoff_delay
        return min(base * (2 ** attempt_count) * self._rng.uniform(0.8, 1.2), top)

    @staticmethod
    def generate_alternate_actions(failed_action: Dict[str, Any], error_info: Dict[str, Any]) -> List[Dict[str, Any]]:
        kind, etype = failed_action.get("type", "unknown"), error_info.get("error_type", "unknown")
        params = dict(failed_action.get("params", {}))
        alts: List[Dict[str, Any]] = []
        if kind == "tool_call":
            tool = failed_action.get("tool", "")
            if etype == "timeout":
                alts.append({"type": "tool_call", "tool": tool, "params": {**params, "timeout": 60}, "reason": "longer timeout"})
            alts.append({"type": "tool_call", "tool": f"{tool}_fallback", "params": params, "reason": "fallback tool"})
        elif kind == "search":
            words = str(params.get("query", failed_action.get("query", ""))).split()
            alts.append({"type": "search", "params": {**params, "query": " ".join(words[: max(1, len(words) // 2)])},
                         "reason": "shorter query"})
        elif kind == "code_exec":
            alts.append({"type": "code_exec", "params": params, "reason": "same code, to be simplified by the model"})
        alts.append({"type": "ask_human", "params": {"question": f"The action '{kind}' failed ({etype}). How should I proceed?"},
                     "reason": "escalate to the user"})
        return alts[:3]

    def should_escalate(self, consecutive_failures: int, error_pattern: str) -> bool:
        if consecutive_failures >= self._max_retry_attempts or error_pattern in self.CRITICAL:
            return True
        p = self._error_patterns.get(error_pattern)
        return bool(p) and p["count"] >= 3 and p["success_rate"] < 0.2

    def learn_from_error(self, error: str, resolution: str, success: bool,
                         action_type: Union[YvReActStepType, str, None] = None) -> None:
        kind = self.classify(error)
        p = self._error_patterns.setdefault(kind, {"count": 0, "resolutions": {}, "success_rate": 0.0, "affected_actions": {}})
        p["count"] += 1
        r = p["resolutions"].setdefault(resolution, {"attempts": 0, "successes": 0})
        r["attempts"] += 1
        r["successes"] += int(success)
        tot_a = sum(v["attempts"] for v in p["resolutions"].values())
        p["success_rate"] = sum(v["successes"] for v in p["resolutions"].values()) / max(tot_a, 1)
        if action_type is not None:
            a = getattr(action_type, "value", str(action_type))
            p["affected_actions"][a] = p["affected_actions"].get(a, 0) + 1
        self._retry_history.setdefault(kind, []).append({"resolution": resolution, "success": success})

    def best_resolution(self, error: str) -> Optional[str]:
        """The resolution with the highest success rate seen for this kind of error (at least one success)."""
        p = self._error_patterns.get(self.classify(error))
        if not p:
            return None
        good = [(v["successes"] / v["attempts"], k) for k, v in p["resolutions"].items() if v["successes"] > 0]
        return max(good)[1] if good else None

    def get_error_pattern_prediction(self, action_type: Union[YvReActStepType, str]) -> float:
        """Share of the recorded errors that hit this kind of action (0.1 with no history)."""
        a = getattr(action_type, "value", str(action_type))
        tot = sum(p["count"] for p in self._error_patterns.values())
        return sum(p["affected_actions"].get(a, 0) for p in self._error_patterns.values()) / tot if tot else 0.1

    def get_retry_statistics(self) -> Dict[str, Any]:
        tot = sum(len(h) for h in self._retry_history.values())
        ok = sum(sum(1 for a in h if a["success"]) for h in self._retry_history.values())
        return {"total_retry_attempts": tot, "successful_retries": ok, "success_rate": ok / max(tot, 1),
                "error_patterns": len(self._error_patterns),
                "most_common_errors": sorted(self._error_patterns, key=lambda k: -self._error_patterns[k]["count"])[:5]}


# ---------------------------------------------------------------------------------------------------------------- the agent
ToolMap = Union[YvToolExecutor, Dict[str, Callable[..., Any]], None]


class YvReActAgentic(nn.Module):
    """understand -> plan -> for each runnable step: think, act, observe, reflect, correct -> result.

    ``run(user_input, generate, tools)`` returns a summary dictionary (goal, step counts, state, answer, history).
    ``tools`` is a ``YvToolExecutor`` or a dictionary of callables keyed by ``search`` / ``execute`` / ``write_file`` /
    ``read_file`` / a tool name; a missing tool is an error of the step, not of the run."""

    def __init__(self, hidden_size: int = 4096, max_steps: int = 20, checkpoint_dir: Optional[str] = None,
                 clock: Callable[[], float] = time.time, sleep: Optional[Callable[[float], None]] = None,
                 checkpoint_interval: float = 300.0):
        super().__init__()
        H = hidden_size
        self.hidden_size, self.max_steps = H, max_steps
        self.goal_understanding = YvGoalUnderstanding(H)
        self.task_decomposition = YvTaskDecomposition(H)
        self.self_correction = YvReActSelfCorrection(H)
        self.thought_generator = nn.Sequential(nn.Linear(3 * H, H), nn.ReLU(), nn.Linear(H, H))
        self.action_selector = nn.Sequential(nn.Linear(H, max(H // 2, 1)), nn.ReLU(), nn.Linear(max(H // 2, 1), len(YvReActStepType)))
        self.confidence_predictor = nn.Sequential(nn.Linear(H, max(H // 4, 1)), nn.ReLU(), nn.Linear(max(H // 4, 1), 1), nn.Sigmoid())
        self.goal_encoder, self.plan_encoder, self.history_encoder = nn.Linear(H, H), nn.Linear(H, H), nn.Linear(H, H)
        self.checkpoint_dir, self._clock, self._sleep = checkpoint_dir, clock, sleep
        self._checkpoint_interval = checkpoint_interval
        self._checkpoint_storage: Dict[str, Dict[str, Any]] = {}
        self._retry_policy = {"max_attempts": 3, "base_delay": 1.0, "max_delay": 60.0}
        self._execution_context: Dict[str, Any] = {}
        self._interruption_flag = False
        self._last_checkpoint_time = 0.0
        self.state = YvReActAgenticState.IDLE

    # -- neural policy heads ------------------------------------------------------------------------------------------------
    def policy(self, goal_state: torch.Tensor, plan_state: torch.Tensor, history_state: torch.Tensor) -> Dict[str, torch.Tensor]:
        """[B, H] x 3 -> a thought state [B, H], action logits over the ten step types and a confidence [B]."""
        t = self.thought_generator(torch.cat([self.goal_encoder(goal_state), self.plan_encoder(plan_state),
                                              self.history_encoder(history_state)], -1))
        return {"thought_state": t, "action_logits": self.action_selector(t), "confidence": self.confidence_predictor(t).squeeze(-1)}

    # -- text-level cycle -------------------------------------------------------------------------------------------------------
    @staticmethod
    def _think(goal: YvReActGoal, step: YvReActStep, history: List[Dict[str, Any]], generate: Callable[[str], str]) -> str:
        recent = "\n".join(f"- {h['action']}: {h['observation']}" for h in history[-3:]) or "(nothing yet)"
        return generate(f"Goal: {goal.intent}\nCurrent step: {step.description}\nRecent results:\n{recent}\n\n"
                        "Think briefly about how to carry out the current step.")

    @staticmethod
    def _fill_params(step: YvReActStep, thought: str, plan: YvReActTaskPlan) -> Dict[str, Any]:
        p = dict(step.params)
        if step.action_type == YvReActStepType.SEARCH:
            p.setdefault("query", step.description)
        elif step.action_type == YvReActStepType.ANSWER:
            p.setdefault("content", thought or step.description)
        p["_inputs"] = {d: plan.steps[d].result for d in step.depends_on if 0 <= d < len(plan.steps)}
        return p

    def _call_tool(self, tools: ToolMap, names: Sequence[str], **kw: Any) -> Tuple[bool, Any, Optional[str]]:
        if isinstance(tools, YvToolExecutor):
            for n in names:
                if n in getattr(tools, "tools", {}):
                    r: YvToolResult = tools.execute(n, **kw)
                    return r.success, r.output if hasattr(r, "output") else getattr(r, "result", None), r.error
            return False, None, f"tool not found: {names[0]}"
        if isinstance(tools, dict):
            for n in names:
                if n in tools:
                    try:
                        return True, tools[n](**kw), None
                    except Exception as e:                      # a failing tool is an observation, not a crash
                        return False, None, f"{type(e).__name__}: {e}"
        return False, None, f"tool not found: {names[0]}"

    def _execute_action(self, action: YvReActStepAction, tools: ToolMap) -> Tuple[bool, Any, Optional[str]]:
        T, p = YvReActStepType, {k: v for k, v in action.params.items() if k != "_inputs"}
        if action.action_type in (T.ANSWER, T.REFLECT, T.PLAN_TASK):
            return True, p.get("content", action.thought), None
        if action.action_type == T.FINISH:
            return True, p.get("content", "finished"), None
        if action.action_type == T.ASK_HUMAN:
            return True, "waiting for human input", None
        if action.action_type == T.SEARCH:
            return self._call_tool(tools, ("search",), query=p.get("query", ""))
        if action.action_type == T.CODE_EXEC:
            return self._call_tool(tools, ("execute", "code_exec"), code=p.get("code", ""))
        if action.action_type == T.WRITE_FILE:
            if isinstance(tools, YvToolExecutor):
                return self._call_tool(tools, ("file",), action="write", path=p.get("path", ""), content=p.get("content", ""))
            return self._call_tool(tools, ("write_file",), path=p.get("path", ""), content=p.get("content", ""))
        if action.action_type == T.READ_FILE:
            if isinstance(tools, YvToolExecutor):
                return self._call_tool(tools, ("file",), action="read", path=p.get("path", ""))
            return self._call_tool(tools, ("read_file",), path=p.get("path", ""))
        name = p.pop("tool", None) or p.pop("name", "")
        return self._call_tool(tools, (name,), **p.get("arguments", p))

    def _run_step(self, plan: YvReActTaskPlan, step: YvReActStep, generate: Callable[[str], str], tools: ToolMap,
                  history: List[Dict[str, Any]]) -> YvReActStepObservation:
        sc = self.self_correction
        step.status = "executing"
        self.state = YvReActAgenticState.EXECUTING
        thought = self._think(plan.goal, step, history, generate)
        params = self._fill_params(step, thought, plan)
        kind = step.action_type
        while True:
            action = YvReActStepAction(kind, params, thought)
            t0 = self._clock()
            ok, result, err = self._execute_action(action, tools)
            obs = YvReActStepObservation(action, result, ok, err, self._clock() - t0)
            self.state = YvReActAgenticState.OBSERVING
            if ok:
                if step.attempts:
                    sc.learn_from_error(step.reflection or "", self._execution_context.get("last_resolution", "retry"), True, kind)
                return obs
            self.state = YvReActAgenticState.REFLECTING
            step.reflection = err
            strategy = sc.determine_retry_strategy(err or "", step.attempts,
                                                   {"has_checkpoint": bool(self._checkpoint_storage)})
            sc.learn_from_error(err or "", strategy.value, False, kind)
            self._execution_context["last_resolution"] = strategy.value
            step.attempts += 1
            K = YvReActRetryKind
            if strategy in (K.ESCALATE, K.ABORT, K.SKIP, K.CHECKPOINT_RESTORE) or step.attempts > self._retry_policy["max_attempts"]:
                obs.error = f"{err} [{strategy.value}]"
                return obs
            if strategy == K.BACKOFF and self._sleep is not None:
                self._sleep(sc.calculate_backoff_time(step.attempts, self._retry_policy["base_delay"], self._retry_policy["max_delay"]))
            if strategy in (K.ALTERNATE, K.DEGRADE):
                alts = sc.generate_alternate_actions({"type": kind.value, "tool": params.get("tool", ""), "params": params},
                                                     sc.analyze_error(err or "", kind))
                alt = alts[0]
                kind = _STEP_ALIASES.get(alt["type"], kind)
                params = {**alt.get("params", {}), "_inputs": params.get("_inputs", {})}
                if "tool" in alt:
                    params["tool"] = alt["tool"]

    def run(self, user_input: str, generate: Callable[[str], str], tools: ToolMap = None, verbose: bool = False,
            _resume: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        start = self._clock()
        self._interruption_flag = False
        if _resume is None:
            self.state = YvReActAgenticState.UNDERSTANDING
            goal = self.goal_understanding.understand(user_input, generate)
            self.state = YvReActAgenticState.PLANNING
            plan = self.task_decomposition.decompose(goal, generate)
            history: List[Dict[str, Any]] = []
        else:
            plan, history = YvReActTaskPlan.from_dict(_resume["plan"]), list(_resume["history"])
            for s in plan.steps:
                if s.status == "executing":
                    s.status = "pending"
        self._execution_context.update(plan=plan, history=history, user_input=user_input, started=start)
        answer, executed = None, 0
        while executed < self.max_steps:
            if self._interruption_flag:
                self.state = YvReActAgenticState.WAITING
                break
            step = plan.get_next_step()
            if step is None:
                break
            plan.current_step = step.step_id
            if step.action_type == YvReActStepType.FINISH:
                plan.update_step(step.step_id, "completed", "finished")
                break
            obs = self._run_step(plan, step, generate, tools, history)
            executed += 1
            text = str(obs.result) if obs.success else str(obs.error)
            history.append({"step": step.step_id, "thought": obs.action.thought, "action": obs.action.action_type.value,
                            "observation": text[:200], "success": obs.success})
            if obs.success:
                plan.update_step(step.step_id, "completed", text)
                if obs.action.action_type == YvReActStepType.ANSWER:
                    answer = text
                if obs.action.action_type == YvReActStepType.ASK_HUMAN:
                    self.state = YvReActAgenticState.WAITING
                    break
            else:
                skipped = "[skip]" in text
                plan.update_step(step.step_id, "skipped" if skipped else "failed", text)
            if self._clock() - self._last_checkpoint_time >= self._checkpoint_interval:
                self.save_execution_state()
        c = plan.counts()
        if self.state != YvReActAgenticState.WAITING:
            done = c["pending"] == 0 and c["executing"] == 0
            self.state = YvReActAgenticState.COMPLETED if done and c["failed"] == 0 else YvReActAgenticState.FAILED
        plan.status = self.state.value
        if answer is None:
            answer = next((s.result for s in reversed(plan.steps) if s.status == "completed" and s.result), None)
        return {"goal": plan.goal.to_dict(), "plan_status": plan.status, "steps_completed": c["completed"],
                "steps_failed": c["failed"], "steps_skipped": c["skipped"], "total_steps": len(plan.steps),
                "history_length": len(history), "history": history, "state": self.state.value, "answer": answer,
                "total_time": self._clock() - start, "success": self.state == YvReActAgenticState.COMPLETED,
                "blocked": plan.blocked(), "retry_statistics": self.self_correction.get_retry_statistics()}

    # -- persistence ------------------------------------------------------------------------------------------------------------
    def save_execution_state(self) -> str:
        ctx = self._execution_context
        plan: Optional[YvReActTaskPlan] = ctx.get("plan")
        cid = f"ckpt_{len(self._checkpoint_storage):04d}_{int(self._clock() * 1000) % 10 ** 9:09d}"
        snap = {"checkpoint_id": cid, "time": self._clock(), "user_input": ctx.get("user_input", ""),
                "plan": plan.to_dict() if plan is not None else None, "history": list(ctx.get("history", [])),
                "state": self.state.value}
        self._checkpoint_storage[cid] = snap
        self._last_checkpoint_time = self._clock()
        if self.checkpoint_dir:
            os.makedirs(self.checkpoint_dir, exist_ok=True)
            tmp = os.path.join(self.checkpoint_dir, cid + ".json.tmp")
            with open(tmp, "w") as f:
                json.dump(snap, f)
            os.replace(tmp, os.path.join(self.checkpoint_dir, cid + ".json"))
        return cid

    def _load(self, checkpoint_id: str) -> Optional[Dict[str, Any]]:
        if checkpoint_id in self._checkpoint_storage:
            return self._checkpoint_storage[checkpoint_id]
        if self.checkpoint_dir:
            p = os.path.join(self.checkpoint_dir, checkpoint_id + ".json")
            if os.path.exists(p):
                with open(p) as f:
                    return json.load(f)
        return None

    def restore_execution_state(self, checkpoint_id: str) -> bool:
        snap = self._load(checkpoint_id)
        if snap is None or snap.get("plan") is None:
            return False
        self._execution_context.update(plan=YvReActTaskPlan.from_dict(snap["plan"]), history=list(snap["history"]),
                                       user_input=snap.get("user_input", ""))
        self.state = YvReActAgenticState(snap.get("state", "idle"))
        return True

    def run_with_persistence(self, user_input: str, generate: Callable[[str], str], tools: ToolMap = None,
                             checkpoint_every_step: bool = True) -> Dict[str, Any]:
        old = self._checkpoint_interval
        if checkpoint_every_step:
            self._checkpoint_interval = 0.0
        try:
            out = self.run(user_input, generate, tools)
        finally:
            self._checkpoint_interval = old
        out["checkpoint_id"] = self.save_execution_state()
        return out

    def resume_from_checkpoint(self, checkpoint_id: str, generate: Callable[[str], str], tools: ToolMap = None) -> Dict[str, Any]:
        snap = self._load(checkpoint_id)
        if snap is None or snap.get("plan") is None:
            raise KeyError(f"no checkpoint {checkpoint_id!r}")
        return self.run(snap.get("user_input", ""), generate, tools, _resume=snap)

    def handle_interruption(self, signal: Optional[str] = None) -> Dict[str, Any]:
        """Ask the running loop to stop before its next step and save where it is."""
        self._interruption_flag = True
        cid = self.save_execution_state() if self._execution_context.get("plan") is not None else None
        return {"interrupted": True, "signal": signal, "checkpoint_id": cid, "state": self.state.value}

    def execute_with_recovery(self, user_input: str, generate: Callable[[str], str], tools: ToolMap = None,
                              max_recoveries: int = 2) -> Dict[str, Any]:
        """Run; when the run fails with steps left, give the failed steps another chance from the last state, up to
        ``max_recoveries`` times."""
        out = self.run_with_persistence(user_input, generate, tools)
        n = 0
        while not out["success"] and out["state"] != YvReActAgenticState.WAITING.value and n < max_recoveries:
            snap = self._load(out["checkpoint_id"])
            for s in snap["plan"]["steps"]:
                if s["status"] == "failed":
                    s["status"], s["attempts"] = "pending", 0
            out = self.run(user_input, generate, tools, _resume=snap)
            out["checkpoint_id"] = self.save_execution_state()
            n += 1
        out["recoveries"] = n
        return out

    def get_execution_progress(self) -> Dict[str, Any]:
        plan: Optional[YvReActTaskPlan] = self._execution_context.get("plan")
        if plan is None:
            return {"state": self.state.value, "progress": 0.0, "total_steps": 0}
        c = plan.counts()
        fin = c["completed"] + c["skipped"] + c["failed"]
        return {"state": self.state.value, "progress": fin / max(len(plan.steps), 1), "total_steps": len(plan.steps),
                "current_step": plan.current_step, **c}

    def estimate_completion_time(self) -> float:
        """Seconds left if the remaining steps take as long as the finished ones did on average (0 with no history)."""
        p = self.get_execution_progress()
        fin = p.get("completed", 0) + p.get("skipped", 0) + p.get("failed", 0)
        if not fin:
            return 0.0
        elapsed = self._clock() - self._execution_context.get("started", self._clock())
        return elapsed / fin * (p["total_steps"] - fin)

    def list_checkpoints(self) -> List[Dict[str, Any]]:
        ids = set(self._checkpoint_storage)
        if self.checkpoint_dir and os.path.isdir(self.checkpoint_dir):
            ids |= {f[:-5] for f in os.listdir(self.checkpoint_dir) if f.endswith(".json")}
        out = []
        for cid in sorted(ids):
            s = self._load(cid) or {}
            out.append({"checkpoint_id": cid, "time": s.get("time"), "state": s.get("state"),
                        "steps": len((s.get("plan") or {}).get("steps", []))})
        return out

    def clear_checkpoints(self) -> None:
        self._checkpoint_storage.clear()
        if self.checkpoint_dir and os.path.isdir(self.checkpoint_dir):
            for f in os.listdir(self.checkpoint_dir):
                if f.startswith("ckpt_") and f.endswith(".json"):
                    os.remove(os.path.join(self.checkpoint_dir, f))


class YvReActFactory:
    @staticmethod
    def create_react_agentic(hidden_size: int = 4096, max_steps: int = 20, **kw: Any) -> YvReActAgentic:
        return YvReActAgentic(hidden_size, max_steps, **kw)

    @staticmethod
    def create_lightweight(hidden_size: int = 256, max_steps: int = 8, **kw: Any) -> YvReActAgentic:
        return YvReActAgentic(hidden_size, max_steps, **kw)


class YvSEERReasoningTool(YvSEERToolBase):
    """A tool whose work is a reasoning call: it formats the question (and optional context) into a prompt for the
    ``reason`` callable and returns its answer.  Lets a plan contain 'think about X' as an ordinary tool step."""

    name, tool_type = "reasoning", YvToolType.REASONING
    description = "reason step by step about a question and return the conclusion"

    def __init__(self, reason: Callable[[str], str], max_context: int = 4000):
        self.reason, self.max_context = reason, max_context

    def run(self, question: str, context: str = "") -> str:
        ctx = f"Context:\n{context[: self.max_context]}\n\n" if context else ""
        return self.reason(f"{ctx}Question: {question}\nReason step by step, then state the conclusion.")


# ---------------------------------------------------------------------------------------------------------------- encoders
def _stable_hash(word: str) -> int:
    h = 2166136261
    for b in word.encode("utf-8"):
        h = ((h ^ b) * 16777619) & 0xFFFFFFFF
    return h


class YvSemanticEncoder(nn.Module):
    """Text -> features without a tokenizer file: words are hashed (FNV-1a, so the ids are the same in every process -
    the reference uses Python's per-process salted ``hash``, semantic_encoder.py:150) into a small embedding table,
    the four role markers ``<|goal|> <|context|> <|action|> <|observation|>`` have their own rows, positions are added,
    and a bidirectional GRU gives the context.  Takes one string or a list (padded, masked)."""

    MARKERS = ("<|goal|>", "<|context|>", "<|action|>", "<|observation|>")
    _SPLIT = re.compile(r"(<\|goal\|>|<\|context\|>|<\|action\|>|<\|observation\|>)", re.IGNORECASE)

    def __init__(self, hidden_size: int = 2048, vocab_size: int = 151646, embedding_dim: int = 512, max_seq_len: int = 512):
        super().__init__()
        assert hidden_size % 2 == 0, "the bidirectional context encoder splits the hidden size in two"
        self.hidden_size, self.vocab_size, self.embedding_dim, self.max_seq_len = hidden_size, vocab_size, embedding_dim, max_seq_len
        self.token_embedding = nn.Embedding(vocab_size, embedding_dim, padding_idx=0)
        self.position_embedding = nn.Embedding(max_seq_len, embedding_dim)
        self.feature_projection = nn.Sequential(nn.Linear(embedding_dim, hidden_size // 2), nn.LayerNorm(hidden_size // 2), nn.GELU(),
                                                nn.Linear(hidden_size // 2, hidden_size), nn.LayerNorm(hidden_size))
        self.context_encoder = nn.GRU(hidden_size, hidden_size // 2, num_layers=2, batch_first=True, bidirectional=True)

    def tokenize(self, text: str) -> List[int]:
        """Ids: 0 padding, 1-4 the role markers, words from 5 upwards."""
        ids: List[int] = []
        for part in self._SPLIT.split(text.strip()):
            low = part.lower()
            if low in self.MARKERS:
                ids.append(1 + self.MARKERS.index(low))
            else:
                ids.extend(5 + _stable_hash(w) % (self.vocab_size - 5) for w in low.split())
        return (ids or [5 + _stable_hash(text.lower()) % (self.vocab_size - 5)])[: self.max_seq_len]

    def forward(self, text: Union[str, Sequence[str]], encode_type: str = "semantic") -> Dict[str, Any]:
        texts = [text] if isinstance(text, str) else list(text)
        toks = [self.tokenize(t) for t in texts]
        L = max(len(t) for t in toks)
        dev = self.token_embedding.weight.device
        ids = torch.zeros(len(toks), L, dtype=torch.long, device=dev)
        for i, t in enumerate(toks):
            ids[i, : len(t)] = torch.tensor(t, device=dev)
        mask = ids != 0
        emb = self.token_embedding(ids)
        if encode_type != "simple":
            emb = emb + self.position_embedding(torch.arange(L, device=dev))[None]
        feats = self.feature_projection(emb) * mask.unsqueeze(-1)
        packed = nn.utils.rnn.pack_padded_sequence(feats, mask.sum(1).cpu(), batch_first=True, enforce_sorted=False)
        ctx, hidden = self.context_encoder(packed)
        ctx, _ = nn.utils.rnn.pad_packed_sequence(ctx, batch_first=True, total_length=L)
        pooled = (ctx * mask.unsqueeze(-1)).sum(1) / mask.sum(1, keepdim=True).clamp_min(1)
        return {"embeddings": feats, "pooled": pooled, "tokens": ids, "mask": mask, "hidden_state": hidden, "context": ctx}

    def encode_goal(self, goal: str) -> torch.Tensor:
        return self(f"<|goal|> {goal}")["pooled"]

    def encode_context(self, context: Any) -> torch.Tensor:
        return self(f"<|context|> {str(context)[:1000]}")["pooled"]

    def encode_with_history(self, current: str, history: Sequence[Dict[str, str]]) -> Dict[str, Any]:
        parts = []
        for h in list(history)[-5:]:
            for key, mark in (("thought", "<|goal|>"), ("action", "<|action|>"), ("observation", "<|observation|>")):
                if key in h:
                    parts.append(f"{mark} {h[key]}")
        return self(" ".join(parts + [current]))


class YvHybridEncoder(nn.Module):
    """The semantic encoder's pooled features, optionally fused with additional features ([B, F] or [F]; resampled to
    the hidden size when F differs) through a learned gate."""

    def __init__(self, hidden_size: int = 2048, vocab_size: int = 151646, embedding_dim: int = 512):
        super().__init__()
        self.hidden_size = hidden_size
        self.semantic_encoder = YvSemanticEncoder(hidden_size, vocab_size, embedding_dim)
        self.feature_fusion = nn.Sequential(nn.Linear(2 * hidden_size, hidden_size), nn.LayerNorm(hidden_size), nn.GELU())
        self.gate = nn.Sequential(nn.Linear(hidden_size, 1), nn.Sigmoid())

    def forward(self, text: Union[str, Sequence[str]], additional_features: Optional[torch.Tensor] = None) -> Dict[str, Any]:
        sem = self.semantic_encoder(text)
        feats = sem["pooled"]
        if additional_features is not None:
            add = additional_features.to(feats.device, feats.dtype)
            add = add.unsqueeze(0) if add.dim() == 1 else add
            if add.shape[-1] != self.hidden_size:
                add = F.adaptive_avg_pool1d(add.unsqueeze(1), self.hidden_size).squeeze(1)
            add = add.expand(feats.shape[0], -1)
            g = self.gate(feats)
            feats = g * self.feature_fusion(torch.cat([feats, add], -1)) + (1 - g) * feats
        return {"semantic_embeddings": sem["embeddings"], "fused_embeddings": feats, "pooled": feats,
                "context": sem["context"], "hidden_state": sem["hidden_state"]}
