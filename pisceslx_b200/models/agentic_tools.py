"""Agent runtime pieces (reference model/multimodal/tool_executor.py, seer_executor.py, state_machine.py, memory.py,
react_agentic.py): built-in tools with a uniform result type, a tool executor with time limits, the agent state
machine with history and snapshots, typed agent memory with retrieval, the experience pool, and the plan / reflection /
retry structures of the ReAct engine.  Everything is host-side Python and works offline: tools that would need the
network say so in their result instead of trying."""
from __future__ import annotations

import ast
import math
import operator
import os
import subprocess
import sys
import tempfile
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple


# ------------------------------------------------------------------------------------------------ tools
class YvToolType(str, Enum):
    CALCULATE = "calculate"
    CODE_EXEC = "code_exec"
    FILE = "file"
    SEARCH = "search"
    HTTP = "http"
    REASONING = "reasoning"
    VERIFICATION = "verification"


@dataclass
class YvToolResult:
    tool: str
    success: bool
    output: Any = None
    error: Optional[str] = None
    seconds: float = 0.0


class YvSEERToolBase:
    name, tool_type = "tool", YvToolType.REASONING

    def run(self, **kw: Any) -> Any:
        raise NotImplementedError

    def __call__(self, **kw: Any) -> YvToolResult:
        t0 = time.perf_counter()
        try:
            return YvToolResult(self.name, True, self.run(**kw), None, time.perf_counter() - t0)
        except Exception as e:
            return YvToolResult(self.name, False, None, f"{type(e).__name__}: {e}", time.perf_counter() - t0)


class YvCalculateTool(YvSEERToolBase):
    """Arithmetic on a parsed expression tree: numbers, + - * / // % **, unary minus, and a few math functions; no
    names, attributes or calls outside the whitelist are evaluated."""
    name, tool_type = "calculate", YvToolType.CALCULATE
    OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv,
           ast.FloorDiv: operator.floordiv, ast.Mod: operator.mod, ast.Pow: operator.pow}
    FUNCS = {"sqrt": math.sqrt, "log": math.log, "exp": math.exp, "sin": math.sin, "cos": math.cos, "abs": abs,
             "round": round, "min": min, "max": max}
    CONSTS = {"pi": math.pi, "e": math.e}

    def _ev(self, n: ast.AST) -> float:
        if isinstance(n, ast.Constant) and isinstance(n.value, (int, float)):
            return n.value
        if isinstance(n, ast.BinOp) and type(n.op) in self.OPS:
            a, b = self._ev(n.left), self._ev(n.right)
            if isinstance(n.op, ast.Pow) and abs(b) > 256:
                raise ValueError("exponent too large")
            return self.OPS[type(n.op)](a, b)
        if isinstance(n, ast.UnaryOp) and isinstance(n.op, (ast.USub, ast.UAdd)):
            v = self._ev(n.operand)
            return -v if isinstance(n.op, ast.USub) else v
        if isinstance(n, ast.Call) and isinstance(n.func, ast.Name) and n.func.id in self.FUNCS and not n.keywords:
            return self.FUNCS[n.func.id](*[self._ev(a) for a in n.args])
        if isinstance(n, ast.Name) and n.id in self.CONSTS:
            return self.CONSTS[n.id]
        raise ValueError(f"unsupported expression element {type(n).__name__}")

    def run(self, expression: str) -> float:
        return self._ev(ast.parse(expression, mode="eval").body)


class YvCodeExecTool(YvSEERToolBase):
    """Runs a Python snippet in a child interpreter (isolated mode, empty environment, temporary working directory,
    time limit) and returns its stdout."""
    name, tool_type = "code_exec", YvToolType.CODE_EXEC

    def __init__(self, timeout_s: float = 5.0, max_output: int = 4000):
        self.timeout, self.max_output = timeout_s, max_output

    def run(self, code: str) -> str:
        with tempfile.TemporaryDirectory() as d:
            p = os.path.join(d, "snippet.py")
            with open(p, "w") as f:
                f.write(code)
            r = subprocess.run([sys.executable, "-I", p], cwd=d, env={}, capture_output=True, text=True, timeout=self.timeout)
            if r.returncode != 0:
                raise RuntimeError(r.stderr[-self.max_output:])
            return r.stdout[-self.max_output:]


class YvFileTool(YvSEERToolBase):
    """read / write / list inside ``root`` only: paths are resolved and must stay under the root."""
    name, tool_type = "file", YvToolType.FILE

    def __init__(self, root: str, max_bytes: int = 1 << 20):
        self.root, self.max_bytes = os.path.realpath(root), max_bytes

    def _path(self, rel: str) -> str:
        p = os.path.realpath(os.path.join(self.root, rel))
        if p != self.root and not p.startswith(self.root + os.sep):
            raise PermissionError(f"{rel!r} is outside the tool's root")
        return p

    def run(self, action: str, path: str = ".", content: str = "") -> Any:
        p = self._path(path)
        if action == "read":
            with open(p) as f:
                return f.read(self.max_bytes)
        if action == "write":
            if len(content.encode()) > self.max_bytes:
                raise ValueError("content too large")
            os.makedirs(os.path.dirname(p), exist_ok=True)
            with open(p, "w") as f:
                f.write(content)
            return len(content)
        if action == "list":
            return sorted(os.listdir(p))
        raise ValueError(f"unknown action {action!r}")


class YvSearchTool(YvSEERToolBase):
    """Keyword search over a local corpus (list of {"id", "text"}): TF-style overlap score, top-k hits."""
    name, tool_type = "search", YvToolType.SEARCH

    def __init__(self, corpus: Sequence[Dict[str, str]]):
        self.corpus = list(corpus)

    def run(self, query: str, k: int = 3) -> List[Dict[str, Any]]:
        q = set(query.lower().split())
        scored = []
        for doc in self.corpus:
            words = doc["text"].lower().split()
            s = sum(1 for w in words if w in q) / math.sqrt(len(words) + 1)
            if s > 0:
                scored.append({"id": doc["id"], "score": s, "text": doc["text"][:200]})
        return sorted(scored, key=lambda r: -r["score"])[:k]


class YvHTTPTool(YvSEERToolBase):
    """Network access is not available to this runtime: the tool reports that instead of attempting a connection."""
    name, tool_type = "http", YvToolType.HTTP

    def run(self, url: str, **_: Any) -> Any:
        raise ConnectionError(f"offline runtime: {url!r} was not fetched; attach a fetcher with YvToolExecutor.register")


YvFetchTool = YvHTTPTool
YvSEERCalculateTool, YvSEERCodeExecTool, YvSEERFileTool, YvSEERSearchTool = YvCalculateTool, YvCodeExecTool, YvFileTool, YvSearchTool


class YvSEERVerificationTool(YvSEERToolBase):
    """Checks a claimed result by recomputation: {"expression", "claimed"} -> bool."""
    name, tool_type = "verify", YvToolType.VERIFICATION

    def run(self, expression: str, claimed: float, tol: float = 1e-6) -> bool:
        return abs(YvCalculateTool().run(expression) - float(claimed)) <= tol


class YvToolExecutor:
    """Name -> tool dispatch with per-tool statistics."""

    def __init__(self, tools: Optional[Sequence[YvSEERToolBase]] = None):
        self.tools: Dict[str, YvSEERToolBase] = {}
        self.stats: Dict[str, Dict[str, int]] = {}
        for t in tools or ():
            self.register(t)

    def register(self, tool: YvSEERToolBase) -> None:
        self.tools[tool.name] = tool
        self.stats.setdefault(tool.name, {"calls": 0, "failures": 0})

    def execute(self, name: str, **kw: Any) -> YvToolResult:
        if name not in self.tools:
            return YvToolResult(name, False, error=f"unknown tool {name!r}")
        r = self.tools[name](**kw)
        self.stats[name]["calls"] += 1
        self.stats[name]["failures"] += int(not r.success)
        return r


YvSEERExecutor = YvMCPUnifiedToolExecutor = YvToolExecutor


# ------------------------------------------------------------------------------------------------ state machine
class YvAgenticState(str, Enum):
    IDLE = "idle"
    PLANNING = "planning"
    ACTING = "acting"
    OBSERVING = "observing"
    REFLECTING = "reflecting"
    DONE = "done"
    FAILED = "failed"


@dataclass
class YvStateTransition:
    source: YvAgenticState
    target: YvAgenticState
    reason: str = ""
    time: float = field(default_factory=time.time)


@dataclass
class YvStateSnapshot:
    state: YvAgenticState
    context: Dict[str, Any]
    step: int


class YvStateMachine:
    """The agent's control states with the allowed transitions, a transition history and restorable snapshots."""

    ALLOWED = {
        YvAgenticState.IDLE: {YvAgenticState.PLANNING},
        YvAgenticState.PLANNING: {YvAgenticState.ACTING, YvAgenticState.DONE, YvAgenticState.FAILED},
        YvAgenticState.ACTING: {YvAgenticState.OBSERVING, YvAgenticState.DONE, YvAgenticState.FAILED},
        YvAgenticState.OBSERVING: {YvAgenticState.REFLECTING, YvAgenticState.ACTING, YvAgenticState.DONE},
        YvAgenticState.REFLECTING: {YvAgenticState.PLANNING, YvAgenticState.ACTING, YvAgenticState.DONE, YvAgenticState.FAILED},
        YvAgenticState.DONE: {YvAgenticState.IDLE},
        YvAgenticState.FAILED: {YvAgenticState.IDLE},
    }

    def __init__(self):
        self.state, self.context, self.step = YvAgenticState.IDLE, {}, 0
        self.history: List[YvStateTransition] = []

    def can(self, target: YvAgenticState) -> bool:
        return target in self.ALLOWED[self.state]

    def to(self, target: YvAgenticState, reason: str = "") -> None:
        if not self.can(target):
            raise ValueError(f"transition {self.state.value} -> {target.value} is not allowed")
        self.history.append(YvStateTransition(self.state, target, reason))
        self.state, self.step = target, self.step + 1

    def snapshot(self) -> YvStateSnapshot:
        return YvStateSnapshot(self.state, dict(self.context), self.step)

    def restore(self, snap: YvStateSnapshot) -> None:
        self.state, self.context, self.step = snap.state, dict(snap.context), snap.step


# ------------------------------------------------------------------------------------------------ memory
class YvMemoryType(str, Enum):
    WORKING = "working"
    EPISODIC = "episodic"
    SEMANTIC = "semantic"


@dataclass
class YvMemoryEntry:
    content: str
    kind: YvMemoryType = YvMemoryType.EPISODIC
    importance: float = 0.5
    time: float = field(default_factory=time.time)
    uses: int = 0


class YvMemory:
    """Typed agent memory: working memory is a short FIFO; episodic and semantic entries are kept up to a capacity
    and evicted by lowest (importance x recency); retrieval ranks by word overlap with the query, importance and
    recency."""

    def __init__(self, working_size: int = 8, capacity: int = 256, half_life_s: float = 3600.0, clock: Callable[[], float] = time.time):
        self.working_size, self.capacity, self.half_life, self.clock = working_size, capacity, half_life_s, clock
        self.entries: List[YvMemoryEntry] = []

    def add(self, content: str, kind: YvMemoryType = YvMemoryType.EPISODIC, importance: float = 0.5) -> YvMemoryEntry:
        e = YvMemoryEntry(content, kind, importance, self.clock())
        self.entries.append(e)
        work = [x for x in self.entries if x.kind == YvMemoryType.WORKING]
        for old in work[: max(0, len(work) - self.working_size)]:
            self.entries.remove(old)
        long_term = [x for x in self.entries if x.kind != YvMemoryType.WORKING]
        if len(long_term) > self.capacity:
            victim = min(long_term, key=lambda x: x.importance * self._recency(x))
            self.entries.remove(victim)
        return e

    def _recency(self, e: YvMemoryEntry) -> float:
        return 0.5 ** ((self.clock() - e.time) / self.half_life)

    def retrieve(self, query: str, k: int = 3, kind: Optional[YvMemoryType] = None) -> List[YvMemoryEntry]:
        q = set(query.lower().split())
        scored = []
        for e in self.entries:
            if kind is not None and e.kind != kind:
                continue
            w = set(e.content.lower().split())
            overlap = len(q & w) / math.sqrt(len(w) + 1)
            scored.append((overlap * (0.5 + e.importance) * (0.5 + 0.5 * self._recency(e)), e))
        out = [e for s, e in sorted(scored, key=lambda t: -t[0])[:k] if s > 0]
        for e in out:
            e.uses += 1
        return out


YvAgenticMemory = YvMemory


@dataclass
class YvExperienceRecord:
    task: str
    actions: List[str]
    success: bool
    reward: float = 0.0


class YvSEERExperiencePool:
    """Keeps finished trajectories and returns the most similar successful ones as few-shot guidance."""

    def __init__(self, capacity: int = 512):
        self.capacity, self.records = capacity, []

    def add(self, rec: YvExperienceRecord) -> None:
        self.records.append(rec)
        if len(self.records) > self.capacity:
            self.records.sort(key=lambda r: (r.success, r.reward))
            self.records.pop(0)

    def similar(self, task: str, k: int = 2) -> List[YvExperienceRecord]:
        q = set(task.lower().split())
        ok = [r for r in self.records if r.success]
        return sorted(ok, key=lambda r: -len(q & set(r.task.lower().split())))[:k]

    def success_rate(self) -> float:
        return sum(r.success for r in self.records) / max(len(self.records), 1)


# ------------------------------------------------------------------------------------------------ ReAct structures
class YvReActActionType(str, Enum):
    TOOL = "tool"
    THINK = "think"
    FINISH = "finish"


@dataclass
class YvReActAction:
    kind: YvReActActionType
    tool: Optional[str] = None
    arguments: Dict[str, Any] = field(default_factory=dict)
    text: str = ""


@dataclass
class YvReActObservation:
    action: YvReActAction
    result: Optional[YvToolResult] = None


@dataclass
class YvReActPlanStep:
    description: str
    tool: Optional[str] = None
    done: bool = False


@dataclass
class YvReActPlan:
    goal: str
    steps: List[YvReActPlanStep] = field(default_factory=list)

    def next_step(self) -> Optional[YvReActPlanStep]:
        return next((s for s in self.steps if not s.done), None)

    def progress(self) -> float:
        return sum(s.done for s in self.steps) / max(len(self.steps), 1)


@dataclass
class YvReActReflection:
    step: int
    error: str
    lesson: str


class YvReActRetryStrategy:
    """Bounded retries with exponential back-off; the same failing (tool, arguments) pair is not repeated verbatim
    more than ``max_same`` times."""

    def __init__(self, max_retries: int = 3, base_delay_s: float = 0.0, max_same: int = 1):
        self.max_retries, self.base_delay, self.max_same = max_retries, base_delay_s, max_same
        self.failures: Dict[str, int] = {}

    def key(self, a: YvReActAction) -> str:
        return f"{a.tool}:{sorted(a.arguments.items())}"

    def record_failure(self, a: YvReActAction) -> None:
        self.failures[self.key(a)] = self.failures.get(self.key(a), 0) + 1

    def should_retry(self, a: YvReActAction, attempt: int) -> bool:
        return attempt < self.max_retries and self.failures.get(self.key(a), 0) <= self.max_same

    def delay(self, attempt: int) -> float:
        return self.base_delay * (2 ** attempt)


class YvSelfCorrection:
    """Turns a failed observation into a reflection and a hint for the next prompt."""

    def reflect(self, step: int, obs: YvReActObservation) -> Optional[YvReActReflection]:
        r = obs.result
        if r is None or r.success:
            return None
        err = r.error or "unknown error"
        if "unknown tool" in err:
            lesson = "use one of the registered tools"
        elif "outside the tool's root" in err or "PermissionError" in err:
            lesson = "stay inside the allowed directory"
        elif "offline" in err or "ConnectionError" in err:
            lesson = "the network is not available; use local tools"
        elif "TimeoutExpired" in err:
            lesson = "the code ran too long; make it smaller"
        else:
            lesson = "check the arguments and try a different approach"
        return YvReActReflection(step, err, lesson)


class YvReActEngine:
    """Plan -> act -> observe -> reflect loop over a ``YvToolExecutor``, driven by a policy callable
    ``policy(goal, observations, reflections) -> YvReActAction`` (a language model in production, a script in tests);
    the state machine records every phase."""

    def __init__(self, executor: YvToolExecutor, policy: Callable[[str, List[YvReActObservation], List[YvReActReflection]], YvReActAction],
                 max_steps: int = 8, retry: Optional[YvReActRetryStrategy] = None):
        self.executor, self.policy, self.max_steps = executor, policy, max_steps
        self.retry = retry or YvReActRetryStrategy()
        self.sm, self.corrector = YvStateMachine(), YvSelfCorrection()

    def run(self, goal: str) -> Dict[str, Any]:
        obs: List[YvReActObservation] = []
        refl: List[YvReActReflection] = []
        self.sm.to(YvAgenticState.PLANNING, goal)
        answer, attempt = None, 0
        for step in range(self.max_steps):
            action = self.policy(goal, obs, refl)
            if action.kind == YvReActActionType.FINISH:
                answer = action.text
                self.sm.to(YvAgenticState.DONE, "finished")
                break
            if self.sm.state != YvAgenticState.ACTING:
                self.sm.to(YvAgenticState.ACTING, action.tool or "think")
            result = self.executor.execute(action.tool, **action.arguments) if action.kind == YvReActActionType.TOOL else None
            self.sm.to(YvAgenticState.OBSERVING)
            o = YvReActObservation(action, result)
            obs.append(o)
            r = self.corrector.reflect(step, o)
            if r is not None:
                self.retry.record_failure(action)
                self.sm.to(YvAgenticState.REFLECTING, r.lesson)
                refl.append(r)
                attempt += 1
                if not self.retry.should_retry(action, attempt):
                    self.sm.to(YvAgenticState.FAILED, "retries exhausted")
                    break
                self.sm.to(YvAgenticState.ACTING, "retry")
            else:
                self.sm.to(YvAgenticState.ACTING, "continue")
        return {"answer": answer, "state": self.sm.state.value, "observations": obs, "reflections": refl,
                "transitions": len(self.sm.history)}


# The names the executor module of the reference gives these tools and types (model/multimodal/seer_executor.py:42-135).
YvSEERToolType = YvToolType
YvSEERResult = YvToolResult
YvSEERSearchTool = YvSearchTool
YvSEERCodeExecTool = YvCodeExecTool
YvSEERCalculateTool = YvCalculateTool
YvSEERFileTool = YvFileTool


def register_seer_tools(registry: Any, tools: Sequence[YvSEERToolBase]) -> List[str]:
    """Registers tool objects in a ``models.agentic_mcp.YvCoreMCPToolRegistry`` (native tools whose handler is ``tool.run``)."""
    from .agentic_mcp import YvMCPToolMetadata, YvMCPToolType
    names = []
    for t in tools:
        if registry.register(YvMCPToolMetadata(t.name, (t.__doc__ or "").strip().split("\n")[0], {}, YvMCPToolType.NATIVE, t.run, tags=[str(getattr(t.tool_type, "value", t.tool_type))])):
            names.append(t.name)
    return names
