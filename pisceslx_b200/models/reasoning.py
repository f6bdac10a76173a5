"""Inference-time reasoning and agent scaffolding (reference model/reasoning/*: ``YvUnifiedReasoner``, CoT / multipath
/ recursive reasoners, ``YvVeriCoT*`` verification; model/agentic/*: ``YvAgentic`` ReAct engine, tool executors, XML
tool-call parser, memory; MCP message types).  These sit off the throughput path (the trainer disables them,
tools/train/core.py:2014-2019): they orchestrate calls to ``generate`` and to registered tools."""
from __future__ import annotations

import json
import re
from collections import Counter
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

GenerateFn = Callable[[str, int], str]          # (prompt, max_new_tokens) -> completion text


@dataclass
class YvReasoningTrace:
    steps: List[str] = field(default_factory=list)
    answer: Optional[str] = None
    votes: Dict[str, int] = field(default_factory=dict)
    verified: Optional[bool] = None


_ANSWER = re.compile(r"(?:final answer|answer)\s*[:=]\s*(.+)", re.I)


def extract_answer(text: str) -> Optional[str]:
    m = _ANSWER.findall(text)
    return m[-1].strip().rstrip(".") if m else None


class YvCoTReasoner:
    """Single chain of thought: prompt for step-by-step reasoning, split the steps, extract the answer."""

    PROMPT = "{question}\nLet's think step by step.\n"

    def __init__(self, generate: GenerateFn, max_new_tokens: int = 256):
        self.generate, self.max_new_tokens = generate, max_new_tokens

    def reason(self, question: str) -> YvReasoningTrace:
        out = self.generate(self.PROMPT.format(question=question), self.max_new_tokens)
        steps = [s.strip() for s in re.split(r"\n+|(?<=\.)\s+(?=Step)", out) if s.strip()]
        return YvReasoningTrace(steps=steps, answer=extract_answer(out))


class YvMultiPathReasoner:
    """Self-consistency: ``n_paths`` sampled chains, majority vote over the extracted answers."""

    def __init__(self, generate: GenerateFn, n_paths: int = 5, max_new_tokens: int = 256):
        self.cot, self.n_paths = YvCoTReasoner(generate, max_new_tokens), n_paths

    def reason(self, question: str) -> YvReasoningTrace:
        traces = [self.cot.reason(question) for _ in range(self.n_paths)]
        votes = Counter(t.answer for t in traces if t.answer is not None)
        best = votes.most_common(1)[0][0] if votes else None
        pick = next((t for t in traces if t.answer == best), traces[0])
        return YvReasoningTrace(steps=pick.steps, answer=best, votes=dict(votes))


class YvRecursiveReasoner:
    """Decompose -> solve sub-questions -> compose, to a bounded depth."""

    def __init__(self, generate: GenerateFn, max_depth: int = 2, max_new_tokens: int = 192):
        self.generate, self.max_depth, self.max_new_tokens = generate, max_depth, max_new_tokens

    def reason(self, question: str, depth: int = 0) -> YvReasoningTrace:
        if depth >= self.max_depth:
            return YvCoTReasoner(self.generate, self.max_new_tokens).reason(question)
        plan = self.generate(f"Break the problem into sub-questions, one per line.\nProblem: {question}\n", self.max_new_tokens)
        subs = [l.strip("-* 0123456789.").strip() for l in plan.splitlines() if l.strip().endswith("?")][:4]
        if not subs:
            return YvCoTReasoner(self.generate, self.max_new_tokens).reason(question)
        solved = [(s, self.reason(s, depth + 1).answer) for s in subs]
        ctx = "\n".join(f"Q: {s}\nA: {a}" for s, a in solved)
        out = self.generate(f"{ctx}\nUsing the answers above, solve: {question}\n", self.max_new_tokens)
        return YvReasoningTrace(steps=[f"{s} -> {a}" for s, a in solved], answer=extract_answer(out) or out.strip())


class YvVeriCoTVerifier:
    """Checks a trace: every arithmetic statement ``a op b = c`` in the steps must hold; optional external checker."""

    _EQ = re.compile(r"(-?\d+(?:\.\d+)?)\s*([+\-*/x×])\s*(-?\d+(?:\.\d+)?)\s*=\s*(-?\d+(?:\.\d+)?)")

    def __init__(self, checker: Optional[Callable[[YvReasoningTrace], bool]] = None):
        self.checker = checker

    def verify(self, trace: YvReasoningTrace) -> bool:
        ok = True
        for step in trace.steps:
            for a, op, b, c in self._EQ.findall(step):
                a, b, c = float(a), float(b), float(c)
                val = {"+": a + b, "-": a - b, "*": a * b, "x": a * b, "×": a * b, "/": a / b if b else float("nan")}[op]
                ok &= abs(val - c) < 1e-6 * max(1.0, abs(c))
        if self.checker is not None:
            ok &= bool(self.checker(trace))
        trace.verified = ok
        return ok


class YvThoughtTreeReasoner:
    """Tree of thoughts with beam search: at every depth each kept partial chain is extended by ``branch`` sampled
    next steps, a value function scores the candidates (default: ask the model to rate the chain 1-10 and parse the
    number), the ``beam`` best survive; a chain ends when a step states an answer.  ``value_fn(question, steps)`` can be
    supplied (a verifier, a reward model) instead of the prompt-based rating."""

    STEP = "{question}\nSteps so far:\n{steps}\nNext step (or 'Answer: ...' if done):\n"
    RATE = "{question}\nSteps so far:\n{steps}\nRate from 1 to 10 how promising this reasoning is. Rating:"

    def __init__(self, generate: GenerateFn, branch: int = 3, beam: int = 2, max_depth: int = 4, max_new_tokens: int = 64,
                 value_fn: Optional[Callable[[str, List[str]], float]] = None):
        self.generate, self.branch, self.beam, self.max_depth = generate, branch, beam, max_depth
        self.max_new_tokens, self.value_fn = max_new_tokens, value_fn
        self.expanded = 0

    def _value(self, question: str, steps: List[str]) -> float:
        if self.value_fn is not None:
            return float(self.value_fn(question, steps))
        out = self.generate(self.RATE.format(question=question, steps="\n".join(steps) or "(none)"), 8)
        m = re.search(r"(\d+(?:\.\d+)?)", out)
        return min(10.0, float(m.group(1))) if m else 0.0

    def reason(self, question: str) -> YvReasoningTrace:
        frontier: List[Tuple[float, List[str]]] = [(0.0, [])]
        done: List[Tuple[float, List[str], str]] = []
        for _ in range(self.max_depth):
            cand: List[Tuple[float, List[str]]] = []
            for _, steps in frontier:
                seen = set()
                for _b in range(self.branch):
                    nxt = self.generate(self.STEP.format(question=question, steps="\n".join(steps) or "(none)"),
                                        self.max_new_tokens).strip().split("\n")[0].strip()
                    if not nxt or nxt in seen:
                        continue
                    seen.add(nxt)
                    self.expanded += 1
                    chain = steps + [nxt]
                    v = self._value(question, chain)
                    ans = extract_answer(nxt)
                    if ans is not None:
                        done.append((v, chain, ans))
                    else:
                        cand.append((v, chain))
            if not cand:
                break
            cand.sort(key=lambda c: -c[0])
            frontier = cand[: self.beam]
        if done:
            v, chain, ans = max(done, key=lambda c: c[0])
            return YvReasoningTrace(steps=chain, answer=ans, votes=dict(Counter(a for _, _, a in done)))
        best = max(frontier, key=lambda c: c[0])[1] if frontier else []
        return YvReasoningTrace(steps=best, answer=None)


class YvCoTMemoryReasoner:
    """Chain of thought with an episodic memory: solved questions are stored with their steps; a new question first
    retrieves the most similar stored ones (token-overlap similarity) and shows them as worked examples."""

    def __init__(self, generate: GenerateFn, capacity: int = 256, shots: int = 2, max_new_tokens: int = 256):
        self.cot, self.capacity, self.shots = YvCoTReasoner(generate, max_new_tokens), capacity, shots
        self.memory: List[Tuple[str, YvReasoningTrace]] = []

    @staticmethod
    def _sim(a: str, b: str) -> float:
        ta, tb = set(a.lower().split()), set(b.lower().split())
        return len(ta & tb) / max(1, len(ta | tb))

    def recall(self, question: str) -> List[Tuple[str, YvReasoningTrace]]:
        ranked = sorted(self.memory, key=lambda m: -self._sim(question, m[0]))
        return [m for m in ranked[: self.shots] if self._sim(question, m[0]) > 0]

    def reason(self, question: str, remember: bool = True) -> YvReasoningTrace:
        shots = self.recall(question)
        prefix = "".join(f"Q: {q}\n" + "\n".join(t.steps) + f"\nAnswer: {t.answer}\n\n" for q, t in shots)
        trace = self.cot.reason(prefix + question if prefix else question)
        if remember and trace.answer is not None:
            self.memory.append((question, trace))
            del self.memory[:-self.capacity]
        return trace


class YvUnifiedReasoner:
    """Front door: picks a strategy by name and optionally verifies, retrying once on a failed check."""

    def __init__(self, generate: GenerateFn, strategy: str = "cot", verify: bool = False, **kw: Any):
        self.impl = {"cot": YvCoTReasoner, "multipath": YvMultiPathReasoner, "recursive": YvRecursiveReasoner,
                     "tree": YvThoughtTreeReasoner, "memory": YvCoTMemoryReasoner}[strategy](generate, **kw)
        self.verifier = YvVeriCoTVerifier() if verify else None

    def reason(self, question: str) -> YvReasoningTrace:
        t = self.impl.reason(question)
        if self.verifier is not None and not self.verifier.verify(t):
            t = self.impl.reason(question + "\n(Check each calculation.)")
            self.verifier.verify(t)
        return t


# ------------------------------------------------------------------------------------------------------ agentic
@dataclass
class YvToolSpec:
    name: str
    description: str
    fn: Callable[..., Any]
    parameters: Dict[str, str] = field(default_factory=dict)


class YvToolRegistry:
    def __init__(self):
        self.tools: Dict[str, YvToolSpec] = {}

    def register(self, name: str, description: str = "", parameters: Optional[Dict[str, str]] = None):
        def deco(fn):
            self.tools[name] = YvToolSpec(name, description, fn, parameters or {})
            return fn
        return deco

    def call(self, name: str, args: Dict[str, Any]) -> Any:
        if name not in self.tools:
            raise KeyError(f"unknown tool {name!r}")
        return self.tools[name].fn(**args)

    def describe(self) -> str:
        return "\n".join(f"- {t.name}({', '.join(t.parameters)}): {t.description}" for t in self.tools.values())


_TOOL_XML = re.compile(r"<tool_call>\s*<name>(.*?)</name>\s*<arguments>(.*?)</arguments>\s*</tool_call>", re.S)


def parse_tool_calls(text: str) -> List[Tuple[str, Dict[str, Any]]]:
    """``<tool_call><name>n</name><arguments>{json}</arguments></tool_call>`` blocks -> [(name, args)]."""
    calls = []
    for name, args in _TOOL_XML.findall(text):
        try:
            calls.append((name.strip(), json.loads(args) if args.strip() else {}))
        except json.JSONDecodeError:
            calls.append((name.strip(), {"_raw": args.strip()}))
    return calls


class YvAgentMemory:
    def __init__(self, max_items: int = 64):
        self.items: List[Tuple[str, str]] = []
        self.max_items = max_items

    def add(self, role: str, content: str) -> None:
        self.items.append((role, content))
        del self.items[:-self.max_items]

    def render(self) -> str:
        return "\n".join(f"{r}: {c}" for r, c in self.items)


class YvAgentic:
    """ReAct loop: think / act / observe until the model answers without a tool call or ``max_turns`` is hit."""

    def __init__(self, generate: GenerateFn, tools: YvToolRegistry, max_turns: int = 6, max_new_tokens: int = 256):
        self.generate, self.tools, self.max_turns, self.max_new_tokens = generate, tools, max_turns, max_new_tokens
        self.memory = YvAgentMemory()

    def run(self, task: str) -> Dict[str, Any]:
        self.memory.add("user", task)
        trajectory: List[Dict[str, Any]] = []
        for turn in range(self.max_turns):
            prompt = f"Tools:\n{self.tools.describe()}\n\n{self.memory.render()}\nassistant:"
            out = self.generate(prompt, self.max_new_tokens)
            calls = parse_tool_calls(out)
            self.memory.add("assistant", out)
            if not calls:
                return {"answer": out.strip(), "turns": turn + 1, "trajectory": trajectory}
            for name, args in calls:
                try:
                    obs = self.tools.call(name, args)
                except Exception as e:                     # the observation carries the failure back to the model
                    obs = f"error: {type(e).__name__}: {e}"
                trajectory.append({"tool": name, "args": args, "observation": obs})
                self.memory.add("tool", f"{name} -> {obs}")
        return {"answer": None, "turns": self.max_turns, "trajectory": trajectory}


@dataclass
class YvMCPMessage:
    """JSON-RPC 2.0 envelope used by the model-context-protocol bridge."""
    method: str
    params: Dict[str, Any] = field(default_factory=dict)
    id: Optional[int] = None

    def to_json(self) -> str:
        d: Dict[str, Any] = {"jsonrpc": "2.0", "method": self.method, "params": self.params}
        if self.id is not None:
            d["id"] = self.id
        return json.dumps(d)

    @staticmethod
    def from_json(s: str) -> "YvMCPMessage":
        d = json.loads(s)
        return YvMCPMessage(d["method"], d.get("params", {}), d.get("id"))


class YvMCPToolBridge:
    """Serves a ``YvToolRegistry`` over MCP-style ``tools/list`` and ``tools/call`` requests."""

    def __init__(self, tools: YvToolRegistry):
        self.tools = tools

    def handle(self, raw: str) -> str:
        msg = YvMCPMessage.from_json(raw)
        try:
            if msg.method == "tools/list":
                result: Any = [{"name": t.name, "description": t.description, "parameters": t.parameters}
                               for t in self.tools.tools.values()]
            elif msg.method == "tools/call":
                result = self.tools.call(msg.params["name"], msg.params.get("arguments", {}))
            else:
                return json.dumps({"jsonrpc": "2.0", "id": msg.id, "error": {"code": -32601, "message": "method not found"}})
            return json.dumps({"jsonrpc": "2.0", "id": msg.id, "result": result})
        except Exception as e:
            return json.dumps({"jsonrpc": "2.0", "id": msg.id, "error": {"code": -32000, "message": str(e)}})
