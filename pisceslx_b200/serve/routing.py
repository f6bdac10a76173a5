"""Request routing in front of the engine: model-id resolution with strategies, availability and load, and detection of
agent / swarm / orchestration / tool patterns in a message (reference tools/infer/model_router.py:62-460,
tools/infer/agent_interceptor.py:81-500).

``serve/server.py`` keeps the small router and the tool-call loop the HTTP service uses; this module is the full form:
typed results, load-balanced and complexity-driven selection over ``serve.infer_config.MODEL_SPECS``, route history, and
the XML pattern interceptor."""
from __future__ import annotations

import json
import re
import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Deque, Dict, List, Optional

from .infer_config import MODEL_SPECS, PiscesLxModelSpec


class PiscesLxRoutingStrategy(str, Enum):
    EXPLICIT = "explicit"
    AUTO = "auto"
    LOAD_BALANCED = "load_balanced"
    FALLBACK = "fallback"


@dataclass
class PiscesLxRouteResult:
    model_spec: Optional[PiscesLxModelSpec]
    model_id: str
    model_size: str
    strategy: PiscesLxRoutingStrategy
    fallback_chain: List[str] = field(default_factory=list)
    metadata: Dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> Dict[str, Any]:
        return {"model_id": self.model_id, "model_size": self.model_size, "strategy": self.strategy.value, "fallback_chain": list(self.fallback_chain),
                "metadata": dict(self.metadata)}


def _size_value(size: str) -> float:
    m = re.match(r"^([0-9.]+)([BMT])$", size.upper())
    if not m:
        return float("inf")
    return float(m.group(1)) * {"M": 1e-3, "B": 1.0, "T": 1e3}[m.group(2)]


class PiscesLxSpecModelRouter:
    """``resolve(model_id)``: ``piscesl1-7b`` / ``yv_0.5B`` / ``7B`` name a size; anything else is ``default_size``.  A size that
    is not available falls back to the nearest smaller available one (then the nearest larger).  With the load-balanced
    strategy, a request without an explicit size goes to the available size with the fewest requests in flight."""

    def __init__(self, available_sizes: Optional[List[str]] = None, default_size: str = "7B", strategy: PiscesLxRoutingStrategy = PiscesLxRoutingStrategy.AUTO,
                 specs: Optional[Dict[str, PiscesLxModelSpec]] = None, history: int = 1000):
        self.specs = dict(specs if specs is not None else MODEL_SPECS)
        self.order = sorted(self.specs, key=_size_value)
        self.available_sizes = [s for s in (available_sizes or [default_size])]
        self.default_size, self.strategy = default_size, PiscesLxRoutingStrategy(strategy)
        self.load: Dict[str, int] = {s: 0 for s in self.available_sizes}
        self.in_flight: Dict[str, int] = {s: 0 for s in self.available_sizes}
        self._history: Deque[Dict[str, Any]] = deque(maxlen=history)

    # -- parsing -----------------------------------------------------------------------------------------------------------------
    def _normalize_size(self, size_str: str) -> Optional[str]:
        s = size_str.strip().upper()
        for known in set(self.order) | set(self.available_sizes):
            if known.upper() == s:
                return known
        return s if re.match(r"^[0-9.]+[BMT]$", s) else None

    def _parse_model_id(self, model_id: str) -> Optional[str]:
        m = re.search(r"(?:^|[-_/:\s])([0-9]+(?:\.[0-9]+)?\s*[bmtBMT])$", model_id.strip())
        return self._normalize_size(m.group(1).replace(" ", "")) if m else None

    # -- fallbacks ---------------------------------------------------------------------------------------------------------------
    def _ranked(self) -> List[str]:
        return sorted(set(self.order) | set(self.available_sizes), key=_size_value)

    def _build_fallback_chain(self, primary_size: str) -> List[str]:
        v = _size_value(primary_size)
        smaller = [s for s in reversed(self._ranked()) if _size_value(s) < v and s in self.available_sizes]
        larger = [s for s in self._ranked() if _size_value(s) > v and s in self.available_sizes]
        return smaller + larger

    def _find_fallback(self, requested_size: str) -> str:
        chain = self._build_fallback_chain(requested_size)
        if chain:
            return chain[0]
        if self.default_size in self.available_sizes:
            return self.default_size
        if not self.available_sizes:
            raise RuntimeError("no model is available")
        return self.available_sizes[0]

    # -- routing -----------------------------------------------------------------------------------------------------------------
    def resolve(self, model_id: str) -> PiscesLxRouteResult:
        size = self._parse_model_id(model_id or "")
        meta: Dict[str, Any] = {}
        if size is not None:
            strategy = PiscesLxRoutingStrategy.EXPLICIT
        elif self.strategy is PiscesLxRoutingStrategy.LOAD_BALANCED and self.available_sizes:
            size = min(self.available_sizes, key=lambda s: (self.in_flight.get(s, 0), _size_value(s)))
            strategy = PiscesLxRoutingStrategy.LOAD_BALANCED
        else:
            size, strategy = self.default_size, PiscesLxRoutingStrategy.AUTO
        if size not in self.available_sizes:
            meta["requested_size"] = size
            size, strategy = self._find_fallback(size), PiscesLxRoutingStrategy.FALLBACK
        res = PiscesLxRouteResult(self.specs.get(size), model_id, size, strategy, self._build_fallback_chain(size), meta)
        self._record_route(res)
        return res

    def _record_route(self, result: PiscesLxRouteResult) -> None:
        self.load[result.model_size] = self.load.get(result.model_size, 0) + 1
        self._history.append(dict(result.to_dict(), time=time.time()))

    def begin(self, size: str) -> None:
        self.in_flight[size] = self.in_flight.get(size, 0) + 1

    def end(self, size: str) -> None:
        self.in_flight[size] = max(self.in_flight.get(size, 0) - 1, 0)

    def get_model_spec(self, model_id: str) -> Optional[PiscesLxModelSpec]:
        return self.resolve(model_id).model_spec

    def list_available_models(self) -> List[Dict[str, Any]]:
        out = []
        for s in sorted(self.available_sizes, key=_size_value):
            spec = self.specs.get(s)
            out.append({"id": f"piscesl1-{s.lower()}", "size": s, "context_length": spec.context_length if spec else None,
                        "hidden_size": spec.hidden_size if spec else None, "num_layers": spec.num_layers if spec else None,
                        "moe_experts": spec.moe_experts if spec else None, "requests": self.load.get(s, 0)})
        return out

    def update_availability(self, size: str, available: bool) -> None:
        size = self._normalize_size(size) or size
        if available and size not in self.available_sizes:
            self.available_sizes.append(size)
            self.load.setdefault(size, 0)
            self.in_flight.setdefault(size, 0)
        elif not available and size in self.available_sizes:
            self.available_sizes.remove(size)

    def get_load_stats(self) -> Dict[str, int]:
        return dict(self.load)

    def reset_load_stats(self) -> None:
        self.load = {s: 0 for s in self.available_sizes}

    def get_route_history(self, limit: int = 100) -> List[Dict[str, Any]]:
        return list(self._history)[-limit:]

    def _estimate_model_size(self, prompt_length: int, task_type: str, max_context_needed: int) -> str:
        """The smallest-to-largest list of available models whose context fits, indexed by the task's weight: general
        and creative work take the middle, code / analysis / reasoning move towards the larger end."""
        need = max(prompt_length * 4, max_context_needed)
        fit = [s for s in sorted(self.available_sizes, key=_size_value) if (self.specs.get(s) is None or self.specs[s].context_length >= need)]
        if not fit:
            return max(self.available_sizes, key=lambda s: self.specs[s].context_length if s in self.specs else 0) if self.available_sizes else self.default_size
        w = {"general": 1.0, "code": 1.2, "reasoning": 1.5, "creative": 1.0, "analysis": 1.3}.get(task_type, 1.0)
        return fit[min(int(len(fit) * w * 0.5), len(fit) - 1)]

    def select_by_complexity(self, prompt_length: int, task_type: str = "general", max_context_needed: int = 0) -> PiscesLxRouteResult:
        if self.strategy is not PiscesLxRoutingStrategy.AUTO:
            return self.resolve(f"piscesl1-{self.default_size.lower()}")
        r = self.resolve(f"piscesl1-{self._estimate_model_size(prompt_length, task_type, max_context_needed).lower()}")
        r.strategy = PiscesLxRoutingStrategy.AUTO
        r.metadata.update(task_type=task_type, prompt_length=prompt_length)
        return r

    def __repr__(self) -> str:
        return f"PiscesLxSpecModelRouter(available={self.available_sizes}, default={self.default_size}, strategy={self.strategy.value})"


# ---- agent patterns ---------------------------------------------------------------------------------------------------------------
class PiscesLxAgentMode(str, Enum):
    NONE = "none"
    SINGLE = "single"
    SWARM = "swarm"
    ORCHESTRATED = "orchestrated"
    TOOL_CALL = "tool_call"
    HYBRID = "hybrid"


@dataclass
class PiscesLxInterceptResult:
    mode: PiscesLxAgentMode
    original_content: str
    processed_content: str
    agent_requests: List[Dict[str, Any]] = field(default_factory=list)
    tool_calls: List[Dict[str, Any]] = field(default_factory=list)
    metadata: Dict[str, Any] = field(default_factory=dict)


_ATTR = re.compile(r'([\w-]+)\s*=\s*(?:"([^"]*)"|\'([^\']*)\'|([^\s>]+))')


def _attrs(tag_open: str) -> Dict[str, str]:
    return {m.group(1): next(g for g in m.groups()[1:] if g is not None) for m in _ATTR.finditer(tag_open)}


class PiscesLxAgentPatternInterceptor:
    """Finds ``<ag>name</ag>``, ``<swarm mode=..>task</swarm>``, ``<orchestrate strategy=..>task</orchestrate>`` (bare or inside
    ``<agentic>``) and ``<tool name=..><args>{json}</args></tool>`` in a message, classifies the message and returns the
    text with the patterns removed.  Attributes may come in any order and quoting (the reference's expressions need
    ``mode`` / ``strategy`` / ``name`` to be written a particular way, agent_interceptor.py:160-186)."""

    PATTERNS = {
        "agentic_block": re.compile(r"<agentic\b[^>]*>(.*?)</agentic>", re.S | re.I),
        "agent_invoke": re.compile(r"<ag\b([^>]*)>(.*?)</ag>", re.S | re.I),
        "swarm_invoke": re.compile(r"<swarm\b([^>]*)>(.*?)</swarm>", re.S | re.I),
        "orchestrate_invoke": re.compile(r"<orchestrate\b([^>]*)>(.*?)</orchestrate>", re.S | re.I),
        "tool_invoke": re.compile(r"<tool\b([^>]*)>(.*?)</tool>", re.S | re.I),
        "tool_args": re.compile(r"<args\b[^>]*>(.*?)</args>", re.S | re.I),
    }

    def __init__(self) -> None:
        self.reset_statistics()

    def reset_statistics(self) -> None:
        self.intercept_count = 0
        self.mode_counts = {m.value: 0 for m in PiscesLxAgentMode}

    def _update_mode_counts(self, mode: PiscesLxAgentMode) -> None:
        self.intercept_count += 1
        self.mode_counts[mode.value] += 1

    def _parse_tool_args(self, content: str) -> Dict[str, Any]:
        m = self.PATTERNS["tool_args"].search(content)
        raw = (m.group(1) if m else content).strip()
        if not raw:
            return {}
        try:
            v = json.loads(raw)
            return v if isinstance(v, dict) else {"value": v}
        except ValueError:
            pairs = dict(re.findall(r"(\w+)\s*[:=]\s*\"?([^,\"\n]+)\"?", raw))
            return pairs or {"raw": raw}

    def has_agent_pattern(self, content: str) -> bool:
        return any(self.PATTERNS[k].search(content) for k in ("agentic_block", "agent_invoke", "swarm_invoke", "orchestrate_invoke", "tool_invoke"))

    def extract_agent_names(self, content: str) -> List[str]:
        return [m.group(2).strip() for m in self.PATTERNS["agent_invoke"].finditer(content) if m.group(2).strip()]

    def extract_tool_calls(self, content: str) -> List[Dict[str, Any]]:
        out = []
        for m in self.PATTERNS["tool_invoke"].finditer(content):
            a = _attrs(m.group(1))
            if a.get("name"):
                out.append({"name": a["name"], "arguments": self._parse_tool_args(m.group(2))})
        return out

    def extract_swarm_config(self, content: str) -> Optional[Dict[str, Any]]:
        m = self.PATTERNS["swarm_invoke"].search(content)
        if not m:
            return None
        a = _attrs(m.group(1))
        return {"mode": a.get("mode", "hierarchical"), "task": m.group(2).strip(), **{k: v for k, v in a.items() if k != "mode"}}

    def extract_orchestrate_config(self, content: str) -> Optional[Dict[str, Any]]:
        m = self.PATTERNS["orchestrate_invoke"].search(content)
        if not m:
            return None
        a = _attrs(m.group(1))
        return {"strategy": a.get("strategy", "dynamic"), "task": m.group(2).strip(), **{k: v for k, v in a.items() if k != "strategy"}}

    def strip_agent_patterns(self, content: str) -> str:
        for k in ("tool_invoke", "swarm_invoke", "orchestrate_invoke", "agent_invoke", "agentic_block"):
            content = self.PATTERNS[k].sub("", content)
        return re.sub(r"\n{3,}", "\n\n", content).strip()

    def intercept(self, content: str) -> PiscesLxInterceptResult:
        agents = [{"type": "agent", "name": n} for n in self.extract_agent_names(content)]
        swarm, orch, tools = self.extract_swarm_config(content), self.extract_orchestrate_config(content), self.extract_tool_calls(content)
        kinds = [bool(agents), swarm is not None, orch is not None, bool(tools)]
        if sum(kinds) > 1:
            mode = PiscesLxAgentMode.HYBRID
        elif swarm is not None:
            mode = PiscesLxAgentMode.SWARM
        elif orch is not None:
            mode = PiscesLxAgentMode.ORCHESTRATED
        elif tools:
            mode = PiscesLxAgentMode.TOOL_CALL
        elif agents:
            mode = PiscesLxAgentMode.SINGLE
        else:
            mode = PiscesLxAgentMode.NONE
        reqs = list(agents)
        if swarm is not None:
            reqs.append({"type": "swarm", **swarm})
        if orch is not None:
            reqs.append({"type": "orchestrate", **orch})
        stripped = self.strip_agent_patterns(content) if mode is not PiscesLxAgentMode.NONE else content
        self._update_mode_counts(mode)
        return PiscesLxInterceptResult(mode, content, stripped, reqs, tools,
                                       {"in_agentic_block": bool(self.PATTERNS["agentic_block"].search(content)), "pattern_count": len(reqs) + len(tools)})

    def get_statistics(self) -> Dict[str, Any]:
        return {"intercept_count": self.intercept_count, "mode_counts": dict(self.mode_counts)}

    def __repr__(self) -> str:
        return f"PiscesLxAgentPatternInterceptor(intercepts={self.intercept_count})"
