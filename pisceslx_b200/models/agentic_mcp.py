"""The model side of the tool protocol: the XML call format the model writes and reads (parser and generator), and the MCP
core - message / metadata / result types, tool registry, executor with a timeout per tool, execution history
(reference model/multimodal/xml_utils.py:64-480, model/multimodal/mcp_protocol.py:61-390).

Call format::

    <agentic mode="swarm" timeout="30">
      <ag context="c1">planner</ag>  or  <ag_group><ag>a</ag><ag>b</ag></ag_group>
      <tool priority="high" fallback="web"><tn>search</tn><tp>{"query": "x"}</tp></tool>
      <context_ref>c1</context_ref>
    </agentic>

Attributes are read in any order and with either kind of quote (the reference's expressions fix the order ``mode`` then
``timeout`` and ``priority`` then ``fallback``, xml_utils.py:118-133, and silently miss a block that writes them the
other way round).  The executor runs a handler on a worker thread and gives up waiting after the tool's ``timeout_s``
(the reference stores ``timeout_s`` and never applies it, mcp_protocol.py:314-362)."""
from __future__ import annotations

import concurrent.futures
import html
import json
import re
import threading
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Tuple


# ---- XML ------------------------------------------------------------------------------------------------------------------------
class YvXMLMode(str, Enum):
    SINGLE = "single"
    SWARM = "swarm"
    SEQUENTIAL = "sequential"


@dataclass
class YvAgenticToolCall:
    tool_name: str
    parameters: Dict[str, Any]
    raw_match: str
    start_pos: int
    end_pos: int
    priority: Optional[str] = None
    fallback: Optional[str] = None


@dataclass
class YvAgenticAgentCall:
    agent_name: str
    raw_match: str
    start_pos: int
    end_pos: int
    timeout: Optional[str] = None
    context: Optional[str] = None


@dataclass
class YvAgenticGroup:
    agents: List[str]
    mode: str
    raw_match: str
    start_pos: int
    end_pos: int


@dataclass
class YvParsedAgenticCall:
    raw_match: str
    start_pos: int
    end_pos: int
    mode: str = "single"
    agents: List[YvAgenticAgentCall] = field(default_factory=list)
    tools: List[YvAgenticToolCall] = field(default_factory=list)
    agent_group: Optional[YvAgenticGroup] = None
    context_refs: List[str] = field(default_factory=list)
    parameters: Dict[str, Any] = field(default_factory=dict)


_ATTR = re.compile(r'([\w-]+)\s*=\s*(?:"([^"]*)"|\'([^\']*)\')')


def _attrs(s: str) -> Dict[str, str]:
    return {m.group(1): (m.group(2) if m.group(2) is not None else m.group(3)) for m in _ATTR.finditer(s or "")}


class YvMCPXMLParser:
    MAX_DEPTH = 64

    def __init__(self) -> None:
        self._setup_patterns()

    def _setup_patterns(self) -> None:
        self.agent_pattern = re.compile(r"<agentic\b([^>]*)>(.*?)</agentic>", re.S)
        self.agent_tag_pattern = re.compile(r"<ag\b([^>]*)>(.*?)</ag>", re.S)
        self.tool_pattern = re.compile(r"<tool\b([^>]*)>(.*?)</tool>", re.S)
        self.tool_name_pattern = re.compile(r"<tn>(.*?)</tn>", re.S)
        self.tool_param_pattern = re.compile(r"<tp>(.*?)</tp>", re.S)
        self.agent_group_pattern = re.compile(r"<ag_group>(.*?)</ag_group>", re.S)
        self.context_ref_pattern = re.compile(r"<context_ref>(.*?)</context_ref>", re.S)
        self.xml_tag_pattern = re.compile(r"<[^>]+>")
        self.param_pattern = re.compile(r"<ap(\d+)>(.+?)</ap\1>", re.S)
        self.legacy_agent_pattern = re.compile(r"<agentic><an>(.+?)</an>(.*?)</agentic>", re.S)

    @staticmethod
    def escape_xml(text: str) -> str:
        return html.escape(str(text), quote=True)

    @staticmethod
    def unescape_xml(text: str) -> str:
        return html.unescape(text)

    def parse_tool_parameters(self, param_text: str) -> Dict[str, Any]:
        t = self.unescape_xml(param_text.strip())
        if not t:
            return {}
        try:
            v = json.loads(t)
            return v if isinstance(v, dict) else {"value": v}
        except RecursionError:
            raise ValueError("JSON content too deeply nested for parsing")
        except ValueError:
            return {"raw": t}

    def _tools(self, body: str, offset: int) -> List[YvAgenticToolCall]:
        out = []
        for m in self.tool_pattern.finditer(body):
            a = _attrs(m.group(1))
            tn = self.tool_name_pattern.search(m.group(2))
            if not tn or not tn.group(1).strip():
                continue
            tp = self.tool_param_pattern.search(m.group(2))
            out.append(YvAgenticToolCall(self.unescape_xml(tn.group(1).strip()), self.parse_tool_parameters(tp.group(1)) if tp else {}, m.group(0),
                                         offset + m.start(), offset + m.end(), a.get("priority"), a.get("fallback")))
        return out

    def extract_agentic_calls(self, text: str) -> List[YvParsedAgenticCall]:
        calls = []
        for m in self.agent_pattern.finditer(text):
            a, body, off = _attrs(m.group(1)), m.group(2), m.start(2)
            if body.lstrip().startswith("<an>"):
                continue                                                                # the older format: extract_legacy_calls
            call = YvParsedAgenticCall(m.group(0), m.start(), m.end(), a.get("mode", "single"))
            if a.get("timeout"):
                call.parameters["timeout"] = a["timeout"]
            gm = self.agent_group_pattern.search(body)
            if gm:
                names = [self.unescape_xml(x.group(2).strip()) for x in self.agent_tag_pattern.finditer(gm.group(1)) if x.group(2).strip()]
                mode = call.mode if call.mode != "single" else "swarm"
                call.agent_group, call.mode = YvAgenticGroup(names, mode, gm.group(0), off + gm.start(), off + gm.end()), mode
            for x in self.agent_tag_pattern.finditer(body):
                if gm and gm.start() <= x.start() < gm.end():
                    continue
                if x.group(2).strip():
                    call.agents.append(YvAgenticAgentCall(self.unescape_xml(x.group(2).strip()), x.group(0), off + x.start(), off + x.end(),
                                                          a.get("timeout"), _attrs(x.group(1)).get("context")))
            call.tools = self._tools(body, off)
            call.context_refs = [c.group(1).strip() for c in self.context_ref_pattern.finditer(body) if c.group(1).strip()]
            calls.append(call)
        return calls

    def extract_tool_calls(self, text: str) -> List[YvAgenticToolCall]:
        """Tool blocks anywhere in the text, inside an ``<agentic>`` block or bare."""
        return self._tools(text, 0)

    def extract_legacy_calls(self, text: str) -> List[Dict[str, Any]]:
        """``<agentic><an>tool</an><ap1>..</ap1><ap2>..</ap2></agentic>``."""
        out = []
        for m in self.legacy_agent_pattern.finditer(text):
            params: Dict[str, Any] = {}
            for p in self.param_pattern.finditer(m.group(2)):
                v = p.group(2).strip()
                try:
                    params[f"ap{p.group(1)}"] = json.loads(v)
                except RecursionError:
                    raise ValueError("JSON content too deeply nested for parsing")
                except ValueError:
                    params[f"ap{p.group(1)}"] = v
            out.append({"tool_name": m.group(1).strip(), "parameters": params, "raw_match": m.group(0), "start_pos": m.start(), "end_pos": m.end()})
        return out

    def remove_agentic_tags(self, text: str, placeholder: str = "") -> str:
        return self.agent_pattern.sub(placeholder, text)

    def strip_all_xml_tags(self, text: str) -> str:
        return self.xml_tag_pattern.sub("", text)

    def validate_xml_structure(self, text: str) -> Tuple[bool, Optional[str]]:
        """Every protocol tag that opens closes, in order, no deeper than ``MAX_DEPTH``; other angle brackets are left alone."""
        known = {"agentic", "ag", "ag_group", "tool", "tn", "tp", "context_ref", "an", "result", "data", "error"}
        stack: List[str] = []
        for m in re.finditer(r"<(/?)([A-Za-z_][\w]*)\b[^>]*?(/?)>", text):
            closing, tag, selfclose = m.group(1) == "/", m.group(2), m.group(3) == "/"
            if tag not in known and not re.fullmatch(r"ap\d+", tag):
                continue
            if selfclose:
                continue
            if not closing:
                stack.append(tag)
                if len(stack) > self.MAX_DEPTH:
                    return False, f"nesting deeper than {self.MAX_DEPTH}"
            else:
                if not stack:
                    return False, f"</{tag}> at {m.start()} closes nothing"
                if stack[-1] != tag:
                    return False, f"</{tag}> at {m.start()} closes <{stack[-1]}>"
                stack.pop()
        return (False, f"<{stack[-1]}> is never closed") if stack else (True, None)


class YvMCPXMLGenerator:
    def __init__(self, parser: Optional[YvMCPXMLParser] = None):
        self.parser = parser or YvMCPXMLParser()

    def _tool(self, tool: Dict[str, Any]) -> str:
        return self.generate_tool_call(tool.get("name", ""), tool.get("params", tool.get("parameters", {})), tool.get("priority"), tool.get("fallback"))

    def generate_tool_call(self, tool_name: str, parameters: Dict[str, Any], priority: Optional[str] = None, fallback: Optional[str] = None) -> str:
        e = self.parser.escape_xml
        attrs = (f' priority="{e(priority)}"' if priority else "") + (f' fallback="{e(fallback)}"' if fallback else "")
        return f"<tool{attrs}><tn>{e(tool_name)}</tn><tp>{e(json.dumps(parameters, ensure_ascii=False))}</tp></tool>"

    def generate_agentic_call(self, agent_name: str, tools: Optional[List[Dict[str, Any]]] = None, mode: str = "single", timeout: Optional[str] = None,
                              context: Optional[str] = None) -> str:
        e = self.parser.escape_xml
        ag = f'<ag{f" context=\"{e(context)}\"" if context else ""}>{e(agent_name)}</ag>'
        attrs = (f' mode="{e(mode)}"' if mode and mode != "single" else "") + (f' timeout="{e(timeout)}"' if timeout else "")
        return f"<agentic{attrs}>{ag}{''.join(self._tool(t) for t in tools or [])}</agentic>"

    def generate_swarm_call(self, agent_names: List[str], tools: Optional[List[Dict[str, Any]]] = None, mode: str = "swarm") -> str:
        e = self.parser.escape_xml
        group = "<ag_group>" + "".join(f"<ag>{e(n)}</ag>" for n in agent_names) + "</ag_group>"
        return f'<agentic mode="{e(mode)}">{group}{"".join(self._tool(t) for t in tools or [])}</agentic>'

    def generate_result_xml(self, success: bool, result: Any = None, agent_name: Optional[str] = None, error_message: Optional[str] = None) -> str:
        e = self.parser.escape_xml
        ag = f' agent="{e(agent_name)}"' if agent_name else ""
        if success:
            body = json.dumps(result, ensure_ascii=False) if isinstance(result, (dict, list)) else str(result)
            return f'<result success="true"{ag}><data>{e(body)}</data></result>'
        return f'<result success="false"{ag}><error>{e(error_message or "Unknown error")}</error></result>'


xml_parser = YvMCPXMLParser()
xml_generator = YvMCPXMLGenerator(xml_parser)


# ---- protocol core ----------------------------------------------------------------------------------------------------------------
class YvMCPMessageType(str, Enum):
    TOOL_CALL = "tool_call"
    TOOL_RESULT = "tool_result"
    TOOL_REGISTER = "tool_register"
    TOOL_LIST = "tool_list"
    HEARTBEAT = "heartbeat"
    ERROR = "error"


class YvMCPToolType(str, Enum):
    NATIVE = "native"          # runs in the model's process
    EXTERNAL = "external"      # runs in a tool host


class YvExecutionMode(str, Enum):
    AUTO = "auto"
    NATIVE_ONLY = "native_only"
    EXTERNAL_ONLY = "external_only"


class YvMCPEnvelope:
    """One message between the model and a tool host (the reference's protocol-level ``YvMCPMessage``, mcp_protocol.py:87-112;
    ``models.reasoning.YvMCPMessage`` is the JSON-RPC form used on the wire)."""

    __slots__ = ("message_type", "sender_id", "receiver_id", "payload", "message_id", "timestamp", "correlation_id")
    _counter = 0
    _lock = threading.Lock()

    def __init__(self, message_type: YvMCPMessageType, sender_id: str, receiver_id: str, payload: Optional[Dict[str, Any]] = None,
                 correlation_id: Optional[str] = None):
        with YvMCPEnvelope._lock:
            YvMCPEnvelope._counter += 1
            n = YvMCPEnvelope._counter
        self.message_type, self.sender_id, self.receiver_id = YvMCPMessageType(message_type), sender_id, receiver_id
        self.payload, self.message_id, self.timestamp, self.correlation_id = dict(payload or {}), f"mcp-{n}", time.time(), correlation_id

    def to_dict(self) -> Dict[str, Any]:
        return {"message_type": self.message_type.value, "sender_id": self.sender_id, "receiver_id": self.receiver_id, "payload": self.payload,
                "message_id": self.message_id, "timestamp": self.timestamp, "correlation_id": self.correlation_id}


class YvMCPToolMetadata:
    __slots__ = ("name", "description", "parameters", "tool_type", "handler", "returns", "timeout_s", "tags")

    def __init__(self, name: str, description: str, parameters: Dict[str, Any], tool_type: YvMCPToolType = YvMCPToolType.NATIVE,
                 handler: Optional[Callable[..., Any]] = None, returns: str = "", timeout_s: float = 30.0, tags: Optional[List[str]] = None):
        self.name, self.description, self.parameters, self.tool_type = name, description, parameters, YvMCPToolType(tool_type)
        self.handler, self.returns, self.timeout_s, self.tags = handler, returns, float(timeout_s), list(tags or [])

    def signature(self) -> Dict[str, Any]:
        return {"name": self.name, "description": self.description, "parameters": self.parameters, "returns": self.returns, "type": self.tool_type.value}

    def missing_required(self, arguments: Dict[str, Any]) -> List[str]:
        """Parameters declared ``{"required": true}`` (or listed under ``"required"``) that the call does not give."""
        req = list(self.parameters.get("required", [])) if isinstance(self.parameters.get("required"), list) else []
        props = self.parameters.get("properties", self.parameters)
        req += [k for k, v in props.items() if isinstance(v, dict) and v.get("required") is True]
        return [k for k in dict.fromkeys(req) if k not in arguments]


class YvMCPExecutionResult:
    __slots__ = ("tool_name", "success", "output", "error", "duration_s", "timestamp")

    def __init__(self, tool_name: str, success: bool, output: Any = None, error: str = "", duration_s: float = 0.0):
        self.tool_name, self.success, self.output, self.error, self.duration_s, self.timestamp = tool_name, bool(success), output, error, duration_s, time.time()

    def is_success(self) -> bool:
        return self.success

    def to_dict(self) -> Dict[str, Any]:
        return {"tool_name": self.tool_name, "success": self.success, "output": self.output, "error": self.error, "duration_s": self.duration_s,
                "timestamp": self.timestamp}


class YvAgenticAction:
    __slots__ = ("tool_name", "arguments", "reasoning", "action_id")

    def __init__(self, tool_name: str, arguments: Optional[Dict[str, Any]] = None, reasoning: str = "", action_id: Optional[str] = None):
        self.tool_name, self.arguments, self.reasoning = tool_name, dict(arguments or {}), reasoning
        self.action_id = action_id or f"act-{int(time.time() * 1e6) & 0xFFFFFFFF:x}"

    def to_dict(self) -> Dict[str, Any]:
        return {"tool_name": self.tool_name, "arguments": self.arguments, "reasoning": self.reasoning, "action_id": self.action_id}

    @classmethod
    def from_tool_call(cls, call: YvAgenticToolCall) -> "YvAgenticAction":
        return cls(call.tool_name, call.parameters)


class YvAgenticObservation:
    __slots__ = ("content", "error", "timestamp")

    def __init__(self, content: Any, error: str = "", timestamp: Optional[float] = None):
        self.content, self.error, self.timestamp = content, error, time.time() if timestamp is None else timestamp

    def failed(self) -> bool:
        return bool(self.error)

    @classmethod
    def from_result(cls, result: YvMCPExecutionResult) -> "YvAgenticObservation":
        return cls(result.output, result.error)


class YvMCPProtocol:
    @staticmethod
    def create_message(message_type: YvMCPMessageType, sender_id: str, receiver_id: str, payload: Optional[Dict[str, Any]] = None,
                       correlation_id: Optional[str] = None) -> YvMCPEnvelope:
        return YvMCPEnvelope(message_type, sender_id, receiver_id, payload, correlation_id)

    @staticmethod
    def tool_call(sender_id: str, receiver_id: str, action: YvAgenticAction, correlation_id: Optional[str] = None) -> YvMCPEnvelope:
        return YvMCPEnvelope(YvMCPMessageType.TOOL_CALL, sender_id, receiver_id, action.to_dict(), correlation_id or action.action_id)

    @staticmethod
    def tool_result(sender_id: str, receiver_id: str, result: YvMCPExecutionResult, correlation_id: Optional[str] = None) -> YvMCPEnvelope:
        return YvMCPEnvelope(YvMCPMessageType.TOOL_RESULT if result.success else YvMCPMessageType.ERROR, sender_id, receiver_id, result.to_dict(), correlation_id)


YvCoreMCPProtocol = YvMCPProtocol


class YvCoreMCPToolRegistry:
    def __init__(self) -> None:
        self._tools: Dict[str, YvMCPToolMetadata] = {}
        self._lock = threading.Lock()

    def register(self, metadata: YvMCPToolMetadata, replace: bool = False) -> bool:
        with self._lock:
            if metadata.name in self._tools and not replace:
                return False
            self._tools[metadata.name] = metadata
            return True

    def register_function(self, fn: Callable[..., Any], name: Optional[str] = None, description: str = "", **kw: Any) -> bool:
        """A plain function as a native tool; its parameters are taken from the signature."""
        import inspect
        props = {p.name: {"type": getattr(p.annotation, "__name__", "any") if p.annotation is not inspect.Parameter.empty else "any",
                          "required": p.default is inspect.Parameter.empty} for p in inspect.signature(fn).parameters.values()
                 if p.kind in (p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY)}
        return self.register(YvMCPToolMetadata(name or fn.__name__, description or (fn.__doc__ or "").strip(), props, YvMCPToolType.NATIVE, fn, **kw))

    def unregister(self, name: str) -> bool:
        with self._lock:
            return self._tools.pop(name, None) is not None

    def get(self, name: str) -> Optional[YvMCPToolMetadata]:
        return self._tools.get(name)

    def list_tools(self, tag: Optional[str] = None) -> List[str]:
        return sorted(n for n, m in self._tools.items() if tag is None or tag in m.tags)

    def schemas(self) -> List[Dict[str, Any]]:
        return [self._tools[n].signature() for n in sorted(self._tools)]

    def __contains__(self, name: str) -> bool:
        return name in self._tools

    def __len__(self) -> int:
        return len(self._tools)


YvMCPToolRegistry = YvCoreMCPToolRegistry


class YvMCPExecutionManager:
    def __init__(self, max_history: int = 1000):
        from collections import deque
        self._history = deque(maxlen=max_history)
        self._lock = threading.Lock()

    def record(self, result: YvMCPExecutionResult) -> None:
        with self._lock:
            self._history.append(result)

    def history(self) -> List[YvMCPExecutionResult]:
        return list(self._history)

    def failure_count(self) -> int:
        return sum(1 for r in self._history if not r.success)

    def stats(self) -> Dict[str, Any]:
        h = list(self._history)
        per: Dict[str, Dict[str, float]] = {}
        for r in h:
            d = per.setdefault(r.tool_name, {"calls": 0, "failures": 0, "total_s": 0.0})
            d["calls"] += 1
            d["failures"] += 0 if r.success else 1
            d["total_s"] += r.duration_s
        return {"calls": len(h), "failures": self.failure_count(), "tools": per}

    def clear(self) -> None:
        with self._lock:
            self._history.clear()


class YvMCPUnifiedToolExecutor:
    """``execute(name, arguments, mode)``: unknown tools, tools without a handler, a mode that rejects the tool's type, missing
    required arguments, a handler that raises and a handler that outlives the tool's timeout all come back as failed
    results (never as exceptions), and every result is recorded."""

    _instance: Optional["YvMCPUnifiedToolExecutor"] = None

    def __init__(self, registry: Optional[YvCoreMCPToolRegistry] = None, max_workers: int = 4):
        self.registry = registry or YvCoreMCPToolRegistry()
        self._manager = YvMCPExecutionManager()
        self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=max_workers, thread_name_prefix="yv-mcp")

    @classmethod
    def get_instance(cls) -> "YvMCPUnifiedToolExecutor":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    @property
    def manager(self) -> YvMCPExecutionManager:
        return self._manager

    def execute(self, tool_name: str, arguments: Optional[Dict[str, Any]] = None, mode: str = YvExecutionMode.AUTO.value) -> YvMCPExecutionResult:
        t0 = time.perf_counter()
        args = dict(arguments or {})
        mode = getattr(mode, "value", mode)

        def fail(msg: str) -> YvMCPExecutionResult:
            r = YvMCPExecutionResult(tool_name, False, error=msg, duration_s=time.perf_counter() - t0)
            self._manager.record(r)
            return r
        md = self.registry.get(tool_name)
        if md is None:
            return fail(f"unknown tool '{tool_name}'")
        if md.handler is None:
            return fail(f"tool '{tool_name}' has no bound handler")
        if mode == YvExecutionMode.NATIVE_ONLY.value and md.tool_type is not YvMCPToolType.NATIVE:
            return fail("native-only mode rejects external tool")
        if mode == YvExecutionMode.EXTERNAL_ONLY.value and md.tool_type is not YvMCPToolType.EXTERNAL:
            return fail("external-only mode rejects native tool")
        missing = md.missing_required(args)
        if missing:
            return fail(f"missing required arguments: {missing}")
        fut = self._pool.submit(md.handler, **args)
        try:
            out = fut.result(timeout=md.timeout_s if md.timeout_s > 0 else None)
        except concurrent.futures.TimeoutError:
            fut.cancel()
            return fail(f"tool '{tool_name}' did not finish within {md.timeout_s:g}s")
        except Exception as e:
            return fail(f"{type(e).__name__}: {e}")
        r = YvMCPExecutionResult(tool_name, True, out, duration_s=time.perf_counter() - t0)
        self._manager.record(r)
        return r

    def execute_action(self, action: YvAgenticAction, mode: str = YvExecutionMode.AUTO.value) -> YvAgenticObservation:
        return YvAgenticObservation.from_result(self.execute(action.tool_name, action.arguments, mode))

    def execute_text(self, text: str, parser: Optional[YvMCPXMLParser] = None, generator: Optional[YvMCPXMLGenerator] = None) -> Tuple[str, List[YvMCPExecutionResult]]:
        """Runs every ``<tool>`` block of ``text`` (trying the block's ``fallback`` tool when the first fails) and returns the text
        with each block replaced by its ``<result>`` element."""
        parser, generator = parser or xml_parser, generator or xml_generator
        results, out, last = [], [], 0
        for call in parser.extract_tool_calls(text):
            r = self.execute(call.tool_name, call.parameters)
            if not r.success and call.fallback:
                r = self.execute(call.fallback, call.parameters)
            results.append(r)
            out.append(text[last:call.start_pos] + generator.generate_result_xml(r.success, r.output, error_message=r.error))
            last = call.end_pos
        return "".join(out) + text[last:], results

    def shutdown(self) -> None:
        self._pool.shutdown(wait=False, cancel_futures=True)


class YvMCPService:
    """Process-wide registry and executor."""

    _registry: Optional[YvCoreMCPToolRegistry] = None
    _executor: Optional[YvMCPUnifiedToolExecutor] = None

    @classmethod
    def registry(cls) -> YvCoreMCPToolRegistry:
        if cls._registry is None:
            cls._registry = YvCoreMCPToolRegistry()
        return cls._registry

    @classmethod
    def executor(cls) -> YvMCPUnifiedToolExecutor:
        if cls._executor is None:
            cls._executor = YvMCPUnifiedToolExecutor(cls.registry())
        return cls._executor

    @classmethod
    def reset(cls) -> None:
        if cls._executor is not None:
            cls._executor.shutdown()
        cls._registry, cls._executor = None, None
