"""Model router (strategies, fallbacks, load, complexity) and the agent-pattern interceptor."""
import pytest

from pisceslx_b200.serve.infer_config import PiscesLxModelSpec
from pisceslx_b200.serve.routing import (PiscesLxAgentMode, PiscesLxAgentPatternInterceptor, PiscesLxInterceptResult, PiscesLxRouteResult,
                                         PiscesLxRoutingStrategy, PiscesLxSpecModelRouter)
from pisceslx_b200.serve.schemas import PiscesLxResponseFormat, PiscesLxServiceStats, PiscesLxTool

SPECS = {"0.5B": PiscesLxModelSpec("0.5B", 640, 16, 10, 8192), "7B": PiscesLxModelSpec("7B", 4096, 32, 32, 131072),
         "70B": PiscesLxModelSpec("70B", 8192, 80, 64, 131072), "671B": PiscesLxModelSpec("671B", 7168, 61, 128, 1048576)}


def test_resolution_and_fallbacks():
    r = PiscesLxSpecModelRouter(["0.5B", "7B", "671B"], "7B", specs=SPECS)
    a = r.resolve("piscesl1-7b")
    assert isinstance(a, PiscesLxRouteResult) and a.model_size == "7B" and a.strategy is PiscesLxRoutingStrategy.EXPLICIT and a.model_spec.hidden_size == 4096
    assert a.fallback_chain == ["0.5B", "671B"]
    assert r.resolve("yv_0.5B").model_size == "0.5B" and r.resolve("671B").model_size == "671B"
    b = r.resolve("gpt-4")
    assert b.model_size == "7B" and b.strategy is PiscesLxRoutingStrategy.AUTO
    c = r.resolve("piscesl1-70b")
    assert c.model_size == "7B" and c.strategy is PiscesLxRoutingStrategy.FALLBACK and c.metadata["requested_size"] == "70B"
    r.update_availability("7B", False)
    assert r.resolve("piscesl1-70b").model_size == "0.5B" and r.resolve("x").model_size == "0.5B"
    r.update_availability("70b", True)
    assert r.resolve("piscesl1-70b").strategy is PiscesLxRoutingStrategy.EXPLICIT
    assert r.get_load_stats()["0.5B"] == 3 and len(r.get_route_history(3)) == 3 and r.get_route_history()[0]["model_id"] == "piscesl1-7b"
    r.reset_load_stats()
    assert sum(r.get_load_stats().values()) == 0
    ids = [m["id"] for m in r.list_available_models()]
    assert ids == ["piscesl1-0.5b", "piscesl1-70b", "piscesl1-671b"]
    assert r.get_model_spec("70B").num_layers == 80 and "available" in repr(r)
    empty = PiscesLxSpecModelRouter(["7B"], "7B", specs=SPECS)
    empty.update_availability("7B", False)
    with pytest.raises(RuntimeError):
        empty.resolve("7B")


def test_load_balanced_and_complexity_selection():
    r = PiscesLxSpecModelRouter(["0.5B", "7B"], "7B", PiscesLxRoutingStrategy.LOAD_BALANCED, specs=SPECS)
    assert r.resolve("anything").model_size == "0.5B"                                  # ties go to the smaller model
    r.begin("0.5B")
    x = r.resolve("anything")
    assert x.model_size == "7B" and x.strategy is PiscesLxRoutingStrategy.LOAD_BALANCED
    r.end("0.5B")
    assert r.resolve("anything").model_size == "0.5B" and r.select_by_complexity(100).model_size == "7B"
    a = PiscesLxSpecModelRouter(["0.5B", "7B", "70B", "671B"], "7B", specs=SPECS)
    assert a.select_by_complexity(100, "general").model_size == "70B"                   # index int(4 * 0.5) of the four that fit
    assert a.select_by_complexity(100, "reasoning").model_size == "671B"
    assert a.select_by_complexity(100_000, "general").model_size == "671B"             # only one context is long enough
    assert a.select_by_complexity(3000, "general").model_size in ("70B", "671B")       # 0.5B's 8k context is too short for 12k
    assert a.select_by_complexity(10**7).model_size == "671B"                           # nothing fits: the longest context


def test_interceptor_modes_and_extraction():
    it = PiscesLxAgentPatternInterceptor()
    r = it.intercept("<ag>code_gen</ag>write a sort")
    assert isinstance(r, PiscesLxInterceptResult) and r.mode is PiscesLxAgentMode.SINGLE and r.processed_content == "write a sort"
    assert r.agent_requests == [{"type": "agent", "name": "code_gen"}]
    s = it.intercept("<agentic>\n<swarm topology=ring mode='mesh'>analyse data</swarm>\n</agentic>")
    assert s.mode is PiscesLxAgentMode.SWARM and s.agent_requests[0] == {"type": "swarm", "mode": "mesh", "task": "analyse data", "topology": "ring"}
    assert s.metadata["in_agentic_block"] and s.processed_content == ""
    o = it.intercept('before <orchestrate strategy="dynamic">research trends</orchestrate> after')
    assert o.mode is PiscesLxAgentMode.ORCHESTRATED and o.agent_requests[0]["strategy"] == "dynamic" and o.processed_content == "before  after"
    t = it.intercept('<tool name="web_search"><args>{"query": "news", "n": 3}</args></tool>')
    assert t.mode is PiscesLxAgentMode.TOOL_CALL and t.tool_calls == [{"name": "web_search", "arguments": {"query": "news", "n": 3}}]
    loose = it.extract_tool_calls("<tool name='calc'><args>expr: 1+1, mode=fast</args></tool><tool><args>{}</args></tool>")
    assert loose == [{"name": "calc", "arguments": {"expr": "1+1", "mode": "fast"}}]
    h = it.intercept('<ag>planner</ag><tool name="x"><args>[1, 2]</args></tool> go')
    assert h.mode is PiscesLxAgentMode.HYBRID and h.tool_calls[0]["arguments"] == {"value": [1, 2]} and h.metadata["pattern_count"] == 2
    n = it.intercept("plain <b>text</b>")
    assert n.mode is PiscesLxAgentMode.NONE and n.processed_content == "plain <b>text</b>" and not it.has_agent_pattern("plain")
    st = it.get_statistics()
    assert st["intercept_count"] == 6 and st["mode_counts"]["hybrid"] == 1 and st["mode_counts"]["none"] == 1
    it.reset_statistics()
    assert it.get_statistics()["intercept_count"] == 0


def test_schema_additions():
    assert PiscesLxResponseFormat().type == "text" and PiscesLxTool(function={"name": "f"}).type == "function"
    s = PiscesLxServiceStats(request_count=3, latency_p50_ms=1.5)
    assert s.model_dump()["request_count"] == 3 and s.latency_p95_ms is None
