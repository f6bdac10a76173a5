"""XML call format (parser / generator) and the MCP core (registry, executor with timeouts, history)."""
import time

import pytest

from pisceslx_b200.models.agentic_mcp import (YvAgenticAction, YvAgenticObservation, YvCoreMCPToolRegistry, YvExecutionMode, YvMCPEnvelope, YvMCPExecutionResult,
                                              YvMCPMessageType, YvMCPProtocol, YvMCPService, YvMCPToolMetadata, YvMCPToolType, YvMCPUnifiedToolExecutor,
                                              YvMCPXMLGenerator, YvMCPXMLParser, YvXMLMode, xml_generator, xml_parser)
from pisceslx_b200.models.agentic_tools import YvCalculateTool, YvSEERCalculateTool, YvSEERResult, register_seer_tools


def test_generator_and_parser_round_trip():
    g, p = YvMCPXMLGenerator(), YvMCPXMLParser()
    xml = g.generate_agentic_call("planner <1>", [{"name": "search", "params": {"query": "a < b & \"c\""}, "priority": "high", "fallback": "web"}],
                                  mode="sequential", timeout="30", context="c1")
    ok, err = p.validate_xml_structure(xml)
    assert ok and err is None
    calls = p.extract_agentic_calls("text before " + xml + " after")
    assert len(calls) == 1
    c = calls[0]
    assert c.mode == YvXMLMode.SEQUENTIAL.value and c.parameters == {"timeout": "30"} and c.start_pos == len("text before ")
    assert c.agents[0].agent_name == "planner <1>" and c.agents[0].context == "c1" and c.agents[0].timeout == "30"
    t = c.tools[0]
    assert t.tool_name == "search" and t.parameters == {"query": "a < b & \"c\""} and t.priority == "high" and t.fallback == "web"
    assert p.remove_agentic_tags("x " + xml + " y", "[call]") == "x [call] y"
    sw = g.generate_swarm_call(["a", "b"], [{"name": "t", "params": {}}])
    s = p.extract_agentic_calls(sw)[0]
    assert s.mode == "swarm" and s.agent_group.agents == ["a", "b"] and s.agents == [] and s.tools[0].tool_name == "t"
    # attributes in the other order and single quotes still parse
    alt = "<agentic timeout='5' mode='swarm'><ag>x</ag><tool fallback='f' priority='low'><tn>k</tn><tp>not json</tp></tool><context_ref>r1</context_ref></agentic>"
    a = p.extract_agentic_calls(alt)[0]
    assert a.mode == "swarm" and a.parameters["timeout"] == "5" and a.tools[0].fallback == "f" and a.tools[0].parameters == {"raw": "not json"} and a.context_refs == ["r1"]


def test_legacy_validation_and_results():
    p = xml_parser
    legacy = '<agentic><an>calc</an><ap1>{"x": 1}</ap1><ap2>plain</ap2></agentic>'
    assert p.extract_legacy_calls(legacy)[0]["parameters"] == {"ap1": {"x": 1}, "ap2": "plain"} and p.extract_agentic_calls(legacy) == []
    assert p.validate_xml_structure("<agentic><ag>x</agentic>") == (False, "</agentic> at 14 closes <ag>")
    assert p.validate_xml_structure("<tool><tn>a</tn>")[1] == "<tool> is never closed" and p.validate_xml_structure("</tn>")[0] is False
    assert p.validate_xml_structure("a < b and <b>bold</b>") == (True, None)
    assert p.strip_all_xml_tags("<a>x</a> y") == "x y" and p.unescape_xml(p.escape_xml("<&>\"'")) == "<&>\"'"
    assert xml_generator.generate_result_xml(True, {"a": 1}, agent_name="ag") == '<result success="true" agent="ag"><data>{&quot;a&quot;: 1}</data></result>'
    assert xml_generator.generate_result_xml(False, error_message="bad <x>") == '<result success="false"><error>bad &lt;x&gt;</error></result>'


def test_registry_and_protocol_messages():
    reg = YvCoreMCPToolRegistry()

    def add(a: int, b: int = 1) -> int:
        """Adds."""
        return a + b
    assert reg.register_function(add, tags=["math"]) and not reg.register_function(add) and "add" in reg and len(reg) == 1
    md = reg.get("add")
    assert md.signature()["type"] == "native" and md.parameters["a"]["required"] and not md.parameters["b"]["required"] and md.missing_required({"b": 2}) == ["a"]
    assert reg.list_tools("math") == ["add"] and reg.list_tools("io") == [] and reg.schemas()[0]["description"] == "Adds."
    act = YvAgenticAction("add", {"a": 2}, reasoning="need a sum")
    msg = YvMCPProtocol.tool_call("model", "host", act)
    assert isinstance(msg, YvMCPEnvelope) and msg.message_type is YvMCPMessageType.TOOL_CALL and msg.correlation_id == act.action_id and msg.to_dict()["payload"]["arguments"] == {"a": 2}
    bad = YvMCPProtocol.tool_result("host", "model", YvMCPExecutionResult("add", False, error="x"), msg.correlation_id)
    assert bad.message_type is YvMCPMessageType.ERROR and bad.message_id != msg.message_id
    assert reg.unregister("add") and not reg.unregister("add")


def test_executor_failure_modes_timeout_and_history():
    reg = YvCoreMCPToolRegistry()
    reg.register(YvMCPToolMetadata("ok", "", {"properties": {"x": {"required": True}}}, YvMCPToolType.NATIVE, lambda x: x * 2))
    reg.register(YvMCPToolMetadata("ext", "", {}, YvMCPToolType.EXTERNAL, lambda: "remote"))
    reg.register(YvMCPToolMetadata("boom", "", {}, handler=lambda: 1 / 0))
    reg.register(YvMCPToolMetadata("slow", "", {}, handler=lambda: time.sleep(1.0), timeout_s=0.05))
    reg.register(YvMCPToolMetadata("unbound", "", {}))
    ex = YvMCPUnifiedToolExecutor(reg)
    assert ex.execute("ok", {"x": 4}).output == 8
    assert ex.execute("ok").error == "missing required arguments: ['x']" and ex.execute("nope").error == "unknown tool 'nope'"
    assert "no bound handler" in ex.execute("unbound").error and "ZeroDivisionError" in ex.execute("boom").error
    t0 = time.perf_counter()
    slow = ex.execute("slow")
    assert not slow.success and "did not finish within 0.05s" in slow.error and time.perf_counter() - t0 < 0.8
    assert ex.execute("ext", mode=YvExecutionMode.NATIVE_ONLY).error == "native-only mode rejects external tool"
    assert ex.execute("ok", {"x": 1}, YvExecutionMode.EXTERNAL_ONLY.value).error == "external-only mode rejects native tool" and ex.execute("ext").output == "remote"
    st = ex.manager.stats()
    assert st["calls"] == 9 and st["failures"] == 7 and ex.manager.failure_count() == 7 and st["tools"]["ok"]["calls"] == 3
    obs = ex.execute_action(YvAgenticAction("boom"))
    assert isinstance(obs, YvAgenticObservation) and obs.failed() and not ex.execute_action(YvAgenticAction("ok", {"x": 1})).failed()
    ex.manager.clear()
    assert ex.manager.history() == []
    ex.shutdown()


def test_execute_text_with_fallback_and_seer_tools():
    YvMCPService.reset()
    reg = YvMCPService.registry()
    assert register_seer_tools(reg, [YvCalculateTool()]) == ["calculate"] and YvSEERCalculateTool is YvCalculateTool and YvSEERResult is not None
    reg.register(YvMCPToolMetadata("flaky", "", {}, handler=lambda **kw: 1 / 0))
    ex = YvMCPService.executor()
    assert ex is YvMCPService.executor() and ex.registry is reg
    text = ('sum: <tool><tn>calculate</tn><tp>{"expression": "2 * (3 + 4)"}</tp></tool> and '
            '<tool fallback="calculate"><tn>flaky</tn><tp>{"expression": "10 / 4"}</tp></tool>.')
    out, results = ex.execute_text(text)
    assert [r.success for r in results] == [True, True] and results[1].tool_name == "calculate"
    assert out == 'sum: <result success="true"><data>14</data></result> and <result success="true"><data>2.5</data></result>.'
    YvMCPService.reset()
