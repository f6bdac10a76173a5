"""MCP service types, tool base and registry, sandbox (child process), monitor, remote client over an injected transport."""
import time

import pytest

from pisceslx_b200.models.agentic_mcp import YvCoreMCPToolRegistry, YvMCPToolMetadata, YvMCPUnifiedToolExecutor
from pisceslx_b200.third_party.mcp_types import (
    POPSSMCPClient, POPSSMCPClientConfig, POPSSMCPConfiguration, POPSSMCPExecutionContext, POPSSMCPHealthCheckStatus, POPSSMCPMonitor, POPSSMCPPerformanceMetrics,
    POPSSMCPPlaza, POPSSMCPSessionMemory, POPSSMCPToolBase, POPSSMCPToolMetadata, POPSSMCPToolRegistry, POPSSMCPToolResult, POPSSSandboxConfig, POPSSToolSandbox)


class Echo(POPSSMCPToolBase):
    name, description, category = "echo", "Repeats a text a number of times", "utility"
    parameters = {"type": "object", "properties": {"text": {"type": "string"}, "times": {"type": "integer"}, "mode": {"type": "string", "enum": ["plain", "upper"]}},
                  "required": ["text"], "additionalProperties": False}

    def execute(self, arguments):
        if arguments.get("text") == "explode":
            raise RuntimeError("kaboom")
        t = arguments["text"] * arguments.get("times", 1)
        return t.upper() if arguments.get("mode") == "upper" else t


def test_types_keep_running_statistics():
    md = POPSSMCPToolMetadata("t", "d")
    md.record_use(True); md.record_use(False)
    assert md.usage_count == 2 and md.error_rate == 0.5 and md.last_used is not None
    pm = POPSSMCPPerformanceMetrics()
    for ok, s in ((True, 1.0), (False, 3.0)):
        pm.record(ok, s)
    assert pm.total_executions == 2 and pm.average_execution_time == 2.0 and pm.error_rate == 0.5
    ctx = POPSSMCPExecutionContext("s", "t", {}).finish(result=1)
    assert ctx.performance_metrics["duration_s"] >= 0 and ctx.result == 1
    mem = POPSSMCPSessionMemory("s")
    for i in range(25):
        mem.remember("tool", f"k{i}", i)
    assert len(mem.tool_memories["tool"]) == 20 and mem.recall("tool", "k0") is None and mem.recall("tool", "k24") == 24 and mem.usage_statistics["tool"] == 25
    assert "calculator" in POPSSMCPConfiguration().blacklisted_tools and POPSSMCPPlaza is not None


def test_tool_base_validation_and_registry():
    t = Echo()
    assert t.execute_sync({"text": "ab", "times": 2, "mode": "upper"}).output == "ABAB"
    for args, frag in (({}, "missing required"), ({"text": 1}, "type string"), ({"text": "a", "times": True}, "type integer"), ({"text": "a", "x": 1}, "unexpected"),
                       ({"text": "a", "mode": "loud"}, "one of")):
        r = t.execute_sync(args)
        assert not r.success and frag in r.error and r.error_type == "ValidationError"
    boom = t.execute_sync({"text": "explode"})
    assert isinstance(boom, POPSSMCPToolResult) and boom.error == "kaboom" and boom.error_type == "RuntimeError" and t.metadata.usage_count == 7
    reg = POPSSMCPToolRegistry()
    assert reg.register(t) and not reg.register(Echo()) and reg.add_alias("say", "echo") and not reg.add_alias("x", "nope")
    assert reg.execute("say", {"text": "hi"}).output == "hi" and reg.execute("nope").error_type == "UnknownTool"
    assert reg.search("repeats") == ["echo"] and reg.list_tools("utility")[0]["name"] == "echo" and reg.list_tools("analytics") == []
    assert [e.success for e in reg.executions] == [True, False]
    blocked = POPSSMCPToolRegistry(POPSSMCPConfiguration(blacklisted_tools={"echo"}))
    assert not blocked.register(Echo())
    core = YvCoreMCPToolRegistry()
    assert reg.export(core) == ["echo"]
    ex = YvMCPUnifiedToolExecutor(core)
    assert ex.execute("echo", {"text": "z", "times": 3}).output == "zzz" and "missing required" in ex.execute("echo", {"times": 3}).error
    ex.shutdown()
    assert reg.unregister("echo") and reg.resolve("say") is None


def test_sandbox_screens_and_contains_code():
    sb = POPSSToolSandbox(POPSSSandboxConfig(timeout=5.0, cpu_seconds=2, memory_limit_mb=256))
    ok = sb.run("import math\nprint(math.factorial(10))")
    assert ok.success and ok.stdout.strip() == "3628800" and ok.return_code == 0
    for code, frag in (("import os", "import of 'os'"), ("open('/etc/passwd')", "call of 'open'"), ("().__class__", "__class__"), ("def f(:", "syntax error"),
                       ("eval('1')", "call of 'eval'")):
        r = sb.run(code)
        assert not r.success and frag in r.error and r.return_code == -1
    assert sb.validate_code("console.log(1)", "javascript")[0] is False
    err = sb.run("print(1/0)")
    assert not err.success and "ZeroDivisionError" in err.error and err.return_code != 0
    slow = POPSSToolSandbox(POPSSSandboxConfig(timeout=0.5, cpu_seconds=5))
    t0 = time.perf_counter()
    r = slow.run("while True:\n    pass")
    assert not r.success and r.timed_out and time.perf_counter() - t0 < 4
    big = sb.run("x = bytearray(1 << 30)\nprint(len(x))")
    assert not big.success and "MemoryError" in (big.stderr + (big.error or ""))
    st = sb.get_stats()
    assert st["runs"] == 3 and st["rejected"] == 5 and st["failures"] == 2
    with pytest.raises(ValueError):
        POPSSSandboxConfig(timeout=0)


def test_monitor_checks_alerts_and_thresholds():
    readings = {"cpu_percent": 10.0, "memory_percent": 50.0, "disk_percent": 30.0}
    mon = POPSSMCPMonitor(POPSSMCPConfiguration(monitoring_interval=0), probes={k: (lambda k=k: readings[k]) for k in readings})
    seen = []
    mon.register_notification_handler("critical", seen.append)
    h = mon.run_health_check()
    assert h.status == "healthy" and h.alerts == [] and set(h.component_statuses) == {"cpu", "memory", "disk", "execution_latency", "queue"}
    readings["cpu_percent"], readings["memory_percent"] = 95.0, 75.0
    h = mon.run_health_check()
    assert h.status == "unhealthy" and h.component_statuses["cpu"] == "unhealthy" and h.component_statuses["memory"] == "degraded" and len(seen) == 1
    active = mon.get_active_alerts()
    assert {a["component"] for a in active} == {"cpu", "memory"} and len(mon.get_active_alerts("critical")) == 1
    mon.run_health_check()
    assert len(mon.get_active_alerts()) == 2                                              # the same conditions do not pile up alerts
    aid = active[0]["alert_id"]
    assert mon.acknowledge_alert(aid, "ops") and not mon.acknowledge_alert("nope") and mon.alerts[aid].acknowledged_by == "ops"
    readings["cpu_percent"], readings["memory_percent"] = 5.0, 5.0
    assert mon.run_health_check().status == "healthy" and mon.get_active_alerts() == [] and len(mon.get_alert_history()) == 2
    for _ in range(20):
        mon.record_execution_time(0.1)
    mon.record_execution_time(9.0)
    mon.record_execution_time(9.0)
    mon.set_threshold("latency_p95_s", 1.0)
    assert mon.run_health_check().component_statuses["execution_latency"] == "unhealthy"
    mon.record_queue_size(900)
    assert mon.get_component_health("execution_latency")["status"] == "unhealthy" and mon.run_health_check().component_statuses["queue"] == "unhealthy"
    mon.add_health_check("custom", lambda: (POPSSMCPHealthCheckStatus.DEGRADED, "meh"))
    mon.add_health_check("broken", lambda: 1 / 0)
    h = mon.run_health_check()
    assert h.component_statuses["custom"] == "degraded" and h.component_statuses["broken"] == "unknown" and mon.remove_health_check("broken")
    for _ in range(10):
        mon.record_execution_time(0.1, success=False)
    assert any("error rate" in a for a in mon.run_health_check().alerts)
    rep = mon.generate_report()
    assert rep["performance"]["total_executions"] == 32 and rep["performance"]["queue_max"] == 900 and rep["thresholds"]["latency_p95_s"] == 1.0
    with pytest.raises(KeyError):
        mon.set_threshold("nope", 1)
    with POPSSMCPMonitor(POPSSMCPConfiguration(monitoring_interval=0), probes={k: (lambda: 1.0) for k in readings}) as m2:
        time.sleep(0.1)
    assert m2.components and m2._thread is None


def test_remote_client_over_a_fake_server():
    tools = {"add": lambda a, b: a + b}
    down = [2]

    def transport(url, env, headers, timeout):
        assert url == "http://h:1/mcp" and headers["Authorization"] == "Bearer k" and env["sender_id"].startswith("client-")
        if down[0] > 0:
            down[0] -= 1
            raise OSError("refused")
        kind, p = env["message_type"], env["payload"]
        if kind == "tool_list":
            return {"tools": [{"name": n} for n in tools]}
        if kind == "tool_call":
            if p["tool_name"] not in tools:
                return {"success": False, "error": "unknown tool"}
            return {"success": True, "output": tools[p["tool_name"]](**p["arguments"])}
        if kind == "tool_register":
            return {"registered": True}
        return {"ok": True}

    slept = []
    c = POPSSMCPClient(POPSSMCPClientConfig(server_url="http://h:1/", api_key="k", max_retries=3), transport, slept.append)
    assert c.list_tools() == [{"name": "add"}] and slept == [0.5, 1.0] and c.connected and c.server.tools == ["add"]
    assert c.call_tool("add", {"a": 2, "b": 3}).output == 5 and c.call_tool("mul").error == "unknown tool"
    assert c.register_tool(YvMCPToolMetadata("x", "", {})) and c.heartbeat() and c.last_heartbeat > 0
    reg = YvCoreMCPToolRegistry()
    reg.register(YvMCPToolMetadata("remote_add", "", {}, "external", c.as_handler("add")))
    ex = YvMCPUnifiedToolExecutor(reg)
    assert ex.execute("remote_add", {"a": 1, "b": 1}).output == 2 and ex.execute("remote_add", {"a": 1, "b": 1}, "native_only").error.startswith("native-only")
    ex.shutdown()
    down[0] = 99
    r = c.call_tool("add", {"a": 1, "b": 1})
    assert not r.success and "unreachable" in r.error and not c.connected and not c.heartbeat() and c.get_stats()["server"]["status"] == "offline"
