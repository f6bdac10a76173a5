"""CPU tests of the agent runtime: tools, executor, state machine, memory, experience pool, ReAct engine."""
from __future__ import annotations

import pytest

from pisceslx_b200.models.agentic_tools import (YvAgenticState, YvCalculateTool, YvCodeExecTool, YvExperienceRecord,
                                                YvFileTool, YvHTTPTool, YvMemory, YvMemoryType, YvReActAction,
                                                YvReActActionType, YvReActEngine, YvReActPlan, YvReActPlanStep,
                                                YvReActRetryStrategy, YvSEERExperiencePool, YvSEERVerificationTool,
                                                YvSearchTool, YvStateMachine, YvToolExecutor)


def test_builtin_tools(tmp_path):
    calc = YvCalculateTool()
    assert calc(expression="2 * (3 + 4) ** 2 - sqrt(16)").output == 94.0
    assert abs(calc(expression="sin(pi / 2)").output - 1.0) < 1e-12
    for bad in ("__import__('os').system('true')", "open('x')", "a.b", "2 ** 100000", "(lambda: 1)()"):
        r = calc(expression=bad)
        assert not r.success and r.error
    code = YvCodeExecTool(timeout_s=5)
    assert code(code="print(sum(range(10)))").output.strip() == "45"
    assert not code(code="raise ValueError('boom')").success
    assert "TimeoutExpired" in YvCodeExecTool(timeout_s=0.5)(code="while True: pass").error
    ft = YvFileTool(str(tmp_path))
    assert ft(action="write", path="a/b.txt", content="hello").output == 5
    assert ft(action="read", path="a/b.txt").output == "hello" and ft(action="list", path="a").output == ["b.txt"]
    esc = ft(action="read", path="../../etc/passwd")
    assert not esc.success and "outside" in esc.error
    st = YvSearchTool([{"id": "d1", "text": "the capital of France is Paris"}, {"id": "d2", "text": "bananas are yellow"}])
    assert st(query="capital France").output[0]["id"] == "d1" and st(query="zebra").output == []
    http = YvHTTPTool()(url="http://example.com")
    assert not http.success and "offline" in http.error
    assert YvSEERVerificationTool()(expression="6*7", claimed=42).output is True


def test_executor_state_machine_memory_and_experience_pool():
    ex = YvToolExecutor([YvCalculateTool()])
    assert ex.execute("calculate", expression="1+1").output == 2 and not ex.execute("nope").success
    ex.execute("calculate", expression="1/0")
    assert ex.stats["calculate"] == {"calls": 2, "failures": 1}
    sm = YvStateMachine()
    sm.to(YvAgenticState.PLANNING)
    snap = sm.snapshot()
    sm.to(YvAgenticState.ACTING); sm.to(YvAgenticState.OBSERVING)
    with pytest.raises(ValueError):
        sm.to(YvAgenticState.PLANNING)                      # observing -> planning goes through reflecting
    assert len(sm.history) == 3 and sm.can(YvAgenticState.DONE)
    sm.restore(snap)
    assert sm.state == YvAgenticState.PLANNING and sm.step == 1
    now = [0.0]
    mem = YvMemory(working_size=2, capacity=3, half_life_s=10.0, clock=lambda: now[0])
    for i in range(4):
        mem.add(f"scratch {i}", YvMemoryType.WORKING)
    assert [e.content for e in mem.entries] == ["scratch 2", "scratch 3"]
    mem.add("an old remark about weather", YvMemoryType.EPISODIC, importance=0.3)
    now[0] = 100.0
    mem.add("user likes green tea", YvMemoryType.SEMANTIC, importance=0.9)
    mem.add("yesterday we fixed a parser bug", YvMemoryType.EPISODIC, importance=0.4)
    mem.add("deploy key lives in a vault", YvMemoryType.SEMANTIC, importance=0.8)
    long_term = [e.content for e in mem.entries if e.kind != YvMemoryType.WORKING]
    assert len(long_term) == 3 and "an old remark about weather" not in long_term   # old and unimportant: evicted
    hit = mem.retrieve("which tea does user like", k=1)
    assert hit and "tea" in hit[0].content and hit[0].uses == 1
    assert mem.retrieve("tea", kind=YvMemoryType.WORKING) == []
    pool = YvSEERExperiencePool(capacity=2)
    pool.add(YvExperienceRecord("sum two numbers", ["calculate"], True, 1.0))
    pool.add(YvExperienceRecord("fetch a page", ["http"], False))
    pool.add(YvExperienceRecord("multiply two numbers", ["calculate"], True, 0.8))
    assert len(pool.records) == 2 and pool.success_rate() == 1.0
    assert pool.similar("add two numbers", 1)[0].task in ("sum two numbers", "multiply two numbers")


def test_react_engine_recovers_from_a_failed_tool_call_and_can_give_up():
    ex = YvToolExecutor([YvCalculateTool(), YvHTTPTool()])
    script = iter([YvReActAction(YvReActActionType.TOOL, "http", {"url": "http://x"}),
                   YvReActAction(YvReActActionType.TOOL, "calculate", {"expression": "6*7"}),
                   YvReActAction(YvReActActionType.FINISH, text="42")])
    seen = []

    def policy(goal, obs, refl):
        seen.append((len(obs), [r.lesson for r in refl]))
        return next(script)
    out = YvReActEngine(ex, policy).run("what is six times seven")
    assert out["answer"] == "42" and out["state"] == "done" and len(out["reflections"]) == 1
    assert "network" in seen[1][1][0] and out["observations"][1].result.output == 42
    stubborn = YvReActEngine(ex, lambda g, o, r: YvReActAction(YvReActActionType.TOOL, "http", {"url": "http://x"}),
                             retry=YvReActRetryStrategy(max_retries=5, max_same=1))
    res = stubborn.run("fetch")
    assert res["state"] == "failed" and res["answer"] is None and len(res["reflections"]) == 2
    plan = YvReActPlan("goal", [YvReActPlanStep("a", done=True), YvReActPlanStep("b")])
    assert plan.next_step().description == "b" and plan.progress() == 0.5
    assert YvReActRetryStrategy(base_delay_s=0.5).delay(2) == 2.0
