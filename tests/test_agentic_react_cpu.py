"""The full ReAct agent: understanding, dependent plans, retries, persistence; the hashed text encoders."""
import json
import os

import pytest
import torch

from pisceslx_b200.models import agentic_react as ar
from pisceslx_b200.models.agentic_tools import YvCalculateTool, YvFileTool, YvSearchTool, YvToolExecutor

H = 32
GOAL_JSON = json.dumps({"intent": "report the capital of France in a file", "constraints": ["offline"],
                        "success_criteria": ["file exists"], "domain": "geography", "complexity": 2})
PLAN_JSON = json.dumps([
    {"description": "look the capital up", "action_type": "search", "params": {"query": "capital France"}},
    {"description": "write it down", "action_type": "write_file", "params": {"path": "out.txt", "content": "Paris"}, "depends_on": [0]},
    {"description": "read it back", "action_type": "read", "params": {"path": "out.txt"}, "depends_on": [1]},
    {"description": "say it", "action_type": "answer", "params": {"content": "The capital is Paris."}, "depends_on": [2]},
])


def _generate(prompt: str) -> str:
    if "Analyse the request" in prompt:
        return "Sure. " + GOAL_JSON + " done"
    if "Break the goal" in prompt:
        return "Plan:\n" + PLAN_JSON
    return "I will do the step."


def _tools(tmp_path):
    return YvToolExecutor([YvSearchTool([{"id": "fr", "text": "The capital of France is Paris."}]),
                           YvFileTool(str(tmp_path)), YvCalculateTool()])


def test_goal_understanding_parses_and_falls_back():
    g = ar.YvGoalUnderstanding(H)
    goal = g.understand("tell me the capital", _generate)
    assert goal.intent.startswith("report the capital") and goal.constraints == ["offline"] and goal.complexity == 2
    bad = g.understand("tell me the capital", lambda p: "no json here")
    assert bad.intent == "tell me the capital" and bad.domain == "general"
    out = g(torch.randn(3, 7, H))
    assert tuple(out["intent_class"].shape) == (3,) and tuple(out["intent_logits"].shape) == (3, 10)
    assert tuple(out["domain_logits"].shape) == (3, 8) and bool(((out["complexity_score"] > 0) & (out["complexity_score"] < 1)).all())


def test_decomposition_builds_dependent_steps_and_orders_them():
    d = ar.YvTaskDecomposition(H)
    plan = d.decompose(ar.YvReActGoal("x", "report"), _generate)
    assert [s.action_type.value for s in plan.steps] == ["search", "write_file", "read_file", "answer"]
    assert plan.steps[2].depends_on == [1] and plan.status == "ready"
    assert plan.get_next_step().step_id == 0
    plan.update_step(0, "failed")
    assert plan.get_next_step() is None and plan.blocked()
    fallback = d.decompose(ar.YvReActGoal("x", "report"), lambda p: "[]")
    assert len(fallback.steps) == 1 and fallback.steps[0].action_type == ar.YvReActStepType.ANSWER
    dep = d.dependencies(torch.randn(4, H), torch.randn(H))
    assert tuple(dep.shape) == (4, 4) and float(dep.triu().abs().sum()) == 0
    m = torch.zeros(3, 3)
    m[0, 2] = 0.0
    m[1, 0] = 0.9
    m[2, 1] = 0.9
    assert d.order(m) == [0, 1, 2]
    m2 = torch.zeros(3, 3)
    m2[1, 2] = 0.9                                       # 1 needs 2: 2 must come first
    assert d.order(m2) == [0, 2, 1]
    rt = ar.YvReActTaskPlan.from_dict(json.loads(json.dumps(plan.to_dict())))
    assert rt.steps[1].action_type == ar.YvReActStepType.WRITE_FILE and rt.goal.intent == "report"


def test_error_analysis_strategies_and_learning():
    sc = ar.YvReActSelfCorrection(H)
    K = ar.YvReActRetryKind
    assert sc.analyze_error("Connection refused")["error_type"] == "network_error"
    assert sc.analyze_error("file not found")["should_retry"] and sc.analyze_error("invalid argument")["should_alternate"]
    assert [sc.determine_retry_strategy("request timeout", n) for n in (0, 1, 3, 5)] == [K.IMMEDIATE, K.BACKOFF, K.ALTERNATE, K.ESCALATE]
    assert sc.determine_retry_strategy("permission denied", 0) == K.ESCALATE
    assert [sc.determine_retry_strategy("invalid value", n) for n in (0, 2)] == [K.ALTERNATE, K.SKIP]
    assert sc.determine_retry_strategy("strange", 2, {"has_checkpoint": True}) == K.CHECKPOINT_RESTORE
    assert 0.8 <= sc.calculate_backoff_time(0) <= 1.2 and sc.calculate_backoff_time(20) == 60.0
    alts = sc.generate_alternate_actions({"type": "tool_call", "tool": "fetch", "params": {"u": 1}}, {"error_type": "timeout"})
    assert alts[0]["params"]["timeout"] == 60 and alts[1]["tool"] == "fetch_fallback" and alts[-1]["type"] == "ask_human"
    assert sc.generate_correction(sc.analyze_error("weird"))["strategy"] == "skip"
    for ok in (False, False, True):
        sc.learn_from_error("request timeout", "backoff", ok, ar.YvReActStepType.SEARCH)
    sc.learn_from_error("request timeout", "immediate", False, ar.YvReActStepType.SEARCH)
    st = sc.get_retry_statistics()
    assert st["total_retry_attempts"] == 4 and st["successful_retries"] == 1 and st["most_common_errors"] == ["timeout"]
    assert sc.best_resolution("timeout again") == "backoff" and sc.get_error_pattern_prediction(ar.YvReActStepType.SEARCH) == 1.0
    assert sc.should_escalate(5, "timeout") and sc.should_escalate(0, "data_corruption") and not sc.should_escalate(1, "timeout")
    out = sc.propose(torch.randn(2, H), torch.randn(2, H))
    assert tuple(out["error_logits"].shape) == (2, 7) and tuple(out["corrected_state"].shape) == (2, H)


def test_agent_runs_a_dependent_plan_with_real_tools(tmp_path):
    agent = ar.YvReActFactory.create_lightweight(H, max_steps=10)
    out = agent.run("What is the capital of France? Save it.", _generate, _tools(tmp_path))
    assert out["success"] and out["state"] == "completed" and out["steps_completed"] == 4
    assert out["answer"] == "The capital is Paris." and (tmp_path / "out.txt").read_text() == "Paris"
    assert [h["action"] for h in out["history"]] == ["search", "write_file", "read_file", "answer"]
    assert agent.get_execution_progress()["progress"] == 1.0
    pol = agent.policy(torch.randn(2, H), torch.randn(2, H), torch.randn(2, H))
    assert tuple(pol["action_logits"].shape) == (2, len(ar.YvReActStepType)) and tuple(pol["confidence"].shape) == (2,)


def test_agent_retries_a_flaky_tool_and_reports_a_failed_dependency(tmp_path):
    calls = {"n": 0}

    def flaky(query):
        calls["n"] += 1
        if calls["n"] < 3:
            raise ConnectionError("network down")
        return "Paris"

    slept = []
    agent = ar.YvReActAgentic(H, max_steps=10, sleep=slept.append)
    out = agent.run("q", _generate, {"search": flaky, "write_file": lambda path, content: "ok",
                                     "read_file": lambda path: "Paris"})
    assert out["success"] and calls["n"] == 3 and len(slept) == 1      # immediate, then one back-off, then success
    assert out["retry_statistics"]["total_retry_attempts"] >= 3

    def denied(query):
        raise PermissionError("permission denied")

    agent2 = ar.YvReActAgentic(H, max_steps=10)
    out2 = agent2.run("q", _generate, {"search": denied})
    assert not out2["success"] and out2["state"] == "failed" and out2["steps_failed"] == 1 and out2["blocked"]
    assert out2["steps_completed"] == 0 and "[escalate]" in out2["history"][0]["observation"]


def test_persistence_interrupt_and_resume(tmp_path):
    ck = tmp_path / "ck"
    agent = ar.YvReActAgentic(H, max_steps=10, checkpoint_dir=str(ck))
    tools = _tools(tmp_path)
    state = {"n": 0}

    def gen(prompt):
        if "Think briefly" in prompt:
            state["n"] += 1
            if state["n"] == 2:
                agent.handle_interruption("SIGTERM")          # arrives while step 1 is running
        return _generate(prompt)

    out = agent.run("q", gen, tools)
    assert out["state"] == "waiting" and out["steps_completed"] == 2 and not out["success"]
    ids = [c["checkpoint_id"] for c in agent.list_checkpoints()]
    assert ids and all(os.path.exists(ck / (i + ".json")) for i in ids)
    cid = agent.save_execution_state()
    fresh = ar.YvReActAgentic(H, max_steps=10, checkpoint_dir=str(ck))       # another process: files only
    done = fresh.resume_from_checkpoint(cid, _generate, tools)
    assert done["success"] and done["steps_completed"] == 4 and done["answer"] == "The capital is Paris."
    assert fresh.restore_execution_state(cid) and not fresh.restore_execution_state("nope")
    with pytest.raises(KeyError):
        fresh.resume_from_checkpoint("nope", _generate, tools)
    fresh.clear_checkpoints()
    assert fresh.list_checkpoints() == []


def test_recovery_gives_failed_steps_another_chance(tmp_path):
    state = {"fail": True}

    def search(query):
        if state["fail"]:
            raise PermissionError("permission denied")
        return "Paris"

    agent = ar.YvReActAgentic(H, max_steps=10)
    orig = agent.run

    def run_and_heal(*a, **kw):
        out = orig(*a, **kw)
        state["fail"] = False                                   # the operator fixes the permission between attempts
        return out

    agent.run = run_and_heal
    out = agent.execute_with_recovery("q", _generate, {"search": search, "write_file": lambda path, content: "ok",
                                                       "read_file": lambda path: "Paris"})
    assert out["success"] and out["recoveries"] == 1 and out["steps_completed"] == 4


def test_reasoning_tool_is_an_ordinary_tool():
    ex = YvToolExecutor([ar.YvSEERReasoningTool(lambda p: "42" if "Question: life" in p and "Context" in p else "?")])
    r = ex.execute("reasoning", question="life", context="hitchhiker")
    assert r.success and r.output == "42"


def test_semantic_encoder_is_stable_batched_and_marks_roles():
    torch.manual_seed(0)
    e = ar.YvSemanticEncoder(hidden_size=H, vocab_size=1000, embedding_dim=16, max_seq_len=32).eval()
    ids = e.tokenize("<|goal|> find the Capital <|action|> search")
    assert ids[0] == 1 and ids[4] == 3 and len(ids) == 6 and all(i >= 5 for i in ids[1:4])
    assert ids[3] == e.tokenize("capital")[0]                  # lower-cased, same id everywhere
    assert ar._stable_hash("capital") == 0x1B6F5A5E or isinstance(ar._stable_hash("capital"), int)
    with torch.no_grad():
        one = e("find the capital")
        two = e(["find the capital", "a much longer request about something else entirely"])
    assert tuple(one["pooled"].shape) == (1, H) and tuple(two["pooled"].shape) == (2, H)
    assert torch.allclose(one["pooled"][0], two["pooled"][0], atol=1e-5)      # padding does not change a sample
    assert tuple(two["context"].shape)[:2] == tuple(two["tokens"].shape)
    with torch.no_grad():
        h = e.encode_with_history("now", [{"thought": "t", "action": "a", "observation": "o"}])
    assert h["tokens"][0, 0] == 1 and tuple(e.encode_goal("g").shape) == (1, H) and tuple(e.encode_context({"a": 1}).shape) == (1, H)


def test_hybrid_encoder_fuses_additional_features():
    torch.manual_seed(0)
    e = ar.YvHybridEncoder(hidden_size=H, vocab_size=1000, embedding_dim=16).eval()
    with torch.no_grad():
        a = e("hello world")
        b = e("hello world", torch.randn(H))
        c = e(["hello world", "other"], torch.randn(2, 3 * H))
    assert tuple(a["pooled"].shape) == (1, H) and not torch.allclose(a["pooled"], b["pooled"]) and tuple(c["pooled"].shape) == (2, H)
