"""Validation and concurrency operators."""
import asyncio
import random

import pytest

from pisceslx_b200.utils import ops_kit as K
from pisceslx_b200.utils.core import PiscesLxCoreError, PiscesLxCoreValidationError


def test_validator_checks_raise_with_context():
    V = K.PiscesLxValidator
    V.require(True, "fine")
    V.expect_type(3, int, "n")
    V.expect_type("a", (str, bytes), "s")
    V.expect_in("b", ["a", "b"], "mode")
    V.expect_range(0.5, 0, 1, "p")
    V.expect_non_empty([1], "items")
    V.expect_length("abc", 1, 3, "code")
    V.expect_match("run-01", r"[a-z]+-\d+", "id")
    for bad in (lambda: V.require(False, "no", why=1), lambda: V.expect_type(True, int, "n"), lambda: V.expect_type(1.5, int, "n"),
                lambda: V.expect_in("c", ["a"], "mode"), lambda: V.expect_range(float("nan"), 0, 1, "p"),
                lambda: V.expect_range(2, 0, 1, "p"), lambda: V.expect_non_empty("  ", "s"), lambda: V.expect_non_empty(None, "s"),
                lambda: V.expect_length([1, 2], 3, 5, "l"), lambda: V.expect_match("Run", r"[a-z]+", "id")):
        with pytest.raises(PiscesLxCoreValidationError):
            bad()
    try:
        V.require(False, "no", why=1)
    except PiscesLxCoreValidationError as e:
        assert e.context.details == {"why": 1} and e.code.id == "P-006"


def test_validator_operator_schema_custom_and_batch():
    op = K.PiscesLxValidatorOperator()
    schema = {"lr": {"type": "float", "required": True, "min": 0, "max": 1}, "mode": {"type": "str", "enum": ["sft", "dpo"]},
              "name": {"type": "str", "pattern": r"[a-z_]+"}, "steps": {"type": "int", "min": 1}}
    ok = op.execute({"check": "schema", "data": {"lr": 0.1, "mode": "sft", "name": "run_a", "extra": 1}, "schema": schema}).output
    assert ok["valid"] and ok["warnings"] == ["unknown fields: ['extra']"]
    bad = op.execute({"check": "schema", "data": {"mode": "ppo", "name": "Run", "steps": True}, "schema": schema}).output
    assert not bad["valid"] and len(bad["errors"]) == 4 and bad["errors"][0] == "lr is required"
    assert not op.execute({"check": "schema", "data": [], "schema": schema}).output["valid"]
    op.add_rule("even", lambda v: (v % 2 == 0, "must be even"))
    assert op.execute({"check": "custom", "rule": "even", "value": 4}).output["valid"]
    assert op.execute({"check": "custom", "rule": "even", "value": 3}).output["errors"] == ["must be even"]
    assert not op.execute({"check": "custom", "rule": "odd", "value": 3}).output["valid"]
    b = op.execute({"check": "batch", "checks": [{"check": "type", "value": 1, "expected": "int"},
                                                 {"check": "range", "value": 5, "min": 0, "max": 1, "name": "p"},
                                                 {"check": "in", "value": "x", "options": ["y"]}, {"check": "length", "value": "ab", "min": 1, "max": 2},
                                                 {"check": "pattern", "value": "ab", "pattern": r"\d+"}, {"check": "nope"}]}).output
    assert not b["valid"] and [e[:3] for e in b["errors"]] == ["[1]", "[2]", "[4]", "[5]"]
    assert not op.execute({"check": "unknown"}).is_success()


def test_timeout_operator():
    t = [0.0]
    clock = lambda: t[0]
    with K.PiscesLxTimeoutOperator(1.0, clock=clock) as g:
        t[0] += 0.5
    assert not g.timed_out and g.elapsed == 0.5
    with pytest.raises(K.PiscesLxTimeoutError):
        with K.PiscesLxTimeoutOperator(1.0, clock=clock):
            t[0] += 2.0
    soft = K.PiscesLxTimeoutOperator(1.0, raise_on_timeout=False, clock=clock)
    with soft:
        t[0] += 2.0
    assert soft.timed_out
    with pytest.raises(ValueError):                              # the body's own error wins
        with K.PiscesLxTimeoutOperator(1.0, clock=clock):
            t[0] += 5
            raise ValueError("x")
    assert K.PiscesLxTimeoutOperator(1.0).call(lambda a, b=1: a + b, 2, b=3) == 5
    import threading
    ev = threading.Event()
    with pytest.raises(K.PiscesLxTimeoutError):
        K.PiscesLxTimeoutOperator(0.05).call(ev.wait, 5.0)
    ev.set()
    with pytest.raises(KeyError):
        K.PiscesLxTimeoutOperator(1.0).call(lambda: {}["k"])


def test_retry_backoff_and_circuit_breaker():
    slept, now = [], [0.0]
    cfg = K.PiscesLxRetryConfig(max_attempts=4, base_delay=0.1, jitter=False, circuit_breaker_threshold=5, circuit_breaker_timeout=10.0)
    r = K.PiscesLxRetryOperator(cfg, sleep=slept.append, clock=lambda: now[0])
    calls = {"n": 0}

    def flaky():
        calls["n"] += 1
        if calls["n"] < 3:
            raise IOError("again")
        return "ok"
    assert r.execute(flaky) == "ok" and slept == [0.1, 0.2] and r.attempts_made == 3 and not r.circuit_open

    def dead():
        raise IOError("down")
    with pytest.raises(K.PiscesLxConcurrencyError) as ei:
        r.execute(dead)
    assert isinstance(ei.value.__cause__, IOError) and slept[2:] == [0.1, 0.2, 0.4]
    with pytest.raises(K.PiscesLxConcurrencyError):
        r.execute(dead)                                          # the fifth consecutive failure opens the breaker
    assert r.circuit_open
    n = r.attempts_made
    with pytest.raises(K.PiscesLxConcurrencyError, match="circuit breaker"):
        r.execute(lambda: "never called")
    assert r.attempts_made == n
    now[0] += 11.0                                               # half-open: one trial goes through and closes it
    assert r.execute(lambda: "back") == "back" and not r.circuit_open
    j = K.PiscesLxRetryOperator(K.PiscesLxRetryConfig(base_delay=1.0, jitter=True), rng=random.Random(1))
    assert all(0.5 <= j.delay_for(0) <= 1.0 for _ in range(20)) and K.PiscesLxRetryOperator(K.PiscesLxRetryConfig(max_delay=3.0, jitter=False)).delay_for(20) == 3.0
    only = K.PiscesLxRetryOperator(K.PiscesLxRetryConfig(exceptions=(KeyError,)), sleep=lambda s: None)
    with pytest.raises(ValueError):
        only.execute(lambda: (_ for _ in ()).throw(ValueError("not retried")))


def _square(x):
    return x * x


def test_parallel_map_keeps_order_and_reports_the_failing_item():
    import time
    p = K.PiscesLxParallelOperator(max_workers=4)
    assert p.map(lambda x: (time.sleep(0.01 * (5 - x)), x * 2)[1], range(5)) == [0, 2, 4, 6, 8] and p.map(_square, []) == []
    with pytest.raises(K.PiscesLxConcurrencyError, match="item 2 failed"):
        p.map(lambda x: 1 // (x - 2), range(4))
    mp = K.PiscesLxParallelOperator(K.PiscesLxConcurrencyBackend.MULTIPROCESSING, max_workers=2, chunk_size=2)
    assert mp.map(_square, [1, 2, 3, 4, 5]) == [1, 4, 9, 16, 25]
    with pytest.raises(K.PiscesLxConcurrencyError):
        K.PiscesLxParallelOperator(K.PiscesLxConcurrencyBackend.ASYNCIO).map(_square, [1])


def test_async_runner_bounds_and_priorities():
    async def main():
        r = K.PiscesLxAsyncOperator(max_concurrent=1, max_queue_size=3)
        order = []
        gate = asyncio.Event()

        def job(tag, wait=False):
            async def run():
                if wait:
                    await gate.wait()
                order.append(tag)
                return tag
            return run

        first = asyncio.ensure_future(r.submit(job("first", wait=True)))
        await asyncio.sleep(0)
        low = asyncio.ensure_future(r.submit(job("low"), K.PiscesLxTaskPriority.LOW))
        normal = asyncio.ensure_future(r.submit(job("normal")))
        crit = asyncio.ensure_future(r.submit(job("critical"), K.PiscesLxTaskPriority.CRITICAL))
        await asyncio.sleep(0)
        assert r.active_count == 1 and r.waiting_count == 3
        with pytest.raises(K.PiscesLxConcurrencyError, match="queue full"):
            await r.submit(job("overflow"))
        gate.set()
        assert await asyncio.gather(first, low, normal, crit) == ["first", "low", "normal", "critical"]
        assert order == ["first", "critical", "normal", "low"]
        await r.shutdown()
        with pytest.raises(K.PiscesLxConcurrencyError):
            await r.submit(job("late"))
    asyncio.run(main())


def test_concurrency_operator_front():
    op = K.PiscesLxConcurrencyOperator()
    assert op.execute({"operation": "timeout", "func": lambda: 7, "seconds": 1}).output == {"result": 7}
    n = {"c": 0}

    def twice():
        n["c"] += 1
        if n["c"] < 2:
            raise RuntimeError("once")
        return "done"
    r = op.execute({"operation": "retry", "func": twice, "sleep": lambda s: None, "base_delay": 0.0})
    assert r.output == {"result": "done", "attempts": 2}
    assert op.execute({"operation": "parallel", "func": _square, "items": [1, 2, 3]}).output == {"results": [1, 4, 9]}

    async def a():
        return "a"

    async def b():
        await asyncio.sleep(0.01)
        return "b"
    assert op.execute({"operation": "async", "coros": [a, b]}).output == {"results": ["a", "b"]}
    bad = op.execute({"operation": "retry", "func": lambda: 1 / 0, "sleep": lambda s: None, "max_attempts": 2})
    assert not bad.is_success() and "exhausted" in bad.error and not op.execute({"operation": "dance"}).is_success()
