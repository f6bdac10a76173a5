"""Validation and concurrency operators (reference opss/validation/__init__.py:53-492,
opss/concurrency/__init__.py:62-502).

Validation: a static checker (``PiscesLxValidator.require / expect_type / expect_in / expect_range / ...``) that raises
``PiscesLxCoreValidationError`` with the offending value in its context, named reusable rules, and an operator that runs
one check, a schema over a dictionary, or a batch of checks and reports every failure instead of the first.

Concurrency: a deadline context manager, a retry helper with exponential back-off, seeded jitter and a circuit
breaker, an order-preserving parallel map over threads or processes, a bounded async task runner with priorities, and
the operator front.  The clock, the sleep function and the random source are injectable, so the tests do not wait.

The deadline works in any thread: it runs the protected call in a worker and abandons it at the deadline
(``call``), or - as a context manager - records the overrun and raises on exit.  The reference arms ``signal.alarm``
in the main thread without installing a handler (concurrency/__init__.py:141-143), which terminates the process when
the alarm fires."""
from __future__ import annotations

import asyncio
import concurrent.futures as cf
import heapq
import random
import re
import threading
import time
from dataclasses import dataclass, field
from enum import Enum, IntEnum
from typing import Any, Awaitable, Callable, Dict, Iterable, List, Optional, Sequence, Set, Tuple, Type, Union

from .core import (PiscesLxCoreConcurrencyError, PiscesLxCoreError, PiscesLxCoreErrorCode, PiscesLxCoreErrorContext,
                   PiscesLxCoreTimeoutError, PiscesLxCoreValidationError)
from .opsc import PiscesLxOperatorInterface

PiscesLxTimeoutError = PiscesLxCoreTimeoutError
PiscesLxConcurrencyError = PiscesLxCoreConcurrencyError


# ---------------------------------------------------------------------------------------------------------------- validation
@dataclass
class PiscesLxValidationRule:
    name: str
    validate: Callable[[Any], Tuple[bool, str]]
    description: str = ""


@dataclass
class PiscesLxValidationResult:
    valid: bool
    errors: List[str] = field(default_factory=list)
    warnings: List[str] = field(default_factory=list)

    def __bool__(self) -> bool:
        return self.valid

    def merge(self, other: "PiscesLxValidationResult") -> "PiscesLxValidationResult":
        return PiscesLxValidationResult(self.valid and other.valid, self.errors + other.errors, self.warnings + other.warnings)


def _fail(message: str, **ctx: Any) -> None:
    raise PiscesLxCoreValidationError(message, PiscesLxCoreErrorContext("validator", "check", details=ctx))


class PiscesLxValidator:
    """Checks that raise on failure.  ``name`` is how the value is called in the message."""

    @staticmethod
    def require(condition: bool, message: str, **ctx: Any) -> None:
        if not condition:
            _fail(message, **ctx)

    @staticmethod
    def expect_type(obj: Any, types: Union[Type, Tuple[Type, ...]], name: str) -> None:
        wanted = types if isinstance(types, tuple) else (types,)
        if isinstance(obj, bool) and bool not in wanted and object not in wanted:
            _fail(f"{name} must be {getattr(types, '__name__', types)}, got bool", value=obj)      # True is not a count
        if not isinstance(obj, types):
            _fail(f"{name} must be {getattr(types, '__name__', types)}, got {type(obj).__name__}", value=repr(obj)[:80])

    @staticmethod
    def expect_in(value: Any, options: Iterable[Any], name: str) -> None:
        opts = list(options)
        if value not in opts:
            _fail(f"{name} must be one of {opts}, got {value!r}", value=value)

    @staticmethod
    def expect_range(value: float, min_val: float, max_val: float, name: str) -> None:
        if not isinstance(value, (int, float)) or isinstance(value, bool) or value != value or not (min_val <= value <= max_val):
            _fail(f"{name} must be in [{min_val}, {max_val}], got {value!r}", value=value)

    @staticmethod
    def expect_non_empty(value: Any, name: str) -> None:
        if value is None or (hasattr(value, "__len__") and len(value) == 0) or (isinstance(value, str) and not value.strip()):
            _fail(f"{name} must not be empty")

    @staticmethod
    def expect_length(value: Any, min_len: int, max_len: int, name: str) -> None:
        if not hasattr(value, "__len__") or not (min_len <= len(value) <= max_len):
            _fail(f"{name} must have between {min_len} and {max_len} items, got {len(value) if hasattr(value, '__len__') else 'no length'}")

    @staticmethod
    def expect_match(value: str, pattern: str, name: str) -> None:
        if not isinstance(value, str) or re.fullmatch(pattern, value) is None:
            _fail(f"{name} must match {pattern!r}, got {value!r}", value=value)


_TYPES = {"str": str, "int": int, "float": (int, float), "bool": bool, "list": list, "dict": dict, "any": object}


class PiscesLxValidatorOperator(PiscesLxOperatorInterface):
    """inputs["check"] selects: ``type`` (value, expected), ``range`` (value, min, max), ``in`` (value, options),
    ``length`` (value, min, max), ``pattern`` (value, pattern), ``schema`` (data, schema: field -> {type, required, enum,
    min, max, pattern}), ``custom`` (value, rule: a registered rule's name), ``batch`` (checks: a list of such inputs).
    The output is {"valid", "errors", "warnings"}; the operator itself fails only on a malformed request."""

    name = "validator"

    def __init__(self) -> None:
        self._rules: Dict[str, PiscesLxValidationRule] = {}

    def add_rule(self, name: str, validate: Callable[[Any], Tuple[bool, str]], description: str = "") -> None:
        self._rules[name] = PiscesLxValidationRule(name, validate, description)

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return inputs.get("check") in ("type", "range", "in", "length", "pattern", "schema", "custom", "batch")

    @staticmethod
    def _guard(fn: Callable[[], None]) -> PiscesLxValidationResult:
        try:
            fn()
            return PiscesLxValidationResult(True)
        except PiscesLxCoreError as e:
            return PiscesLxValidationResult(False, [e.message])

    def _schema(self, data: Any, schema: Dict[str, Dict[str, Any]]) -> PiscesLxValidationResult:
        if not isinstance(data, dict):
            return PiscesLxValidationResult(False, ["data must be a dictionary"])
        V, res = PiscesLxValidator, PiscesLxValidationResult(True)
        for key, spec in schema.items():
            if key not in data or data[key] is None:
                if spec.get("required", False):
                    res = res.merge(PiscesLxValidationResult(False, [f"{key} is required"]))
                continue
            v = data[key]
            checks: List[Callable[[], None]] = []
            if "type" in spec:
                checks.append(lambda v=v, s=spec, k=key: V.expect_type(v, _TYPES.get(s["type"], object), k))
            if "enum" in spec:
                checks.append(lambda v=v, s=spec, k=key: V.expect_in(v, s["enum"], k))
            if "min" in spec or "max" in spec:
                checks.append(lambda v=v, s=spec, k=key: V.expect_range(v, s.get("min", float("-inf")), s.get("max", float("inf")), k))
            if "pattern" in spec:
                checks.append(lambda v=v, s=spec, k=key: V.expect_match(v, s["pattern"], k))
            for c in checks:
                r = self._guard(c)
                res = res.merge(r)
                if not r:
                    break
        unknown = sorted(set(data) - set(schema))
        if unknown:
            res.warnings.append(f"unknown fields: {unknown}")
        return res

    def check(self, inputs: Dict[str, Any]) -> PiscesLxValidationResult:
        V, kind, name = PiscesLxValidator, inputs["check"], inputs.get("name", "value")
        if kind == "type":
            exp = inputs["expected"]
            return self._guard(lambda: V.expect_type(inputs["value"], _TYPES.get(exp, exp) if isinstance(exp, str) else exp, name))
        if kind == "range":
            return self._guard(lambda: V.expect_range(inputs["value"], inputs.get("min", float("-inf")), inputs.get("max", float("inf")), name))
        if kind == "in":
            return self._guard(lambda: V.expect_in(inputs["value"], inputs["options"], name))
        if kind == "length":
            return self._guard(lambda: V.expect_length(inputs["value"], inputs.get("min", 0), inputs.get("max", 1 << 62), name))
        if kind == "pattern":
            return self._guard(lambda: V.expect_match(inputs["value"], inputs["pattern"], name))
        if kind == "schema":
            return self._schema(inputs["data"], inputs["schema"])
        if kind == "custom":
            rule = self._rules.get(inputs["rule"])
            if rule is None:
                return PiscesLxValidationResult(False, [f"unknown rule {inputs['rule']!r}"])
            ok, msg = rule.validate(inputs["value"])
            return PiscesLxValidationResult(bool(ok), [] if ok else [msg or f"rule {rule.name} failed"])
        res = PiscesLxValidationResult(True)
        for i, sub in enumerate(inputs["checks"]):
            r = self.check(sub) if self.validate_inputs(sub) else PiscesLxValidationResult(False, ["malformed check"])
            res = res.merge(PiscesLxValidationResult(r.valid, [f"[{i}] {e}" for e in r.errors], r.warnings))
        return res

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        r = self.check(inputs)
        return {"valid": r.valid, "errors": r.errors, "warnings": r.warnings}


# ---------------------------------------------------------------------------------------------------------------- concurrency
class PiscesLxTaskPriority(IntEnum):
    CRITICAL = 0
    HIGH = 1
    NORMAL = 2
    LOW = 3
    BACKGROUND = 4


class PiscesLxConcurrencyBackend(str, Enum):
    THREADING = "threading"
    MULTIPROCESSING = "multiprocessing"
    ASYNCIO = "asyncio"


@dataclass
class PiscesLxConcurrencyConfig:
    max_workers: int = 4
    max_memory_mb: Optional[int] = None
    timeout_seconds: float = 300.0
    retry_attempts: int = 3
    retry_delay: float = 1.0
    backend: PiscesLxConcurrencyBackend = PiscesLxConcurrencyBackend.THREADING
    enable_profiling: bool = False


@dataclass
class PiscesLxRetryConfig:
    max_attempts: int = 3
    base_delay: float = 0.2
    max_delay: float = 60.0
    exponential_base: float = 2.0
    jitter: bool = True
    exceptions: Tuple[Type[BaseException], ...] = (Exception,)
    circuit_breaker_threshold: int = 5
    circuit_breaker_timeout: float = 300.0


class PiscesLxTimeoutOperator:
    """``with PiscesLxTimeoutOperator(2.0): ...`` raises ``PiscesLxTimeoutError`` on exit when the body took longer
    (the body is not interrupted); ``PiscesLxTimeoutOperator(2.0).call(fn, *args)`` runs ``fn`` in a worker thread and
    raises at the deadline, leaving the worker to finish in the background."""

    def __init__(self, seconds: float, raise_on_timeout: bool = True, clock: Callable[[], float] = time.perf_counter) -> None:
        self.seconds, self.raise_on_timeout, self._clock = float(seconds), raise_on_timeout, clock
        self._start: Optional[float] = None
        self._timeout_occurred = False
        self.elapsed = 0.0

    def __enter__(self) -> "PiscesLxTimeoutOperator":
        self._start, self._timeout_occurred = self._clock(), False
        return self

    def __exit__(self, exc_type, exc, tb) -> bool:
        self.elapsed = self._clock() - (self._start or 0.0)
        self._timeout_occurred = self.elapsed > self.seconds
        if self._timeout_occurred and self.raise_on_timeout and exc_type is None:
            raise PiscesLxTimeoutError(f"operation took {self.elapsed:.3f}s, limit {self.seconds}s",
                                       PiscesLxCoreErrorContext("timeout", "exit", details={"seconds": self.seconds}))
        return False

    @property
    def timed_out(self) -> bool:
        return self._timeout_occurred

    def call(self, fn: Callable[..., Any], *args: Any, **kwargs: Any) -> Any:
        box: Dict[str, Any] = {}

        def work() -> None:
            try:
                box["value"] = fn(*args, **kwargs)
            except BaseException as e:                      # delivered to the caller below
                box["error"] = e

        t = threading.Thread(target=work, daemon=True, name="pisceslx-timeout")
        t.start()
        t.join(self.seconds)
        if t.is_alive():
            self._timeout_occurred = True
            if self.raise_on_timeout:
                raise PiscesLxTimeoutError(f"operation exceeded {self.seconds}s",
                                           PiscesLxCoreErrorContext("timeout", "call", details={"seconds": self.seconds}))
            return None
        if "error" in box:
            raise box["error"]
        return box.get("value")


class PiscesLxRetryOperator:
    """execute(func): up to ``max_attempts`` calls, sleeping base x exponential_base^attempt (capped, with jitter in
    [0.5, 1.0] of the delay) between them.  Consecutive failures across calls open a circuit breaker after
    ``circuit_breaker_threshold``; while open, ``execute`` fails at once; after ``circuit_breaker_timeout`` one trial
    call is let through (half-open) and a success closes the breaker."""

    def __init__(self, config: Optional[PiscesLxRetryConfig] = None, sleep: Callable[[float], None] = time.sleep,
                 clock: Callable[[], float] = time.monotonic, rng: Optional[random.Random] = None):
        self.config = config or PiscesLxRetryConfig()
        self._sleep, self._clock, self._rng = sleep, clock, rng or random.Random(0)
        self._failure_count = 0
        self._circuit_open = False
        self._last_failure_time = 0.0
        self.attempts_made = 0

    def _is_circuit_open(self) -> bool:
        if not self._circuit_open:
            return False
        if self._clock() - self._last_failure_time > self.config.circuit_breaker_timeout:
            return False                                    # half-open: let one call try
        return True

    def _record_failure(self) -> None:
        self._failure_count += 1
        self._last_failure_time = self._clock()
        if self._failure_count >= self.config.circuit_breaker_threshold:
            self._circuit_open = True

    def delay_for(self, attempt: int) -> float:
        c = self.config
        d = min(c.base_delay * (c.exponential_base ** attempt), c.max_delay)
        return d * (0.5 + 0.5 * self._rng.random()) if c.jitter else d

    def execute(self, func: Callable[[], Any]) -> Any:
        c = self.config
        if self._is_circuit_open():
            raise PiscesLxConcurrencyError("circuit breaker is open", PiscesLxCoreErrorContext("retry", "execute", details={"failures": self._failure_count}))
        last: Optional[BaseException] = None
        for attempt in range(c.max_attempts):
            self.attempts_made += 1
            try:
                out = func()
                self._failure_count, self._circuit_open = 0, False
                return out
            except c.exceptions as e:
                last = e
                self._record_failure()
                if self._circuit_open or attempt == c.max_attempts - 1:
                    break
                self._sleep(self.delay_for(attempt))
        err = PiscesLxConcurrencyError(f"retry attempts exhausted: {type(last).__name__}: {last}",
                                       PiscesLxCoreErrorContext("retry", "execute", details={"attempts": c.max_attempts}))
        err.__cause__ = last
        raise err

    @property
    def circuit_open(self) -> bool:
        return self._is_circuit_open()


class PiscesLxParallelOperator:
    """map(func, items) with the results in the order of the items.  Threads by default; with the multiprocessing
    backend ``func`` and the items must pickle and the items are sent in chunks of ``chunk_size``.  A failing item
    raises ``PiscesLxConcurrencyError`` carrying the item's index."""

    def __init__(self, backend: PiscesLxConcurrencyBackend = PiscesLxConcurrencyBackend.THREADING,
                 max_workers: Optional[int] = None, chunk_size: int = 1, timeout: Optional[float] = None):
        self.backend, self.max_workers, self.chunk_size, self.timeout = PiscesLxConcurrencyBackend(backend), max_workers, chunk_size, timeout

    def map(self, func: Callable[[Any], Any], items: Sequence[Any]) -> List[Any]:
        items = list(items)
        if not items:
            return []
        workers = self.max_workers or min(len(items), 16)
        if self.backend == PiscesLxConcurrencyBackend.THREADING:
            pool: cf.Executor = cf.ThreadPoolExecutor(workers, thread_name_prefix="pisceslx-map")
        elif self.backend == PiscesLxConcurrencyBackend.MULTIPROCESSING:
            pool = cf.ProcessPoolExecutor(workers)
        else:
            raise PiscesLxConcurrencyError(f"unsupported backend for map: {self.backend.value}")
        try:
            if self.backend == PiscesLxConcurrencyBackend.MULTIPROCESSING:
                return list(pool.map(func, items, chunksize=self.chunk_size, timeout=self.timeout))
            futs = [pool.submit(func, it) for it in items]
            out = []
            for i, f in enumerate(futs):
                try:
                    out.append(f.result(timeout=self.timeout))
                except cf.TimeoutError:
                    raise PiscesLxTimeoutError(f"item {i} timed out after {self.timeout}s")
                except Exception as e:
                    raise PiscesLxConcurrencyError(f"item {i} failed: {type(e).__name__}: {e}",
                                                   PiscesLxCoreErrorContext("parallel", "map", details={"index": i})) from e
            return out
        finally:
            pool.shutdown(wait=False, cancel_futures=True)


class PiscesLxAsyncOperator:
    """Runs coroutines with at most ``max_concurrent`` active.  Waiting submissions are admitted by priority (then in
    order of arrival); more than ``max_queue_size`` waiting is refused."""

    def __init__(self, max_concurrent: int = 100, max_queue_size: int = 1000):
        self.max_concurrent, self.max_queue_size = max_concurrent, max_queue_size
        self._running: Set[asyncio.Task] = set()
        self._waiting: List[Tuple[int, int, asyncio.Future]] = []
        self._seq = 0
        self._shutdown = False
        self.started_order: List[int] = []

    @property
    def active_count(self) -> int:
        return len(self._running)

    @property
    def waiting_count(self) -> int:
        return len(self._waiting)

    def _admit(self) -> None:
        while self._waiting and len(self._running) < self.max_concurrent:
            _, _, gate = heapq.heappop(self._waiting)
            if not gate.done():
                gate.set_result(None)
                return

    async def submit(self, coro: Callable[[], Awaitable[Any]], priority: PiscesLxTaskPriority = PiscesLxTaskPriority.NORMAL) -> Any:
        if self._shutdown:
            raise PiscesLxConcurrencyError("the async runner is shut down")
        self._seq += 1
        ticket = self._seq
        if len(self._running) >= self.max_concurrent:
            if len(self._waiting) >= self.max_queue_size:
                raise PiscesLxConcurrencyError(f"queue full ({self.max_queue_size} waiting)")
            gate: asyncio.Future = asyncio.get_running_loop().create_future()
            heapq.heappush(self._waiting, (int(priority), ticket, gate))
            await gate
        task = asyncio.ensure_future(coro())
        self._running.add(task)
        self.started_order.append(ticket)
        try:
            return await task
        finally:
            self._running.discard(task)
            self._admit()

    async def shutdown(self, timeout: float = 30.0) -> None:
        self._shutdown = True
        for _, _, gate in self._waiting:
            if not gate.done():
                gate.set_exception(PiscesLxConcurrencyError("the async runner is shut down"))
        self._waiting.clear()
        tasks = list(self._running)
        for t in tasks:
            t.cancel()
        if tasks:
            await asyncio.wait(tasks, timeout=timeout)


class PiscesLxConcurrencyOperator(PiscesLxOperatorInterface):
    """operation ``timeout`` (func, seconds), ``retry`` (func, optional retry settings), ``parallel`` (func, items,
    optional backend) or ``async`` (coros: a list of coroutine functions, run to completion on a private loop)."""

    name = "concurrency"

    def __init__(self, config: Optional[PiscesLxConcurrencyConfig] = None):
        self.config = config or PiscesLxConcurrencyConfig()

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return inputs.get("operation") in ("timeout", "retry", "parallel", "async")

    def run(self, inputs: Dict[str, Any]) -> Any:
        c, op = self.config, inputs["operation"]
        if op == "timeout":
            return {"result": PiscesLxTimeoutOperator(float(inputs.get("seconds", c.timeout_seconds))).call(inputs["func"])}
        if op == "retry":
            rc = PiscesLxRetryConfig(max_attempts=int(inputs.get("max_attempts", c.retry_attempts)),
                                     base_delay=float(inputs.get("base_delay", c.retry_delay)), jitter=bool(inputs.get("jitter", True)))
            r = PiscesLxRetryOperator(rc, sleep=inputs.get("sleep", time.sleep))
            return {"result": r.execute(inputs["func"]), "attempts": r.attempts_made}
        if op == "parallel":
            p = PiscesLxParallelOperator(inputs.get("backend", c.backend), inputs.get("max_workers", c.max_workers),
                                         int(inputs.get("chunk_size", 1)), inputs.get("timeout"))
            return {"results": p.map(inputs["func"], inputs["items"])}

        async def drive() -> List[Any]:
            runner = PiscesLxAsyncOperator(int(inputs.get("max_concurrent", c.max_workers)))
            return list(await asyncio.gather(*(runner.submit(f) for f in inputs["coros"])))
        return {"results": asyncio.run(drive())}
