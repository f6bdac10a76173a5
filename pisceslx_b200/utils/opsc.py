"""Operator runtime (reference utils/opsc/{interface,base,core,executor,registry,resources}.py): the operator ABI
(``execute(inputs) -> result`` with a status enum), a registry, an executor with timeout / retry / parallel fan-out
(opss concurrency operators), and the CUDA stream / event pool that operators borrow from
(resources.py:210-1130)."""
from __future__ import annotations

import concurrent.futures as cf
import threading
import time
import traceback
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, List, Optional

import torch


class PiscesLxOperatorStatus(str, Enum):
    PENDING = "PENDING"
    RUNNING = "RUNNING"
    SUCCESS = "SUCCESS"
    FAILED = "FAILED"
    CANCELLED = "CANCELLED"


@dataclass
class PiscesLxOperatorResult:
    operator_name: str
    status: PiscesLxOperatorStatus
    output: Any = None
    error: Optional[str] = None
    execution_time: float = 0.0
    metadata: Dict[str, Any] = field(default_factory=dict)

    def is_success(self) -> bool:
        return self.status == PiscesLxOperatorStatus.SUCCESS


class PiscesLxOperatorInterface:
    """Base class: subclasses implement ``run``; ``execute`` wraps it with status, timing and error capture."""

    name: str = "operator"
    version: str = "1.0"

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return True

    def run(self, inputs: Dict[str, Any]) -> Any:
        raise NotImplementedError

    def execute(self, inputs: Dict[str, Any]) -> PiscesLxOperatorResult:
        t0 = time.perf_counter()
        if not self.validate_inputs(inputs):
            return PiscesLxOperatorResult(self.name, PiscesLxOperatorStatus.FAILED, error="invalid inputs")
        try:
            out = self.run(inputs)
            return PiscesLxOperatorResult(self.name, PiscesLxOperatorStatus.SUCCESS, out, None, time.perf_counter() - t0)
        except Exception as e:
            return PiscesLxOperatorResult(self.name, PiscesLxOperatorStatus.FAILED, None,
                                          f"{type(e).__name__}: {e}\n{traceback.format_exc(limit=3)}",
                                          time.perf_counter() - t0)


class PiscesLxFunctionOperator(PiscesLxOperatorInterface):
    def __init__(self, name: str, fn: Callable[[Dict[str, Any]], Any]):
        self.name, self.fn = name, fn

    def run(self, inputs: Dict[str, Any]) -> Any:
        return self.fn(inputs)


class PiscesLxOperatorRegistry:
    def __init__(self):
        self._ops: Dict[str, Callable[[], PiscesLxOperatorInterface]] = {}
        self._lock = threading.Lock()

    def register(self, name: str, factory: Callable[[], PiscesLxOperatorInterface]) -> None:
        with self._lock:
            self._ops[name] = factory

    def create(self, name: str) -> PiscesLxOperatorInterface:
        if name not in self._ops:
            raise KeyError(f"operator {name!r} is not registered")
        return self._ops[name]()

    def names(self) -> List[str]:
        return sorted(self._ops)


class PiscesLxOperatorExecutor:
    """Runs operators with a deadline, retries with back-off, and fans out independent calls on a thread pool."""

    def __init__(self, registry: Optional[PiscesLxOperatorRegistry] = None, max_workers: int = 4):
        self.registry = registry or PiscesLxOperatorRegistry()
        self.pool = cf.ThreadPoolExecutor(max_workers=max_workers, thread_name_prefix="opsc")
        self.history: List[PiscesLxOperatorResult] = []

    def _op(self, op: Any) -> PiscesLxOperatorInterface:
        return self.registry.create(op) if isinstance(op, str) else op

    def execute(self, op: Any, inputs: Dict[str, Any], timeout: Optional[float] = None, retries: int = 0,
                backoff: float = 0.05) -> PiscesLxOperatorResult:
        operator = self._op(op)
        res = PiscesLxOperatorResult(operator.name, PiscesLxOperatorStatus.PENDING)
        for attempt in range(retries + 1):
            fut = self.pool.submit(operator.execute, inputs)
            try:
                res = fut.result(timeout=timeout)
            except cf.TimeoutError:
                fut.cancel()
                res = PiscesLxOperatorResult(operator.name, PiscesLxOperatorStatus.CANCELLED,
                                             error=f"timed out after {timeout}s")
            res.metadata["attempt"] = attempt + 1
            if res.is_success():
                break
            time.sleep(backoff * (2 ** attempt))
        self.history.append(res)
        return res

    def execute_parallel(self, calls: List[tuple], timeout: Optional[float] = None) -> List[PiscesLxOperatorResult]:
        futs = [self.pool.submit(self._op(op).execute, inputs) for op, inputs in calls]
        out = []
        for (op, _), f in zip(calls, futs):
            try:
                out.append(f.result(timeout=timeout))
            except cf.TimeoutError:
                out.append(PiscesLxOperatorResult(getattr(op, "name", str(op)), PiscesLxOperatorStatus.CANCELLED,
                                                  error="timed out"))
        return out

    def shutdown(self) -> None:
        self.pool.shutdown(wait=False, cancel_futures=True)


class PiscesLxStreamPool:
    """Pool of CUDA streams and events handed out to operators that want to overlap work (side copies, collectives
    next to compute).  On CPU the pool hands out ``None`` so that callers keep one code path."""

    def __init__(self, device: Optional[torch.device] = None, n_streams: int = 4):
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                                 else torch.device("cpu"))
        self.cuda = self.device.type == "cuda"
        self._streams = [torch.cuda.Stream(self.device) for _ in range(n_streams)] if self.cuda else []
        self._free_events: List[Any] = []
        self._next = 0
        self._lock = threading.Lock()

    def stream(self) -> Optional["torch.cuda.Stream"]:
        if not self.cuda:
            return None
        with self._lock:
            s = self._streams[self._next % len(self._streams)]
            self._next += 1
        return s

    def event(self) -> Optional["torch.cuda.Event"]:
        if not self.cuda:
            return None
        with self._lock:
            return self._free_events.pop() if self._free_events else torch.cuda.Event()

    def recycle(self, ev: Any) -> None:
        if ev is not None:
            with self._lock:
                self._free_events.append(ev)

    def fork_join(self, fns: List[Callable[[], Any]]) -> List[Any]:
        """Run each callable on its own stream after the current stream's work, and make the current stream wait
        for all of them."""
        if not self.cuda:
            return [f() for f in fns]
        cur = torch.cuda.current_stream(self.device)
        outs = []
        for f in fns:
            s = self.stream()
            s.wait_stream(cur)
            with torch.cuda.stream(s):
                outs.append(f())
            cur.wait_stream(s)
        return outs
