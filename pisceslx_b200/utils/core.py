"""Application kit (reference utils/dc.py:89-1382): error types, configuration, filesystem, request context, token
budgets, prompt templates, an LLM client front, a batch processor, lifecycle hooks and service modules, devices and a
resource pool, system metrics.  The reference implements these as wrappers over an external service-framework
package; here they are self-contained (standard library + psutil when present), and the device layer describes the
GPUs of this node through NVML when it is available.

``utils/dc.py`` keeps the logger, metrics, tracing and memory budget; this module imports them."""
from __future__ import annotations

import asyncio
import json
import os
import re
import shutil
import tempfile
import threading
import time
from dataclasses import asdict, dataclass, field
from enum import Enum
from typing import Any, AsyncIterator, Awaitable, Callable, Dict, Iterable, List, Optional, Sequence, Tuple, Union

from .dc import PiscesLxLogger, PiscesLxMetrics


# ---------------------------------------------------------------------------------------------------------------- errors
class PiscesLxCoreLogLevel(str, Enum):
    DEBUG = "debug"
    INFO = "info"
    WARNING = "warning"
    ERROR = "error"
    CRITICAL = "critical"


class PiscesLxCoreErrorCode(Enum):
    INTERNAL_ERROR = ("P-001", "Internal server error")
    CONFIG_PARSE_ERROR = ("P-002", "Configuration parse error")
    FILESYSTEM_ERROR = ("P-003", "Filesystem operation error")
    TOKEN_LIMIT_EXCEEDED = ("P-004", "Token limit exceeded")
    LLM_REQUEST_FAILED = ("P-005", "LLM request failed")
    VALIDATION_ERROR = ("P-006", "Validation error")
    SERVICE_UNAVAILABLE = ("P-007", "Service unavailable")
    TIMEOUT_ERROR = ("P-008", "Operation timeout")
    MEMORY_ERROR = ("P-009", "Memory budget exceeded")
    NETWORK_ERROR = ("P-010", "Network operation failed")
    CONCURRENCY_ERROR = ("P-011", "Concurrency violation")

    @property
    def id(self) -> str:
        return self.value[0]

    @property
    def text(self) -> str:
        return self.value[1]


@dataclass(frozen=True)
class PiscesLxCoreErrorContext:
    component: str = "unknown"
    operation: str = "unknown"
    request_id: Optional[str] = None
    correlation_id: Optional[str] = None
    details: Dict[str, Any] = field(default_factory=dict)


class PiscesLxCoreError(Exception):
    default_code = PiscesLxCoreErrorCode.INTERNAL_ERROR

    def __init__(self, code: Optional[PiscesLxCoreErrorCode] = None, message: Optional[str] = None,
                 context: Optional[PiscesLxCoreErrorContext] = None):
        self.code = code or self.default_code
        self.message = message or self.code.text
        self.context = context or PiscesLxCoreErrorContext()
        super().__init__(f"[{self.code.id}] {self.message}")

    def to_dict(self) -> Dict[str, Any]:
        return {"code": self.code.id, "name": self.code.name, "message": self.message, "context": asdict(self.context)}


def _subclass(name: str, code: PiscesLxCoreErrorCode) -> type:
    return type(name, (PiscesLxCoreError,), {"default_code": code, "__doc__": code.text,
                                             "__init__": lambda self, message=None, context=None, code=None:
                                             PiscesLxCoreError.__init__(self, code, message, context)})


PiscesLxCoreValidationError = _subclass("PiscesLxCoreValidationError", PiscesLxCoreErrorCode.VALIDATION_ERROR)
PiscesLxCoreTimeoutError = _subclass("PiscesLxCoreTimeoutError", PiscesLxCoreErrorCode.TIMEOUT_ERROR)
PiscesLxCoreMemoryError = _subclass("PiscesLxCoreMemoryError", PiscesLxCoreErrorCode.MEMORY_ERROR)
PiscesLxCoreNetworkError = _subclass("PiscesLxCoreNetworkError", PiscesLxCoreErrorCode.NETWORK_ERROR)
PiscesLxCoreConcurrencyError = _subclass("PiscesLxCoreConcurrencyError", PiscesLxCoreErrorCode.CONCURRENCY_ERROR)


# ---------------------------------------------------------------------------------------------------------------- config / fs
class PiscesLxConfiguration:
    """Layered key-value configuration with dotted keys.  Later sources win: files (JSON or YAML), dictionaries,
    environment variables (``PREFIX_A__B=1`` sets ``a.b``; values are parsed as JSON when they parse), ``set``."""

    def __init__(self, initial: Optional[Dict[str, Any]] = None):
        self._data: Dict[str, Any] = {}
        if initial:
            self.load_from_dict(initial)

    @staticmethod
    def _merge(dst: Dict[str, Any], src: Dict[str, Any]) -> None:
        for k, v in src.items():
            if isinstance(v, dict) and isinstance(dst.get(k), dict):
                PiscesLxConfiguration._merge(dst[k], v)
            else:
                dst[k] = v

    def load_from_dict(self, config: Dict[str, Any]) -> None:
        self._merge(self._data, config)

    def load_from_env(self, prefix: str = "PISCES_", environ: Optional[Dict[str, str]] = None) -> int:
        n = 0
        for key, raw in (environ if environ is not None else os.environ).items():
            if not key.startswith(prefix):
                continue
            try:
                val: Any = json.loads(raw)
            except ValueError:
                val = raw
            self.set(key[len(prefix):].lower().replace("__", "."), val)
            n += 1
        return n

    def load_from_file(self, file_path: str) -> None:
        try:
            with open(file_path, encoding="utf-8") as f:
                text = f.read()
            if file_path.endswith((".yaml", ".yml")):
                import yaml
                data = yaml.safe_load(text) or {}
            else:
                data = json.loads(text)
            if not isinstance(data, dict):
                raise ValueError("the top level must be a mapping")
        except (OSError, ValueError) as e:
            raise PiscesLxCoreError(PiscesLxCoreErrorCode.CONFIG_PARSE_ERROR, f"{file_path}: {e}",
                                    PiscesLxCoreErrorContext("configuration", "load_from_file"))
        self.load_from_dict(data)

    def get(self, key: str, default: Any = None) -> Any:
        cur: Any = self._data
        for part in key.split("."):
            if not isinstance(cur, dict) or part not in cur:
                return default
            cur = cur[part]
        return cur

    def set(self, key: str, value: Any) -> None:
        cur = self._data
        parts = key.split(".")
        for part in parts[:-1]:
            nxt = cur.get(part)
            if not isinstance(nxt, dict):
                nxt = cur[part] = {}
            cur = nxt
        cur[parts[-1]] = value

    def get_int(self, key: str, default: int = 0) -> int:
        try:
            return int(self.get(key, default))
        except (TypeError, ValueError):
            return default

    def get_float(self, key: str, default: float = 0.0) -> float:
        try:
            return float(self.get(key, default))
        except (TypeError, ValueError):
            return default

    def get_bool(self, key: str, default: bool = False) -> bool:
        v = self.get(key, default)
        return v.strip().lower() in ("1", "true", "yes", "on") if isinstance(v, str) else bool(v)

    def to_dict(self) -> Dict[str, Any]:
        return json.loads(json.dumps(self._data))


class PiscesLxFilesystem:
    """File operations confined to ``base_path`` (a path that escapes it raises) with atomic writes."""

    def __init__(self, base_path: Optional[str] = None):
        self.base_path = os.path.realpath(base_path or os.getcwd())

    def _resolve(self, path: str) -> str:
        p = os.path.realpath(path if os.path.isabs(path) else os.path.join(self.base_path, path))
        if p != self.base_path and not p.startswith(self.base_path + os.sep):
            raise PiscesLxCoreError(PiscesLxCoreErrorCode.FILESYSTEM_ERROR, f"{path!r} is outside {self.base_path!r}",
                                    PiscesLxCoreErrorContext("filesystem", "resolve"))
        return p

    def _atomic(self, path: str, data: bytes) -> None:
        p = self._resolve(path)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        fd, tmp = tempfile.mkstemp(dir=os.path.dirname(p), prefix=".tmp_")
        try:
            with os.fdopen(fd, "wb") as f:
                f.write(data)
                f.flush()
                os.fsync(f.fileno())
            os.replace(tmp, p)
        except BaseException:
            if os.path.exists(tmp):
                os.remove(tmp)
            raise

    def read(self, path: str) -> str:
        with open(self._resolve(path), encoding="utf-8") as f:
            return f.read()

    def write(self, path: str, content: str) -> None:
        self._atomic(path, content.encode("utf-8"))

    def read_bytes(self, path: str) -> bytes:
        with open(self._resolve(path), "rb") as f:
            return f.read()

    def write_bytes(self, path: str, content: bytes) -> None:
        self._atomic(path, content)

    def exists(self, path: str) -> bool:
        return os.path.exists(self._resolve(path))

    def delete(self, path: str) -> bool:
        p = self._resolve(path)
        if os.path.isdir(p):
            shutil.rmtree(p)
            return True
        if os.path.exists(p):
            os.remove(p)
            return True
        return False

    def list_dir(self, path: str = ".") -> List[str]:
        return sorted(os.listdir(self._resolve(path)))

    def mkdir(self, path: str) -> None:
        os.makedirs(self._resolve(path), exist_ok=True)


class PiscesLxCoreContext:
    """What a component needs to do its work: a named logger, the process metrics, a configuration, a filesystem and
    the ids of the request being served.  Usable as a (sync or async) context manager that logs an escaping error."""

    _shared_metrics: Optional[PiscesLxMetrics] = None

    def __init__(self, name: str = "pisceslx", config: Optional[PiscesLxConfiguration] = None,
                 base_path: Optional[str] = None):
        self.name = name
        self._request_id: Optional[str] = None
        self._correlation_id: Optional[str] = None
        self._config = config or PiscesLxConfiguration()
        self._fs = PiscesLxFilesystem(base_path)
        self._logger = PiscesLxLogger(name)

    @classmethod
    def create(cls, name: str = "pisceslx", **kw: Any) -> "PiscesLxCoreContext":
        return cls(name, **kw)

    logger = property(lambda self: self._logger)
    config = property(lambda self: self._config)
    filesystem = property(lambda self: self._fs)

    @property
    def metrics(self) -> PiscesLxMetrics:
        if PiscesLxCoreContext._shared_metrics is None:
            PiscesLxCoreContext._shared_metrics = PiscesLxMetrics()
        return PiscesLxCoreContext._shared_metrics

    def set_request_id(self, request_id: str) -> None:
        self._request_id = request_id

    def get_request_id(self) -> Optional[str]:
        return self._request_id

    def set_correlation_id(self, correlation_id: str) -> None:
        self._correlation_id = correlation_id

    def get_correlation_id(self) -> Optional[str]:
        return self._correlation_id

    def error_context(self, component: str, operation: str, **details: Any) -> PiscesLxCoreErrorContext:
        return PiscesLxCoreErrorContext(component, operation, self._request_id, self._correlation_id, details)

    def __enter__(self) -> "PiscesLxCoreContext":
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        if exc_type is not None:
            self._logger.error(f"context exited with {exc_type.__name__}: {exc}")

    async def __aenter__(self) -> "PiscesLxCoreContext":
        return self

    async def __aexit__(self, exc_type, exc, tb) -> None:
        self.__exit__(exc_type, exc, tb)


# ---------------------------------------------------------------------------------------------------------------- LLM front
class PiscesLxTokenManager:
    """Per-model token limits and a token count.  ``counter(text) -> int`` (a tokenizer's ``len(encode(.))``) gives
    exact counts; without one the estimate is a quarter of the characters, or one per CJK character."""

    def __init__(self, counter: Optional[Callable[[str], int]] = None, limits: Optional[Dict[str, int]] = None):
        self._counter = counter
        self._limits: Dict[str, int] = dict(limits or {})

    def count_tokens(self, text: str, model: str = "pisces") -> int:
        if self._counter is not None:
            return int(self._counter(text))
        cjk = sum(1 for c in text if "぀" <= c <= "鿿" or "가" <= c <= "힯")
        return cjk + (len(text) - cjk + 3) // 4

    def get_limit(self, model: str) -> int:
        return self._limits.get(model, -1)

    def set_limit(self, model: str, limit: int) -> None:
        self._limits[model] = int(limit)

    def is_within_limit(self, text: str, model: str = "pisces") -> bool:
        lim = self.get_limit(model)
        return lim < 0 or self.count_tokens(text, model) <= lim

    def require(self, text: str, model: str = "pisces") -> int:
        n = self.count_tokens(text, model)
        lim = self.get_limit(model)
        if 0 <= lim < n:
            raise PiscesLxCoreError(PiscesLxCoreErrorCode.TOKEN_LIMIT_EXCEEDED, f"{n} tokens > limit {lim} of {model}",
                                    PiscesLxCoreErrorContext("token_manager", "require", details={"tokens": n, "limit": lim}))
        return n

    def truncate(self, text: str, model: str = "pisces") -> str:
        """The longest prefix of ``text`` inside the model's limit (binary search on the count)."""
        lim = self.get_limit(model)
        if lim < 0 or self.count_tokens(text, model) <= lim:
            return text
        lo, hi = 0, len(text)
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self.count_tokens(text[:mid], model) <= lim:
                lo = mid
            else:
                hi = mid - 1
        return text[:lo]


class PiscesLxPromptTemplate:
    """``{name}`` placeholders.  ``render`` fills the ones it is given and leaves the rest (``strict=True`` raises on a
    missing one); ``{{`` and ``}}`` are literal braces; ``partial`` returns a template with some variables fixed."""

    _VAR = re.compile(r"(?<!\{)\{(\w+)\}(?!\})")

    def __init__(self, template: str):
        self.template = template
        self._variables = list(dict.fromkeys(self._VAR.findall(template)))

    def get_variables(self) -> List[str]:
        return list(self._variables)

    def render(self, strict: bool = False, **kwargs: Any) -> str:
        missing = [v for v in self._variables if v not in kwargs]
        if strict and missing:
            raise PiscesLxCoreError(PiscesLxCoreErrorCode.VALIDATION_ERROR, f"missing template variables: {missing}",
                                    PiscesLxCoreErrorContext("prompt_template", "render"))
        out = self._VAR.sub(lambda m: str(kwargs[m.group(1)]) if m.group(1) in kwargs else m.group(0), self.template)
        return out if missing else out.replace("{{", "{").replace("}}", "}")

    def partial(self, **kwargs: Any) -> "PiscesLxPromptTemplate":
        return PiscesLxPromptTemplate(self._VAR.sub(
            lambda m: str(kwargs[m.group(1)]).replace("{", "{{").replace("}", "}}") if m.group(1) in kwargs else m.group(0),
            self.template))


@dataclass
class PiscesLxLLMResponse:
    content: str
    model: str
    token_count: int
    duration_ms: float
    finish_reason: str = "complete"
    metadata: Dict[str, Any] = field(default_factory=dict)


class PiscesLxLLMClient:
    """Async front of a text generator.  ``backend(prompt, max_tokens=..., temperature=..., **kw)`` returns a string,
    an awaitable of one, or (for streaming) an iterator / async iterator of pieces; the serving engine's ``generate``
    fits.  Prompts over the model's token limit are refused before the backend is called; failures of the backend
    surface as ``LLM_REQUEST_FAILED``."""

    def __init__(self, ctx: Optional[PiscesLxCoreContext] = None, model: str = "pisces",
                 backend: Optional[Callable[..., Any]] = None, token_manager: Optional[PiscesLxTokenManager] = None,
                 clock: Callable[[], float] = time.perf_counter):
        self.ctx, self.model, self._backend, self._clock = ctx or PiscesLxCoreContext(), model, backend, clock
        self._token_manager = token_manager or PiscesLxTokenManager()

    def _need_backend(self) -> Callable[..., Any]:
        if self._backend is None:
            raise PiscesLxCoreError(PiscesLxCoreErrorCode.SERVICE_UNAVAILABLE, "no generation backend is attached",
                                    self.ctx.error_context("llm_client", "generate"))
        return self._backend

    async def generate(self, prompt: str, max_tokens: Optional[int] = None, temperature: float = 0.7, **kwargs: Any) -> PiscesLxLLMResponse:
        backend = self._need_backend()
        n_in = self._token_manager.require(prompt, self.model)
        t0 = self._clock()
        try:
            out = backend(prompt, max_tokens=max_tokens, temperature=temperature, **kwargs)
            if asyncio.iscoroutine(out) or isinstance(out, asyncio.Future):
                out = await out
        except PiscesLxCoreError:
            raise
        except Exception as e:
            raise PiscesLxCoreError(PiscesLxCoreErrorCode.LLM_REQUEST_FAILED, f"{type(e).__name__}: {e}",
                                    self.ctx.error_context("llm_client", "generate", model=self.model))
        text = str(out)
        n_out = self._token_manager.count_tokens(text, self.model)
        cut = max_tokens is not None and n_out >= max_tokens
        return PiscesLxLLMResponse(text, self.model, n_in + n_out, (self._clock() - t0) * 1e3, "length" if cut else "complete",
                                   {"prompt_tokens": n_in, "completion_tokens": n_out})

    async def generate_stream(self, prompt: str, max_tokens: Optional[int] = None, temperature: float = 0.7,
                              **kwargs: Any) -> AsyncIterator[str]:
        backend = self._need_backend()
        self._token_manager.require(prompt, self.model)
        out = backend(prompt, max_tokens=max_tokens, temperature=temperature, stream=True, **kwargs)
        if asyncio.iscoroutine(out):
            out = await out
        if hasattr(out, "__aiter__"):
            async for piece in out:
                yield str(piece)
        elif isinstance(out, str):
            yield out
        else:
            for piece in out:
                yield str(piece)
                await asyncio.sleep(0)


class PiscesLxBatchProcessor:
    """Runs an async ``processor`` over items with at most ``max_concurrent`` in flight, optionally no more than
    ``rate_limit`` starts per second, a per-item ``timeout``; results keep the order of the items.  With
    ``return_exceptions`` a failed item yields its exception instead of cancelling the batch."""

    def __init__(self, max_concurrent: int = 5, rate_limit: Optional[float] = None, timeout: Optional[float] = 30.0):
        self.max_concurrent, self.rate_limit, self.timeout = max_concurrent, rate_limit, timeout

    async def process_all(self, items: Sequence[Any], processor: Callable[[Any], Awaitable[Any]],
                          return_exceptions: bool = False) -> List[Any]:
        sem = asyncio.Semaphore(self.max_concurrent)
        gap = 1.0 / self.rate_limit if self.rate_limit else 0.0
        lock = asyncio.Lock()
        next_start = [0.0]

        async def one(item: Any) -> Any:
            async with sem:
                if gap:
                    async with lock:
                        now = asyncio.get_running_loop().time()
                        wait = next_start[0] - now
                        next_start[0] = max(now, next_start[0]) + gap
                    if wait > 0:
                        await asyncio.sleep(wait)
                try:
                    return await asyncio.wait_for(processor(item), self.timeout)
                except asyncio.TimeoutError:
                    raise PiscesLxCoreTimeoutError(f"item timed out after {self.timeout}s")

        return list(await asyncio.gather(*(one(i) for i in items), return_exceptions=return_exceptions))

    def run(self, items: Sequence[Any], processor: Callable[[Any], Awaitable[Any]], **kw: Any) -> List[Any]:
        """Blocking form for callers without an event loop."""
        return asyncio.run(self.process_all(items, processor, **kw))


# ---------------------------------------------------------------------------------------------------------------- lifecycle
class PiscesLxHookKind(str, Enum):
    BEFORE_INIT = "before_init"
    AFTER_INIT = "after_init"
    BEFORE_START = "before_start"
    AFTER_START = "after_start"
    BEFORE_SHUTDOWN = "before_shutdown"
    AFTER_SHUTDOWN = "after_shutdown"


HookFn = Callable[[PiscesLxCoreContext], Any]


class PiscesLxHooks:
    """Callbacks per lifecycle point, sync or async, run in registration order."""

    def __init__(self) -> None:
        self._hooks: Dict[PiscesLxHookKind, List[HookFn]] = {k: [] for k in PiscesLxHookKind}

    def register(self, hook_kind: PiscesLxHookKind, callback: HookFn) -> None:
        self._hooks[hook_kind].append(callback)

    async def emit(self, hook_kind: PiscesLxHookKind, ctx: PiscesLxCoreContext) -> int:
        for cb in self._hooks[hook_kind]:
            r = cb(ctx)
            if asyncio.iscoroutine(r):
                await r
        return len(self._hooks[hook_kind])

    def emit_sync(self, hook_kind: PiscesLxHookKind, ctx: PiscesLxCoreContext) -> int:
        for cb in self._hooks[hook_kind]:
            r = cb(ctx)
            if asyncio.iscoroutine(r):
                asyncio.run(r)
        return len(self._hooks[hook_kind])

    def on_before_init(self, cb: HookFn) -> None: self.register(PiscesLxHookKind.BEFORE_INIT, cb)
    def on_after_init(self, cb: HookFn) -> None: self.register(PiscesLxHookKind.AFTER_INIT, cb)
    def on_before_start(self, cb: HookFn) -> None: self.register(PiscesLxHookKind.BEFORE_START, cb)
    def on_after_start(self, cb: HookFn) -> None: self.register(PiscesLxHookKind.AFTER_START, cb)
    def on_before_shutdown(self, cb: HookFn) -> None: self.register(PiscesLxHookKind.BEFORE_SHUTDOWN, cb)
    def on_after_shutdown(self, cb: HookFn) -> None: self.register(PiscesLxHookKind.AFTER_SHUTDOWN, cb)


class PiscesLxServiceModule:
    """A unit of the application with a name, a priority, dependencies on other modules and three lifecycle methods to
    override (``on_init`` / ``on_start`` / ``on_shutdown``).  A non-critical module may fail without stopping the
    application."""

    def __init__(self, name: str, priority: int = 0, dependencies: Sequence[str] = (), critical: bool = True):
        self._name, self._priority, self._dependencies, self._is_critical = name, priority, list(dependencies), critical
        self._ctx: Optional[PiscesLxCoreContext] = None
        self.state = "created"

    def name(self) -> str: return self._name
    def is_critical(self) -> bool: return self._is_critical
    def priority(self) -> int: return self._priority
    def dependencies(self) -> List[str]: return list(self._dependencies)

    def init(self, ctx: Optional[PiscesLxCoreContext] = None) -> None:
        self._ctx = ctx or PiscesLxCoreContext(self._name)
        self.on_init(self._ctx)
        self.state = "initialized"

    def start(self, ctx: Optional[PiscesLxCoreContext] = None) -> None:
        if self._ctx is not None:
            self.on_start(self._ctx)
            self.state = "started"

    def shutdown(self, ctx: Optional[PiscesLxCoreContext] = None) -> None:
        if self._ctx is not None:
            self.on_shutdown(self._ctx)
            self.state = "stopped"

    def on_init(self, ctx: PiscesLxCoreContext) -> None: ...
    def on_start(self, ctx: PiscesLxCoreContext) -> None: ...
    def on_shutdown(self, ctx: PiscesLxCoreContext) -> None: ...


class PiscesLxAsyncServiceModule(PiscesLxServiceModule):
    """The same with coroutine lifecycle methods."""

    async def init(self, ctx: Optional[PiscesLxCoreContext] = None) -> None:  # type: ignore[override]
        self._ctx = ctx or PiscesLxCoreContext(self._name)
        await self.on_init(self._ctx)
        self.state = "initialized"

    async def start(self, ctx: Optional[PiscesLxCoreContext] = None) -> None:  # type: ignore[override]
        if self._ctx is not None:
            await self.on_start(self._ctx)
            self.state = "started"

    async def shutdown(self, ctx: Optional[PiscesLxCoreContext] = None) -> None:  # type: ignore[override]
        if self._ctx is not None:
            await self.on_shutdown(self._ctx)
            self.state = "stopped"

    async def on_init(self, ctx: PiscesLxCoreContext) -> None: ...  # type: ignore[override]
    async def on_start(self, ctx: PiscesLxCoreContext) -> None: ...  # type: ignore[override]
    async def on_shutdown(self, ctx: PiscesLxCoreContext) -> None: ...  # type: ignore[override]


class PiscesLxApplication:
    """Runs service modules through their lifecycle in dependency order (then by descending priority), emitting the
    hooks around every phase; shutdown goes in reverse.  A failing non-critical module is logged and skipped."""

    def __init__(self, name: str = "pisceslx", ctx: Optional[PiscesLxCoreContext] = None):
        self.ctx = ctx or PiscesLxCoreContext(name)
        self.hooks = PiscesLxHooks()
        self._modules: Dict[str, PiscesLxServiceModule] = {}
        self.failed: Dict[str, str] = {}
        self._order: List[str] = []

    def add(self, module: PiscesLxServiceModule) -> "PiscesLxApplication":
        self._modules[module.name()] = module
        return self

    def order(self) -> List[str]:
        done: List[str] = []
        left = sorted(self._modules.values(), key=lambda m: (-m.priority(), m.name()))
        while left:
            ready = [m for m in left if all(d in done or d not in self._modules for d in m.dependencies())]
            if not ready:
                raise PiscesLxCoreError(PiscesLxCoreErrorCode.VALIDATION_ERROR,
                                        f"dependency cycle among {[m.name() for m in left]}",
                                        self.ctx.error_context("application", "order"))
            done.append(ready[0].name())
            left.remove(ready[0])
        return done

    async def _phase(self, names: Sequence[str], method: str, before: PiscesLxHookKind, after: PiscesLxHookKind) -> None:
        await self.hooks.emit(before, self.ctx)
        for n in names:
            m = self._modules[n]
            if n in self.failed or any(d in self.failed for d in m.dependencies()):
                self.failed.setdefault(n, "a dependency failed")
                continue
            try:
                r = getattr(m, method)(None)
                if asyncio.iscoroutine(r):
                    await r
            except Exception as e:
                if m.is_critical():
                    raise
                self.failed[n] = f"{type(e).__name__}: {e}"
                self.ctx.logger.warning(f"module {n} failed in {method}: {e}")
        await self.hooks.emit(after, self.ctx)

    async def start(self) -> None:
        K = PiscesLxHookKind
        self._order = self.order()
        await self._phase(self._order, "init", K.BEFORE_INIT, K.AFTER_INIT)
        await self._phase(self._order, "start", K.BEFORE_START, K.AFTER_START)

    async def shutdown(self) -> None:
        K = PiscesLxHookKind
        await self._phase(list(reversed(self._order)), "shutdown", K.BEFORE_SHUTDOWN, K.AFTER_SHUTDOWN)


# ---------------------------------------------------------------------------------------------------------------- devices
class PiscesLxDeviceType(str, Enum):
    CPU = "cpu"
    GPU = "gpu"
    TPU = "tpu"
    NPU = "npu"
    MEMORY = "memory"
    STORAGE = "storage"
    NETWORK = "network"
    ACCELERATOR = "accelerator"
    CUSTOM = "custom"


class PiscesLxDeviceStatus(str, Enum):
    UNKNOWN = "unknown"
    AVAILABLE = "available"
    BUSY = "busy"
    ERROR = "error"
    OFFLINE = "offline"
    MAINTENANCE = "maintenance"
    DEGRADED = "degraded"
    ALLOCATED = "allocated"


@dataclass
class PiscesLxDeviceCapabilities:
    compute_units: int = 0
    memory_gb: float = 0.0
    storage_gb: float = 0.0
    bandwidth_gbps: float = 0.0
    custom: Dict[str, float] = field(default_factory=dict)

    def meets_requirements(self, required: "PiscesLxDeviceCapabilities") -> bool:
        return (self.compute_units >= required.compute_units and self.memory_gb >= required.memory_gb
                and self.storage_gb >= required.storage_gb and self.bandwidth_gbps >= required.bandwidth_gbps
                and all(self.custom.get(k, 0.0) >= v for k, v in required.custom.items()))


@dataclass
class PiscesLxDeviceHealthMetrics:
    cpu_usage_percent: float = 0.0
    memory_usage_percent: float = 0.0
    temperature_celsius: float = 0.0
    error_count: int = 0
    throughput: int = 0
    network_latency_ms: float = 0.0
    disk_iops: int = 0
    battery_level_percent: float = 100.0
    response_time_ms: float = 0.0
    uptime_seconds: int = 0

    @property
    def health_score(self) -> float:
        s = 100.0
        s -= max(self.cpu_usage_percent - 80, 0) * 0.5
        s -= max(self.memory_usage_percent - 80, 0) * 0.5
        s -= max(self.temperature_celsius - 70, 0) * 0.3
        s -= min(self.error_count * 5, 30)
        return max(0.0, min(100.0, s))

    @property
    def is_healthy(self) -> bool:
        return self.health_score >= 50.0


class PiscesLxDevice:
    def __init__(self, device_id: str, device_type: PiscesLxDeviceType = PiscesLxDeviceType.CPU, name: Optional[str] = None):
        self._id, self._type, self._name = device_id, device_type, name or device_id
        self._status = PiscesLxDeviceStatus.UNKNOWN
        self._capabilities = PiscesLxDeviceCapabilities()
        self._health_metrics = PiscesLxDeviceHealthMetrics()
        self._metadata: Dict[str, Any] = {}

    id = property(lambda self: self._id)
    name = property(lambda self: self._name)
    device_type = property(lambda self: self._type)
    status = property(lambda self: self._status)
    capabilities = property(lambda self: self._capabilities)
    health_metrics = property(lambda self: self._health_metrics)
    metadata = property(lambda self: self._metadata)
    health_score = property(lambda self: self._health_metrics.health_score)

    def set_status(self, status: PiscesLxDeviceStatus) -> None: self._status = status
    def set_capabilities(self, caps: PiscesLxDeviceCapabilities) -> None: self._capabilities = caps
    def set_health_metrics(self, metrics: PiscesLxDeviceHealthMetrics) -> None: self._health_metrics = metrics
    def set_metadata(self, key: str, value: Any) -> None: self._metadata[key] = value

    @property
    def is_healthy(self) -> bool:
        return self._health_metrics.is_healthy and self._status not in (
            PiscesLxDeviceStatus.ERROR, PiscesLxDeviceStatus.OFFLINE, PiscesLxDeviceStatus.MAINTENANCE)

    @property
    def is_available(self) -> bool:
        return self._status == PiscesLxDeviceStatus.AVAILABLE and self.is_healthy


@dataclass
class PiscesLxResourcePoolStatus:
    total_devices: int = 0
    available_devices: int = 0
    allocated_devices: int = 0
    total_capacity: float = 0.0
    available_capacity: float = 0.0
    allocated_capacity: float = 0.0
    utilization_percent: float = 0.0
    average_health_score: float = 0.0
    status_distribution: Dict[str, int] = field(default_factory=dict)

    @property
    def is_healthy(self) -> bool:
        return self.available_devices > 0 or self.allocated_devices > 0


@dataclass
class PiscesLxResourcePoolStatistics:
    total_devices: int = 0
    available_devices: int = 0
    busy_devices: int = 0
    offline_devices: int = 0
    error_devices: int = 0
    total_compute_units: int = 0
    total_memory_gb: float = 0.0
    total_storage_gb: float = 0.0
    total_bandwidth_gbps: float = 0.0
    average_health_score: float = 0.0
    status_distribution: Dict[str, int] = field(default_factory=dict)


@dataclass
class PiscesLxConnectionPoolStatistics:
    total_connections: int = 0
    active_connections: int = 0
    idle_connections: int = 0
    unhealthy_connections: int = 0
    total_successful_ops: int = 0
    total_failed_ops: int = 0
    average_response_time_ms: float = 0.0
    health_check_interval_secs: int = 30

    @property
    def success_rate(self) -> float:
        n = self.total_successful_ops + self.total_failed_ops
        return self.total_successful_ops / n if n else 1.0


class PiscesLxResourcePool:
    """Named set of devices with allocation: ``allocate`` picks the healthiest available device that meets the
    requirements and marks it ALLOCATED; ``release`` returns it.  Capacity is counted in compute units.  Thread-safe."""

    def __init__(self, name: str = "default"):
        self.name = name
        self._devices: Dict[str, PiscesLxDevice] = {}
        self._owners: Dict[str, str] = {}
        self._lock = threading.RLock()

    def add_device(self, device: PiscesLxDevice) -> None:
        with self._lock:
            self._devices[device.id] = device

    def remove_device(self, device_id: str) -> bool:
        with self._lock:
            self._owners.pop(device_id, None)
            return self._devices.pop(device_id, None) is not None

    def get_device(self, device_id: str) -> Optional[PiscesLxDevice]:
        return self._devices.get(device_id)

    def get_all_devices(self) -> List[PiscesLxDevice]:
        return list(self._devices.values())

    def get_available_devices(self) -> List[PiscesLxDevice]:
        return [d for d in self._devices.values() if d.is_available]

    def select_best_device(self, requirements: Optional[PiscesLxDeviceCapabilities] = None,
                           device_type: Optional[PiscesLxDeviceType] = None) -> Optional[PiscesLxDevice]:
        c = [d for d in self.get_available_devices()
             if (device_type is None or d.device_type == device_type)
             and (requirements is None or d.capabilities.meets_requirements(requirements))]
        return max(c, key=lambda d: (d.health_score, -d.capabilities.memory_gb, d.id)) if c else None

    def allocate(self, owner: str, requirements: Optional[PiscesLxDeviceCapabilities] = None,
                 device_type: Optional[PiscesLxDeviceType] = None) -> Optional[PiscesLxDevice]:
        with self._lock:
            d = self.select_best_device(requirements, device_type)
            if d is not None:
                d.set_status(PiscesLxDeviceStatus.ALLOCATED)
                self._owners[d.id] = owner
            return d

    def release(self, device_id: str) -> bool:
        with self._lock:
            d = self._devices.get(device_id)
            if d is None or d.status != PiscesLxDeviceStatus.ALLOCATED:
                return False
            d.set_status(PiscesLxDeviceStatus.AVAILABLE)
            self._owners.pop(device_id, None)
            return True

    def owner_of(self, device_id: str) -> Optional[str]:
        return self._owners.get(device_id)

    def get_status(self) -> PiscesLxResourcePoolStatus:
        with self._lock:
            ds = list(self._devices.values())
            avail = [d for d in ds if d.is_available]
            alloc = [d for d in ds if d.status == PiscesLxDeviceStatus.ALLOCATED]
            total = float(sum(d.capabilities.compute_units for d in ds))
            free = float(sum(d.capabilities.compute_units for d in avail))
            dist: Dict[str, int] = {}
            for d in ds:
                dist[d.status.value] = dist.get(d.status.value, 0) + 1
            return PiscesLxResourcePoolStatus(len(ds), len(avail), len(alloc), total, free, total - free,
                                              (total - free) / total * 100 if total else 0.0,
                                              sum(d.health_score for d in ds) / len(ds) if ds else 0.0, dist)

    def get_statistics(self) -> PiscesLxResourcePoolStatistics:
        st, ds = self.get_status(), list(self._devices.values())
        S = PiscesLxDeviceStatus
        return PiscesLxResourcePoolStatistics(
            st.total_devices, st.available_devices, sum(d.status == S.BUSY for d in ds), sum(d.status == S.OFFLINE for d in ds),
            sum(d.status == S.ERROR for d in ds), sum(d.capabilities.compute_units for d in ds),
            sum(d.capabilities.memory_gb for d in ds), sum(d.capabilities.storage_gb for d in ds),
            sum(d.capabilities.bandwidth_gbps for d in ds), st.average_health_score, st.status_distribution)

    def is_healthy(self) -> bool:
        return self.get_status().is_healthy

    @classmethod
    def from_local_gpus(cls, name: str = "gpus", nvml: Any = None) -> "PiscesLxResourcePool":
        """One device per GPU of this node, described through NVML (read-only queries: name, memory, multiprocessor
        count, temperature, utilisation).  ``nvml`` is the module to use (``pynvml`` by default); without NVML or without
        GPUs the pool is empty."""
        pool = cls(name)
        try:
            if nvml is None:
                import pynvml as nvml                    # provided by nvidia-ml-py
            nvml.nvmlInit()
        except Exception:
            return pool
        try:
            for i in range(nvml.nvmlDeviceGetCount()):
                h = nvml.nvmlDeviceGetHandleByIndex(i)
                nm = nvml.nvmlDeviceGetName(h)
                d = PiscesLxDevice(f"gpu:{i}", PiscesLxDeviceType.GPU, nm.decode() if isinstance(nm, bytes) else str(nm))
                mem = nvml.nvmlDeviceGetMemoryInfo(h)
                sms = 0
                try:
                    sms = int(nvml.nvmlDeviceGetNumGpuCores(h)) // 128
                except Exception:
                    pass
                d.set_capabilities(PiscesLxDeviceCapabilities(sms, mem.total / 2 ** 30))
                hm = PiscesLxDeviceHealthMetrics(memory_usage_percent=100.0 * mem.used / max(mem.total, 1))
                try:
                    hm.temperature_celsius = float(nvml.nvmlDeviceGetTemperature(h, 0))
                    hm.cpu_usage_percent = float(nvml.nvmlDeviceGetUtilizationRates(h).gpu)
                except Exception:
                    pass
                d.set_health_metrics(hm)
                d.set_status(PiscesLxDeviceStatus.AVAILABLE)
                pool.add_device(d)
        finally:
            try:
                nvml.nvmlShutdown()
            except Exception:
                pass
        return pool


# ---------------------------------------------------------------------------------------------------------------- system metrics
@dataclass
class PiscesLxSystemMetrics:
    timestamp: float = 0.0
    cpu: Dict[str, Any] = field(default_factory=dict)
    memory: Dict[str, Any] = field(default_factory=dict)
    disk: Dict[str, Any] = field(default_factory=dict)
    network: Dict[str, Any] = field(default_factory=dict)

    cpu_usage_percent = property(lambda self: float(self.cpu.get("total_usage_percent", 0.0)))
    memory_usage_percent = property(lambda self: float(self.memory.get("usage_percent", 0.0)))
    disk_usage_percent = property(lambda self: float(self.disk.get("usage_percent", 0.0)))

    def to_dict(self) -> Dict[str, Any]:
        return {"timestamp": self.timestamp, "cpu": dict(self.cpu), "memory": dict(self.memory), "disk": dict(self.disk),
                "network": dict(self.network)}

    @classmethod
    def collect(cls, path: str = "/", previous: Optional["PiscesLxSystemMetrics"] = None) -> "PiscesLxSystemMetrics":
        """One sample of the host: psutil when it is installed, /proc and ``shutil.disk_usage`` otherwise.  With a
        ``previous`` sample the network rates are filled in."""
        now = time.time()
        m = cls(now)
        du = shutil.disk_usage(path)
        m.disk = {"total_bytes": du.total, "used_bytes": du.used, "free_bytes": du.free,
                  "usage_percent": 100.0 * du.used / max(du.total, 1)}
        try:
            import psutil
            vm, sw, net = psutil.virtual_memory(), psutil.swap_memory(), psutil.net_io_counters()
            per = psutil.cpu_percent(interval=None, percpu=True)
            st = psutil.cpu_stats()
            m.cpu = {"total_usage_percent": sum(per) / max(len(per), 1), "per_core_usage": per,
                     "context_switches": st.ctx_switches, "interrupts": st.interrupts}
            m.memory = {"total_bytes": vm.total, "used_bytes": vm.used, "free_bytes": vm.available, "usage_percent": vm.percent,
                        "swap_total_bytes": sw.total, "swap_used_bytes": sw.used, "swap_free_bytes": sw.free,
                        "swap_usage_percent": sw.percent}
            m.network = {"total_received_bytes": net.bytes_recv, "total_transmitted_bytes": net.bytes_sent}
        except ImportError:
            info: Dict[str, int] = {}
            try:
                with open("/proc/meminfo") as f:
                    for line in f:
                        k, v = line.split(":", 1)
                        info[k] = int(v.split()[0]) * 1024
            except OSError:
                pass
            tot, free = info.get("MemTotal", 0), info.get("MemAvailable", 0)
            m.memory = {"total_bytes": tot, "used_bytes": tot - free, "free_bytes": free,
                        "usage_percent": 100.0 * (tot - free) / max(tot, 1)}
            load = os.getloadavg()[0] if hasattr(os, "getloadavg") else 0.0
            m.cpu = {"total_usage_percent": min(100.0, 100.0 * load / max(os.cpu_count() or 1, 1)), "per_core_usage": []}
            m.network = {"total_received_bytes": 0, "total_transmitted_bytes": 0}
        if previous is not None and now > previous.timestamp:
            dt = now - previous.timestamp
            m.network["received_bytes_per_sec"] = (m.network["total_received_bytes"] - previous.network.get("total_received_bytes", 0)) / dt
            m.network["transmitted_bytes_per_sec"] = (m.network["total_transmitted_bytes"] - previous.network.get("total_transmitted_bytes", 0)) / dt
        return m
