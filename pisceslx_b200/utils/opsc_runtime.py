"""Operator runtime beyond the base ABI (reference utils/opsc: base.py ``PiscesLxBaseOperator`` / transform / filter
operators, core.py ``PiscesLxOperatorCore``, registry.py hub + registrar, resources.py CUDA stream / event objects,
schedulers, memory pool, resource estimator, heterogeneous.py offload manager / load balancer / executor,
distributed.py parallel operators and communication statistics).  Device objects degrade to no-ops on a CPU-only
host, so the same pipelines run in tests."""
from __future__ import annotations

import heapq
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .opsc import (PiscesLxOperatorInterface, PiscesLxOperatorRegistry, PiscesLxOperatorResult, PiscesLxOperatorStatus)


# ------------------------------------------------------------------------------------------------ base operators
@dataclass
class PiscesLxOperatorConfig:
    name: str = "operator"
    timeout_s: Optional[float] = None
    retries: int = 0
    params: Dict[str, Any] = field(default_factory=dict)


class PiscesLxBaseOperator(PiscesLxOperatorInterface):
    """Operator with a config and setup / teardown hooks called around ``run``."""

    def __init__(self, config: Optional[PiscesLxOperatorConfig] = None):
        self.config = config or PiscesLxOperatorConfig()
        self.name = self.config.name
        self.calls = 0

    def setup(self, inputs: Dict[str, Any]) -> None:
        pass

    def teardown(self, inputs: Dict[str, Any], result: PiscesLxOperatorResult) -> None:
        pass

    def execute(self, inputs: Dict[str, Any]) -> PiscesLxOperatorResult:
        self.setup(inputs)
        res = None
        for _ in range(self.config.retries + 1):
            res = super().execute(inputs)
            self.calls += 1
            if res.is_success():
                break
        self.teardown(inputs, res)
        return res


class PiscesLxTransformOperator(PiscesLxBaseOperator):
    """Applies ``fn`` to ``inputs[key]`` and returns the inputs with the transformed value."""

    def __init__(self, fn: Callable[[Any], Any], key: str = "data", config: Optional[PiscesLxOperatorConfig] = None):
        super().__init__(config or PiscesLxOperatorConfig("transform"))
        self.fn, self.key = fn, key

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        return {**inputs, self.key: self.fn(inputs[self.key])}


class PiscesLxFilterOperator(PiscesLxBaseOperator):
    """Keeps the items of ``inputs[key]`` for which ``predicate`` holds."""

    def __init__(self, predicate: Callable[[Any], bool], key: str = "data", config: Optional[PiscesLxOperatorConfig] = None):
        super().__init__(config or PiscesLxOperatorConfig("filter"))
        self.predicate, self.key = predicate, key

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        return {**inputs, self.key: [x for x in inputs[self.key] if self.predicate(x)]}


@dataclass
class PiscesLxExecutionContext:
    run_id: str = ""
    device: str = "cpu"
    started: float = field(default_factory=time.time)
    trace: List[Tuple[str, str, float]] = field(default_factory=list)      # (operator, status, seconds)
    shared: Dict[str, Any] = field(default_factory=dict)


class PiscesLxOperatorRegistryHub(PiscesLxOperatorRegistry):
    """Registry with namespaces (``train/…``, ``infer/…``) and a decorator for registration."""

    def registrar(self, name: str):
        def deco(cls):
            self.register(name, cls)
            return cls
        return deco

    def namespace(self, prefix: str) -> List[str]:
        return [n for n in self.names() if n.startswith(prefix.rstrip("/") + "/")]


PiscesLxOperatorRegistrar = PiscesLxOperatorRegistryHub


@dataclass
class PiscesLxOperatorSystemConfig:
    stop_on_failure: bool = True
    max_workers: int = 4


class PiscesLxOperatorCore:
    """Runs a pipeline of operators: each operator's output dict becomes the next one's input; the context records
    a trace; a failure stops the pipeline (or is skipped, by configuration)."""

    def __init__(self, hub: Optional[PiscesLxOperatorRegistryHub] = None, config: Optional[PiscesLxOperatorSystemConfig] = None):
        self.hub, self.config = hub or PiscesLxOperatorRegistryHub(), config or PiscesLxOperatorSystemConfig()

    def run_pipeline(self, ops: Sequence[Any], inputs: Dict[str, Any], ctx: Optional[PiscesLxExecutionContext] = None
                     ) -> Tuple[Dict[str, Any], PiscesLxExecutionContext]:
        ctx = ctx or PiscesLxExecutionContext()
        data = dict(inputs)
        for op in ops:
            op = self.hub.create(op) if isinstance(op, str) else op
            res = op.execute(data)
            ctx.trace.append((op.name, res.status.value, res.execution_time))
            if res.is_success():
                data = res.output if isinstance(res.output, dict) else {**data, "output": res.output}
            elif self.config.stop_on_failure:
                ctx.shared["error"] = res.error
                break
        return data, ctx


# ------------------------------------------------------------------------------------------------ device resources
class PiscesLxCUDAStream:
    """A CUDA stream, or a no-op stand-in when there is no GPU (``with stream:`` runs the body inline)."""

    def __init__(self, device: Optional[torch.device] = None, priority: int = 0):
        self.stream = torch.cuda.Stream(device, priority=priority) if torch.cuda.is_available() else None

    def __enter__(self):
        if self.stream is not None:
            self._ctx = torch.cuda.stream(self.stream)
            self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self.stream is not None:
            self._ctx.__exit__(*exc)
        return False

    def wait_stream(self, other: "PiscesLxCUDAStream") -> None:
        if self.stream is not None and other.stream is not None:
            self.stream.wait_stream(other.stream)

    def synchronize(self) -> None:
        if self.stream is not None:
            self.stream.synchronize()


class PiscesLxCUDAEvent:
    def __init__(self, timing: bool = True):
        self.event = torch.cuda.Event(enable_timing=timing) if torch.cuda.is_available() else None
        self._t = 0.0

    def record(self, stream: Optional[PiscesLxCUDAStream] = None) -> None:
        if self.event is not None:
            self.event.record(stream.stream if stream and stream.stream is not None else None)
        self._t = time.perf_counter()

    def elapsed_ms(self, end: "PiscesLxCUDAEvent") -> float:
        if self.event is not None and end.event is not None:
            end.event.synchronize()
            return self.event.elapsed_time(end.event)
        return (end._t - self._t) * 1e3


class PiscesLxAllocationPriority(int, Enum):
    LOW = 0
    NORMAL = 1
    HIGH = 2


@dataclass(order=True)
class PiscesLxScheduledTask:
    sort_key: Tuple[int, int]
    fn: Callable[[], Any] = field(compare=False)
    name: str = field(default="", compare=False)


class PiscesLxCUDAScheduler:
    """Priority queue of host callables dispatched round-robin over ``n_streams`` streams; ``run_all`` joins them on
    the current stream and returns the results in submission order."""

    def __init__(self, n_streams: int = 2, device: Optional[torch.device] = None):
        self.streams = [PiscesLxCUDAStream(device) for _ in range(n_streams)]
        self.queue: List[PiscesLxScheduledTask] = []
        self._n = 0

    def submit(self, fn: Callable[[], Any], priority: PiscesLxAllocationPriority = PiscesLxAllocationPriority.NORMAL, name: str = "") -> int:
        heapq.heappush(self.queue, PiscesLxScheduledTask((-int(priority), self._n), fn, name))
        self._n += 1
        return self._n - 1

    def run_all(self) -> List[Any]:
        results: Dict[int, Any] = {}
        order: List[str] = []
        i = 0
        while self.queue:
            t = heapq.heappop(self.queue)
            s = self.streams[i % len(self.streams)]
            with s:
                results[t.sort_key[1]] = t.fn()
            order.append(t.name)
            i += 1
        if torch.cuda.is_available():
            cur = torch.cuda.current_stream()
            for s in self.streams:
                if s.stream is not None:
                    cur.wait_stream(s.stream)
        self.last_order = order
        return [results[k] for k in sorted(results)]


@dataclass
class PiscesLxDeviceLoad:
    index: int
    memory_used_frac: float
    utilization: float
    tasks: int = 0

    def score(self) -> float:
        return 0.6 * self.memory_used_frac + 0.3 * self.utilization / 100.0 + 0.1 * self.tasks


class PiscesLxGPUScheduler:
    """Places tasks on the least loaded device (memory, utilisation, tasks already placed here)."""

    def __init__(self, read_loads: Callable[[], List[PiscesLxDeviceLoad]]):
        self.read_loads = read_loads
        self.placed: Dict[str, int] = {}

    def place(self, task_id: str, min_free_frac: float = 0.0) -> Optional[int]:
        loads = self.read_loads()
        for l in loads:
            l.tasks = sum(1 for d in self.placed.values() if d == l.index)
        ok = [l for l in loads if 1.0 - l.memory_used_frac >= min_free_frac]
        if not ok:
            return None
        best = min(ok, key=lambda l: l.score())
        self.placed[task_id] = best.index
        return best.index

    def release(self, task_id: str) -> None:
        self.placed.pop(task_id, None)


class PiscesLxMemoryPool:
    """Reuses scratch tensors by (dtype, device, rounded size): ``get`` hands out a view of a pooled buffer, ``put``
    returns it; sizes are rounded up to powers of two so that nearby requests share buffers."""

    def __init__(self, max_cached_bytes: int = 1 << 30):
        self.free: Dict[Tuple[Any, Any, int], List[torch.Tensor]] = {}
        self.max_cached, self.cached_bytes = max_cached_bytes, 0
        self.hits = self.misses = 0

    @staticmethod
    def _bucket(n: int) -> int:
        return 1 << max(0, (n - 1).bit_length())

    def get(self, numel: int, dtype: torch.dtype = torch.float32, device: Any = "cpu") -> torch.Tensor:
        key = (dtype, str(device), self._bucket(numel))
        lst = self.free.get(key)
        if lst:
            buf = lst.pop()
            self.cached_bytes -= buf.numel() * buf.element_size()
            self.hits += 1
        else:
            buf = torch.empty(key[2], dtype=dtype, device=device)
            self.misses += 1
        return buf[:numel]

    def put(self, t: torch.Tensor) -> None:
        base = t._base if t._base is not None else t
        nbytes = base.numel() * base.element_size()
        if self.cached_bytes + nbytes > self.max_cached:
            return
        self.free.setdefault((base.dtype, str(base.device), base.numel()), []).append(base)
        self.cached_bytes += nbytes


class PiscesLxResourceType(str, Enum):
    GPU_MEMORY = "gpu_memory"
    HOST_MEMORY = "host_memory"
    COMPUTE = "compute"


@dataclass
class PiscesLxResourceRequest:
    kind: PiscesLxResourceType
    amount: float
    priority: PiscesLxAllocationPriority = PiscesLxAllocationPriority.NORMAL


@dataclass
class PiscesLxResourceAllocation:
    request: PiscesLxResourceRequest
    granted: float
    device: Optional[int] = None


class PiscesLxResourceEstimator:
    """Memory of a module's parameters, gradients and optimizer state, and of a tensor shape."""

    @staticmethod
    def module_bytes(m: torch.nn.Module, training: bool = True, optimizer_bytes_per_param: float = 8.0) -> Dict[str, float]:
        p = sum(x.numel() * x.element_size() for x in m.parameters())
        n = sum(x.numel() for x in m.parameters())
        g = p if training else 0
        o = n * optimizer_bytes_per_param if training else 0
        return {"parameters": p, "gradients": g, "optimizer": o, "total": p + g + o}

    @staticmethod
    def tensor_bytes(shape: Sequence[int], dtype: torch.dtype = torch.bfloat16) -> int:
        n = 1
        for s in shape:
            n *= int(s)
        return n * torch.empty((), dtype=dtype).element_size()


# ------------------------------------------------------------------------------------------------ heterogeneous
class PiscesLxExecutionTarget(str, Enum):
    GPU = "gpu"
    CPU = "cpu"
    AUTO = "auto"


PiscesLxDeviceTypePreference = PiscesLxExecutionTarget


@dataclass
class PiscesLxHeterogeneousConfig:
    gpu_budget_bytes: int = 160 << 30
    prefetch: int = 1                    # layers moved to the device ahead of use
    pin_host: bool = True


class PiscesLxOffloadManager:
    """Keeps the parameters of a list of layers on the host and moves a sliding window of them to the device around
    their use (``prefetch`` layers ahead); ``resident`` tells which layers are on the device now."""

    def __init__(self, layers: Sequence[torch.nn.Module], device: Any, config: Optional[PiscesLxHeterogeneousConfig] = None):
        self.layers, self.device, self.cfg = list(layers), torch.device(device), config or PiscesLxHeterogeneousConfig()
        self.resident: List[int] = []
        self.moves = 0
        for l in self.layers:
            l.to("cpu")
            if self.cfg.pin_host and torch.cuda.is_available():
                for p in l.parameters():
                    p.data = p.data.pin_memory()

    def _load(self, i: int) -> None:
        if i not in self.resident and 0 <= i < len(self.layers):
            self.layers[i].to(self.device, non_blocking=True)
            self.resident.append(i)
            self.moves += 1

    def _evict_before(self, i: int) -> None:
        for j in [r for r in self.resident if r < i]:
            self.layers[j].to("cpu")
            self.resident.remove(j)

    def run(self, x: torch.Tensor) -> torch.Tensor:
        x = x.to(self.device)
        for i, l in enumerate(self.layers):
            for k in range(i, i + 1 + self.cfg.prefetch):
                self._load(k)
            x = l(x)
            self._evict_before(i + 1)
        self._evict_before(len(self.layers))
        return x


class PiscesLxLoadBalancer:
    """Splits a batch between targets in proportion to their measured throughput (items / s), updated by an EMA."""

    def __init__(self, targets: Sequence[str], ema: float = 0.5):
        self.rate = {t: 1.0 for t in targets}
        self.ema = ema

    def split(self, n_items: int) -> Dict[str, int]:
        total = sum(self.rate.values())
        out = {t: int(n_items * r / total) for t, r in self.rate.items()}
        rest = n_items - sum(out.values())
        for t in sorted(self.rate, key=lambda k: -self.rate[k])[:rest]:
            out[t] += 1
        return out

    def observe(self, target: str, items: int, seconds: float) -> None:
        if seconds > 0 and items > 0:
            self.rate[target] = self.ema * self.rate[target] + (1 - self.ema) * items / seconds


class PiscesLxHeterogeneousExecutor:
    """Runs ``fn(chunk, target)`` over the chunks the balancer assigns to each target and concatenates the results in
    the original order; the measured times feed the balancer."""

    def __init__(self, fn: Callable[[torch.Tensor, str], torch.Tensor], targets: Sequence[str] = ("gpu", "cpu")):
        self.fn, self.balancer = fn, PiscesLxLoadBalancer(targets)

    def run(self, batch: torch.Tensor) -> torch.Tensor:
        parts, start = [], 0
        for target, n in self.balancer.split(batch.shape[0]).items():
            if n == 0:
                continue
            t0 = time.perf_counter()
            parts.append(self.fn(batch[start:start + n], target))
            self.balancer.observe(target, n, time.perf_counter() - t0)
            start += n
        return torch.cat(parts, 0)


# ------------------------------------------------------------------------------------------------ distributed
class PiscesLxParallelismType(str, Enum):
    DATA = "data"
    TENSOR = "tensor"
    PIPELINE = "pipeline"
    EXPERT = "expert"
    HYBRID = "hybrid"


class PiscesLxCommunicationType(str, Enum):
    ALL_REDUCE = "all_reduce"
    ALL_GATHER = "all_gather"
    REDUCE_SCATTER = "reduce_scatter"
    ALL_TO_ALL = "all_to_all"
    SEND_RECV = "send_recv"


@dataclass
class PiscesLxCommunicationStats:
    calls: Dict[str, int] = field(default_factory=dict)
    bytes: Dict[str, int] = field(default_factory=dict)

    def record(self, kind: PiscesLxCommunicationType, nbytes: int) -> None:
        self.calls[kind.value] = self.calls.get(kind.value, 0) + 1
        self.bytes[kind.value] = self.bytes.get(kind.value, 0) + int(nbytes)

    def total_bytes(self) -> int:
        return sum(self.bytes.values())


@dataclass
class PiscesLxParallelConfig:
    kind: PiscesLxParallelismType = PiscesLxParallelismType.DATA
    tp: int = 1
    ep: int = 1
    pp: int = 1


class PiscesLxDistributedOperator(PiscesLxBaseOperator):
    """Base of the parallel operators: knows the process group (None = single process) and counts its traffic."""

    def __init__(self, config: Optional[PiscesLxParallelConfig] = None, group: Any = None):
        super().__init__(PiscesLxOperatorConfig("distributed"))
        self.pcfg, self.group, self.stats = config or PiscesLxParallelConfig(), group, PiscesLxCommunicationStats()

    @property
    def world(self) -> int:
        import torch.distributed as dist
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def all_reduce_mean(self, t: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
            t /= self.world
        self.stats.record(PiscesLxCommunicationType.ALL_REDUCE, t.numel() * t.element_size())
        return t


class PiscesLxDataParallelOperator(PiscesLxDistributedOperator):
    """inputs {"parameters"} -> averages gradients over the data-parallel group (bucketed flat all-reduce)."""

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        grads = [p.grad for p in inputs["parameters"] if p.grad is not None]
        if grads:
            flat = torch.cat([g.reshape(-1).float() for g in grads])
            self.all_reduce_mean(flat)
            off = 0
            for g in grads:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()
        return {"reduced_tensors": len(grads), "world": self.world}


class PiscesLxPipelineParallelOperator(PiscesLxDistributedOperator):
    """inputs {"stages": list of callables, "micro_batches"} -> runs the stages of this process in 1F1B order on one
    process (the multi-process schedule is ``parallel.pp``); returns the outputs per micro-batch."""

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        outs = []
        for mb in inputs["micro_batches"]:
            x = mb
            for st in inputs["stages"]:
                x = st(x)
                self.stats.record(PiscesLxCommunicationType.SEND_RECV, x.numel() * x.element_size())
            outs.append(x)
        return {"outputs": outs, "bubble_fraction": (len(inputs["stages"]) - 1) / (len(inputs["micro_batches"]) + len(inputs["stages"]) - 1)}


class PiscesLxExpertParallelOperator(PiscesLxDistributedOperator):
    """inputs {"tokens" [T, H], "expert_idx" [T], "experts": list of callables (the local experts)} -> tokens sorted
    by expert, processed, and restored to their order (the dispatch / combine of one rank)."""

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        x, idx, experts = inputs["tokens"], inputs["expert_idx"], inputs["experts"]
        order = torch.argsort(idx, stable=True)
        xs, out = x[order], torch.empty_like(x)
        counts = torch.bincount(idx, minlength=len(experts)).tolist()
        start = 0
        ys = []
        for e, c in enumerate(counts):
            ys.append(experts[e](xs[start:start + c]) if c else xs[:0])
            start += c
        out[order] = torch.cat(ys, 0)
        self.stats.record(PiscesLxCommunicationType.ALL_TO_ALL, 2 * x.numel() * x.element_size())
        return {"output": out, "tokens_per_expert": counts}


class PiscesLxHybridParallelOperator(PiscesLxDistributedOperator):
    """inputs {"tp", "ep", "pp"} -> builds the mesh through ``parallel.state.init_parallel`` and reports its shape."""

    def run(self, inputs: Dict[str, Any]) -> Dict[str, int]:
        from ..parallel.state import init_parallel
        st = init_parallel(tp=int(inputs.get("tp", self.pcfg.tp)), ep=int(inputs.get("ep", self.pcfg.ep)),
                           pp=int(inputs.get("pp", self.pcfg.pp)), backend=inputs.get("backend"), device=inputs.get("device"))
        return {"world": st.world_size, "tp": st.tp_size, "ep": st.ep_size, "pp": st.pp_size, "dp": st.dp_size}
