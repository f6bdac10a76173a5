"""The MoE runtime operator for serving (reference opss/infer/moe_runtime.py:84-1643): routing with an adaptive
temperature, dynamic capacity, a routing cache, request sharing, load statistics, brownout of unimportant expert
groups and the switch between expert- and tensor-parallel execution of the expert layer.

``serve/runtime.py`` holds the building blocks (expert residency cache, load balancer, batch sharing, tri-route
decision, brownout grouper, layout choice by bytes moved); this module adds the configured operator around a model's
gate and the remaining classes.

Host reads are kept off the per-call path: the load window is a device tensor that is only looked at every
``adaptive_temp_interval`` / ``capacity_update_interval`` calls, and the routing cache is keyed by a hash of the token
ids the caller already has on the host (the reference hashes ``hidden_states`` through ``.cpu().numpy().tobytes()`` on
every call, moe_runtime.py:320-330, which synchronises the stream and copies the activations for each lookup).  The
count of dropped assignments is returned as a tensor."""
from __future__ import annotations

import json
import time
from collections import OrderedDict
from dataclasses import asdict, dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..utils.opsc import PiscesLxOperatorInterface
from .runtime import PiscesLxBatchSharing, PiscesLxBrownoutMoEGrouper, moebius_choose_layout


class PiscesLxMoERoutingStrategy(str, Enum):
    TOP_K = "top_k"
    ADAPTIVE = "adaptive"            # top-k with the adaptive temperature
    CAPACITY = "capacity"            # top-k, then assignments over the capacity are dropped
    PRIORITY = "priority"            # tokens with a weight above the threshold are served first when capacity binds


@dataclass
class PiscesLxMoERuntimeConfig:
    routing_strategy: str = "adaptive"
    routing_temp: float = 1.12
    top_k: int = 2
    capacity_factor: float = 1.0
    min_capacity: int = 4
    noise_std: float = 0.0
    load_balance_alpha: float = 0.01
    enable_load_balancing: bool = True
    utilization_high: float = 1.5
    utilization_low: float = 0.5
    enable_expert_cache: bool = True
    expert_cache_size: int = 10000
    enable_batch_expert_sharing: bool = True
    batch_sharing_threshold: int = 32
    dynamic_capacity: bool = True
    capacity_update_interval: int = 16
    capacity_margin: float = 0.1
    enable_adaptive_temp: bool = True
    adaptive_temp_step: float = 0.03
    adaptive_temp_interval: int = 16
    adaptive_temp_cap: float = 1.30
    adaptive_temp_floor: float = 0.5
    priority_threshold: float = 0.5
    drop_tokens: bool = True

    def __post_init__(self) -> None:
        self.routing_strategy = PiscesLxMoERoutingStrategy(getattr(self.routing_strategy, "value", self.routing_strategy)).value
        if self.top_k < 1:
            raise ValueError("top_k must be at least 1")

    @classmethod
    def from_model_config(cls, model_config: Any) -> "PiscesLxMoERuntimeConfig":
        get = (lambda k, d: model_config.get(k, d)) if isinstance(model_config, dict) else (lambda k, d: getattr(model_config, k, d))
        return cls(routing_temp=float(get("routing_temp", 1.12)), top_k=int(get("moe_top_k", 2)),
                   capacity_factor=float(get("moe_capacity_factor", 1.0)), min_capacity=int(get("moe_min_capacity", 4)),
                   load_balance_alpha=float(get("moe_load_balance_alpha", 0.01)), drop_tokens=bool(get("moe_drop_tokens", True)))

    @classmethod
    def from_json(cls, config_path: str) -> "PiscesLxMoERuntimeConfig":
        with open(config_path, encoding="utf-8") as f:
            d = json.load(f)
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


@dataclass
class PiscesLxExpertStats:
    expert_id: int
    token_count: int = 0
    call_count: int = 0
    total_latency_ms: float = 0.0

    def update(self, token_count: int, latency_ms: float = 0.0) -> None:
        self.token_count += int(token_count)
        self.call_count += 1
        self.total_latency_ms += float(latency_ms)

    @property
    def avg_latency_ms(self) -> float:
        return self.total_latency_ms / self.call_count if self.call_count else 0.0

    @property
    def avg_tokens(self) -> float:
        return self.token_count / self.call_count if self.call_count else 0.0


class PiscesLxExpertCacheEntry:
    def __init__(self, cache_key: str, expert_indices: torch.Tensor, routing_probs: torch.Tensor):
        self.cache_key, self.expert_indices, self.routing_probs = cache_key, expert_indices, routing_probs
        self.hits, self.created = 0, time.time()

    def hit(self) -> None:
        self.hits += 1

    def to_dict(self) -> Dict[str, Any]:
        return {"cache_key": self.cache_key, "hits": self.hits, "tokens": int(self.expert_indices.shape[0]), "age_s": time.time() - self.created}


class PiscesLxExpertCacheManager:
    """Routing decisions by a key of the token ids (a prompt prefix routed before routes the same way again): an LRU of
    ``PiscesLxExpertCacheEntry``.  Lookups never touch the device."""

    def __init__(self, max_entries: int = 10000):
        self.max_entries = max_entries
        self._entries: "OrderedDict[str, PiscesLxExpertCacheEntry]" = OrderedDict()
        self.hits = self.misses = self.evictions = 0

    @staticmethod
    def key_for(token_ids: Sequence[int], layer: int = 0) -> str:
        h = 1469598103934665603
        for t in token_ids:
            h = ((h ^ (int(t) & 0xFFFFFFFF)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
        return f"{layer}:{len(token_ids)}:{h:016x}"

    def get(self, cache_key: str) -> Optional[PiscesLxExpertCacheEntry]:
        e = self._entries.get(cache_key)
        if e is None:
            self.misses += 1
            return None
        self._entries.move_to_end(cache_key)
        e.hit()
        self.hits += 1
        return e

    def insert(self, cache_key: str, expert_indices: torch.Tensor, routing_probs: torch.Tensor) -> PiscesLxExpertCacheEntry:
        e = PiscesLxExpertCacheEntry(cache_key, expert_indices.detach(), routing_probs.detach())
        self._entries[cache_key] = e
        self._entries.move_to_end(cache_key)
        while len(self._entries) > self.max_entries:
            self._entries.popitem(last=False)
            self.evictions += 1
        return e

    def get_hit_rate(self) -> float:
        n = self.hits + self.misses
        return self.hits / n if n else 0.0

    def get_stats(self) -> Dict[str, Any]:
        return {"entries": len(self._entries), "hits": self.hits, "misses": self.misses, "evictions": self.evictions, "hit_rate": self.get_hit_rate()}

    def clear(self) -> None:
        self._entries.clear()


class PiscesLxBatchExpertSharing:
    """Requests with a long common token prefix route that prefix identically and can share its keys / values.
    ``find_similar_requests`` returns, for a new request, the cached requests whose common-prefix share reaches the
    threshold; ``share_prefix_kv`` reports how many tokens of which request to reuse."""

    def __init__(self, similarity_threshold: float = 0.8, max_tracked: int = 1024):
        self.similarity_threshold, self.max_tracked = similarity_threshold, max_tracked
        self._requests: "OrderedDict[str, Tuple[int, ...]]" = OrderedDict()
        self.shared_tokens = self.lookups = 0

    @staticmethod
    def common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
        n = 0
        for x, y in zip(a, b):
            if x != y:
                break
            n += 1
        return n

    def compute_similarity(self, input_ids_1: Sequence[int], input_ids_2: Sequence[int]) -> float:
        """Length of the common prefix over the shorter length."""
        m = min(len(input_ids_1), len(input_ids_2))
        return self.common_prefix(input_ids_1, input_ids_2) / m if m else 0.0

    def register(self, request_id: str, input_ids: Sequence[int]) -> None:
        self._requests[request_id] = tuple(input_ids)
        self._requests.move_to_end(request_id)
        while len(self._requests) > self.max_tracked:
            self._requests.popitem(last=False)

    def find_similar_requests(self, input_ids: Sequence[int], k: int = 1) -> List[Tuple[str, float, int]]:
        self.lookups += 1
        out = []
        for rid, ids in self._requests.items():
            p = self.common_prefix(input_ids, ids)
            s = p / min(len(input_ids), len(ids)) if ids and input_ids else 0.0
            if s >= self.similarity_threshold and p > 0:
                out.append((rid, s, p))
        return sorted(out, key=lambda t: (-t[2], t[0]))[:k]

    def share_prefix_kv(self, input_ids: Sequence[int]) -> Optional[Dict[str, Any]]:
        hit = self.find_similar_requests(input_ids, 1)
        if not hit:
            return None
        rid, s, p = hit[0]
        self.shared_tokens += p
        return {"source_request": rid, "shared_tokens": p, "similarity": s, "remaining_tokens": len(input_ids) - p}

    def group_by_experts(self, expert_sets: List[set], max_group: int = 8) -> List[List[int]]:
        return PiscesLxBatchSharing.group(expert_sets, max_group)

    def get_stats(self) -> Dict[str, Any]:
        return {"tracked": len(self._requests), "lookups": self.lookups, "shared_tokens": self.shared_tokens}


@dataclass
class PiscesLxBrownoutExpertGroup:
    """One co-activation group of experts with its running importance and whether it is switched on."""
    group_id: int
    expert_ids: List[int]
    importance: float = 1.0
    active: bool = True

    @classmethod
    def from_grouper(cls, grouper: PiscesLxBrownoutMoEGrouper) -> List["PiscesLxBrownoutExpertGroup"]:
        return [cls(g, list(m), float(grouper.importance[g]), bool(grouper.active[g])) for g, m in enumerate(grouper.groups)]


class PiscesLxMoebiusParallelismMode(str, Enum):
    EXPERT_PARALLEL = "ep"
    TENSOR_PARALLEL = "tp"


class PiscesLxMoebiusParallelismSwitch:
    """Chooses how the expert layer runs for the next step: with few tokens per step (decode) every expert's whole
    weight would be read for a handful of rows, so splitting each expert across ranks (tensor parallel) reads 1/n of it
    per rank; with many tokens (prefill) moving tokens to whole experts (expert parallel) is cheaper.  The decision is
    the byte count of ``serve.runtime.moebius_choose_layout`` with hysteresis, so that a batch size near the break-even
    point does not flip the layout every step."""

    def __init__(self, world_size: int = 1, hidden: int = 4096, ffn: int = 1408, top_k: int = 2, hysteresis: float = 0.15,
                 switcher: Optional[Callable[[PiscesLxMoebiusParallelismMode], None]] = None, clock: Callable[[], float] = time.perf_counter):
        self.world_size, self.hidden, self.ffn, self.top_k, self.hysteresis = world_size, hidden, ffn, top_k, hysteresis
        self.mode = PiscesLxMoebiusParallelismMode.EXPERT_PARALLEL
        self._switcher, self._clock = switcher, clock
        self.switch_count, self._latencies = 0, []

    def preferred(self, batch_tokens: int, num_experts: int) -> Tuple[PiscesLxMoebiusParallelismMode, float]:
        r = moebius_choose_layout(batch_tokens, self.hidden, self.ffn, num_experts, self.top_k, self.world_size)
        lo, hi = sorted((float(r["ep_time_s"]), float(r["tp_time_s"])))
        return PiscesLxMoebiusParallelismMode(r["layout"]), ((hi - lo) / hi if hi > 0 else 0.0)

    def should_switch(self, batch_tokens: int, num_experts: int) -> bool:
        if self.world_size <= 1:
            return False
        mode, margin = self.preferred(batch_tokens, num_experts)
        return mode is not self.mode and margin >= self.hysteresis

    def switch(self, new_mode: PiscesLxMoebiusParallelismMode) -> float:
        t0 = self._clock()
        if self._switcher is not None and new_mode is not self.mode:
            self._switcher(new_mode)
        dt = self._clock() - t0
        if new_mode is not self.mode:
            self.mode = new_mode
            self.switch_count += 1
            self._latencies.append(dt)
        return dt

    def step(self, batch_tokens: int, num_experts: int) -> PiscesLxMoebiusParallelismMode:
        if self.should_switch(batch_tokens, num_experts):
            self.switch(self.preferred(batch_tokens, num_experts)[0])
        return self.mode

    def get_avg_switch_latency(self) -> float:
        return sum(self._latencies) / len(self._latencies) if self._latencies else 0.0


class PiscesLxMoERuntimeOperator(PiscesLxOperatorInterface):
    """``set_model(model)`` finds the gates (modules with a ``gate`` linear whose output width is the expert count);
    ``route(hidden [T, H], layer=0, token_ids=None)`` returns the chosen experts and their weights.

    Adaptive temperature: every ``adaptive_temp_interval`` calls the utilisation ratio of each expert (its share of
    the recent assignments x E) is looked at; experts above ``utilization_high`` or under ``utilization_low`` raise the
    temperature by one step (flatter routing), a balanced state lowers it back towards the configured value.
    Dynamic capacity: ceil(T k / E x capacity_factor x (1 + margin)), at least ``min_capacity``, recomputed every
    ``capacity_update_interval`` calls from the observed peak / mean load ratio."""

    name = "moe_runtime"

    def __init__(self, config: Optional[PiscesLxMoERuntimeConfig] = None):
        self.config = c = config or PiscesLxMoERuntimeConfig()
        self.cache = PiscesLxExpertCacheManager(c.expert_cache_size) if c.enable_expert_cache else None
        self.sharing = PiscesLxBatchExpertSharing() if c.enable_batch_expert_sharing else None
        self._gates: List[nn.Module] = []
        self.num_experts = 0
        self._adaptive_temp = c.routing_temp
        self._calls = 0
        self._load: Optional[torch.Tensor] = None
        self._capacity_scale = 1.0
        self.expert_stats: Dict[int, PiscesLxExpertStats] = {}
        self._dropped: Optional[torch.Tensor] = None
        self.brownout: Optional[PiscesLxBrownoutMoEGrouper] = None

    @property
    def dropped(self) -> int:
        return int(self._dropped) if self._dropped is not None else 0

    # -- model -------------------------------------------------------------------------------------------------------------------
    def set_model(self, model: nn.Module) -> int:
        self._gates = []
        for m in model.modules():
            g = getattr(m, "gate", None)
            if isinstance(g, nn.Linear) and hasattr(m, "num_experts") and g.out_features == m.num_experts:
                self._gates.append(m)
        if self._gates:
            self.num_experts = int(self._gates[0].num_experts)
            self._load = torch.zeros(self.num_experts, device=self._gates[0].gate.weight.device)
            self.expert_stats = {e: PiscesLxExpertStats(e) for e in range(self.num_experts)}
            self.brownout = PiscesLxBrownoutMoEGrouper(self.num_experts, group_size=max(1, min(4, self.num_experts // 2 or 1)))
        return len(self._gates)

    def brownout_groups(self, load_factor: float = 1.0) -> List[PiscesLxBrownoutExpertGroup]:
        """Applies the brownout at this load factor (above 1 switches more groups off) and returns the groups; later
        ``route`` calls mask the experts of inactive groups."""
        self.brownout.brownout(load_factor)
        self._mask = self.brownout.logit_mask(self._load.device) if not all(self.brownout.active) else None
        return PiscesLxBrownoutExpertGroup.from_grouper(self.brownout)

    # -- adaptation --------------------------------------------------------------------------------------------------------------
    def get_utilization_ratios(self) -> torch.Tensor:
        if self._load is None:
            return torch.ones(max(self.num_experts, 1))
        tot = self._load.sum()
        return torch.where(tot > 0, self._load / tot.clamp_min(1e-20) * self.num_experts, torch.ones_like(self._load))

    def _update_routing_temperature(self) -> float:
        c = self.config
        u = self.get_utilization_ratios()
        skewed = bool(((u > c.utilization_high) | (u < c.utilization_low)).any())
        t = self._adaptive_temp + c.adaptive_temp_step if skewed else max(c.routing_temp, self._adaptive_temp - c.adaptive_temp_step)
        return min(max(t, c.adaptive_temp_floor), max(c.adaptive_temp_cap, c.routing_temp))

    def capacity(self, tokens: int) -> int:
        c = self.config
        base = tokens * c.top_k / max(self.num_experts, 1) * c.capacity_factor * (1.0 + c.capacity_margin) * self._capacity_scale
        return max(int(-(-base // 1)), c.min_capacity)

    def _adaptive_adjust(self) -> None:
        c = self.config
        if c.enable_adaptive_temp and self._calls % max(c.adaptive_temp_interval, 1) == 0:
            self._adaptive_temp = self._update_routing_temperature()
        if c.dynamic_capacity and self._calls % max(c.capacity_update_interval, 1) == 0 and self._load is not None:
            u = self.get_utilization_ratios()
            self._capacity_scale = float(min(2.0, max(1.0, float(u.max()))))       # room for the busiest expert's share
        if self._load is not None:
            self._load.mul_(0.9)                                                   # a window, not an all-time total

    # -- routing -----------------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def route(self, hidden_states: torch.Tensor, layer: int = 0, token_ids: Optional[Sequence[int]] = None,
              token_weights: Optional[torch.Tensor] = None, temperature: Optional[float] = None,
              return_aux_loss: bool = False) -> Dict[str, Any]:
        c = self.config
        if not self._gates:
            raise RuntimeError("set_model(model) first: no gate to route with")
        x = hidden_states.reshape(-1, hidden_states.shape[-1])
        T = x.shape[0]
        key = PiscesLxExpertCacheManager.key_for(token_ids, layer) if (self.cache is not None and token_ids is not None and len(token_ids) == T) else None
        if key is not None:
            e = self.cache.get(key)
            if e is not None:
                return {"expert_indices": e.expert_indices, "routing_probs": e.routing_probs, "routing_temp": self._adaptive_temp,
                        "cache_hit": True, "capacity": self.capacity(T), "dropped": torch.zeros((), dtype=torch.long), "load_balance_loss": None}
        gate = self._gates[min(layer, len(self._gates) - 1)]
        logits = torch.nn.functional.linear(x.to(gate.gate.weight.dtype), gate.gate.weight).float()
        bias = getattr(gate, "expert_bias", None)
        if bias is not None:
            logits = logits + bias.float()
        if getattr(self, "_mask", None) is not None:
            logits = logits + self._mask.to(logits.device)
        temp = float(temperature) if temperature is not None else (self._adaptive_temp if c.routing_strategy != "top_k" else 1.0)
        probs = torch.softmax(logits / temp, -1)
        k = min(c.top_k, probs.shape[-1])
        top_p, top_i = probs.topk(k, -1)
        top_p = top_p / top_p.sum(-1, keepdim=True).clamp_min(1e-20)
        cap, dropped = self.capacity(T), torch.zeros((), dtype=torch.long, device=x.device)
        if c.drop_tokens and c.routing_strategy in ("capacity", "priority"):
            score = top_p.clone()
            if c.routing_strategy == "priority" and token_weights is not None:
                score = score + (token_weights.reshape(-1, 1).float() >= c.priority_threshold).float() * 2.0    # served first
            flat_e, flat_s = top_i.reshape(-1), score.reshape(-1)
            order = torch.argsort(flat_e.double() * 4.0 + (3.0 - flat_s.double().clamp(0, 3)), stable=True)
            counts = torch.bincount(flat_e, minlength=self.num_experts)
            starts = torch.cumsum(counts, 0) - counts
            rank = torch.empty_like(order)
            rank[order] = torch.arange(order.numel(), device=order.device) - starts[flat_e[order]]
            keep = (rank < cap).view(T, k)
            dropped = (~keep).sum()
            top_p = top_p * keep
            top_p = top_p / top_p.sum(-1, keepdim=True).clamp_min(1e-20) * keep.any(-1, keepdim=True)
        counts = torch.bincount(top_i.reshape(-1), minlength=self.num_experts).float()
        if self._load is not None:
            self._load += counts.to(self._load.device)
        self._calls += 1
        self._dropped = self._dropped + dropped.to(self._dropped.device) if self._dropped is not None else dropped.clone()
        self._adaptive_adjust()
        aux = None
        if return_aux_loss:
            f = counts / counts.sum().clamp_min(1.0)
            aux = c.load_balance_alpha * self.num_experts * (f * probs.mean(0)).sum()
        if key is not None:
            self.cache.insert(key, top_i, top_p)
        return {"expert_indices": top_i, "routing_probs": top_p, "routing_temp": temp, "cache_hit": False, "capacity": cap,
                "dropped": dropped, "load_balance_loss": aux}

    def record_execution(self, counts: Sequence[int], latency_ms: float = 0.0) -> None:
        """Per-expert token counts of an executed layer (and its latency) for the statistics."""
        for e, n in enumerate(counts):
            if n and e in self.expert_stats:
                self.expert_stats[e].update(int(n), latency_ms)

    # -- front -------------------------------------------------------------------------------------------------------------------
    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return inputs.get("action", "route") in ("route", "stats", "reset", "share")

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        a = inputs.get("action", "route")
        if a == "route":
            return self.route(inputs["hidden_states"], int(inputs.get("layer", 0)), inputs.get("token_ids"), inputs.get("token_weights"),
                              inputs.get("temperature"), bool(inputs.get("return_aux_loss", False)))
        if a == "share":
            if self.sharing is None:
                return {"shared": None}
            out = self.sharing.share_prefix_kv(inputs["input_ids"])
            self.sharing.register(str(inputs.get("request_id", len(self.sharing._requests))), inputs["input_ids"])
            return {"shared": out}
        if a == "reset":
            self.reset()
            return {}
        return self.get_stats()

    def get_stats(self) -> Dict[str, Any]:
        u = self.get_utilization_ratios()
        return {"calls": self._calls, "routing_temp": self._adaptive_temp, "capacity_scale": self._capacity_scale, "dropped": self.dropped,
                "utilization_max": float(u.max()), "utilization_min": float(u.min()),
                "overutilized": [int(i) for i in (u > self.config.utilization_high).nonzero().flatten()],
                "underutilized": [int(i) for i in (u < self.config.utilization_low).nonzero().flatten()],
                "cache": self.cache.get_stats() if self.cache else None, "sharing": self.sharing.get_stats() if self.sharing else None,
                "experts": {e: {"tokens": s.token_count, "avg_latency_ms": s.avg_latency_ms} for e, s in self.expert_stats.items() if s.call_count}}

    def reset(self) -> None:
        self._adaptive_temp, self._calls, self._capacity_scale, self._dropped, self._mask = self.config.routing_temp, 0, 1.0, None, None
        if self._load is not None:
            self._load.zero_()
        if self.cache is not None:
            self.cache.clear()
        for s in self.expert_stats.values():
            s.token_count = s.call_count = 0
            s.total_latency_ms = 0.0

    cleanup = reset


class PiscesLxMoeRuntime:
    @staticmethod
    def create_moe_runtime_operator(config: Optional[PiscesLxMoERuntimeConfig] = None, model: Optional[nn.Module] = None) -> PiscesLxMoERuntimeOperator:
        op = PiscesLxMoERuntimeOperator(config)
        if model is not None:
            op.set_model(model)
        return op

    @staticmethod
    def from_model(model: nn.Module) -> PiscesLxMoERuntimeOperator:
        cfg = PiscesLxMoERuntimeConfig.from_model_config(getattr(model, "cfg", {}))
        return PiscesLxMoeRuntime.create_moe_runtime_operator(cfg, model)
