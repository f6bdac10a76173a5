"""Serving-side runtime helpers (reference opss/infer/moe_runtime.py ``PiscesLxMoERuntimeOperator``: expert cache,
batch sharing, load balancer, the "Moebius" EP<->TP switch heuristic :1563-1625; opss/infer/vllm.py chunked-prefill
scheduler and multi-LoRA registry; opss/infer/tpo.py test-time preference optimisation)."""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch


class PiscesLxExpertCache:
    """LRU residency of expert weights on the device when not all experts fit (host copies stay pinned)."""

    def __init__(self, capacity: int, loader: Callable[[int], Any]):
        self.capacity, self.loader = capacity, loader
        self.resident: "OrderedDict[int, Any]" = OrderedDict()
        self.hits = self.misses = 0

    def get(self, expert: int) -> Any:
        if expert in self.resident:
            self.resident.move_to_end(expert)
            self.hits += 1
            return self.resident[expert]
        self.misses += 1
        w = self.loader(expert)
        self.resident[expert] = w
        if len(self.resident) > self.capacity:
            self.resident.popitem(last=False)
        return w

    def prefetch(self, experts: List[int]) -> None:
        for e in experts:
            self.get(e)


class PiscesLxExpertLoadBalancer:
    """Tracks expert load with an exponential moving average and proposes a placement of experts on ranks that
    evens out the expected tokens per rank (greedy longest-processing-time)."""

    def __init__(self, num_experts: int, decay: float = 0.9):
        self.load = torch.zeros(num_experts)
        self.decay = decay

    def observe(self, counts: torch.Tensor) -> None:
        self.load = self.decay * self.load + (1 - self.decay) * counts.float().cpu()

    def imbalance(self) -> float:
        m = float(self.load.mean())
        return float(self.load.max()) / m if m > 0 else 1.0

    def placement(self, n_ranks: int) -> List[List[int]]:
        per = len(self.load) // n_ranks
        ranks: List[List[int]] = [[] for _ in range(n_ranks)]
        tot = [0.0] * n_ranks
        for e in torch.argsort(self.load, descending=True).tolist():
            r = min((i for i in range(n_ranks) if len(ranks[i]) < per), key=lambda i: tot[i])
            ranks[r].append(e)
            tot[r] += float(self.load[e])
        return ranks


class PiscesLxBatchSharing:
    """Groups requests whose routed expert sets overlap so that one expert-weight read serves several requests."""

    @staticmethod
    def group(expert_sets: List[set], max_group: int = 8) -> List[List[int]]:
        left = list(range(len(expert_sets)))
        groups: List[List[int]] = []
        while left:
            seed = left.pop(0)
            g, union = [seed], set(expert_sets[seed])
            left.sort(key=lambda i: -len(union & expert_sets[i]))
            while left and len(g) < max_group and len(union & expert_sets[left[0]]) > 0:
                i = left.pop(0)
                g.append(i)
                union |= expert_sets[i]
                left.sort(key=lambda j: -len(union & expert_sets[j]))
            groups.append(g)
        return groups


def moebius_choose_layout(tokens_per_step: int, hidden: int, ffn: int, n_experts: int, top_k: int, n_gpus: int,
                          nvlink_gbs: float = 770.0, hbm_gbs: float = 6500.0) -> Dict[str, Any]:
    """EP vs TP for the expert layer of one decode / prefill step, from bytes moved: expert parallelism moves
    activations (2 * tokens * top_k * hidden * 2 B over NVLink) and reads each rank's resident experts once; tensor
    parallelism reads 1/n of every expert on every rank and all-reduces the output."""
    w_bytes = 3 * hidden * ffn * 2
    active = min(n_experts, tokens_per_step * top_k)
    ep_comm = 2 * tokens_per_step * top_k * hidden * 2 * (n_gpus - 1) / n_gpus / n_gpus
    ep_time = ep_comm / (nvlink_gbs * 1e9) + (active / n_gpus) * w_bytes / (hbm_gbs * 1e9)
    tp_comm = 2 * tokens_per_step * hidden * 2 * (n_gpus - 1) / n_gpus
    tp_time = tp_comm / (nvlink_gbs * 1e9) + active * w_bytes / n_gpus / (hbm_gbs * 1e9)
    return {"layout": "ep" if ep_time <= tp_time else "tp", "ep_time_s": ep_time, "tp_time_s": tp_time}


@dataclass
class _PrefillJob:
    request_id: int
    tokens: List[int]
    done: int = 0


class PiscesLxChunkedPrefillScheduler:
    """Token-budget scheduler: every step carries all running decodes (one token each) and fills the remaining budget
    with prompt chunks, so that a long prompt does not stall the decodes (bounded inter-token latency)."""

    def __init__(self, token_budget: int = 2048, chunk: int = 512):
        self.token_budget, self.chunk = token_budget, chunk
        self.prefill: List[_PrefillJob] = []
        self.decoding: List[int] = []

    def add(self, request_id: int, tokens: List[int]) -> None:
        self.prefill.append(_PrefillJob(request_id, tokens))

    def step(self) -> Dict[str, Any]:
        budget = self.token_budget - len(self.decoding)
        chunks: List[Tuple[int, int, int]] = []
        for job in list(self.prefill):
            if budget <= 0:
                break
            n = min(self.chunk, len(job.tokens) - job.done, budget)
            chunks.append((job.request_id, job.done, job.done + n))
            job.done += n
            budget -= n
            if job.done == len(job.tokens):
                self.prefill.remove(job)
                self.decoding.append(job.request_id)
        return {"decode": list(self.decoding), "prefill_chunks": chunks}

    def finish(self, request_id: int) -> None:
        if request_id in self.decoding:
            self.decoding.remove(request_id)


class PiscesLxMultiLoRARegistry:
    """Adapters by name; a batch with mixed adapters applies y += scale * (x A_i^T) B_i^T row-group by row-group."""

    def __init__(self):
        self.adapters: Dict[str, Tuple[torch.Tensor, torch.Tensor, float]] = {}

    def register(self, name: str, a: torch.Tensor, b: torch.Tensor, scale: float = 1.0) -> None:
        self.adapters[name] = (a, b, scale)

    def apply(self, x: torch.Tensor, base_out: torch.Tensor, adapter_names: List[Optional[str]]) -> torch.Tensor:
        out = base_out.clone()
        for name in set(n for n in adapter_names if n is not None):
            rows = torch.tensor([i for i, n in enumerate(adapter_names) if n == name], device=x.device)
            a, b, s = self.adapters[name]
            out[rows] += s * (x[rows] @ a.t().to(x.dtype)) @ b.t().to(x.dtype)
        return out


class PiscesLxTPO:
    """Test-time preference optimisation: sample candidates, score them with a reward function, feed the best and
    the worst back as a textual critique, repeat; returns the best candidate seen."""

    def __init__(self, generate: Callable[[str, int], str], reward: Callable[[str, str], float], n: int = 4, rounds: int = 2):
        self.generate, self.reward, self.n, self.rounds = generate, reward, n, rounds

    def run(self, prompt: str, max_new_tokens: int = 128) -> Dict[str, Any]:
        best, best_r, ctx = None, float("-inf"), prompt
        for _ in range(self.rounds):
            cands = [self.generate(ctx, max_new_tokens) for _ in range(self.n)]
            scored = sorted(((self.reward(prompt, c), c) for c in cands), key=lambda t: t[0])
            if scored[-1][0] > best_r:
                best_r, best = scored[-1]
            ctx = (f"{prompt}\nA weaker answer was:\n{scored[0][1]}\nA stronger answer was:\n{scored[-1][1]}\n"
                   f"Write an answer better than both.\n")
        return {"answer": best, "reward": best_r}


class PiscesLxTriRouteDecision(torch.nn.Module):
    """One small router that decides three things per token from its hidden state (reference
    opss/infer/moe_runtime.py:1391): the attention mode per head (full / sparse / linear), an additive adjustment of the
    expert logits, and the KV-cache bit width for the token (one of ``bit_options``)."""

    def __init__(self, hidden: int, n_head: int, n_experts: int, n_modes: int = 3,
                 bit_options: Tuple[int, ...] = (2, 4, 8, 16), bottleneck: int = 64):
        super().__init__()
        self.n_head, self.n_modes, self.bit_options = n_head, n_modes, tuple(bit_options)
        self.trunk = torch.nn.Sequential(torch.nn.Linear(hidden, bottleneck), torch.nn.GELU())
        self.mode_head = torch.nn.Linear(bottleneck, n_head * n_modes)
        self.expert_head = torch.nn.Linear(bottleneck, n_experts)
        self.bit_head = torch.nn.Linear(bottleneck, len(bit_options))
        torch.nn.init.zeros_(self.expert_head.weight)
        torch.nn.init.zeros_(self.expert_head.bias)

    def forward(self, h: torch.Tensor) -> Dict[str, torch.Tensor]:
        z = self.trunk(h.float())
        mode_logits = self.mode_head(z).view(*h.shape[:-1], self.n_head, self.n_modes)
        bit_logits = self.bit_head(z)
        bits = torch.tensor(self.bit_options, device=h.device)[bit_logits.argmax(-1)]
        return {"attention_mode": mode_logits.argmax(-1), "mode_logits": mode_logits,
                "expert_logit_delta": self.expert_head(z), "kv_bits": bits, "bit_logits": bit_logits}

    def cost(self, out: Dict[str, torch.Tensor], mode_cost: Tuple[float, ...] = (1.0, 0.35, 0.1)) -> torch.Tensor:
        """Differentiable expected compute / memory cost (for training the router against a quality loss)."""
        pm = torch.softmax(out["mode_logits"], -1)
        pb = torch.softmax(out["bit_logits"], -1)
        mc = torch.tensor(mode_cost[: self.n_modes], device=pm.device)
        bc = torch.tensor(self.bit_options, device=pb.device, dtype=torch.float32) / 16.0
        return (pm * mc).sum(-1).mean() + (pb * bc).sum(-1).mean()


class PiscesLxBrownoutMoEGrouper:
    """Experts are clustered into co-activation groups (experts that fire together go together); at run time groups
    whose running importance falls under ``threshold`` are switched off and the router's logits for their experts
    are masked, trading a little quality for throughput under load (reference :1451-1560)."""

    def __init__(self, n_experts: int, group_size: int = 4, threshold: float = 0.3, ema: float = 0.1,
                 min_active_groups: int = 1):
        self.E, self.gs, self.thr, self.ema, self.min_active = n_experts, group_size, threshold, ema, min_active_groups
        self.groups: List[List[int]] = [list(range(i, min(i + group_size, n_experts))) for i in range(0, n_experts, group_size)]
        self.importance = [1.0] * len(self.groups)
        self.active = [True] * len(self.groups)

    def fit(self, idx: torch.Tensor) -> None:
        """Greedy grouping from routing decisions idx [T, k]: repeatedly seed a group with the busiest unassigned
        expert and add the unassigned experts that co-occur with the group most."""
        onehot = torch.zeros(idx.shape[0], self.E).scatter_(1, idx.long().cpu(), 1.0)
        co = onehot.t() @ onehot
        load = co.diagonal().clone()
        co.fill_diagonal_(0)
        free = set(range(self.E))
        groups = []
        while free:
            seed = max(free, key=lambda e: float(load[e]))
            g = [seed]
            free.discard(seed)
            while len(g) < self.gs and free:
                nxt = max(free, key=lambda e: float(co[g, e].sum()))
                g.append(nxt)
                free.discard(nxt)
            groups.append(sorted(g))
        self.groups = groups
        self.importance, self.active = [1.0] * len(groups), [True] * len(groups)

    def observe(self, weights: torch.Tensor, idx: torch.Tensor) -> None:
        """Updates group importance from one batch of routing (share of the routed weight that went to the group,
        relative to a uniform share)."""
        mass = torch.zeros(self.E).scatter_add_(0, idx.flatten().long().cpu(), weights.flatten().float().cpu())
        total = float(mass.sum()) or 1.0
        for g, members in enumerate(self.groups):
            rel = float(mass[members].sum()) / total * len(self.groups)
            self.importance[g] = (1 - self.ema) * self.importance[g] + self.ema * rel

    def brownout(self, load_factor: float) -> List[int]:
        """Switches groups off while the server is overloaded (``load_factor`` > 1 scales the threshold up); returns the
        ids of inactive groups.  The ``min_active_groups`` most important groups always stay on."""
        thr = self.thr * max(0.0, load_factor)
        order = sorted(range(len(self.groups)), key=lambda g: -self.importance[g])
        keep = set(order[: self.min_active])
        self.active = [g in keep or self.importance[g] >= thr for g in range(len(self.groups))]
        return [g for g, a in enumerate(self.active) if not a]

    def logit_mask(self, device=None) -> torch.Tensor:
        """Additive mask [E] for the router logits: -inf on experts of inactive groups."""
        m = torch.zeros(self.E, device=device)
        for g, members in enumerate(self.groups):
            if not self.active[g]:
                m[members] = float("-inf")
        return m


class PiscesLxSemanticCache:
    """Answers cached by the MEANING of the prompt: a prompt whose embedding is within ``threshold`` cosine similarity
    of a stored one gets the stored answer.  ``embed`` maps text to a vector (the engine's ``embeddings``); entries
    leave in least-recently-used order."""

    def __init__(self, embed, capacity: int = 1024, threshold: float = 0.97):
        self.embed, self.capacity, self.threshold = embed, capacity, threshold
        self._keys: List[torch.Tensor] = []
        self._vals: List[str] = []
        self._used: List[int] = []
        self._clock = 0
        self.hits = self.misses = 0

    def _vec(self, text: str) -> torch.Tensor:
        v = torch.as_tensor(self.embed(text), dtype=torch.float32).flatten()
        return v / v.norm().clamp_min(1e-12)

    def get(self, prompt: str) -> Optional[str]:
        self._clock += 1
        if self._keys:
            sims = torch.stack(self._keys) @ self._vec(prompt)
            i = int(sims.argmax())
            if float(sims[i]) >= self.threshold:
                self._used[i] = self._clock
                self.hits += 1
                return self._vals[i]
        self.misses += 1
        return None

    def put(self, prompt: str, answer: str) -> None:
        self._clock += 1
        if len(self._keys) >= self.capacity:
            i = min(range(len(self._used)), key=self._used.__getitem__)
            for lst in (self._keys, self._vals, self._used):
                lst.pop(i)
        self._keys.append(self._vec(prompt))
        self._vals.append(answer)
        self._used.append(self._clock)

    def stats(self) -> Dict[str, float]:
        n = self.hits + self.misses
        return {"entries": len(self._keys), "hits": self.hits, "misses": self.misses, "hit_rate": self.hits / n if n else 0.0}
