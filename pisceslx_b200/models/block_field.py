"""Subconscious Block Field: a large set of knowledge blocks of which a few are resident on the device at a time.

Reference: model/core/block_field.py (``YvKnowledgeBlockModule`` :63, ``YvResidentBlockPool`` :154,
``YvSubconsciousBlockField`` :263) and model/core/block_addresser.py (``YvAddressingStatistics`` :54,
``YvResonantTraceAddresser`` :123).  What the parts guarantee, and what the tests check:

* A block is an associative memory read (``M`` rows of width ``d`` behind rank-``r`` query / key projections) that
  emits a BOUNDED modulation: ``|gamma| <= gamma_max`` (scaled tanh) and ``|beta| <= c * |h|`` (direction of the
  read, radius ``c |h|``, smooth at zero).  Hence ``|h' - h| <= alpha (gamma_max + c) |h|`` for ANY block: choosing
  a wrong block can only fail to help.
* The addresser scores a token against one trace per block in a small trace space and picks the arg-max; over a
  sequence a block, once chosen, is kept for at least ``min_dwell`` tokens before another may take over (a rule that
  looks at the past only), because every switch may cost a host-to-device transfer of a whole block.
* The pool keeps ``slots`` blocks on the device (least recently used leaves first; an evicted block is committed back
  to the host store by a callback, so its updates are not lost).  Only resident blocks take part in a step, so only
  they receive gradients.
* Selection ends in an arg-max, which would leave the traces without gradient; the block's contribution is therefore
  multiplied by ``1 + (p_c - detach(p_c))`` (value exactly 1, gradient ``d/dp_c``), so the language-model loss alone
  trains the addresser.

The field is applied ONCE per forward, to the embeddings before the first layer (reference model/core/model.py:2209-2217).
Host storage here is CPU tensors (a state dict per block); the device is whatever the hidden states live on.
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class YvKnowledgeBlockModule(nn.Module):
    def __init__(self, hidden: int, rows: int, rank: int, gamma_max: float = 0.5, beta_bound: float = 0.25,
                 seed: Optional[int] = None):
        super().__init__()
        g = torch.Generator().manual_seed(seed) if seed is not None else None
        self.hidden, self.rows, self.rank = hidden, rows, rank
        self.gamma_max, self.beta_bound, self.beta_eps = gamma_max, beta_bound, 1e-6
        self.memory = nn.Parameter(torch.randn(rows, hidden, generator=g) * 0.02)
        self.query = nn.Parameter(torch.randn(rank, hidden, generator=g) * hidden ** -0.5)
        self.key = nn.Parameter(torch.randn(rank, hidden, generator=g) * hidden ** -0.5)
        self.out = nn.Parameter(torch.randn(hidden, hidden, generator=g) * hidden ** -0.5)
        self.log_temperature = nn.Parameter(torch.zeros(()))

    @property
    def param_count(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def forward(self, h: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """h [..., d] -> (gamma, beta), both [..., d] and bounded as stated in the module docstring."""
        x = h.float()
        mem = F.normalize(self.memory.float(), dim=-1)
        scores = (x @ self.query.float().t()) @ (mem @ self.key.float().t()).t()
        scores = scores * self.log_temperature.exp().clamp_min(1e-3) * self.rank ** -0.5
        read = torch.softmax(scores, -1) @ mem                        # fp32 softmax over the memory rows
        proj = read @ self.out.float().t()
        gamma = self.gamma_max * torch.tanh(proj)
        beta = self.beta_bound * x.norm(dim=-1, keepdim=True) * proj / (proj.norm(dim=-1, keepdim=True) + self.beta_eps)
        return gamma, beta


class YvAddressingStatistics:
    """Switch rate and dwell lengths of the observed selections."""

    def __init__(self) -> None:
        self.tokens = self.switches = 0
        self.runs: List[int] = []

    def record(self, selected: torch.Tensor) -> None:
        """selected [B, T] block ids after the dwell constraint."""
        sel = selected.detach().cpu()
        for row in sel:
            self.tokens += int(row.numel())
            change = (row[1:] != row[:-1]).nonzero().flatten().tolist()
            self.switches += len(change)
            edges = [0] + [c + 1 for c in change] + [int(row.numel())]
            self.runs += [b - a for a, b in zip(edges[:-1], edges[1:])]
        del self.runs[:-4096]

    def switch_rate(self) -> float:
        return self.switches / max(self.tokens - 1, 1)

    def mean_dwell(self) -> float:
        r = self.switch_rate()
        return float("inf") if r == 0 else 1.0 / r

    def tail_dwell(self, q: float = 0.05) -> float:
        """Dwell length below which a fraction ``q`` of the runs fall (runs that end a sequence included)."""
        if not self.runs:
            return float("inf")
        s = sorted(self.runs)
        return float(s[min(len(s) - 1, int(q * len(s)))])

    def snapshot(self) -> Dict[str, float]:
        return {"tokens": float(self.tokens), "switches": float(self.switches), "switch_rate": self.switch_rate(),
                "mean_dwell": self.mean_dwell(), "tail_dwell": self.tail_dwell()}


class YvResonantTraceAddresser(nn.Module):
    """Token -> block by the best-matching trace.  ``project`` maps the hidden state into the trace space; a trace
    is one unit vector per block; ``hysteresis`` is the margin a challenger needs over the block in use in the
    token-by-token (serving) form; ``min_dwell`` is enforced structurally in the sequence form."""

    def __init__(self, hidden: int, n_blocks: int, trace_dim: int = 64, min_dwell: int = 17, hysteresis: float = 0.05,
                 temperature: float = 0.1, seed: Optional[int] = None):
        super().__init__()
        g = torch.Generator().manual_seed(seed) if seed is not None else None
        self.n_blocks, self.trace_dim, self.min_dwell = n_blocks, trace_dim, max(1, int(min_dwell))
        self.hysteresis, self.temperature = hysteresis, temperature
        self.project = nn.Parameter(torch.randn(trace_dim, hidden, generator=g) * hidden ** -0.5)
        self.traces = nn.Parameter(F.normalize(torch.randn(n_blocks, trace_dim, generator=g), dim=-1))
        self.stats = YvAddressingStatistics()
        self._prev: Optional[int] = None

    def scores(self, hidden: torch.Tensor) -> torch.Tensor:
        """[..., d] -> [..., n_blocks] cosine similarities over the temperature."""
        z = F.normalize(hidden.float() @ self.project.float().t(), dim=-1)
        return z @ F.normalize(self.traces.float(), dim=-1).t() / self.temperature

    @torch.no_grad()
    def select(self, hidden: torch.Tensor) -> Tuple[int, torch.Tensor]:
        """One state [d] (decode): stay with the previous block unless another beats it by the hysteresis margin."""
        s = self.scores(hidden.reshape(-1, hidden.shape[-1]).mean(0))
        best = int(s.argmax())
        if self._prev is not None and best != self._prev and float(s[best] - s[self._prev]) < self.hysteresis / self.temperature:
            best = self._prev
        self._prev = best
        return best, s

    def reset(self) -> None:
        self._prev = None

    @staticmethod
    def apply_dwell_constraint(selected: torch.Tensor, min_dwell: int) -> torch.Tensor:
        """[B, T] raw arg-max ids -> ids in which a switch happens only after the block in use has been kept for at
        least ``min_dwell`` tokens.  The rule looks at the past only (the reference merges short runs after the fact,
        which lets a token's block depend on later tokens; this form gives the same dwell floor and is also what
        token-by-token serving can reproduce).  The last run of a row may be shorter: the sequence ended."""
        if min_dwell <= 1:
            return selected
        out = selected.clone()
        for b, row in enumerate(selected.detach().cpu().tolist()):
            cur, run = row[0], 0
            fixed = []
            for v in row:
                if v != cur and run >= min_dwell:
                    cur, run = v, 0
                fixed.append(cur)
                run += 1
            out[b] = torch.tensor(fixed, dtype=selected.dtype, device=selected.device)
        return out

    def select_sequence(self, hidden: torch.Tensor, max_distinct: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """hidden [B, T, d] -> (ids [B, T], scores [B, T, n_blocks] with grad).  The ids obey the dwell floor and, with
        ``max_distinct``, use at most that many different blocks in the whole call (what fits the device at once): a
        request for one block too many is answered with the best-scoring block among those already in use.  Every
        decision depends on earlier tokens of the row (and on earlier rows of the batch) only."""
        s = self.scores(hidden)
        raw = s.argmax(-1)
        if max_distinct is None:
            ids = self.apply_dwell_constraint(raw, self.min_dwell)
        else:
            sc = s.detach().float().cpu()
            used: List[int] = []
            ids = raw.clone()
            for b, row in enumerate(raw.detach().cpu().tolist()):
                cur, run, fixed = None, 0, []
                for t, v in enumerate(row):
                    if cur is None or (v != cur and run >= self.min_dwell):
                        if v not in used:
                            if len(used) < max_distinct:
                                used.append(v)
                            else:
                                v = used[int(sc[b, t, used].argmax())]
                        if v != cur:
                            cur, run = v, 0
                    fixed.append(cur)
                    run += 1
                ids[b] = torch.tensor(fixed, dtype=raw.dtype, device=raw.device)
        self.stats.record(ids)
        return ids, s

    def residence_memory_bytes(self) -> int:
        return (self.traces.numel() + self.project.numel()) * self.traces.element_size()


class YvResidentBlockPool(nn.Module):
    """``slots`` blocks on the device, least recently used first out.  ``install`` returns the id of the block it
    evicted (after handing it to ``evict_callback``), or None."""

    def __init__(self, slots: int):
        super().__init__()
        if slots < 1:
            raise ValueError(f"a pool needs at least one slot, got {slots}")
        self.slots = slots
        self.resident = nn.ModuleDict()                       # str(block id) -> module: parameters are visible to optimizers
        self._order: "OrderedDict[int, None]" = OrderedDict()
        self.stats = {"hits": 0, "misses": 0, "evictions": 0}

    def resident_block_ids(self) -> List[int]:
        return sorted(self._order)

    def slot_module(self, block_id: int) -> Optional[YvKnowledgeBlockModule]:
        key = str(block_id)
        return self.resident[key] if key in self.resident else None

    def touch(self, block_id: int) -> None:
        self._order.pop(block_id, None)
        self._order[block_id] = None

    def install(self, block_id: int, module: YvKnowledgeBlockModule,
                evict_callback: Optional[Callable[[int, YvKnowledgeBlockModule], None]] = None) -> Optional[int]:
        if str(block_id) in self.resident:
            self.stats["hits"] += 1
            self.touch(block_id)
            return None
        self.stats["misses"] += 1
        evicted = None
        if len(self._order) >= self.slots:
            evicted, _ = self._order.popitem(last=False)
            victim = self.resident[str(evicted)]
            if evict_callback is not None:
                evict_callback(evicted, victim)
            del self.resident[str(evicted)]
            self.stats["evictions"] += 1
        self.resident[str(block_id)] = module
        self.touch(block_id)
        return evicted


class YvSubconsciousBlockField(nn.Module):
    """``block_count`` knowledge blocks; ``pool_slots`` of them resident; one addresser.

    Blocks that are not resident live in ``_host`` as CPU state dicts (created on first use from a per-block seed, so
    the field's nominal capacity costs no memory until a block is touched).  ``read_and_modulate`` selects a block per
    token, makes the selected blocks resident (evicting with commit-back), applies each block once to all of its
    tokens and returns the modulated states with diagnostics."""

    def __init__(self, hidden: int, block_count: int = 16, memory_rows: int = 64, rank: int = 32, pool_slots: int = 2,
                 gamma_max: float = 0.5, beta_bound: float = 0.25, alpha: float = 0.1, min_dwell: int = 17,
                 trace_dim: int = 64, seed: int = 0):
        super().__init__()
        self.hidden, self.block_count, self.memory_rows, self.rank = hidden, block_count, memory_rows, rank
        self.gamma_max, self.beta_bound, self.alpha, self.seed = gamma_max, beta_bound, alpha, seed
        self.addresser = YvResonantTraceAddresser(hidden, block_count, trace_dim, min_dwell, seed=seed)
        self.pool = YvResidentBlockPool(pool_slots)
        self._host: Dict[int, Dict[str, torch.Tensor]] = {}
        self._paired = False

    @classmethod
    def from_config(cls, cfg: Any, block_count: Optional[int] = None, memory_rows: Optional[int] = None) -> "YvSubconsciousBlockField":
        return cls(cfg.hidden_size, block_count or cfg.block_count, memory_rows or cfg.block_memory_rows or 64,
                   min(cfg.block_rank, cfg.hidden_size), cfg.block_pool_slots, cfg.block_gamma_max, cfg.block_beta_bound,
                   cfg.block_inject_alpha, cfg.block_min_dwell_tokens)

    # ---- blocks: host store <-> pool -------------------------------------------------------------------------
    def _make_block(self, block_id: int) -> YvKnowledgeBlockModule:
        return YvKnowledgeBlockModule(self.hidden, self.memory_rows, self.rank, self.gamma_max, self.beta_bound,
                                      seed=self.seed * 1_000_003 + block_id + 1)

    def commit_block(self, block_id: int, module: YvKnowledgeBlockModule) -> None:
        """Write a (possibly updated) block back to the host store."""
        self._host[block_id] = {k: v.detach().to("cpu", copy=True) for k, v in module.state_dict().items()}

    def load_block(self, block_id: int) -> YvKnowledgeBlockModule:
        m = self._make_block(block_id)
        if block_id in self._host:
            m.load_state_dict(self._host[block_id])
        return m

    def _ensure_resident(self, block_id: int, device: torch.device) -> YvKnowledgeBlockModule:
        m = self.pool.slot_module(block_id)
        if m is None:
            self.pool.install(block_id, self.load_block(block_id).to(device), evict_callback=self.commit_block)
            m = self.pool.slot_module(block_id)
        else:
            self.pool.touch(block_id)
        return m

    # ---- paired initialisation -----------------------------------------------------------------------------------
    @torch.no_grad()
    def paired_initialize(self, n_blocks: Optional[int] = None) -> None:
        """Point every block's trace at the direction that block responds to: the trace of block i becomes the image,
        in trace space, of the block's dominant query direction (the first right-singular vector of its query / key
        read path), so that at initialisation a token is routed to a block whose memory it actually excites instead
        of to a random one.  Deterministic (blocks are built from their seeds)."""
        n = min(n_blocks or self.block_count, self.block_count)
        P = self.addresser.project.float()
        for i in range(n):
            blk = self.load_block(i)
            direction = torch.linalg.svd(blk.query.float(), full_matrices=False).Vh[0]       # [hidden]
            t = P @ direction
            self.addresser.traces[i].copy_(F.normalize(t, dim=0).to(self.addresser.traces.dtype))
        self._paired = True

    # ---- the read ------------------------------------------------------------------------------------------------
    def relative_perturbation_bound(self) -> float:
        """kappa = alpha (gamma_max + c): |h' - h| <= kappa |h| whatever block was chosen."""
        return self.alpha * (self.gamma_max + self.beta_bound)

    def _straight_through_gate(self, scores: torch.Tensor, selected: torch.Tensor) -> Optional[torch.Tensor]:
        if not (self.training and torch.is_grad_enabled() and scores.requires_grad):
            return None
        p = torch.softmax(scores.float(), -1).gather(-1, selected.unsqueeze(-1).long())
        return (1.0 + (p - p.detach())).reshape(-1, 1)        # exactly 1 in value; carries d/dp of the chosen block

    def read_and_modulate(self, hidden: torch.Tensor) -> Tuple[torch.Tensor, Dict[str, Any]]:
        """hidden [B, T, d] -> (h + alpha (gamma * h + beta) with the per-token block, diagnostics)."""
        if hidden.dim() != 3:
            raise ValueError(f"read_and_modulate expects [B, T, d], got {tuple(hidden.shape)}")
        B, T, d = hidden.shape
        # at most ``slots`` different blocks per call: all of them are resident together, so none is evicted while
        # the autograd graph of this forward still points at its parameters
        selected, scores = self.addresser.select_sequence(hidden, max_distinct=self.pool.slots)
        gate = self._straight_through_gate(scores, selected)
        flat = hidden.reshape(B * T, d)
        ids = selected.reshape(-1)
        served = uniq = torch.unique(ids).tolist()
        out = flat.float()
        for u in served:
            m = self._ensure_resident(int(u), hidden.device)
            pos = (ids == u).nonzero().flatten()
            h_u = flat[pos].float()
            gamma, beta = m(h_u)
            delta = self.alpha * (gamma * h_u + beta)
            if gate is not None:
                delta = gate[pos] * delta
            out = out.index_add(0, pos, delta)
        diag = {"selected": selected, "distinct_blocks": len(uniq), "served_blocks": [int(u) for u in served],
                "resident_blocks": self.pool.resident_block_ids(), **self.addresser.stats.snapshot()}
        return out.to(hidden.dtype).view(B, T, d), diag

    @torch.no_grad()
    def modulate_token(self, hidden: torch.Tensor) -> torch.Tensor:
        """Decode form: one state [..., d]; the addresser's hysteresis decides whether the block changes."""
        block_id, _ = self.addresser.select(hidden)
        m = self._ensure_resident(block_id, hidden.device)
        gamma, beta = m(hidden.float())
        return (hidden.float() + self.alpha * (gamma * hidden.float() + beta)).to(hidden.dtype)

    def measurable_capacity(self) -> Dict[str, float]:
        per_block = float(self.memory_rows * self.hidden + 2 * self.rank * self.hidden + self.hidden * self.hidden + 1)
        resident = float(sum(m.param_count for m in self.pool.resident.values()))
        return {"block_count": float(self.block_count), "params_per_block": per_block,
                "nominal_capacity": per_block * self.block_count, "resident_params": resident,
                "host_blocks": float(len(self._host)), "switch_rate": self.addresser.stats.switch_rate(),
                "mean_dwell": self.addresser.stats.mean_dwell()}

    def commit_all(self) -> None:
        for bid in self.pool.resident_block_ids():
            self.commit_block(bid, self.pool.slot_module(bid))
