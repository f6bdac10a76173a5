"""The research router in full (reference model/moe/gate.py:103-844, ``YvMoEGate``): the standard linear gate plus four
auxiliary routing heads behind learned sparse gates, a modal affinity bias, warm-up phases, history-driven capacity
scaling, adaptive temperature and bias, dynamic and importance-tiered top-k, forced rebalancing and a routing cache
shared by the layers of a stage.  Selected with ``moe_gate_type = "research"``.

What differs from the reference, on purpose:

  * No host synchronisation.  The reference reads the usage statistics back (``.tolist()`` / ``.item()``) to pick a
    temperature target, a bias rate, a top-k and the tokens to move.  Here all of these are tensor expressions with
    ``torch.where`` chains, so the router can sit inside a captured graph and never stalls the stream.
  * Static shapes.  The reference changes ``k`` from call to call.  Here the number of slots per token is fixed
    (``slots``) and a smaller effective ``k`` - from the load state or from the token's importance tier - is a mask on
    the trailing slots followed by a renormalisation, so the dispatch plan keeps its size.
  * The capacity scaling of the scores is folded into the logits as ``log(limit)``, which is the same distribution
    after the softmax, and the selection then runs through the fused gate kernel.
  * The graph-of-tokens head smooths its logits over the *preceding* tokens of the token's cluster only (a running
    mean), so the route of a token never depends on tokens after it.  (The reference builds the clusters and then
    leaves them unused, gate.py:340-345.)
  * The importance projection that picks the tier is trained: the tier mask is a straight-through product of step
    functions, so its gradient is that of the matching sigmoids.

Each auxiliary head is multiplied by a value-neutral straight-through factor of its sparse gate (value exactly 1,
gradient of the sigmoid), and ``sparsity_loss`` - a function of the gate parameters only - is what pushes a gate down;
the trunk folds it into the objective unconditionally (``YvModel.sparsity_objective``).  ``prune_routing_heads`` removes
the heads whose gate has closed."""
from __future__ import annotations

import math
from typing import Optional, Set, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import YvConfig
from ..ops import functional as F_
from ..ops import moe as moe_ops
from .moe import YvStableMoEGate, capacity_mask
from .routers import YvDGEncoder

SPARSE_GATE_INIT = 5.0           # sigmoid(5) = 0.993: every head starts open
HEADS = ("hicl", "got", "soft_moe", "expert_orient")


def straight_through_gate(g: torch.Tensor) -> torch.Tensor:
    """Factor with value exactly 1 whose gradient with respect to ``g`` is that of ``sigmoid(g)``."""
    s = torch.sigmoid(g.float())
    return torch.ones_like(s) + (s - s.detach())


def _step_ste(x: torch.Tensor, tau: float = 0.1) -> torch.Tensor:
    """1[x >= 0] with the gradient of sigmoid(x / tau)."""
    soft = torch.sigmoid(x / tau)
    return (x >= 0).to(soft.dtype) + (soft - soft.detach())


class YvResearchMoEGate(YvStableMoEGate):
    def __init__(self, cfg: YvConfig, num_experts: Optional[int] = None, top_k: Optional[int] = None):
        super().__init__(cfg, num_experts, top_k)
        ex = cfg.extra
        H, E = cfg.hidden_size, self.num_experts
        std = cfg.initializer_range
        # phases
        self.noise_std = float(cfg.moe_noise_std)
        self.random_to_gradient_steps = int(ex.get("moe_random_to_gradient_steps", 2000))
        self.routing_head_warmup_steps = max(self.random_to_gradient_steps, int(ex.get("moe_routing_head_warmup_min", 500)))
        self.logit_warmup_steps = int(ex.get("moe_gate_warmup_steps", 100))
        self.gate_warmup_alpha = float(ex.get("moe_gate_warmup_alpha", 0.05))
        self.current_step = 0
        # temperature
        self.min_temperature = float(ex.get("moe_temperature_min", 1.5))
        self.max_temperature = float(ex.get("moe_temperature_max", 5.0))
        self.long_sequence_temp = float(ex.get("moe_attention_mamba_temp", 0.3))
        self.register_buffer("temperature", torch.tensor(float(ex.get("moe_research_temperature", 3.0))))
        # history
        self.register_buffer("expert_usage", torch.zeros(E, dtype=torch.float32))
        self.register_buffer("total_routed", torch.zeros((), dtype=torch.float32))
        self.expert_capacity_limit = float(ex.get("moe_expert_capacity_limit", 1.2))
        self.load_balance_threshold = float(ex.get("moe_load_balance_threshold", 0.15))
        self.load_balance_alpha = float(cfg.moe_load_balance_alpha)
        self.z_loss_alpha = float(cfg.moe_z_loss_alpha)
        # slots and effective k
        self.k_min = int(ex.get("moe_dynamic_top_k_min", max(1, self.top_k - 1)))
        self.k_max = min(int(ex.get("moe_dynamic_top_k_max", self.top_k)), E)
        self.slots = max(self.top_k, self.k_max)
        self.tier_thresholds = (float(ex.get("ultra_sparse_tier1_threshold", 0.3)),
                                float(ex.get("ultra_sparse_tier2_threshold", 0.8)))
        self.tier_topk = (int(ex.get("ultra_sparse_tier1_topk", 1)), int(ex.get("ultra_sparse_tier2_topk", 2)))
        self.importance_proj = nn.Sequential(nn.Linear(H, max(H // 4, 1), bias=False), nn.SiLU(),
                                             nn.Linear(max(H // 4, 1), 1, bias=False))
        # auxiliary heads
        self.hicl_dg_encoder = YvDGEncoder(H, int(ex.get("hicl_expansion", 4)), int(ex.get("hicl_sparsity_k", 32)))
        self.hicl_prototypes = nn.Parameter(torch.randn(E, H * int(ex.get("hicl_expansion", 4))) * 0.02)
        self.w_hicl = nn.Parameter(torch.tensor(0.1))
        self.got_dim = int(ex.get("graph_of_tokens_dim", 64))
        self.got_embed = nn.Linear(H, self.got_dim, bias=False)
        self.got_threshold = nn.Parameter(torch.tensor(0.3))
        self.got_cluster_proj = nn.Linear(H, E, bias=False)
        self.w_got = nn.Parameter(torch.tensor(0.05))
        self.soft_moe_temperature = float(ex.get("soft_moe_temperature", 1.0))
        self.gate_k = nn.Linear(H, E, bias=False)
        self.gate_v = nn.Linear(H, E, bias=False)
        self.register_buffer("soft_moe_budget", torch.tensor(float(ex.get("soft_moe_mean_k", self.top_k))))
        self.w_soft = nn.Parameter(torch.tensor(0.05))
        D = max(64, H // 64)
        self.expert_embeddings = nn.Parameter(torch.randn(E, D))
        self.input_encoder = nn.Sequential(nn.Linear(H, D, bias=False), nn.SiLU(), nn.Linear(D, D, bias=False))
        self.expert_capability_encoder = nn.Sequential(nn.Linear(D, D, bias=False), nn.SiLU(),
                                                       nn.Linear(D, D, bias=False))
        self.w_expert_orient = nn.Parameter(torch.tensor(0.05))
        for m in (self.got_embed, self.got_cluster_proj, self.gate_k, self.gate_v):
            nn.init.normal_(m.weight, std=std)
        self.sparse_gate_hicl = nn.Parameter(torch.tensor(SPARSE_GATE_INIT))
        self.sparse_gate_got = nn.Parameter(torch.tensor(SPARSE_GATE_INIT))
        self.sparse_gate_soft_moe = nn.Parameter(torch.tensor(SPARSE_GATE_INIT))
        self.sparse_gate_expert_orient = nn.Parameter(torch.tensor(SPARSE_GATE_INIT))
        self.sparsity_reg_weight = float(ex.get("sparsity_reg_weight", 1e-4))
        self._pruned_heads: Set[str] = set()
        # modal affinity
        self.n_modalities = int(ex.get("n_modalities", 5))
        self.expert_modal_affinity = nn.Parameter(torch.zeros(E, self.n_modalities))
        self.affinity_alpha = 1.0
        # routing shared by the layers of one stage
        self.path_stage_size = int(ex.get("path_moe_stage_size", 1))
        self._path_pos = 0
        self._path_cache: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None
        self._path_signature: Optional[Tuple[int, bool]] = None
        self.last_soft_active: Optional[torch.Tensor] = None

    # ---- heads ----------------------------------------------------------------------------------------------------------
    def _head_active(self, name: str) -> bool:
        if name in self._pruned_heads:
            return False
        if not self.training:
            return True
        return self.current_step >= self.routing_head_warmup_steps

    def _got_logits(self, x: torch.Tensor) -> torch.Tensor:
        """Expert logits of the cluster projection, averaged over the preceding tokens of the token's cluster.
        A cluster is a run of adjacent tokens whose embedded cosine similarity passes the learned threshold."""
        raw = self.got_cluster_proj(x).float()                                     # [T, E]
        z = F.normalize(self.got_embed(x).float(), dim=-1)
        link = (z[1:] * z[:-1]).sum(-1) >= self.got_threshold                      # token t+1 continues t's cluster
        start = torch.cat([torch.ones(1, dtype=torch.bool, device=x.device), ~link])
        pos = torch.arange(x.shape[0], device=x.device)
        first = torch.cummax(torch.where(start, pos, torch.zeros_like(pos)), 0).values   # index of the cluster's first token
        csum = raw.cumsum(0)
        before = torch.where(first[:, None] > 0, csum[(first - 1).clamp_min(0)], torch.zeros_like(csum))
        return (csum - before) / (pos - first + 1).to(raw.dtype)[:, None]

    def _auxiliary_logits(self, x: torch.Tensor) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        extra = x.new_zeros((x.shape[0], self.num_experts), dtype=torch.float32)
        soft = None
        if self._head_active("hicl"):
            sim = self.hicl_dg_encoder(x) @ self.hicl_prototypes.float().t()
            extra = extra + (self.w_hicl.float() * straight_through_gate(self.sparse_gate_hicl)) * sim
        if self._head_active("got"):
            extra = extra + (self.w_got.float() * straight_through_gate(self.sparse_gate_got)) * self._got_logits(x)
        if self._head_active("soft_moe"):
            lk, lv = self.gate_k(x).float(), self.gate_v(x).float()
            thr = lk.median(dim=-1, keepdim=True).values
            sw = torch.sigmoid((lk - thr) / self.soft_moe_temperature)
            soft = sw * lv.softmax(-1)
            soft = soft / soft.sum(-1, keepdim=True).clamp_min(1e-8)
            self.last_soft_active = sw
            extra = extra + (self.w_soft.float() * straight_through_gate(self.sparse_gate_soft_moe)) * soft
        if self._head_active("expert_orient"):
            sim = self.input_encoder(x).float() @ self.expert_capability_encoder(self.expert_embeddings).float().t()
            extra = extra + (self.w_expert_orient.float()
                             * straight_through_gate(self.sparse_gate_expert_orient)) * sim
        return extra, soft

    def sparsity_loss(self) -> torch.Tensor:
        """Regulariser over the sparse gates of the heads that are still present; parameters only."""
        gates = [getattr(self, "sparse_gate_" + n) for n in HEADS if n not in self._pruned_heads]
        if not gates:
            return self.gate.weight.new_zeros(())
        return self.sparsity_reg_weight * sum(torch.sigmoid(g.float()) for g in gates)

    @torch.no_grad()
    def prune_routing_heads(self, prune_threshold: float = 0.05) -> Set[str]:
        """After training: drop every head whose gate value fell under ``prune_threshold`` together with its
        parameters.  The standard gate always stays.  Returns the names pruned by this call."""
        owned = {"hicl": ("hicl_dg_encoder", "hicl_prototypes", "w_hicl"),
                 "got": ("got_embed", "got_threshold", "got_cluster_proj", "w_got"),
                 "soft_moe": ("gate_k", "gate_v", "w_soft"),
                 "expert_orient": ("expert_embeddings", "input_encoder", "expert_capability_encoder",
                                   "w_expert_orient")}
        done: Set[str] = set()
        for name in HEADS:
            if name in self._pruned_heads:
                continue
            if float(torch.sigmoid(getattr(self, "sparse_gate_" + name).float())) < prune_threshold:
                self._pruned_heads.add(name)
                done.add(name)
                for attr in owned[name] + ("sparse_gate_" + name,):
                    delattr(self, attr)
        return done

    def drop_heads(self, names) -> None:
        """Remove the named heads without looking at their gates (rebuilding a pruned router before its weights are
        loaded)."""
        for n in names:
            if n in HEADS and n not in self._pruned_heads:
                getattr(self, "sparse_gate_" + n).data.fill_(-30.0)
        self.prune_routing_heads(0.5)

    def get_extra_state(self):
        return {"current_step": self.current_step, "calls": self._calls, "pruned": sorted(self._pruned_heads)}

    def set_extra_state(self, state) -> None:
        self.current_step = int(state.get("current_step", 0))
        self._calls = int(state.get("calls", 0))
        self.drop_heads(state.get("pruned", ()))

    # ---- history-driven state, all on the device ------------------------------------------------------------------------
    def _usage_rate(self) -> torch.Tensor:
        return self.expert_usage / self.total_routed.clamp_min(1.0)

    def _capacity_log_limits(self) -> torch.Tensor:
        lim = (self.expert_capacity_limit * (1.5 - self._usage_rate())).clamp(0.1, 1.0)
        return torch.where(self.total_routed > 0, lim.log(), torch.zeros_like(lim))

    def _load_ratio(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(max / min of the non-zero usage shares, variance of the shares, whether two or more experts were used)."""
        u = self._usage_rate()
        nz = u > 1e-8
        mx = torch.where(nz, u, torch.zeros_like(u)).max()
        mn = torch.where(nz, u, torch.full_like(u, float("inf"))).min()
        ok = nz.sum() >= 2
        ratio = torch.where(ok, mx / (mn + 1e-8), torch.ones_like(mx))
        return ratio, u.var(unbiased=True) if u.numel() > 1 else u.new_zeros(()), ok

    def _effective_k(self) -> torch.Tensor:
        """Scalar tensor: top_k + 1 when the load is badly spread, top_k - 1 when it is well spread, inside
        [k_min, k_max]."""
        base = torch.full((), float(self.top_k), device=self.expert_usage.device)
        if not self.training or self.recomputing:
            return base
        ratio, var, _ = self._load_ratio()
        score = 0.7 * var + 0.3 * (ratio - 1.0)
        k = torch.where(score > self.load_balance_threshold, base + 1,
                        torch.where(score < 0.5 * self.load_balance_threshold, base - 1, base))
        k = torch.where(self.total_routed > 0, k, base)
        return k.clamp(float(self.k_min), float(self.k_max))

    @torch.no_grad()
    def _adapt(self, counts: torch.Tensor, tokens: int) -> None:
        self.expert_usage += counts.float()
        self.total_routed += float(tokens)
        ratio, var, ok = self._load_ratio()
        sig = torch.log(ratio + 1e-8)
        mx_t = torch.full_like(var, self.max_temperature)
        target = torch.where(
            ratio > 50.0, torch.minimum(mx_t, 2.0 + 0.3 * sig),
            torch.where(ratio > 10.0, torch.minimum(mx_t, torch.maximum(1.5 + 15 * var, 1.0 + 0.2 * sig)),
                        torch.where(var > 0.1, torch.minimum(mx_t, torch.maximum(1.0 + 10 * var, 1.0 + 0.1 * sig)),
                                    torch.where(var > 0.05, (1.0 + 5 * var).clamp_min(1.0),
                                                (1.0 - 2 * var).clamp_min(self.min_temperature)))))
        new = (0.8 * self.temperature + 0.2 * target).clamp(self.min_temperature, self.max_temperature)
        self.temperature.copy_(torch.where(ok & (self.total_routed >= 10), new, self.temperature))
        self._calls += 1
        if self._calls % self.bias_update_freq == 0:
            rate = self.bias_update_rate * torch.where(ratio > 20.0, 3.0, torch.where(ratio > 10.0, 2.0,
                                                       torch.where(ratio > 5.0, 1.5, 1.0)))
            dev = 1.0 / self.num_experts - self._usage_rate()
            self.expert_bias.copy_((self.expert_bias + rate * dev).clamp(-2.0, 2.0))

    def _rebalance(self, idx: torch.Tensor, probs: torch.Tensor) -> torch.Tensor:
        """When the max / min usage ratio passes 10, move a fraction (up to 30 %) of the assignments that point at an
        expert with more than twice its share to the token's best-scoring expert with under half its share that the
        token does not already use.  Which assignments move is a fixed hash of (token, slot, step)."""
        ratio, _, ok = self._load_ratio()
        u = self._usage_rate()
        over, under = u > 2.0 / self.num_experts, u < 0.5 / self.num_experts
        rate = ((ratio - 10.0) / 100.0).clamp(0.0, 0.3)
        rate = torch.where(ok & (self.total_routed >= 100) & over.any() & under.any(), rate, torch.zeros_like(rate))
        T, K = idx.shape
        tok = torch.arange(T, device=idx.device, dtype=torch.int64)
        chosen = torch.zeros(T, self.num_experts, dtype=torch.bool, device=idx.device)
        chosen.scatter_(1, idx.long(), True)
        out = idx.clone()
        for s in range(K):
            cur = out[:, s].long()
            h = ((tok * 2654435761 + s * 40503 + self.current_step * 9973) % 1000).float() / 1000.0
            cand_score = probs.masked_fill(chosen | ~under[None, :], float("-inf"))
            best = cand_score.argmax(-1)
            can = torch.isfinite(cand_score.gather(1, best[:, None]).squeeze(1))
            move = over[cur] & (h < rate) & can
            new = torch.where(move, best, cur)
            chosen.scatter_(1, new[:, None], True)
            out[:, s] = new.to(idx.dtype)
        return out

    # ---- forward --------------------------------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, modal_id: Optional[torch.Tensor] = None,
                seq_len: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """x [..., H] -> weights [T, slots] (rows sum to 1), idx [T, slots], routing loss.  ``modal_id`` [T] (or one
        id per sequence) adds each expert's learned affinity for the token's modality."""
        x2 = x.reshape(-1, x.shape[-1])
        T, E, K = x2.shape[0], self.num_experts, self.slots
        live = self.training and not self.recomputing
        if live:
            self.current_step += 1
        if self.path_stage_size > 1:
            sig = (T, self.training)
            if sig != self._path_signature:                 # another batch or phase: the cached rows are not its rows
                self._path_pos, self._path_cache, self._path_signature = 0, None, sig
            if self._path_pos != 0 and self._path_cache is not None:
                self._path_pos = (self._path_pos + 1) % self.path_stage_size
                w, idx, counts = self._path_cache
                self.last_counts = counts
                return w, idx, x2.new_zeros((), dtype=torch.float32)
        logits = F_.linear(x2, self._gate_weight(), out_fp32=True)
        extra, soft = self._auxiliary_logits(x2)
        logits = logits + extra
        if modal_id is not None:
            m = modal_id.reshape(-1).long()
            if m.numel() != T:
                assert T % m.numel() == 0, "modal_id must have one id per token or per sequence"
                m = m.repeat_interleave(T // m.numel())
            logits = logits + self.affinity_alpha * self.expert_modal_affinity.float().t()[m]
        logits = logits + self.expert_bias
        if live and self.current_step < self.logit_warmup_steps:
            logits = logits * (self.gate_warmup_alpha
                               + (1.0 - self.gate_warmup_alpha) * self.current_step / self.logit_warmup_steps)
        if live and self.noise_std > 0:
            logits = logits + torch.randn_like(logits) * self.noise_std
        temp = self.temperature * (self.long_sequence_temp if (seq_len or 0) >= 8192 else 1.0)
        logits = logits / temp.clamp(0.1, self.max_temperature)
        raw_logits = logits
        if live:
            logits = logits + self._capacity_log_limits()
        random_phase = live and self.current_step <= self.random_to_gradient_steps
        if random_phase:
            _, idx, counts, _ = moe_ops.gate_topk(torch.rand_like(logits), None, K, True, 1)
            weights = torch.full((T, K), 1.0 / K, device=x2.device, dtype=torch.float32)
            probs = torch.softmax(logits, -1)
        else:
            weights, idx, counts, probs = moe_ops.gate_topk(logits, None, K, True, 1)
            if live:
                moved = self._rebalance(idx, probs)
                if self.num_experts > 1:
                    full = torch.softmax(logits, -1)
                    sel = full.gather(1, moved.long())
                    weights = torch.where(moved == idx, weights, sel)            # a moved slot takes its own score
                    weights = weights / weights.sum(-1, keepdim=True).clamp_min(1e-20)
                    idx = moved
                    counts = torch.bincount(idx.flatten().long(), minlength=E).to(counts.dtype)
        # effective k: trailing slots are masked out, by the load state and by the token's importance tier
        slot = torch.arange(K, device=x2.device, dtype=torch.float32)
        imp = torch.sigmoid(self.importance_proj(x2).float()).squeeze(-1)                           # [T]
        t1, t2 = self.tier_thresholds
        k1, k2 = self.tier_topk
        tier = torch.ones(T, K, device=x2.device, dtype=torch.float32)
        tier = tier * torch.where(slot[None, :] >= k1, _step_ste(imp - t1)[:, None], torch.ones_like(tier))
        tier = tier * torch.where(slot[None, :] >= k2, _step_ste(imp - t2)[:, None], torch.ones_like(tier))
        keep = tier * (slot[None, :] < self._effective_k()).float()
        keep = torch.cat([torch.ones(T, 1, device=x2.device), keep[:, 1:]], 1)       # the first slot always stays
        weights = weights * keep
        weights = weights / weights.sum(-1, keepdim=True).clamp_min(1e-20)
        if self.drop_tokens:
            weights = capacity_mask(weights, idx, probs, self.capacity(T), counts)
        # losses
        p = torch.softmax(raw_logits.float(), -1)
        ideal = 1.0 / E
        lb = self.load_balance_alpha * (p.mean(0) - ideal).pow(2).sum()
        if self.training:
            actual = counts.float() / max(T * K, 1)
            lb = 0.5 * lb + 0.5 * self.load_balance_alpha * (actual - ideal).pow(2).sum()
        over = torch.relu(self._usage_rate() - self.expert_capacity_limit).pow(2).sum()
        z = self.z_loss_alpha * torch.nan_to_num(raw_logits.float(), nan=0.0, posinf=1e4, neginf=-1e4).pow(2).mean()
        aux = lb + 0.005 * over + z
        if soft is not None and self.last_soft_active is not None:
            aux = aux + 0.01 * (self.last_soft_active.sum(-1).mean() - self.soft_moe_budget).pow(2)
        self.last_counts = counts
        if live and not random_phase:
            self._adapt(counts, T)
        elif live:
            with torch.no_grad():
                self.total_routed += float(T)
        if self.path_stage_size > 1:
            self._path_cache = (weights.detach(), idx, counts)      # later calls reuse the route, not its graph
            self._path_pos = (self._path_pos + 1) % self.path_stage_size
        return weights, idx, aux
