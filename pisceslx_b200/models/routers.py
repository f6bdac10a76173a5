"""Alternative MoE routers (reference model/moe/gate.py: ``YvExpertOrientedRouter`` :1250, ``YvPathMoEGate`` :1756,
``YvPhiBalancing`` :1841, ``YvModalAwareRouter`` :1927, ``YvUltraSparseGate`` :2039; model/moe/layer.py:
``YvExpertChoiceRouter`` :124, ``YvFineGrainedRouter`` :262).

All routers return ``(weights [T, k], indices [T, k], aux)`` like the trunk's gates (``models.moe``), so that the
grouped-GEMM expert layer can take any of them; a slot with weight 0 is an unused slot."""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as F_


def _topk_renorm(probs: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    w, idx = probs.topk(k, -1)
    return w / w.sum(-1, keepdim=True).clamp_min(1e-9), idx


class YvExpertChoiceRouter(nn.Module):
    """Experts pick tokens: each expert takes its ``capacity`` highest-scoring tokens, so load is equal by
    construction.  Returned in token-major form: up to ``max_k`` slots per token (a token can be unpicked)."""

    def __init__(self, hidden: int, n_experts: int, capacity_factor: float = 1.0, max_k: int = 4):
        super().__init__()
        self.w = nn.Parameter(torch.empty(n_experts, hidden).normal_(std=0.02))
        self.cf, self.max_k = capacity_factor, max_k

    def forward(self, x: torch.Tensor):
        T, E = x.shape[0], self.w.shape[0]
        probs = torch.softmax(F_.linear(x, self.w.to(x.dtype)).float(), -1)          # [T, E]
        cap = max(1, min(T, int(self.cf * T * self.max_k / E / 2 + 0.5)))
        top_t = probs.topk(cap, 0).indices                                             # [cap, E]
        picked = torch.zeros(T, E, dtype=torch.bool, device=x.device).scatter_(0, top_t, True)
        w, idx = (probs * picked).topk(min(self.max_k, E), -1)
        aux = {"tokens_per_expert": picked.sum(0), "unrouted": int((~picked.any(-1)).sum())}
        return w, idx, aux


class YvFineGrainedRouter(nn.Module):
    """``n_groups`` groups of ``n_sub`` sub-experts: top-``k`` groups are chosen by the group's best sub-expert score,
    then the best sub-expert inside each chosen group.  Indices are flat: group * n_sub + sub."""

    def __init__(self, hidden: int, n_groups: int, n_sub: int, top_k: int):
        super().__init__()
        self.g, self.s, self.k = n_groups, n_sub, top_k
        self.w = nn.Parameter(torch.empty(n_groups * n_sub, hidden).normal_(std=0.02))

    def forward(self, x: torch.Tensor):
        p = torch.softmax(F_.linear(x, self.w.to(x.dtype)).float(), -1).view(-1, self.g, self.s)
        best, sub = p.max(-1)                                                          # [T, G]
        w, grp = _topk_renorm(best, self.k)
        idx = grp * self.s + torch.gather(sub, 1, grp)
        me = p.view(-1, self.g * self.s).mean(0)
        ce = torch.zeros_like(me).scatter_add_(0, idx.flatten(), torch.ones(idx.numel(), device=x.device)) / idx.numel()
        return w, idx, {"load_balance": self.g * self.s * (me * ce).sum()}


class YvExpertOrientedRouter(nn.Module):
    """Logits = linear gate + ``sim_weight`` * cosine similarity between the token (projected) and a learned
    capability embedding per expert; a running load estimate is subtracted as a correction."""

    def __init__(self, hidden: int, n_experts: int, top_k: int, embed_dim: int = 64, sim_weight: float = 1.0,
                 load_correction: float = 0.1):
        super().__init__()
        self.k, self.sw, self.lc = top_k, sim_weight, load_correction
        self.w = nn.Parameter(torch.empty(n_experts, hidden).normal_(std=0.02))
        self.proj = nn.Parameter(torch.empty(embed_dim, hidden).normal_(std=0.02))
        self.capability = nn.Parameter(torch.randn(n_experts, embed_dim) * 0.1)
        self.register_buffer("load", torch.full((n_experts,), 1.0 / n_experts))

    def forward(self, x: torch.Tensor):
        E = self.w.shape[0]
        t = F.normalize(F_.linear(x, self.proj.to(x.dtype)).float(), dim=-1)
        sim = t @ F.normalize(self.capability.float(), dim=-1).t()
        logits = F_.linear(x, self.w.to(x.dtype)).float() + self.sw * sim - self.lc * E * (self.load - 1.0 / E)
        w, idx = _topk_renorm(torch.softmax(logits, -1), self.k)
        if self.training:
            with torch.no_grad():
                cnt = torch.zeros(E, device=x.device).scatter_add_(0, idx.flatten(), torch.ones(idx.numel(), device=x.device))
                self.load.mul_(0.9).add_(cnt / cnt.sum().clamp_min(1), alpha=0.1)
        return w, idx, {"similarity": sim}


class YvPathMoEGate(nn.Module):
    """One inner gate shared by ``stage_size`` consecutive MoE layers: the first call of a stage routes, the next
    ``stage_size - 1`` calls return the same assignment; no auxiliary loss."""

    def __init__(self, inner: nn.Module, stage_size: int):
        super().__init__()
        self.inner, self.stage_size = inner, stage_size
        self._cached: Optional[Tuple[Any, ...]] = None
        self._calls = 0

    def reset(self) -> None:
        self._cached, self._calls = None, 0

    def forward(self, x: torch.Tensor):
        if self._cached is None or self._calls % self.stage_size == 0 or self._cached[0].shape[0] != x.shape[0]:
            self._cached = tuple(self.inner(x))
            self._calls = 0
        self._calls += 1
        return self._cached


class YvPhiBalancing:
    """Population-level mirror descent on the routing bias: ``pi`` is an EMA of the mean routing probability per
    expert; ``bias -= lr * (pi - 1/E) / sqrt(pi + eps)``, clamped to +-``clamp``."""

    def __init__(self, n_experts: int, lr: float = 0.01, ema: float = 0.99, clamp: float = 2.0, eps: float = 1e-6):
        self.E, self.lr, self.ema, self.clamp, self.eps = n_experts, lr, ema, clamp, eps
        self.pi = torch.full((n_experts,), 1.0 / n_experts)
        self.bias = torch.zeros(n_experts)

    @torch.no_grad()
    def update(self, routing_prob: torch.Tensor) -> torch.Tensor:
        """routing_prob [T, E] (or the per-expert mean [E]); returns the bias to add to the logits."""
        p = routing_prob.float().mean(0) if routing_prob.dim() == 2 else routing_prob.float()
        self.pi = self.pi.to(p.device) * self.ema + p * (1 - self.ema)
        g = self.pi - 1.0 / self.E
        self.bias = (self.bias.to(p.device) - self.lr * g / torch.sqrt(self.pi + self.eps)).clamp(-self.clamp, self.clamp)
        return self.bias


class YvModalAwareRouter(nn.Module):
    """Top-k gate with a learned (expert, modality) affinity bias; tokens of the cross-modal class
    (``modal_id == n_modalities - 1``) always get the ``n_cross`` dedicated experts (the last ones) in their first
    slots."""

    def __init__(self, hidden: int, n_experts: int, top_k: int, n_modalities: int = 4, n_cross: int = 1):
        super().__init__()
        self.k, self.nm, self.nc = top_k, n_modalities, min(n_cross, top_k)
        self.w = nn.Parameter(torch.empty(n_experts, hidden).normal_(std=0.02))
        self.affinity = nn.Parameter(torch.zeros(n_modalities, n_experts))

    def forward(self, x: torch.Tensor, modal_ids: Optional[torch.Tensor] = None):
        E = self.w.shape[0]
        logits = F_.linear(x, self.w.to(x.dtype)).float()
        select = logits
        if modal_ids is not None:
            logits = logits + self.affinity.float()[modal_ids]
            cross = modal_ids == self.nm - 1
            forced = torch.zeros_like(logits)
            forced[:, E - self.nc:] = 1e4
            # the forcing term decides the selection only; the combine weights come from the unforced probabilities
            select = torch.where(cross[:, None], logits + forced, logits)
        idx = select.topk(self.k, -1).indices
        w = torch.gather(torch.softmax(logits, -1), 1, idx)
        return w / w.sum(-1, keepdim=True).clamp_min(1e-9), idx, {}


class YvUltraSparseGate(nn.Module):
    """Tiered sparsity: a small scorer rates each token's importance; tier 1 tokens use 1 expert, tier 2 use 2,
    tier 3 use ``k_max`` (quantile thresholds ``q1 < q2`` over the batch, so the tier shares stay fixed).
    Cross-modal tokens are forced into tier 3.  Unused slots have weight 0."""

    def __init__(self, hidden: int, n_experts: int, tiers: Tuple[int, int, int] = (1, 2, 4), q1: float = 0.90, q2: float = 0.99):
        super().__init__()
        self.tiers, self.q1, self.q2 = tiers, q1, q2
        self.w = nn.Parameter(torch.empty(n_experts, hidden).normal_(std=0.02))
        self.scorer = nn.Sequential(nn.Linear(hidden, 32), nn.GELU(), nn.Linear(32, 1))

    def forward(self, x: torch.Tensor, force_high: Optional[torch.Tensor] = None):
        imp = self.scorer(x.float()).squeeze(-1)
        t1, t2 = torch.quantile(imp.detach(), self.q1), torch.quantile(imp.detach(), self.q2)
        tier_k = torch.full_like(imp, self.tiers[0], dtype=torch.long)
        tier_k[imp > t1] = self.tiers[1]
        tier_k[imp > t2] = self.tiers[2]
        if force_high is not None:
            tier_k[force_high] = self.tiers[2]
        probs = torch.softmax(F_.linear(x, self.w.to(x.dtype)).float(), -1)
        w, idx = probs.topk(self.tiers[2], -1)
        live = torch.arange(self.tiers[2], device=x.device)[None, :] < tier_k[:, None]
        w = w * live
        # the scorer learns through a straight-through factor on the weights
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-9) * (1 + imp - imp.detach())[:, None]
        return w, idx, {"tier_k": tier_k, "mean_k": tier_k.float().mean()}


class YvDGEncoder(nn.Module):
    """Sparse pattern separator (reference model/moe/hicl_router.py:44): project to ``expansion`` x hidden, keep the
    ``sparsity_k`` largest activations per token, L2-normalise."""

    def __init__(self, hidden: int, expansion: int = 4, sparsity_k: int = 32):
        super().__init__()
        self.proj = nn.Parameter(torch.empty(hidden * expansion, hidden).normal_(std=hidden ** -0.5))
        self.k = min(sparsity_k, hidden * expansion)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        z = torch.relu(F_.linear(x, self.proj.to(x.dtype)).float())
        thr = z.topk(self.k, -1).values[..., -1:]
        return F.normalize(torch.where(z >= thr, z, torch.zeros_like(z)), dim=-1)


class YvHiClRouter(nn.Module):
    """Prototype router (reference :89): tokens are sparse-coded by ``YvDGEncoder`` and matched by cosine similarity
    against one prototype per expert; prototypes follow the codes routed to them by an EMA (no gradient), so the
    router has no trained gate matrix."""

    def __init__(self, hidden: int, n_experts: int, top_k: int = 2, dg_expansion: int = 4, dg_sparsity_k: int = 32,
                 momentum: float = 0.99, temperature: float = 0.1):
        super().__init__()
        self.enc = YvDGEncoder(hidden, dg_expansion, dg_sparsity_k)
        self.k, self.m, self.t = top_k, momentum, temperature
        self.register_buffer("prototypes", F.normalize(torch.randn(n_experts, hidden * dg_expansion), dim=-1))

    def forward(self, x: torch.Tensor):
        code = self.enc(x)
        sim = code @ self.prototypes.t()
        w, idx = _topk_renorm(torch.softmax(sim / self.t, -1), self.k)
        if self.training:
            with torch.no_grad():
                top1 = idx[:, 0]
                sums = torch.zeros_like(self.prototypes).index_add_(0, top1, code.detach())
                cnt = torch.zeros(self.prototypes.shape[0], device=x.device).index_add_(0, top1, torch.ones_like(top1, dtype=torch.float))
                seen = cnt > 0
                upd = F.normalize(sums[seen] / cnt[seen, None], dim=-1)
                self.prototypes[seen] = F.normalize(self.m * self.prototypes[seen] + (1 - self.m) * upd, dim=-1)
        return w, idx, {"similarity": sim}


class YvTokenGraphBuilder(nn.Module):
    """Token affinity graph (reference model/moe/graph_of_tokens.py:59): cosine similarity of projected tokens times a
    positional decay exp(-decay |i - j|), thresholded by a learned value; clusters are the connected runs of the
    thresholded chain (adjacent tokens whose affinity passes the threshold share a cluster)."""

    def __init__(self, hidden: int, dim: int = 64, pos_decay: float = 0.1, max_clusters: int = 8):
        super().__init__()
        self.proj = nn.Parameter(torch.empty(dim, hidden).normal_(std=hidden ** -0.5))
        self.threshold = nn.Parameter(torch.tensor(0.3))
        self.decay, self.max_clusters = pos_decay, max_clusters

    def affinity(self, x: torch.Tensor) -> torch.Tensor:
        z = F.normalize(F_.linear(x, self.proj.to(x.dtype)).float(), dim=-1)
        pos = torch.arange(x.shape[0], device=x.device, dtype=torch.float32)
        return (z @ z.t()) * torch.exp(-self.decay * (pos[:, None] - pos[None, :]).abs())

    def clusters(self, x: torch.Tensor) -> torch.Tensor:
        """x [T, H] (one sequence) -> cluster id per token [T], at most ``max_clusters`` clusters."""
        A = self.affinity(x)
        link = torch.diagonal(A, 1) >= self.threshold                    # token t+1 joins token t's cluster
        cid = torch.cat([torch.zeros(1, dtype=torch.long, device=x.device), (~link).long().cumsum(0)])
        return cid.clamp_max(self.max_clusters - 1)


class YvRoMARegularizer(nn.Module):
    """Routing manifold alignment (reference :127): samples whose task embeddings are neighbours should route alike.
    Loss = mean over each sample's ``n_neighbors`` nearest neighbours (in embedding space) of the squared distance
    between their routing distributions."""

    def __init__(self, hidden: int, n_neighbors: int = 8):
        super().__init__()
        self.embed = nn.Linear(hidden, hidden)
        self.n_neighbors = n_neighbors

    def forward(self, pooled_hidden: torch.Tensor, routing_probs: torch.Tensor) -> torch.Tensor:
        e = F.normalize(self.embed(pooled_hidden.float()), dim=-1)
        sim = e @ e.t()
        sim.fill_diagonal_(float("-inf"))
        k = min(self.n_neighbors, max(1, e.shape[0] - 1))
        nbr = sim.topk(k, -1).indices                                    # [N, k]
        diff = routing_probs.float()[:, None, :] - routing_probs.float()[nbr]
        return diff.pow(2).sum(-1).mean()


class YvGraphOfTokensRouter(nn.Module):
    """Two-stage routing (reference :196): tokens are clustered along the sequence; every cluster picks its top-k
    experts from the mean of its tokens' logits, and each token then takes its own softmax weights restricted to its
    cluster's experts, so that a phrase is processed by one set of experts."""

    def __init__(self, hidden: int, n_experts: int, top_k: int = 2, max_clusters: int = 8):
        super().__init__()
        self.graph = YvTokenGraphBuilder(hidden, max_clusters=max_clusters)
        self.w = nn.Parameter(torch.empty(n_experts, hidden).normal_(std=0.02))
        self.k = top_k

    def forward(self, x: torch.Tensor):
        """x [T, H]: the tokens of one sequence, in order."""
        logits = F_.linear(x, self.w.to(x.dtype)).float()
        cid = self.graph.clusters(x)
        n_c = int(cid.max()) + 1
        onehot = F.one_hot(cid, n_c).float()
        mean_logits = (onehot.t() @ logits) / onehot.sum(0).clamp_min(1)[:, None]      # [C, E]
        c_idx = mean_logits.topk(self.k, -1).indices                                    # [C, k]
        idx = c_idx[cid]                                                                # [T, k]
        w = torch.softmax(torch.gather(logits, 1, idx), -1)
        return w, idx, {"clusters": cid, "n_clusters": n_c}
