"""Tree-shaped latent reasoning (reference model/reasoning/reasoner/recursive_depth.py:117-1452): recursive
decomposition of a problem into sub-problems with aggregation and bidirectional verification, and a value-guided search
over a tree of thoughts.

The reference walks both trees in Python, one sample and one node at a time, and reads a scalar back from the device
at every node (``.item()`` for the number of children, the depth, the value of a node).  Both trees here are DENSE and
LEVEL-BATCHED:

  * Decomposition: level ``l`` holds ``[B, width**l, H]`` node embeddings; one call of the decomposer produces all
    children of a level, one call of the reasoning block solves all leaves (siblings attend to one another), one call
    of the aggregator folds a level into its parents.  How many children a node uses (2..width) and how deep a sample
    goes are masks and ``torch.where`` selections, so shapes are static and nothing is read back.
  * Search: the full ``beam_width``-ary tree of depth ``tree_depth`` is expanded once, level by level (a few hundred
    nodes), its values are one matrix ``[B, nodes]``, and every simulation is index arithmetic on ``[B]`` vectors:
    descend by UCB with gathers, back the leaf value up along the ancestor chain with scatters.  All samples of the
    batch search at once."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .compat import YvCrossAttention
from .reasoning_engine import _ReasoningLayer


@dataclass
class YvRecursiveReasoningConfig:
    hidden_size: int = 2048
    max_depth: int = 10            # bound of the predicted depth
    min_depth: int = 1
    width: int = 4                 # children per node
    temperature: float = 0.7
    use_aggregation: bool = True
    use_verification: bool = True
    threshold_complexity: float = 0.5
    early_exit_threshold: float = 0.9
    tree_levels: int = 3           # levels of the dense tree; a predicted depth beyond it adds refinement passes
    n_head: int = 8


def _heads(hidden: int, want: int) -> int:
    for h in range(min(want, hidden), 0, -1):
        if hidden % h == 0:
            return h
    return 1


class _YvSubProblemDecomposer(nn.Module):
    """Node [.., H] + context + complexity -> ``width`` child embeddings and how many of them are used (2..width).
    Children differ by a learned offset per child slot (the reference separates them with random noise only)."""

    def __init__(self, hidden_size: int, width: int = 4):
        super().__init__()
        H = hidden_size
        self.width = width
        self.decomposition_net = nn.Sequential(nn.Linear(3 * H, H), nn.GELU(), nn.Linear(H, H), nn.LayerNorm(H))
        self.child_proj = nn.Linear(H, H)
        self.child_slots = nn.Parameter(torch.randn(width, H) * 0.02)
        self.num_subproblems_predictor = nn.Linear(H, width - 1 if width > 1 else 1)

    def forward(self, problem_embedding: torch.Tensor, context: torch.Tensor, complexity_score: torch.Tensor,
                noise_scale: float = 0.0) -> Dict[str, torch.Tensor]:
        """problem_embedding [..., H]; context broadcastable to it; complexity_score [..., 1] or a scalar."""
        c = complexity_score if torch.is_tensor(complexity_score) else problem_embedding.new_tensor(complexity_score)
        feats = self.decomposition_net(torch.cat([problem_embedding, context.expand_as(problem_embedding),
                                                  problem_embedding * c], -1))
        kids = feats.unsqueeze(-2) + self.child_proj(feats).unsqueeze(-2) * 0.5 + self.child_slots.to(feats.dtype)
        if noise_scale > 0:
            kids = kids + torch.randn_like(kids) * noise_scale
        n = 2 + self.num_subproblems_predictor(problem_embedding).float().argmax(-1) if self.width > 1 else \
            torch.ones(problem_embedding.shape[:-1], dtype=torch.long, device=problem_embedding.device)
        n = n.clamp(max=self.width)
        active = torch.arange(self.width, device=kids.device) < n.unsqueeze(-1)                    # [..., width]
        return {"sub_problem_embeddings": kids, "num_subproblems": n, "active": active, "decomposed_features": feats}


class _YvRecursiveReasoningBlock(nn.Module):
    """Two attention layers over a set of nodes [N, L, H] (siblings, or the tokens of a sequence) + a projection."""

    def __init__(self, hidden_size: int, num_layers: int = 2, n_head: int = 8, causal: bool = False):
        super().__init__()
        H = hidden_size
        self.reasoning_layers = nn.ModuleList([_ReasoningLayer(H, _heads(H, n_head), causal) for _ in range(num_layers)])
        self.output_proj = nn.Sequential(nn.Linear(H, H), nn.LayerNorm(H), nn.GELU(), nn.Linear(H, H))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for layer in self.reasoning_layers:
            x = layer(x)
        return self.output_proj(x)


class _YvSubProblemAggregator(nn.Module):
    """Parent [N, H] + children [N, W, H] (+ mask of the children in use) -> parent solution: the parent attends to
    its children, the attended value is mixed with their (masked, optionally weighted) mean and gated against the
    parent itself."""

    def __init__(self, hidden_size: int, num_heads: int = 8):
        super().__init__()
        H = hidden_size
        self.attention = YvCrossAttention(H, H, _heads(H, num_heads))
        self.gate_net = nn.Sequential(nn.Linear(2 * H, H), nn.Sigmoid())
        self.output_proj = nn.Sequential(nn.Linear(H, H), nn.LayerNorm(H))

    def forward(self, problem_embedding: torch.Tensor, sub_problem_results: Any,
                weights: Optional[torch.Tensor] = None, active: Optional[torch.Tensor] = None) -> torch.Tensor:
        if isinstance(sub_problem_results, (list, tuple)):
            if len(sub_problem_results) == 0:
                return problem_embedding
            sub_problem_results = torch.stack(list(sub_problem_results), 1)
        kids = sub_problem_results                                                                   # [N, W, H]
        N, W, H = kids.shape
        if active is None:
            active = torch.ones(N, W, dtype=torch.bool, device=kids.device)
        w = torch.ones(N, W, device=kids.device) if weights is None else torch.softmax(weights.float(), -1).expand(N, W)
        w = w * active.float()
        w = (w / w.sum(-1, keepdim=True).clamp_min(1e-8)).to(kids.dtype)
        masked = kids * active.unsqueeze(-1).to(kids.dtype)              # children not in use contribute nothing
        attended = self.attention(problem_embedding.unsqueeze(1), masked).squeeze(1)
        agg = (w.unsqueeze(-1) * kids).sum(1) + 0.3 * attended
        gate = self.gate_net(torch.cat([problem_embedding, agg], -1))
        return self.output_proj(agg * gate + problem_embedding * (1 - gate))


class _YvBidirectionalVerifier(nn.Module):
    """Forward pass hypothesis -> conclusion, backward pass evidence -> hypothesis, a consistency score in [0, 1] from
    (hypothesis, forward, backward) and the fusion of both passes."""

    def __init__(self, hidden_size: int):
        super().__init__()
        H = hidden_size
        mk = lambda: nn.Sequential(nn.Linear(2 * H, H), nn.GELU(), nn.Linear(H, H), nn.LayerNorm(H))
        self.forward_reasoner, self.backward_reasoner = mk(), mk()
        self.consistency_checker = nn.Sequential(nn.Linear(3 * H, H), nn.GELU(), nn.Linear(H, max(H // 2, 1)), nn.GELU(),
                                                 nn.Linear(max(H // 2, 1), 1), nn.Sigmoid())
        self.fusion_proj = nn.Sequential(nn.Linear(2 * H, H), nn.LayerNorm(H))

    def forward(self, hypothesis: torch.Tensor, evidence: torch.Tensor, context: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        fwd = self.forward_reasoner(torch.cat([hypothesis, context.expand_as(hypothesis)], -1))
        bwd = self.backward_reasoner(torch.cat([evidence, fwd], -1))
        score = self.consistency_checker(torch.cat([hypothesis, fwd, bwd], -1))
        return self.fusion_proj(torch.cat([fwd, bwd], -1)), score


class YvRecursiveDepthReasoner(nn.Module):
    """Problem -> tree of sub-problems -> solved leaves -> aggregated back to the root -> verified.

    ``forward(hidden_states [B, S, H])`` returns ``reasoning_output`` [B, H] (the root solution), ``reasoning_states``
    [B, S, H] (the input with the solution mixed in by the confidence), ``confidence`` [B, 1], ``complexity`` [B, 1],
    ``optimal_depth`` [B] and ``num_subproblems`` [B] (leaves in use)."""

    TASK_DEPTH_CAP = {"planning": 8, "mathematical": 10}

    def __init__(self, config: Optional[YvRecursiveReasoningConfig] = None):
        super().__init__()
        self.config = config = config or YvRecursiveReasoningConfig()
        H = self.hidden_size = config.hidden_size
        self.max_depth, self.min_depth, self.width = config.max_depth, config.min_depth, config.width
        self.levels = max(1, min(config.tree_levels, config.max_depth))
        self.decomposer = _YvSubProblemDecomposer(H, self.width)
        self.recursive_block = _YvRecursiveReasoningBlock(H, 2, config.n_head)
        self.aggregator = _YvSubProblemAggregator(H, config.n_head) if config.use_aggregation else None
        self.verifier = _YvBidirectionalVerifier(H) if config.use_verification else None
        g = lambda i, o: (nn.Linear(i, o), nn.GELU())
        self.complexity_predictor = nn.Sequential(*g(H, max(H // 2, 1)), *g(max(H // 2, 1), max(H // 4, 1)),
                                                  nn.Linear(max(H // 4, 1), 1), nn.Sigmoid())
        self.confidence_predictor = nn.Sequential(*g(3 * H, H), *g(H, max(H // 2, 1)), nn.Linear(max(H // 2, 1), 1),
                                                  nn.Sigmoid())
        self.depth_predictor = nn.Sequential(*g(H, max(H // 2, 1)), nn.Linear(max(H // 2, 1), self.max_depth))
        self._init_weights()

    def _init_weights(self) -> None:
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.xavier_uniform_(m.weight)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

    @staticmethod
    def _pool(hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor]) -> torch.Tensor:
        if attention_mask is None:
            return hidden_states.mean(1)
        m = attention_mask.to(hidden_states.dtype).unsqueeze(-1)
        return (hidden_states * m).sum(1) / m.sum(1).clamp_min(1.0)

    def _calculate_problem_complexity(self, hidden_states: torch.Tensor,
                                      attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self._pool(hidden_states, attention_mask) if hidden_states.dim() == 3 else hidden_states
        return self.complexity_predictor(x)

    def _predict_optimal_depth(self, pooled: torch.Tensor, complexity: torch.Tensor, cap: int) -> torch.Tensor:
        """[B] long: 0.6 x the expected depth of the predictor + 0.4 x (complexity x max depth), inside
        [min_depth, cap]."""
        p = torch.softmax(self.depth_predictor(pooled).float(), -1)
        expected = (p * torch.arange(1, self.max_depth + 1, device=p.device)).sum(-1)
        base = (complexity.float().squeeze(-1) * self.max_depth).floor().clamp(self.min_depth, self.max_depth)
        return (0.6 * expected + 0.4 * base).floor().clamp(self.min_depth, cap).long()

    def _solve_tree(self, root: torch.Tensor, context: torch.Tensor, depth: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """root [B, H], context [B, H], depth [B] -> (root solution [B, H], leaves in use [B])."""
        B, H = root.shape
        W, L = self.width, self.levels
        nodes, actives = [root.unsqueeze(1)], []                                   # level l: [B, W**l, H]
        alive = [torch.ones(B, 1, dtype=torch.bool, device=root.device)]           # node exists for this sample
        for l in range(L):
            cur = nodes[-1]
            d = self.decomposer(cur, context.unsqueeze(1), self.complexity_predictor(cur),
                                0.1 * (1 - l / L) if self.training else 0.0)
            expand = alive[-1] & (depth > l).unsqueeze(1)                          # deeper than this level?
            act = d["active"] & expand.unsqueeze(-1)                               # [B, n, W]
            nodes.append(d["sub_problem_embeddings"].reshape(B, -1, H))
            actives.append(act)
            alive.append(act.reshape(B, -1))
        # every node is solved together with its siblings; the root forms a group of one
        solved = []
        for l, n in enumerate(nodes):
            grp = n.reshape(-1, W if l > 0 else 1, H)
            solved.append(self.recursive_block(grp).reshape(B, -1, H))
        # fold the levels upwards: a node with children in use takes their aggregate, otherwise its own solution
        up = solved[L]
        for l in range(L - 1, -1, -1):
            kids = up.reshape(-1, W, H)
            act = actives[l].reshape(-1, W)
            own = solved[l].reshape(-1, H)
            if self.aggregator is not None:
                agg = self.aggregator(own, kids, None, act)
            else:
                wt = act.to(kids.dtype).unsqueeze(-1)
                agg = (kids * wt).sum(1) / wt.sum(1).clamp_min(1.0)
            up = torch.where(act.any(-1, keepdim=True), agg, own).reshape(B, -1, H)
        leaves = alive[L].sum(-1)
        for l in range(L - 1, -1, -1):                                             # nodes that stopped early are leaves too
            leaves = leaves + (alive[l] & ~actives[l].any(-1)).sum(-1)
        return up.squeeze(1), leaves

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                task_type: str = "reasoning", return_intermediate: bool = False) -> Dict[str, Any]:
        B, S, H = hidden_states.shape
        cap = min(self.max_depth, self.TASK_DEPTH_CAP.get(task_type, 6))
        pooled = self._pool(hidden_states, attention_mask)
        complexity = self.complexity_predictor(pooled)
        depth = self._predict_optimal_depth(pooled, complexity, cap)
        solution, leaves = self._solve_tree(pooled, pooled, depth)
        passes = ((depth - 1) // self.levels).clamp_min(0)                         # depth beyond the tree: refine again
        for r in range(int(math.ceil(max(cap - self.levels, 0) / self.levels))):
            again, _ = self._solve_tree(solution, pooled, depth - (r + 1) * self.levels)
            solution = torch.where((passes > r).unsqueeze(-1), again, solution)
        out: Dict[str, Any] = {}
        if self.verifier is not None:
            evidence = self._pool(self.recursive_block(hidden_states + solution.unsqueeze(1)), attention_mask)
            solution, consistency = self.verifier(solution, evidence, pooled)
            out["consistency_scores"] = consistency
            out["verification_passed"] = consistency.squeeze(-1) > self.config.threshold_complexity
        confidence = self.confidence_predictor(torch.cat([solution, pooled, solution - pooled], -1))
        out.update(reasoning_output=solution, confidence=confidence, complexity=complexity, optimal_depth=depth,
                   num_subproblems=leaves,
                   reasoning_states=hidden_states + confidence.unsqueeze(1).to(hidden_states.dtype) * solution.unsqueeze(1))
        if not return_intermediate:
            out.pop("consistency_scores", None)
        return out


class YvLatentThoughtTree(nn.Module):
    """Value-guided search over a dense tree of thoughts.  ``forward(problem [B, H], context [B, H])`` returns the
    embedding of the best-valued node per sample (``thought_tree_output`` [B, H]), its value, a confidence relative to
    the best sample of the batch, the visit counts [B, nodes] and the best node's path (node indices, root first)."""

    def __init__(self, hidden_size: int, tree_depth: int = 5, beam_width: int = 3, exploration_weight: float = 1.414):
        super().__init__()
        H = hidden_size
        self.hidden_size, self.tree_depth, self.beam_width, self.c = H, tree_depth, beam_width, exploration_weight
        self.thought_encoder = nn.Sequential(nn.Linear(2 * H, H), nn.GELU(), nn.LayerNorm(H))
        self.value_head = nn.Linear(H, 1)
        self.policy_head = nn.Linear(H, H)
        # the beam_width expansion networks as two batched weights
        self.expand_in = nn.Parameter(torch.empty(beam_width, H, 2 * H))
        self.expand_in_bias = nn.Parameter(torch.zeros(beam_width, 2 * H))
        self.expand_out = nn.Parameter(torch.empty(beam_width, 2 * H, H))
        self.expand_out_bias = nn.Parameter(torch.zeros(beam_width, H))
        for w in (self.expand_in, self.expand_out):
            for i in range(beam_width):
                nn.init.xavier_uniform_(w[i])
        self.level_start = [0]
        for l in range(tree_depth):
            self.level_start.append(self.level_start[-1] + beam_width ** l)
        self.num_nodes = self.level_start[-1] + beam_width ** tree_depth

    def _ucb_score(self, node_value: torch.Tensor, visit_count: torch.Tensor, parent_visits: torch.Tensor) -> torch.Tensor:
        explore = self.c * torch.sqrt(torch.log(parent_visits.clamp_min(1.0)) / visit_count.clamp_min(1e-8))
        return torch.where(visit_count > 0, node_value + explore, torch.full_like(node_value, float("inf")))

    def expand_tree(self, problem_embedding: torch.Tensor, context: torch.Tensor) -> torch.Tensor:
        """All node embeddings [B, nodes, H] in breadth-first order (children of node i are i * W + 1 .. i * W + W)."""
        root = self.thought_encoder(torch.cat([problem_embedding, context], -1))
        levels = [root.unsqueeze(1)]
        for _ in range(self.tree_depth):
            cur = levels[-1]                                                        # [B, n, H]
            hid = F.gelu(torch.einsum("bnh,whk->bnwk", cur, self.expand_in.to(cur.dtype)) + self.expand_in_bias.to(cur.dtype))
            kid = torch.einsum("bnwk,wkh->bnwh", hid, self.expand_out.to(cur.dtype)) + self.expand_out_bias.to(cur.dtype)
            levels.append((cur.unsqueeze(2) + 0.1 * kid).reshape(cur.shape[0], -1, cur.shape[-1]))
        return torch.cat(levels, 1)

    def forward(self, problem_embedding: torch.Tensor, context: torch.Tensor, num_simulations: int = 100) -> Dict[str, Any]:
        B, W, D = problem_embedding.shape[0], self.beam_width, self.tree_depth
        dev = problem_embedding.device
        states = self.expand_tree(problem_embedding, context)
        prior = self.value_head(states).squeeze(-1).float()                         # [B, N] the network's value
        with torch.no_grad():
            values, visits = prior.detach().clone(), torch.zeros_like(prior)
            visits[:, 0] = 1.0
            rows = torch.arange(B, device=dev)
            kid_off = torch.arange(1, W + 1, device=dev)
            for _ in range(num_simulations):
                node = torch.zeros(B, dtype=torch.long, device=dev)
                path = [node]
                for _l in range(D):
                    kids = node.unsqueeze(1) * W + kid_off                          # [B, W]
                    ucb = self._ucb_score(values.gather(1, kids), visits.gather(1, kids),
                                          visits.gather(1, node.unsqueeze(1)))
                    node = kids.gather(1, ucb.argmax(-1, keepdim=True)).squeeze(1)
                    path.append(node)
                leaf_value = prior[rows, node]
                for n in path:                                                      # running mean along the chain
                    v, c = values[rows, n], visits[rows, n]
                    values[rows, n] = torch.where(c > 0, (v * c + leaf_value) / (c + 1), leaf_value)
                    visits[rows, n] = c + 1
            searched = torch.where(visits > 0, values, torch.full_like(values, float("-inf")))
            best = searched.argmax(-1)                                              # [B]
            chain = [best]
            for _l in range(D):
                chain.append(torch.where(chain[-1] > 0, (chain[-1] - 1) // W, chain[-1]))
            best_path = torch.stack(chain[::-1], 1)                                 # root first; the root repeats if short
            best_value = searched[rows, best]
            top = best_value.max()
            confidence = torch.where(top > 0, (best_value / (top + 1e-8)).clamp(max=1.0), torch.ones_like(best_value))
        out_emb = states[rows, best]
        return {"thought_tree_output": out_emb, "confidence": confidence.unsqueeze(-1), "best_values": best_value,
                "best_node": best, "best_path": best_path, "visit_counts": visits, "node_values": values,
                "policy": self.policy_head(out_emb), "tree_depth": D, "beam_width": W, "num_nodes": self.num_nodes}


# name of the reference, for code that imports it from here (the prompt-level tree search is models.reasoning.YvThoughtTreeReasoner)
YvThoughtTreeReasoner = YvLatentThoughtTree
