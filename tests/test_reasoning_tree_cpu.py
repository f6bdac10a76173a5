"""Level-batched decomposition tree and the dense value-guided thought search."""
import inspect

import torch

from pisceslx_b200.models.reasoning_tree import (YvLatentThoughtTree, YvRecursiveDepthReasoner,
                                                 YvRecursiveReasoningConfig, _YvBidirectionalVerifier,
                                                 _YvSubProblemAggregator, _YvSubProblemDecomposer)

H = 32


def _reasoner(**kw):
    torch.manual_seed(0)
    return YvRecursiveDepthReasoner(YvRecursiveReasoningConfig(hidden_size=H, n_head=4, **kw)).eval()


def test_decomposer_children_and_counts():
    torch.manual_seed(0)
    d = _YvSubProblemDecomposer(H, width=4)
    out = d(torch.randn(3, 5, H), torch.randn(3, 1, H), torch.rand(3, 5, 1))
    assert tuple(out["sub_problem_embeddings"].shape) == (3, 5, 4, H)
    n = out["num_subproblems"]
    assert int(n.min()) >= 2 and int(n.max()) <= 4
    assert torch.equal(out["active"].sum(-1), n)
    kids = out["sub_problem_embeddings"]
    assert float((kids[..., 0, :] - kids[..., 1, :]).abs().max()) > 0     # children are distinct


def test_aggregator_ignores_children_not_in_use():
    torch.manual_seed(0)
    a = _YvSubProblemAggregator(H, 4).eval()
    parent, kids = torch.randn(2, H), torch.randn(2, 4, H)
    act = torch.tensor([[True, True, False, False], [True, True, True, True]])
    base = a(parent, kids, None, act)
    kids2 = kids.clone()
    kids2[0, 2:] = torch.randn(2, H)                                      # unused children of sample 0 change
    again = a(parent, kids2, None, act)
    assert torch.allclose(base[0], again[0], atol=1e-6)
    assert tuple(a(parent, [kids[:, 0], kids[:, 1]]).shape) == (2, H) and a(parent, []) is parent


def test_verifier_score_range():
    torch.manual_seed(0)
    v = _YvBidirectionalVerifier(H)
    fused, s = v(torch.randn(3, H), torch.randn(3, H), torch.randn(3, H))
    assert tuple(fused.shape) == (3, H) and tuple(s.shape) == (3, 1) and bool(((s >= 0) & (s <= 1)).all())


def test_recursive_reasoner_outputs_and_depth_masks():
    r = _reasoner()
    hs = torch.randn(3, 10, H)
    out = r(hs, return_intermediate=True)
    assert tuple(out["reasoning_output"].shape) == (3, H) and tuple(out["reasoning_states"].shape) == (3, 10, H)
    assert tuple(out["confidence"].shape) == (3, 1) and tuple(out["optimal_depth"].shape) == (3,)
    assert int(out["optimal_depth"].min()) >= 1 and int(out["optimal_depth"].max()) <= 6
    assert tuple(out["consistency_scores"].shape) == (3, 1) and out["verification_passed"].dtype == torch.bool
    assert int(out["num_subproblems"].min()) >= 1
    assert "consistency_scores" not in r(hs)
    # depth 0: no decomposition, the root is the only leaf; depth 1: between 2 and width leaves
    pooled = hs.mean(1)
    _, leaves0 = r._solve_tree(pooled, pooled, torch.zeros(3, dtype=torch.long))
    _, leaves1 = r._solve_tree(pooled, pooled, torch.ones(3, dtype=torch.long))
    _, leaves3 = r._solve_tree(pooled, pooled, torch.full((3,), 3))
    assert leaves0.tolist() == [1, 1, 1]
    assert all(2 <= v <= 4 for v in leaves1.tolist()) and bool((leaves3 >= leaves1).all())
    assert all(v <= 4 ** 3 for v in leaves3.tolist())


def test_recursive_reasoner_per_sample_depth_is_independent_of_the_batch():
    r = _reasoner(use_verification=False)
    hs = torch.randn(4, 6, H)
    together = r(hs)["reasoning_output"]
    alone = torch.cat([r(hs[i:i + 1])["reasoning_output"] for i in range(4)])
    assert torch.allclose(together, alone, atol=1e-5)


def test_recursive_reasoner_trains_and_has_no_read_back():
    torch.manual_seed(0)
    r = YvRecursiveDepthReasoner(YvRecursiveReasoningConfig(hidden_size=H, n_head=4, use_aggregation=False)).train()
    out = r(torch.randn(2, 5, H), attention_mask=torch.ones(2, 5), task_type="mathematical")
    (out["reasoning_output"].pow(2).mean() + out["confidence"].mean()).backward()
    assert r.decomposer.child_slots.grad is not None and float(r.decomposer.child_slots.grad.abs().sum()) > 0
    src = inspect.getsource(YvRecursiveDepthReasoner._solve_tree) + inspect.getsource(YvRecursiveDepthReasoner.forward)
    assert ".item()" not in src and ".tolist()" not in src


def test_thought_tree_layout_and_search():
    torch.manual_seed(0)
    t = YvLatentThoughtTree(H, tree_depth=3, beam_width=3).eval()
    assert t.num_nodes == 1 + 3 + 9 + 27 and t.level_start == [0, 1, 4, 13]
    p, c = torch.randn(2, H), torch.randn(2, H)
    states = t.expand_tree(p, c)
    assert tuple(states.shape) == (2, 40, H)
    out = t(p, c, num_simulations=30)
    assert tuple(out["thought_tree_output"].shape) == (2, H) and tuple(out["confidence"].shape) == (2, 1)
    vis = out["visit_counts"]
    assert vis[:, 0].tolist() == [31.0, 31.0]                             # the root is on every path
    assert torch.allclose(vis[:, 1:4].sum(-1), torch.full((2,), 30.0))   # one child of the root per simulation
    assert torch.allclose(vis[:, 13:].sum(-1), torch.full((2,), 30.0))   # one leaf per simulation
    bp = out["best_path"]
    assert bp[:, 0].tolist() == [0, 0] and torch.equal(bp[:, -1], out["best_node"])
    for b in range(2):                                                    # consecutive entries are parent and child
        for u, v in zip(bp[b, :-1].tolist(), bp[b, 1:].tolist()):
            assert v == u or (v - 1) // 3 == u
    assert torch.equal(out["thought_tree_output"], states[torch.arange(2), out["best_node"]])


def test_thought_tree_prefers_the_branch_with_the_highest_values():
    torch.manual_seed(0)
    t = YvLatentThoughtTree(H, tree_depth=2, beam_width=2).eval()
    p, c = torch.randn(1, H), torch.randn(1, H)
    out = t(p, c, num_simulations=64)
    prior = t.value_head(t.expand_tree(p, c)).squeeze(-1)[0]
    vis = out["visit_counts"][0]
    better_child = 1 if float(prior[3:5].max()) > float(prior[5:7].max()) else 2
    assert float(vis[better_child]) >= float(vis[3 - better_child])
    t.train()
    o = t(p, c, num_simulations=4)
    (o["thought_tree_output"].pow(2).sum() + o["policy"].sum()).backward()
    assert t.expand_in.grad is not None and t.thought_encoder[0].weight.grad is not None
