"""Gradient-clustering expert initialisation: streamed statistics, sketches, k-means, elbow, displacement by cluster."""
import pytest
import torch
import torch.nn as nn

from pisceslx_b200.models.expert_init import YvClusterInfo, YvGradientClusterInitializer, YvGradientStatistics


def test_streamed_statistics_match_the_buffered_definition():
    torch.manual_seed(0)
    m = nn.Linear(6, 4)
    init = YvGradientClusterInitializer(6, 4, 2)
    grads = []
    for _ in range(5):
        m.zero_grad()
        m(torch.randn(3, 6)).pow(2).sum().backward()
        grads.append(m.weight.grad.flatten().clone())
        st = init.collect_gradients(m, param_filter="weight")
    assert list(st) == ["weight"] and isinstance(st["weight"], YvGradientStatistics) and st["weight"].count == 5
    G = torch.stack(grads)
    assert torch.allclose(st["weight"].mean, G.mean(0), atol=1e-5) and torch.allclose(st["weight"].std, G.std(0), atol=1e-5)
    assert torch.allclose(st["weight"].norm, G.norm(dim=1).mean(), atol=1e-5) and st["weight"].param_shape == (4, 6)
    assert abs(float(st["weight"].direction.norm()) - 1) < 1e-5
    assert len(init._acc["weight"]) == 5 and init._acc["weight"]["mean"].numel() == 24       # fixed footprint, no list of gradients
    init.reset_statistics()
    assert init.gradient_features == {} and init._collection_count == 0


def _stats(groups=3, per=6, shape=(8, 16), seed=0):
    g = torch.Generator().manual_seed(seed)
    out = {}
    bases = [torch.randn(shape, generator=g) for _ in range(groups)]
    for c in range(groups):
        for i in range(per):
            mean = (bases[c] + 0.05 * torch.randn(shape, generator=g)).flatten() * 1e-3
            out[f"g{c}.p{i}"] = YvGradientStatistics(mean, mean.abs() * 0.1, mean.norm(), mean / mean.norm(), 10, shape, f"g{c}.p{i}")
    return out


def test_sketch_preserves_direction_similarity_and_clusters_recover_groups():
    st = _stats()
    init = YvGradientClusterInitializer(16, 8, 6, min_clusters=2, max_clusters=6)
    f, names = init._extract_clustering_features(st)
    assert f.shape == (18, 2 * 128 + 3)
    same = torch.nn.functional.cosine_similarity(f[0, :128], f[1, :128], dim=0)
    diff = torch.nn.functional.cosine_similarity(f[0, :128], f[7, :128], dim=0)
    assert same > 0.9 and abs(float(diff)) < 0.5
    clusters = init.discover_expert_specializations(st, auto_detect_k=False, num_clusters=3, seed=1)
    assert sorted(c.size for c in clusters) == [6, 6, 6] and all(isinstance(c, YvClusterInfo) for c in clusters)
    for c in clusters:
        assert len({n.split(".")[0] for n in c.member_names}) == 1                       # every cluster is one planted group
    assert init.auto_detect_clusters(f, 2, 6) == 3                                        # the elbow is at the planted count
    assert len(init.discover_expert_specializations(st)) == 3
    assert init.get_cluster_summary()["num_clusters"] == 3
    with pytest.raises(ValueError):
        init.discover_expert_specializations({})
    with pytest.raises(ValueError):
        init.discover_expert_specializations(st, auto_detect_k=False)


def test_parameters_of_different_shapes_cluster_together():
    g = torch.Generator().manual_seed(0)
    st = {}
    for i, shape in enumerate([(4, 8), (16, 2), (8, 8), (3, 5)]):
        m = torch.randn(shape, generator=g).flatten()
        st[f"p{i}"] = YvGradientStatistics(m, m.abs(), m.norm(), m / m.norm(), 3, shape, f"p{i}")
    init = YvGradientClusterInitializer(8, 8, 2, min_clusters=2, max_clusters=3)
    cl = init.discover_expert_specializations(st, auto_detect_k=False, num_clusters=2)
    assert sum(c.size for c in cl) == 4


def test_assignment_is_proportional():
    mk = lambda n: YvClusterInfo(0, torch.zeros(1), list(range(n)), [], 0.0, n)
    a = YvGradientClusterInitializer._assign_clusters_to_experts(8, 3, [mk(10), mk(5), mk(1)])
    assert len(a) == 8 and a.count(0) > a.count(1) >= a.count(2) >= 1
    b = YvGradientClusterInitializer._assign_clusters_to_experts(2, 3, [mk(1), mk(9), mk(5)])
    assert b == [1, 2]                                                                 # fewer experts than clusters: the largest clusters


def test_experts_are_displaced_by_cluster_and_stay_functional():
    torch.manual_seed(0)
    st = _stats(groups=2, per=3, shape=(8, 16))
    init = YvGradientClusterInitializer(16, 8, 4, min_clusters=2, max_clusters=2)
    init.discover_expert_specializations(st, auto_detect_k=False, num_clusters=2, seed=0)
    dense = nn.Linear(16, 8)
    experts = nn.ModuleList([nn.Linear(16, 8) for _ in range(4)])
    for e in experts:
        e.load_state_dict(dense.state_dict())                                          # up-cycling: every expert starts as the dense layer
    assign = init.initialize_experts_from_clusters(experts, init_scale=0.05, gradient_stats=st)
    assert sorted(assign) == [0, 0, 1, 1]
    delta = [(e.weight - dense.weight).detach().flatten() for e in experts]
    cos = lambda a, b: float(torch.nn.functional.cosine_similarity(a, b, dim=0))
    i0, i1 = [i for i, a in enumerate(assign) if a == 0], [i for i, a in enumerate(assign) if a == 1]
    assert cos(delta[i0[0]], delta[i0[1]]) > 0.9 and cos(delta[i0[0]], delta[i1[0]]) < 0.5
    rel = float(delta[0].norm() / dense.weight.detach().norm())
    assert 0.03 < rel < 0.08                                                            # a displacement, not an overwrite
    assert all(torch.equal(e.bias, dense.bias) for e in experts)
    member = st[init.clusters[assign[0]].member_names[0]]
    assert cos(delta[0], -member.direction) > 0.9                                       # against the mean gradient
    # different shape and preserve_structure: untouched
    other = nn.ModuleList([nn.Linear(5, 5)])
    w = other[0].weight.clone()
    init.initialize_experts_from_clusters(other, gradient_stats=st)
    assert torch.equal(other[0].weight, w)
    init.initialize_experts_from_clusters(other, gradient_stats=st, preserve_structure=False)
    assert not torch.equal(other[0].weight, w)
    # no clusters: default initialisation
    assert YvGradientClusterInitializer(5, 5, 1).initialize_experts_from_clusters(other) == []
