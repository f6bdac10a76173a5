"""Fused MoE dispatch front: stacked SwiGLU path and sort-based path against the per-expert mask loop."""
import pytest
import torch
import torch.nn as nn

from pisceslx_b200.models.moe import YvSwiGLUExpert
from pisceslx_b200.serve.fused_moe import PiscesLxFusedMoe, PiscesLxFusedMoEDispatch


def _route(T, E, k, seed=0):
    g = torch.Generator().manual_seed(seed)
    p = torch.softmax(torch.randn(T, E, generator=g), -1)
    w, i = p.topk(k, -1)
    return w / w.sum(-1, keepdim=True), i


def test_generic_experts_match_the_mask_loop_and_skip_idle_experts():
    torch.manual_seed(0)
    experts = nn.ModuleList([nn.Sequential(nn.Linear(16, 24), nn.GELU(), nn.Linear(24, 16)) for _ in range(6)])
    x = torch.randn(20, 16)
    w, i = _route(20, 6, 2)
    i[i == 5] = 4                                                                       # expert 5 gets nothing
    d = PiscesLxFusedMoEDispatch(6, 2)
    out = d(x, w, i, experts)
    assert torch.allclose(out, PiscesLxFusedMoe.reference_dispatch(x, w, i, experts), atol=1e-5)
    out2, stats = d(x, w, i, experts, collect_stats=True)
    assert torch.allclose(out2, out) and len(stats) == len(set(i.flatten().tolist()))
    out.sum().backward()
    assert experts[0][0].weight.grad is not None and experts[5][0].weight.grad is None
    with pytest.raises(ValueError):
        d(x, w[:10], i[:10], experts)


def test_uniform_swiglu_experts_take_the_stacked_path():
    torch.manual_seed(0)
    experts = nn.ModuleList([YvSwiGLUExpert(16, 32) for _ in range(4)])
    x = torch.randn(12, 16)
    w, i = _route(12, 4, 2, seed=1)
    d = PiscesLxFusedMoEDispatch(4, 2)
    with torch.no_grad():
        out = d(x, w, i, experts)
        ref = PiscesLxFusedMoe.reference_dispatch(x, w, i, experts)
    assert d._stack is not None and d._stack[1].shape == (4, 64, 16) and torch.allclose(out, ref, atol=1e-4)
    key = d._stack[0]
    with torch.no_grad():
        d(x, w, i, experts)
        assert d._stack[0] == key                                                        # cached
        experts[0].w2.mul_(2.0)
        out3 = d(x, w, i, experts)
    assert d._stack[0] != key and torch.allclose(out3, PiscesLxFusedMoe.reference_dispatch(x, w, i, experts), atol=1e-4)
    assert torch.allclose(PiscesLxFusedMoe.fused_moe_dispatch(x, w, i, experts, 4, 2), d(x, w, i, experts), atol=1e-4)   # trainable experts: the differentiable path
