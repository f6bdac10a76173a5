"""Configured experts: types, lookup mode, shared and attention experts, factory registration."""
import pytest
import torch

from pisceslx_b200.models.moe_extras import (YvAttentionExpert, YvExpertBase, YvExpertConfig, YvExpertFactory, YvExpertMode, YvExpertType, YvSharedExpert,
                                             create_expert, register_expert)


@pytest.mark.parametrize("kind", ["standard", "swiglu", "geglu", "multi_layer", "shared", "attention"])
def test_every_type_keeps_shape_and_trains(kind):
    torch.manual_seed(0)
    e = YvExpertFactory.create_from_config(YvExpertConfig(hidden_size=16, intermediate_size=24, expert_type=kind, num_heads=4))
    assert isinstance(e, YvExpertBase) and e.config.expert_type is YvExpertType(kind)
    for shape in ((5, 16), (2, 3, 16)):
        x = torch.randn(*shape, requires_grad=True)
        y = e(x)
        assert y.shape == x.shape
        y.sum().backward()
        assert x.grad is not None
    assert any(p.grad is not None for p in e.parameters())


def test_lookup_mode_freezes_and_dropout_applies():
    e = create_expert(YvExpertConfig(hidden_size=8, intermediate_size=8, mode="pure_lookup"))
    assert e.mode is YvExpertMode.PURE_LOOKUP and not any(p.requires_grad for p in e.parameters())
    over = create_expert(YvExpertConfig(hidden_size=8, intermediate_size=8), mode=YvExpertMode.PURE_LOOKUP)
    assert not any(p.requires_grad for p in over.parameters())
    d = create_expert(YvExpertConfig(hidden_size=8, intermediate_size=8, dropout=0.5)).train()
    torch.manual_seed(0)
    assert (d(torch.ones(64, 8)) == 0).any()
    with pytest.raises(ValueError):
        YvExpertConfig(activation="tanh")
    with pytest.raises(ValueError):
        YvExpertConfig(expert_type="conv")


def test_shared_gate_starts_at_one_and_attention_expert_is_causal():
    torch.manual_seed(0)
    s = YvSharedExpert(YvExpertConfig(hidden_size=8, intermediate_size=12))
    x = torch.randn(4, 8)
    assert torch.allclose(s(x), s.core(x), atol=1e-6)                                    # sigmoid(0) x 2 = 1
    a = YvAttentionExpert(YvExpertConfig(hidden_size=8, num_heads=2)).eval()
    seq = torch.randn(1, 6, 8)
    changed = seq.clone()
    changed[:, -1] += 1.0
    assert torch.allclose(a(seq)[:, :-1], a(changed)[:, :-1], atol=1e-6) and torch.allclose(a(seq[0]), a(seq)[0], atol=1e-6)
    with pytest.raises(ValueError):
        YvAttentionExpert(YvExpertConfig(hidden_size=10, num_heads=4))


def test_registration_and_base_is_abstract():
    class Double(YvExpertBase):
        def body(self, x):
            return 2 * x
    register_expert(YvExpertType.STANDARD, Double)
    try:
        assert torch.equal(create_expert(YvExpertConfig(hidden_size=4, expert_type="standard"))(torch.ones(2, 4)), 2 * torch.ones(2, 4))
    finally:
        from pisceslx_b200.models import moe_extras
        moe_extras._EXPERT_REGISTRY.pop(YvExpertType.STANDARD)
    with pytest.raises(NotImplementedError):
        YvExpertBase(YvExpertConfig(hidden_size=4))(torch.ones(1, 4))
    assert YvExpertFactory.create("swiglu", 8, 8) is not None
