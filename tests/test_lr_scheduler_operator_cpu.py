"""Learning-rate scheduler operator family."""
import math

import pytest
import torch

from pisceslx_b200.optim import lr as L


def test_warmup_shapes_and_cosine():
    s = L.PiscesLxCosineWarmupScheduler(max_lr=1.0, min_lr=0.0, warmup_steps=10, total_steps=110)
    vals = [s.get_lr_at_step(i) for i in range(120)]
    assert vals[0] == pytest.approx(0.01 + 0.99 * 0.1) and vals[9] == pytest.approx(1.0) and vals[10] == pytest.approx(1.0)
    assert vals[60] == pytest.approx(0.5) and vals[110] == pytest.approx(0.0) and vals[119] == pytest.approx(0.0)
    assert all(a <= b + 1e-12 for a, b in zip(vals[:10], vals[1:10])) and all(a >= b - 1e-12 for a, b in zip(vals[10:], vals[11:]))
    cub = L.PiscesLxLRSchedulerOperator(L.PiscesLxLRSchedulerConfig(max_lr=1.0, warmup_steps=10, warmup_type="cubic"))
    exp = L.PiscesLxLRSchedulerOperator(L.PiscesLxLRSchedulerConfig(max_lr=1.0, warmup_steps=10, warmup_type="exponential"))
    assert cub.get_lr_at_step(4) < s.get_lr_at_step(4) < exp.get_lr_at_step(4) and exp.get_lr_at_step(9) == pytest.approx(1.0)
    with pytest.raises(ValueError):
        L.PiscesLxLRSchedulerConfig(warmup_type="spline")
    with pytest.raises(ValueError):
        L.PiscesLxLRSchedulerConfig(type="zigzag")
    assert L.PiscesLxLRSchedulerConfig(warmup_ratio=0.1, total_steps=500).warmup_steps == 50


def test_every_type_has_the_expected_shape():
    mk = lambda **kw: L.PiscesLxLRSchedulerOperator(L.PiscesLxLRSchedulerConfig(max_lr=1.0, min_lr=0.01, warmup_steps=0, **kw))
    assert mk(type="linear", total_steps=100).get_lr_at_step(50) == pytest.approx(1 - 0.99 * 0.5)
    assert mk(type="polynomial", total_steps=100, power=2.0).get_lr_at_step(50) == pytest.approx(0.01 + 0.99 * 0.25)
    assert mk(type="step", decay_steps=10, decay_ratio=0.5).get_lr_at_step(25) == pytest.approx(0.25)
    assert mk(type="exponential", decay_steps=10, decay_gamma=1.0).get_lr_at_step(10) == pytest.approx(math.exp(-1))
    assert mk(type="step", decay_steps=1, decay_ratio=0.1).get_lr_at_step(50) == 0.01             # floored at min_lr
    assert mk(type="constant").get_lr_at_step(12345) == 1.0
    assert mk(type="warmup_decay", total_steps=100, power=1.0).get_lr_at_step(25) == pytest.approx(0.75)
    inv = L.PiscesLxInverseSquareRootScheduler(max_lr=1.0, min_lr=0.0, warmup_steps=16)
    assert inv.get_lr_at_step(15) == pytest.approx(1.0) and inv.get_lr_at_step(16) == pytest.approx(1.0)
    assert inv.get_lr_at_step(16 + 48) == pytest.approx(0.5)                                      # sqrt(16 / 64)
    wsd = mk(type="wsd", total_steps=100, stable_ratio=0.8)
    assert wsd.get_lr_at_step(79) == 1.0 and wsd.get_lr_at_step(90) == pytest.approx(0.01 + 0.99 * 0.5) and wsd.get_lr_at_step(100) == pytest.approx(0.01)
    late = L.PiscesLxLRSchedulerOperator(L.PiscesLxLRSchedulerConfig(type="linear", max_lr=1.0, min_lr=0.0, warmup_steps=0, total_steps=10, apply_at_step=5))
    assert late.get_lr_at_step(3) == 1.0 and late.get_lr_at_step(10) == pytest.approx(0.5)


def test_cosine_restarts_closed_form_and_seekable():
    c = L.PiscesLxLRSchedulerConfig(type="cosine_with_restarts", max_lr=1.0, min_lr=0.0, cycle_min_lr=0.0, warmup_steps=0,
                                    cycle_first_step=10, cycle_scaling_factor=2.0, cycle_peak_decay=0.5)
    s = L.PiscesLxLRSchedulerOperator(c)
    # cycles: [0, 10) peak 1, [10, 30) peak 0.5, [30, 70) peak 0.25
    assert [s._cycle_of(t)[0] for t in (0, 9, 10, 29, 30, 69, 70)] == [0, 0, 1, 1, 2, 2, 3]
    assert s.get_lr_at_step(0) == pytest.approx(1.0) and s.get_lr_at_step(5) == pytest.approx(0.5)
    assert s.get_lr_at_step(10) == pytest.approx(0.5) and s.get_lr_at_step(20) == pytest.approx(0.25) and s.get_lr_at_step(30) == pytest.approx(0.25)
    late_first = s.get_lr_at_step(65)
    assert s.get_lr_at_step(3) == pytest.approx(0.5 * (1 + math.cos(math.pi * 0.3))) and s.get_lr_at_step(65) == late_first   # order of queries is free
    same = L.PiscesLxLRSchedulerOperator(L.PiscesLxLRSchedulerConfig(type="cosine_with_restarts", max_lr=1.0, cycle_min_lr=0.0, min_lr=0.0,
                                                                     warmup_steps=0, cycle_first_step=10))
    assert same.get_lr_at_step(25) == pytest.approx(same.get_lr_at_step(5))


def test_stateful_side_groups_accumulation_history_and_resume():
    w1, w2 = torch.nn.Parameter(torch.zeros(1)), torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([{"params": [w1], "lr": 1.0}, {"params": [w2], "lr": 0.1}])
    s = L.PiscesLxLrScheduler.create_scheduler("linear", opt, max_lr=1.0, min_lr=0.0, warmup_steps=0, total_steps=10,
                                               gradient_accumulation_steps=2)
    assert isinstance(s, L.PiscesLxLinearWarmupScheduler) and s.get_last_lr() == [1.0, pytest.approx(0.1)]
    seen = [s.step() for _ in range(6)]                                   # three optimizer steps
    assert seen == [1.0, pytest.approx(0.9), pytest.approx(0.9), pytest.approx(0.8), pytest.approx(0.8), pytest.approx(0.7)]
    assert s.current_step == 3 and s.get_last_lr() == [pytest.approx(0.7), pytest.approx(0.07)]
    assert s.get_lr_history() == [1.0, pytest.approx(0.9), pytest.approx(0.8), pytest.approx(0.7)]
    sd = s.state_dict()
    opt2 = torch.optim.SGD([{"params": [w1], "lr": 1.0}, {"params": [w2], "lr": 0.1}])
    s2 = L.PiscesLxLrScheduler.create_scheduler("linear", opt2, max_lr=1.0, min_lr=0.0, warmup_steps=0, total_steps=10,
                                                gradient_accumulation_steps=2)
    s2.load_state_dict(sd)
    assert s2.get_last_lr() == [pytest.approx(0.7), pytest.approx(0.07)] and s2.step() == pytest.approx(0.7) and s2.step() == pytest.approx(0.6)
    s.reset()
    assert s.current_step == 0 and s.get_last_lr()[0] == 1.0
    gen = L.PiscesLxLrScheduler.create_scheduler("polynomial", max_lr=1.0, min_lr=0.0, warmup_steps=0, total_steps=4, power=2.0)
    assert type(gen) is L.PiscesLxLRSchedulerOperator and gen.execute({"action": "get_lr", "step": 2}).output == {"lr": pytest.approx(0.25)}
    assert gen.execute({"action": "step"}).output["step"] == 1 and len(gen.execute({"action": "history"}).output["history"]) == 1
    assert not gen.execute({"action": "jump"}).is_success()
