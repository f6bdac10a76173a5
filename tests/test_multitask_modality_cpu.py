"""Task-uncertainty weighting and per-modality learning-rate schedules."""
import math

import pytest
import torch
from torch import nn

from pisceslx_b200.optim import multitask_modality as MM


def test_uncertainty_weighting_formula_and_types():
    c = MM.PiscesLxMultiTaskConfig(num_tasks=2, task_types=["regression", "classification"], task_names=["depth", "label"])
    op = MM.PiscesLxMultiTaskOperator(c)
    with torch.no_grad():
        op.log_uncertainty.copy_(torch.tensor([math.log(2.0), math.log(0.5)]))
    l1, l2 = torch.tensor(3.0), torch.tensor(1.0)
    total = op.compute_loss([l1, l2])
    want = 0.5 * 3.0 / 4.0 + 1.0 / 0.25 + math.log(2.0) + math.log(0.5)
    assert float(total) == pytest.approx(want, rel=1e-6)
    assert op.get_uncertainties() == [pytest.approx(2.0), pytest.approx(0.5)]
    assert op.get_task_weights() == {"depth": pytest.approx(0.125), "label": pytest.approx(4.0)}
    with pytest.raises(ValueError):
        op.compute_loss([l1])
    with pytest.raises(ValueError):
        MM.PiscesLxMultiTaskConfig(num_tasks=0)
    assert MM.PiscesLxMultiTaskConfig(num_tasks=3).task_names == ["task_0", "task_1", "task_2"]


def test_sigmas_learn_the_scale_of_each_task():
    torch.manual_seed(0)
    op = MM.PiscesLxMultiTaskOperator(MM.PiscesLxMultiTaskConfig(num_tasks=2))
    opt = torch.optim.Adam([op.param_group(model_lr=0.05)])
    for _ in range(400):
        losses = [torch.tensor(100.0), torch.tensor(0.01)]          # fixed, very different scales
        opt.zero_grad()
        op.compute_loss(losses).backward()
        opt.step()
    s = op.get_uncertainties()                                      # the optimum is sigma_i^2 = L_i
    assert s[0] == pytest.approx(10.0, rel=0.05) and s[1] == pytest.approx(0.1, rel=0.05)
    w = op.get_task_weights()
    assert w["task_0"] * 100.0 == pytest.approx(w["task_1"] * 0.01, rel=0.1)     # both terms now weigh the same
    assert op.get_statistics()["steps"] == 400 and opt.param_groups[0]["weight_decay"] == 0.0


def test_warmup_clamp_freeze_shared_and_empirical_init():
    op = MM.PiscesLxMultiTaskOperator(MM.PiscesLxMultiTaskConfig(num_tasks=2, warmup_steps=2))
    losses = [torch.tensor(4.0, requires_grad=True), torch.tensor(2.0, requires_grad=True)]
    assert float(op.compute_loss(losses)) == 3.0 and op.get_statistics()["in_warmup"]
    op.compute_loss(losses)
    assert float(op.compute_loss(losses)) == pytest.approx(0.5 * 4 + 0.5 * 2)             # sigma = 1 after the warm-up
    cl = MM.PiscesLxMultiTaskOperator(MM.PiscesLxMultiTaskConfig(num_tasks=1, clamp_uncertainty=True, uncertainty_min=0.5, uncertainty_max=2.0))
    with torch.no_grad():
        cl.log_uncertainty.fill_(5.0)
    assert cl.get_uncertainties() == [pytest.approx(2.0)]
    cl.freeze_uncertainty()
    assert not cl.log_uncertainty.requires_grad
    cl.unfreeze_uncertainty()
    assert cl.log_uncertainty.requires_grad
    sh = MM.PiscesLxMultiTaskOperator(MM.PiscesLxMultiTaskConfig(num_tasks=3, separate_uncertainty=False))
    assert sh.log_uncertainty.shape == (1,) and len(sh.get_uncertainties()) == 3
    em = MM.PiscesLxMultiTaskOperator(MM.PiscesLxMultiTaskConfig(num_tasks=2, uncertainty_init_strategy="empirical"))
    em.compute_loss([torch.tensor(16.0), torch.tensor(0.25)])
    assert em.get_uncertainties() == [pytest.approx(4.0), pytest.approx(0.5)]
    em.reset()
    assert em.get_uncertainties() == [1.0, 1.0] and em.steps == 0
    r = em.execute({"task_losses": [torch.tensor(1.0), torch.tensor(1.0)]})
    assert r.is_success() and "loss" in r.output and not em.execute({"task_losses": [torch.tensor(1.0)]}).is_success()
    f = MM.PiscesLxMultiTaskFacade(2, ["a", "b"])
    assert float(f.compute_loss([torch.tensor(2.0), torch.tensor(2.0)])) == 2.0 and len(list(f.parameters())) == 1
    lazy = MM.PiscesLxTaskUncertaintyWeighting()
    assert float(lazy.compute([torch.tensor(2.0), torch.tensor(4.0), torch.tensor(6.0)])) == 6.0 and lazy.operator.config.num_tasks == 3


class Multi(nn.Module):
    def __init__(self):
        super().__init__()
        self.vision_encoder = nn.Linear(4, 4)
        self.audio_encoder = nn.Linear(4, 4)
        self.modal_fusion = nn.Linear(4, 4)
        self.layers = nn.ModuleList([nn.Linear(4, 4)])
        self.lm_head = nn.Linear(4, 4)
        self.misc = nn.Parameter(torch.zeros(2))


def test_modality_detection_and_groups():
    d = MM.PiscesLxModalitySchedulerOperator._detect_modality
    T = MM.PiscesLxModalityType
    assert d("model.vision_encoder.blocks.0.qkv") is T.VISION and d("audio_encoder.conv.weight") is T.AUDIO
    assert d("model.modal_fusion.gate") is T.FUSION and d("model.layers.3.attention.o_proj") is T.TEXT
    assert d("lm_head") is T.TEXT and d("misc") is T.OTHER and d("vision_fusion_proj") is T.FUSION
    op = MM.PiscesLxModalitySchedulerOperator(MM.PiscesLxModalitySchedulerConfig(lr_multipliers={"vision": 0.1}))
    groups = op.build_param_groups(Multi(), lr=1e-3, weight_decay=0.0)
    tags = {g["modality"]: g for g in groups}
    assert set(tags) == {"vision", "audio", "fusion", "text", "other"} and tags["vision"]["lr"] == pytest.approx(1e-4)
    assert len(tags["text"]["params"]) == 4 and tags["other"]["params"][0].shape == (2,)


def test_each_modality_follows_its_own_cycle():
    m = Multi()
    f = MM.PiscesLxModalitySchedulerFacade(vision_t0=4, vision_t_mult=2.0, vision_eta_min=0.0, fusion_t0=2, fusion_t_mult=1.0, fusion_eta_min=0.0,
                                           text_t0=8, text_eta_min=0.0, audio_eta_min=0.0, other_eta_min=0.0)
    opt = torch.optim.SGD(f.param_groups(m, lr=1.0))
    assert f.setup(opt) == {"vision": 1, "audio": 1, "fusion": 1, "text": 1, "other": 1}
    hist = {k: [v] for k, v in f.get_lr().items()}
    for _ in range(12):
        f.step()
        for k, v in f.get_lr().items():
            hist[k].append(v)
    assert hist["fusion"][:5] == [pytest.approx(1.0), pytest.approx(0.5), pytest.approx(1.0), pytest.approx(0.5), pytest.approx(1.0)]
    assert hist["vision"][0] == pytest.approx(1.0) and hist["vision"][2] == pytest.approx(0.5) and hist["vision"][4] == pytest.approx(1.0)
    assert hist["vision"][8] == pytest.approx(0.5) and hist["vision"][12] == pytest.approx(1.0)      # the second cycle is 8 long
    assert hist["text"][4] == pytest.approx(0.5) and hist["text"][8] == pytest.approx(1.0)
    assert len({round(hist[k][3], 6) for k in ("vision", "fusion", "text")}) == 3                   # three different rates at once
    sd = f.operator.state_dict()
    f2 = MM.PiscesLxModalitySchedulerFacade(f.operator.config)
    opt2 = torch.optim.SGD(f2.param_groups(m, lr=1.0))
    f2.setup(opt2)
    f2.operator.load_state_dict(sd)
    assert f2.get_lr() == pytest.approx(f.get_lr())
    f.step(epoch=0)
    assert f.get_lr()["vision"] == pytest.approx(1.0)


def test_joint_warmup_untagged_groups_and_operator_front():
    m = Multi()
    op = MM.PiscesLxModalitySchedulerOperator(MM.PiscesLxModalitySchedulerConfig(warmup_steps=4, warmup_lr=0.0, text_t0=100, text_eta_min=0.0))
    opt = torch.optim.SGD([{"params": list(m.layers.parameters()) + list(m.lm_head.parameters()), "lr": 2.0},
                           {"params": list(m.vision_encoder.parameters()), "lr": 1.0}])
    r = op.execute({"action": "setup", "optimizer": opt, "model": m})
    assert r.output == {"groups": {"text": 1, "vision": 1}} and opt.param_groups[0]["modality"] == "text"
    assert opt.param_groups[0]["lr"] == pytest.approx(0.5)                  # step 0 of a 4-step warm-up to 2.0
    for _ in range(3):
        out = op.execute({"action": "step"}).output
    assert out["step"] == 3 and out["lr"]["text"] == pytest.approx(2.0) and out["lr"]["vision"] == pytest.approx(1.0)
    assert op.execute({"action": "get_lr"}).output["lr"]["text"] == pytest.approx(2.0)
    assert not op.execute({"action": "rewind"}).is_success()
