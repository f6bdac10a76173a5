"""Rollout-based alignment trainers on a tiny model (CPU): GRPO with DAPO options, agentic multi-turn RL, PPO with a
value head, reward model, KTO / BCO, preference data processing."""
import torch

from pisceslx_b200 import YvConfig
from pisceslx_b200.engine import rl
from pisceslx_b200.models import build_model

TARGET = 7


def tiny(seed=0, vocab=32):
    cfg = YvConfig.tiny_text_moe(vocab_size=vocab)
    cfg.n_layer, cfg.hidden_size, cfg.n_head, cfg.n_kv_head, cfg.head_dim = 1, 64, 2, 1, 32
    cfg.moe_num_experts, cfg.moe_top_k = 2, 1
    cfg.use_gradient_checkpointing = False
    return build_model(cfg, "cpu", torch.float32, seed=seed)


def reward_target(prompt, resp):
    return float((resp == TARGET).float().mean()) if resp.numel() else 0.0


def test_token_logprobs_and_sampling_masks():
    m = tiny()
    prompts = torch.randint(0, 32, (3, 4), generator=torch.Generator().manual_seed(0))
    ids, mask = rl.sample_responses(m, prompts, 6, eos_token_id=5)
    assert ids.shape == (3, 10) and not mask[:, :4].any()
    for i in range(3):                                            # nothing after the first EOS is part of the response
        resp = ids[i, 4:]
        if (resp == 5).any():
            first = int((resp == 5).nonzero()[0])
            assert mask[i, 4:4 + first + 1].all() and not mask[i, 4 + first + 1:].any()
    lp, msk = rl.token_logprobs(m, ids, mask)
    assert lp.shape == (3, 9) and (lp <= 0).all() and float(lp[:, :3].abs().sum()) == 0.0


def test_grpo_raises_the_reward_and_first_update_has_unit_ratio():
    torch.manual_seed(0)
    m = tiny()
    opt = torch.optim.AdamW(m.parameters(), lr=2e-2, weight_decay=0.0)
    cfg = rl.PiscesLxGRPOConfig(group_size=8, max_new_tokens=6, kl_coef=0.02, clip_high=0.28, dynamic_sampling=True,
                                diversity_weight=0.0, inner_epochs=1)
    op = rl.PiscesLxGRPOOperator(m, opt, reward_target, cfg)
    prompts = [torch.randint(0, 32, (4,), generator=torch.Generator().manual_seed(i)) for i in range(4)]
    tr = rl.PiscesLxGRPOTrainer(op, prompts, prompts_per_step=2)
    hist = tr.train(25)
    first, last = sum(h["reward_mean"] for h in hist[:5]) / 5, sum(h["reward_mean"] for h in hist[-5:]) / 5
    assert last > first + 0.15, (first, last)
    done = [h for h in hist if "ratio_mean" in h]
    assert abs(done[0]["ratio_mean"] - 1.0) < 1e-4 and done[0]["clipfrac"] == 0.0 and done[0]["kl"] < 1e-6
    assert all(0.0 <= h["groups_kept"] <= 1.0 for h in hist)


def test_grpo_options_refinement_diversity_checkpoint(tmp_path):
    torch.manual_seed(1)
    m = tiny(1)
    opt = torch.optim.SGD(m.parameters(), lr=1e-3)
    cfg = rl.PiscesLxGRPOConfig(group_size=4, max_new_tokens=4, kl_coef=0.0, refine_rounds=1, diversity_weight=0.5,
                                overlong_penalty=0.1, token_level_loss=False, minibatch_size=4, inner_epochs=2)
    op = rl.PiscesLxGRPOOperator(m, opt, reward_target, cfg, step_reward_fn=lambda p, r: [0.0, 1.0])
    assert op.ref is None                                          # no KL term, no reference copy
    tr = rl.PiscesLxGRPOTrainer(op, [torch.arange(3), torch.arange(3) + 5], save_dir=str(tmp_path), save_steps=2)
    hist = tr.train(2)
    assert len(op.replay) == 16 and all("loss" in h for h in hist)
    path = tmp_path / "grpo_step_2.pt"
    assert path.exists()
    tr2 = rl.PiscesLxGRPOTrainer(rl.PiscesLxGRPOOperator(tiny(2), torch.optim.SGD(tiny(2).parameters(), lr=1e-3),
                                                         reward_target, cfg), [torch.arange(3)])
    tr2.op.opt = torch.optim.SGD(tr2.op.model.parameters(), lr=1e-3)
    tr2.load_checkpoint(str(path))
    assert tr2.step == 2
    for a, b in zip(m.state_dict().values(), tr2.op.model.state_dict().values()):
        assert torch.equal(a, b)


class CountingEnv:
    """Reward 1 per turn whose action contains the target token; three turns."""

    def __init__(self):
        self.t = 0

    def reset(self):
        self.t = 0
        return torch.tensor([1, 2, 3])

    def step(self, action):
        self.t += 1
        return torch.tensor([4, self.t]), float((action == TARGET).any()), self.t >= 3


def test_agentic_multi_turn_rollouts_and_update():
    torch.manual_seed(2)
    m = tiny(3)
    tr = rl.PiscesLxAgenticRLTrainer(m, torch.optim.AdamW(m.parameters(), lr=1e-2), CountingEnv, group_size=4, max_turns=5,
                                     max_new_tokens=3)
    traj = tr._collect_agent_trajectory(CountingEnv())
    assert len(traj["returns"]) == 3                              # the environment ended the episode
    n_act = int(traj["mask"].sum())
    assert n_act == 9 and traj["ids"].shape[0] == 3 + 9 + 2 * 2   # reset obs + 3 actions + 2 observations
    assert set(traj["turn_of"][traj["mask"]].tolist()) == {0, 1, 2}
    assert traj["returns"][0] >= traj["returns"][1] >= traj["returns"][2]
    before = [p.detach().clone() for p in m.parameters()]
    stats = tr.train(2)
    assert stats[0]["turns_mean"] == 3.0 and stats[0]["tokens"] == 36.0
    assert any(not torch.equal(a, b) for a, b in zip(before, m.parameters()))


def test_ppo_with_value_head_and_reward_model():
    torch.manual_seed(3)
    m = tiny(4)
    opt = torch.optim.AdamW(m.parameters(), lr=5e-3)
    ppo = rl.PiscesLxPPOOperator(m, opt, reward_target, max_new_tokens=5, ppo_epochs=2)
    prompts = torch.randint(0, 32, (6, 4), generator=torch.Generator().manual_seed(1))
    s1 = ppo.step(prompts)
    assert abs(s1["kl"]) < 1e-5 and s1["value_loss"] >= 0 and len(opt.param_groups) == 2     # value head joined
    for _ in range(3):
        s = ppo.step(prompts)
    assert s["kl_coef"] > 0 and all(torch.isfinite(p).all() for p in m.parameters())
    rm_model = tiny(5)
    rm = rl.PiscesLxRewardModelOperator(rm_model, torch.optim.AdamW(rm_model.parameters(), lr=1e-2))
    chosen = torch.full((8, 6), TARGET)
    rejected = torch.randint(8, 32, (8, 6), generator=torch.Generator().manual_seed(2))
    for _ in range(30):
        st = rm.step(chosen, rejected)
    assert st["accuracy"] == 1.0 and st["margin"] > 0.5


def test_kto_bco_and_preference_processor():
    torch.manual_seed(4)
    m = tiny(6)
    kto = rl.PiscesLxKTOOperator(m, torch.optim.AdamW(m.parameters(), lr=1e-2), beta=0.5)
    prompts = torch.randint(0, 32, (8, 3), generator=torch.Generator().manual_seed(3))
    good = torch.full((4, 4), TARGET)
    bad = torch.full((4, 4), 9)
    comp = torch.cat([good, bad])
    desirable = torch.tensor([1, 1, 1, 1, 0, 0, 0, 0], dtype=torch.bool)
    for _ in range(15):
        st = kto.step(prompts, comp, desirable)
    assert st["reward_desirable"] > st["reward_undesirable"] and st["kl_ref"] >= 0
    m2 = tiny(7)
    bco = rl.PiscesLxBCOOperator(m2, torch.optim.AdamW(m2.parameters(), lr=1e-2), beta=0.5)
    l0 = bco.step(prompts, comp, desirable)["loss"]
    for _ in range(15):
        l1 = bco.step(prompts, comp, desirable)["loss"]
    assert l1 < l0

    class Tok:
        def encode(self, s):
            return [ord(c) % 32 for c in s]

    proc = rl.PiscesLxPreferenceDataProcessor(Tok(), max_length=8)
    pairs = proc.pairs([{"prompt": "ab", "chosen": "cde", "rejected": "f"}, {"prompt": "a", "chosen": "b", "rejected": "cdefghijk"}])
    assert pairs["chosen"].shape == (2, 5) and pairs["rejected"].shape == (2, 8)
    assert pairs["chosen_labels"][0].tolist() == [-100, -100, 3, 4, 5] and pairs["rejected_labels"][1, 0] == -100
    singles = proc.singles([{"prompt": "ab", "completion": "c", "label": 1}, {"prompt": "a", "completion": "bc", "label": 0}])
    assert singles["desirable"].tolist() == [True, False] and singles["labels"].shape == (2, 3)
