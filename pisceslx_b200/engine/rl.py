"""On-policy alignment trainers with their rollout loops: GRPO (+ DAPO options), PPO with a value head, agentic
multi-turn RL, and the off-policy KTO / BCO operators that need a running KL / reward baseline.

Reference surface: ``PiscesLxGRPOOperator`` / ``PiscesLxGRPOTrainer`` / ``PiscesLxAgenticRLTrainer``
(opss/train/grpo.py:259-2408: group sampling, reference log-probs, group-relative advantages, clipped update with a
KL term, iterative refinement, diversity-aware reward mixing from a replay buffer, step-quality rewards, token-level
advantages), ``PiscesLxPPOOperator`` / ``PiscesLxRewardModelOperator`` / ``PiscesLxKTOOperator`` /
``PiscesLxBCOOperator`` / ``PiscesLxPreferenceDataProcessor`` (opss/train/pref_align.py:243-955).  The objectives
themselves live in ``engine.alignment``; this module adds what turns them into training loops.

Design: rollouts are BATCHED - the G responses of a group (and the groups of several prompts) are sampled in one
``model.generate`` call over the paged KV cache, and old / reference / new log-probabilities are one forward each over
the padded batch; the reference samples its group members one by one (grpo.py:648-751).
"""
from __future__ import annotations

import copy
import math
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .alignment import bco_loss, dapo_filter_groups, gae, group_relative_advantages, kto_loss


# --------------------------------------------------------------------------------------------------
# shared pieces
# --------------------------------------------------------------------------------------------------
def token_logprobs(model: Any, ids: torch.Tensor, response_mask: torch.Tensor, return_hidden: bool = False):
    """Per-token log-probabilities of ``ids[:, 1:]`` under ``model`` as ``[B, S-1]`` (0 outside the response mask).
    ``response_mask [B, S]`` marks the generated positions."""
    out = model(input_ids=ids, return_logits=True, return_hidden=return_hidden)
    logits = out.logits[:, :-1].float()
    lp = torch.log_softmax(logits, -1).gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1)
    m = response_mask[:, 1:].to(lp.dtype)
    if return_hidden:
        return lp * m, m, out["hidden_states"]
    return lp * m, m


@torch.no_grad()
def sample_responses(model: Any, prompts: torch.Tensor, max_new_tokens: int, temperature: float = 1.0,
                     top_p: float = 1.0, eos_token_id: Optional[int] = None, pad_token_id: int = 0):
    """One batched rollout: ``prompts [B, P]`` -> ``(ids [B, P + T], response_mask [B, P + T])``; positions after a
    sequence's end-of-sequence token are padding and masked out."""
    from ..models.generation import YvSampler, YvSamplingConfig
    sampler = YvSampler(YvSamplingConfig(strategy="top_k_top_p", temperature=max(temperature, 1e-5), top_k=0, top_p=top_p))
    ids, _ = model.generate(prompts, max_new_tokens=max_new_tokens, sampler=sampler,
                            eos_token_id=-1 if eos_token_id is None else eos_token_id)
    B, P = prompts.shape
    mask = torch.zeros_like(ids, dtype=torch.bool)
    mask[:, P:] = True
    if eos_token_id is not None and eos_token_id >= 0:
        resp = ids[:, P:]
        ended = (resp == eos_token_id).cumsum(1)
        after = (ended - (resp == eos_token_id).long()) > 0          # strictly after the first EOS
        mask[:, P:] &= ~after
    return ids, mask


class YvAdaptiveKLController:
    """Keeps the measured KL near a target by scaling the penalty coefficient (PPO's proportional controller)."""

    def __init__(self, init_coef: float = 0.05, target: float = 6.0, horizon: int = 10000):
        self.coef, self.target, self.horizon = init_coef, target, horizon

    def update(self, kl: float, n_steps: int) -> float:
        err = max(min(kl / self.target - 1.0, 0.2), -0.2)
        self.coef *= 1.0 + err * n_steps / self.horizon
        return self.coef


# --------------------------------------------------------------------------------------------------
# GRPO
# --------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxGRPOConfig:
    group_size: int = 8
    max_new_tokens: int = 64
    temperature: float = 1.0
    top_p: float = 1.0
    clip_low: float = 0.2
    clip_high: float = 0.2                 # > clip_low = DAPO's clip-higher
    kl_coef: float = 0.04                  # weight of the k3 estimate of KL(policy || reference); 0 = no reference
    inner_epochs: int = 1
    minibatch_size: int = 0                # 0 = the whole rollout batch at once
    token_level_loss: bool = True          # average over all response tokens of the batch (DAPO) instead of per sequence
    dynamic_sampling: bool = False         # drop groups whose rewards are all equal (no learning signal)
    overlong_penalty: float = 0.0          # subtracted when a response hits max_new_tokens without EOS
    refine_rounds: int = 0                 # iterative refinement: re-sample conditioned on the best response so far
    diversity_weight: float = 0.0          # MMR-style bonus for responses unlike those in the replay buffer
    replay_size: int = 256
    max_grad_norm: float = 1.0
    eos_token_id: Optional[int] = None
    pad_token_id: int = 0


@dataclass
class PiscesLxTrajectoryEntry:
    prompt: torch.Tensor
    ids: torch.Tensor
    mask: torch.Tensor
    reward: float
    info: Dict[str, Any] = field(default_factory=dict)


class PiscesLxGRPOOperator:
    """Group-relative policy optimisation.  ``reward_fn(prompt_ids [P], response_ids [T]) -> float``."""

    def __init__(self, model: Any, optimizer: torch.optim.Optimizer, reward_fn: Callable[[torch.Tensor, torch.Tensor], float],
                 config: Optional[PiscesLxGRPOConfig] = None, ref_model: Any = None,
                 step_reward_fn: Optional[Callable[[torch.Tensor, torch.Tensor], Sequence[float]]] = None):
        self.model, self.opt, self.reward_fn = model, optimizer, reward_fn
        self.cfg = config or PiscesLxGRPOConfig()
        self.ref = ref_model
        if self.ref is None and self.cfg.kl_coef > 0:
            self.ref = copy.deepcopy(model).eval().requires_grad_(False)
        self.step_reward_fn = step_reward_fn
        self.replay: List[torch.Tensor] = []                 # bag-of-token embeddings of past responses (diversity)
        self.stats_history: List[Dict[str, float]] = []

    # ---- rollout ------------------------------------------------------------------------------------------
    def _sample_group_responses(self, prompts: torch.Tensor):
        c = self.cfg
        rep = prompts.repeat_interleave(c.group_size, dim=0)
        ids, mask = sample_responses(self.model, rep, c.max_new_tokens, c.temperature, c.top_p, c.eos_token_id, c.pad_token_id)
        for _ in range(c.refine_rounds):
            # iterative refinement: the best response of each group so far is appended to the prompt as a draft and a
            # new group is sampled; the better of old and new is kept per slot
            r_old = self._compute_rewards(rep, ids, mask)
            best = r_old.view(-1, c.group_size).argmax(1) + torch.arange(0, rep.shape[0], c.group_size, device=r_old.device)
            draft = ids[best][:, prompts.shape[1]:]
            ctx = torch.cat([prompts, draft], dim=1).repeat_interleave(c.group_size, dim=0)
            ids2, mask2 = sample_responses(self.model, ctx, c.max_new_tokens, c.temperature, c.top_p, c.eos_token_id,
                                           c.pad_token_id)
            new_resp, new_mask = ids2[:, ctx.shape[1]:], mask2[:, ctx.shape[1]:]
            cand = torch.cat([rep, new_resp], dim=1)
            cmask = torch.cat([torch.zeros_like(rep, dtype=torch.bool), new_mask], dim=1)
            r_new = self._compute_rewards(rep, cand, cmask)
            take = (r_new > r_old).view(-1, 1)
            ids, mask = torch.where(take, cand, ids), torch.where(take, cmask, mask)
        return rep, ids, mask

    def _compute_rewards(self, prompts: torch.Tensor, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        P = prompts.shape[1]
        out = []
        for i in range(ids.shape[0]):
            resp = ids[i, P:][mask[i, P:]]
            r = float(self.reward_fn(prompts[i], resp))
            if self.step_reward_fn is not None:               # verifiable per-step quality folded into the outcome
                steps = list(self.step_reward_fn(prompts[i], resp))
                if steps:
                    r += sum(steps) / len(steps)
            if c.overlong_penalty and int(mask[i, P:].sum()) >= c.max_new_tokens and \
                    (c.eos_token_id is None or not bool((resp == c.eos_token_id).any())):
                r -= c.overlong_penalty
            out.append(r)
        return torch.tensor(out, dtype=torch.float32, device=ids.device)

    def _diversify_rewards(self, ids: torch.Tensor, mask: torch.Tensor, rewards: torch.Tensor) -> torch.Tensor:
        """MMR-style bonus: cosine distance of a response's mean token embedding to the nearest replayed response."""
        c = self.cfg
        if c.diversity_weight <= 0:
            return rewards
        with torch.no_grad():
            emb = self.model.model.embed.weight.detach().float()
            m = mask.float()
            feat = F.normalize((emb[ids] * m.unsqueeze(-1)).sum(1) / m.sum(1, keepdim=True).clamp_min(1), dim=-1)
            if self.replay:
                bank = torch.stack(self.replay).to(feat.device)
                novelty = 1.0 - (feat @ bank.t()).max(dim=1).values
                rewards = rewards + c.diversity_weight * novelty
            self.replay.extend(feat.cpu().unbind(0))
            del self.replay[:-c.replay_size]
        return rewards

    # ---- update ---------------------------------------------------------------------------------------------
    def compute_group_advantages(self, rewards: torch.Tensor) -> torch.Tensor:
        return group_relative_advantages(rewards, self.cfg.group_size)

    def _policy_loss(self, ids, mask, old_lp, ref_lp, adv):
        c = self.cfg
        lp, m = token_logprobs(self.model, ids, mask)
        ratio = torch.exp(lp - old_lp)
        a = adv.unsqueeze(1)
        surr = torch.minimum(ratio * a, ratio.clamp(1 - c.clip_low, 1 + c.clip_high) * a)
        per_tok = -surr
        kl = torch.zeros((), device=ids.device)
        if ref_lp is not None and c.kl_coef > 0:
            d = ref_lp - lp
            k3 = (torch.exp(d) - d - 1.0) * m                  # unbiased, non-negative estimate of KL(pi || ref)
            per_tok = per_tok + c.kl_coef * k3
            kl = k3.sum() / m.sum().clamp_min(1)
        if c.token_level_loss:
            loss = (per_tok * m).sum() / m.sum().clamp_min(1)
        else:
            loss = ((per_tok * m).sum(1) / m.sum(1).clamp_min(1)).mean()
        clipfrac = (((ratio - 1).abs() > max(c.clip_low, c.clip_high)) * m).sum() / m.sum().clamp_min(1)
        return loss, {"kl": float(kl), "clipfrac": float(clipfrac), "ratio_mean": float((ratio * m).sum() / m.sum().clamp_min(1))}

    def train_on_prompts(self, prompts: torch.Tensor) -> Dict[str, float]:
        """One GRPO iteration over ``prompts [N, P]``: sample N x G responses, score, update."""
        c = self.cfg
        was_training = self.model.training
        rep, ids, mask = self._sample_group_responses(prompts)
        rewards = self._compute_rewards(rep, ids, mask)
        shaped = self._diversify_rewards(ids, mask, rewards)
        adv = self.compute_group_advantages(shaped)
        keep = torch.ones_like(adv, dtype=torch.bool)
        if c.dynamic_sampling:
            keep = dapo_filter_groups(shaped, c.group_size)
        stats = {"reward_mean": float(rewards.mean()), "reward_std": float(rewards.std(unbiased=False)),
                 "groups_kept": float(keep.float().mean()), "response_len": float(mask.sum(1).float().mean())}
        if not bool(keep.any()):
            self.stats_history.append({**stats, "loss": 0.0, "skipped": 1.0})
            return self.stats_history[-1]
        ids, mask, adv = ids[keep], mask[keep], adv[keep]
        self.model.eval()
        with torch.no_grad():
            old_lp, _ = token_logprobs(self.model, ids, mask)
            ref_lp = token_logprobs(self.ref, ids, mask)[0] if (self.ref is not None and c.kl_coef > 0) else None
        self.model.train()
        n = ids.shape[0]
        mb = c.minibatch_size or n
        last: Dict[str, float] = {}
        losses = []
        for _ in range(c.inner_epochs):
            perm = torch.randperm(n, device=ids.device) if mb < n else torch.arange(n, device=ids.device)
            for s in range(0, n, mb):
                j = perm[s:s + mb]
                loss, last = self._policy_loss(ids[j], mask[j], old_lp[j], None if ref_lp is None else ref_lp[j], adv[j])
                self.opt.zero_grad(set_to_none=True)
                loss.backward()
                if c.max_grad_norm > 0:
                    torch.nn.utils.clip_grad_norm_([p for p in self.model.parameters() if p.grad is not None], c.max_grad_norm)
                self.opt.step()
                losses.append(float(loss))
        self.model.train(was_training)
        stats.update(last, loss=sum(losses) / len(losses))
        self.stats_history.append(stats)
        return stats


class PiscesLxGRPOTrainer:
    """Loop + checkpoints around the operator (reference grpo.py:1886-2010)."""

    def __init__(self, operator: PiscesLxGRPOOperator, prompts: Sequence[torch.Tensor], prompts_per_step: int = 2,
                 save_dir: Optional[str] = None, save_steps: int = 0):
        self.op, self.prompts, self.n = operator, list(prompts), prompts_per_step
        self.save_dir, self.save_steps, self.step = save_dir, save_steps, 0

    def train(self, steps: int) -> List[Dict[str, float]]:
        hist = []
        for _ in range(steps):
            batch = [self.prompts[(self.step * self.n + i) % len(self.prompts)] for i in range(self.n)]
            hist.append(self.op.train_on_prompts(torch.stack(batch)))
            self.step += 1
            if self.save_dir and self.save_steps and self.step % self.save_steps == 0:
                self._save_checkpoint(self.save_dir, self.step)
        return hist

    def _save_checkpoint(self, save_dir: str, step: int) -> str:
        os.makedirs(save_dir, exist_ok=True)
        path = os.path.join(save_dir, f"grpo_step_{step}.pt")
        torch.save({"model_state_dict": self.op.model.state_dict(), "optimizer_state_dict": self.op.opt.state_dict(),
                    "step": step, "stats": self.op.stats_history[-50:]}, path)
        return path

    def load_checkpoint(self, path: str) -> None:
        ck = torch.load(path, map_location="cpu", weights_only=False)
        self.op.model.load_state_dict(ck["model_state_dict"])
        self.op.opt.load_state_dict(ck["optimizer_state_dict"])
        self.step = int(ck.get("step", 0))


# --------------------------------------------------------------------------------------------------
# agentic multi-turn RL
# --------------------------------------------------------------------------------------------------
class PiscesLxAgenticRLTrainer:
    """Multi-turn rollouts against an environment.  ``env.reset() -> observation ids``; ``env.step(action ids) ->
    (observation ids, reward, done)``.  A trajectory's context is observation, action, observation, ...; only action
    tokens are trained.  Advantages: discounted return-to-go per turn, normalised over the group of trajectories that
    started from the same reset (reference grpo.py:2012-2408)."""

    def __init__(self, model: Any, optimizer: torch.optim.Optimizer, env_factory: Callable[[], Any], group_size: int = 4,
                 max_turns: int = 4, max_new_tokens: int = 16, gamma: float = 1.0, clip: float = 0.2, temperature: float = 1.0,
                 eos_token_id: Optional[int] = None):
        self.model, self.opt, self.env_factory = model, optimizer, env_factory
        self.G, self.max_turns, self.T, self.gamma, self.clip = group_size, max_turns, max_new_tokens, gamma, clip
        self.temperature, self.eos = temperature, eos_token_id

    @torch.no_grad()
    def _collect_agent_trajectory(self, env: Any) -> Dict[str, Any]:
        dev = next(self.model.parameters()).device
        ctx = env.reset().to(dev).view(1, -1)
        mask = torch.zeros_like(ctx, dtype=torch.bool)
        turn_of = torch.full_like(ctx, -1)
        rewards: List[float] = []
        for turn in range(self.max_turns):
            ids, m = sample_responses(self.model, ctx, self.T, self.temperature, 1.0, self.eos)
            new = ids.shape[1] - ctx.shape[1]
            act = ids[0, ctx.shape[1]:][m[0, ctx.shape[1]:]]
            obs, r, done = env.step(act.cpu())
            rewards.append(float(r))
            mask = torch.cat([mask, m[:, -new:]], dim=1)
            turn_of = torch.cat([turn_of, torch.full((1, new), turn, device=dev, dtype=turn_of.dtype)], dim=1)
            ctx = ids
            if done:
                break
            obs = obs.to(dev).view(1, -1)
            ctx = torch.cat([ctx, obs], dim=1)
            mask = torch.cat([mask, torch.zeros_like(obs, dtype=torch.bool)], dim=1)
            turn_of = torch.cat([turn_of, torch.full_like(obs, -1)], dim=1)
        g, rtg = 0.0, []
        for r in reversed(rewards):
            g = r + self.gamma * g
            rtg.append(g)
        return {"ids": ctx[0], "mask": mask[0], "turn_of": turn_of[0], "returns": list(reversed(rtg)), "reward": sum(rewards)}

    def _compute_agent_advantages(self, trajs: List[Dict[str, Any]]) -> List[torch.Tensor]:
        tot = torch.tensor([t["returns"][0] for t in trajs])
        mean, std = tot.mean(), tot.std(unbiased=False).clamp_min(1e-6)
        out = []
        for t in trajs:
            per_turn = (torch.tensor(t["returns"]) - mean) / std          # credit every turn with what followed it
            adv = torch.zeros(t["ids"].shape[0])
            for k, a in enumerate(per_turn):
                adv[(t["turn_of"] == k).cpu()] = a
            out.append(adv)
        return out

    def agentic_rl_update(self) -> Dict[str, float]:
        was_training = self.model.training
        self.model.eval()
        trajs = [self._collect_agent_trajectory(self.env_factory()) for _ in range(self.G)]
        advs = self._compute_agent_advantages(trajs)
        dev = next(self.model.parameters()).device
        L = max(t["ids"].shape[0] for t in trajs)
        ids = torch.zeros(self.G, L, dtype=torch.long, device=dev)
        mask = torch.zeros(self.G, L, dtype=torch.bool, device=dev)
        adv = torch.zeros(self.G, L, device=dev)
        for i, (t, a) in enumerate(zip(trajs, advs)):
            n = t["ids"].shape[0]
            ids[i, :n], mask[i, :n], adv[i, :n] = t["ids"], t["mask"], a.to(dev)
        with torch.no_grad():
            old_lp, _ = token_logprobs(self.model, ids, mask)
        self.model.train()
        lp, m = token_logprobs(self.model, ids, mask)
        ratio = torch.exp(lp - old_lp)
        a = adv[:, 1:]
        loss = -(torch.minimum(ratio * a, ratio.clamp(1 - self.clip, 1 + self.clip) * a) * m).sum() / m.sum().clamp_min(1)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        self.model.train(was_training)
        return {"loss": float(loss), "reward_mean": sum(t["reward"] for t in trajs) / self.G,
                "turns_mean": sum(len(t["returns"]) for t in trajs) / self.G, "tokens": float(m.sum())}

    def train(self, steps: int) -> List[Dict[str, float]]:
        return [self.agentic_rl_update() for _ in range(steps)]


# --------------------------------------------------------------------------------------------------
# PPO with a value head, reward model
# --------------------------------------------------------------------------------------------------
class YvValueHead(nn.Module):
    def __init__(self, hidden: int):
        super().__init__()
        self.proj = nn.Linear(hidden, 1)
        nn.init.zeros_(self.proj.weight)
        nn.init.zeros_(self.proj.bias)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.proj(hidden_states.float()).squeeze(-1)


class PiscesLxPPOOperator:
    """PPO-clip with GAE: rollout -> per-token reward = -kl_coef * (logp - ref_logp), plus the scalar reward at the last
    response token -> advantages -> ``ppo_epochs`` passes of minibatch updates of policy and value head."""

    def __init__(self, model: Any, optimizer: torch.optim.Optimizer, reward_fn: Callable[[torch.Tensor, torch.Tensor], float],
                 ref_model: Any = None, value_head: Optional[YvValueHead] = None, clip: float = 0.2, vf_coef: float = 0.5,
                 gamma: float = 1.0, lam: float = 0.95, ppo_epochs: int = 2, max_new_tokens: int = 32,
                 kl: Optional[YvAdaptiveKLController] = None, temperature: float = 1.0, eos_token_id: Optional[int] = None):
        self.model, self.opt, self.reward_fn = model, optimizer, reward_fn
        self.ref = ref_model if ref_model is not None else copy.deepcopy(model).eval().requires_grad_(False)
        self.value_head = value_head or YvValueHead(model.cfg.hidden_size).to(next(model.parameters()).device)
        if not any(p is q for g in optimizer.param_groups for q in g["params"] for p in self.value_head.parameters()):
            optimizer.add_param_group({"params": list(self.value_head.parameters())})
        self.clip, self.vf_coef, self.gamma, self.lam, self.epochs, self.T = clip, vf_coef, gamma, lam, ppo_epochs, max_new_tokens
        self.kl = kl or YvAdaptiveKLController()
        self.temperature, self.eos = temperature, eos_token_id

    def step(self, prompts: torch.Tensor) -> Dict[str, float]:
        was_training = self.model.training
        self.model.eval()
        ids, mask = sample_responses(self.model, prompts, self.T, self.temperature, 1.0, self.eos)
        P = prompts.shape[1]
        with torch.no_grad():
            old_lp, m, hid = token_logprobs(self.model, ids, mask, return_hidden=True)
            ref_lp, _ = token_logprobs(self.ref, ids, mask)
            old_v = self.value_head(hid)[:, :-1] * m
            kl_tok = (old_lp - ref_lp) * m
            rewards = -self.kl.coef * kl_tok
            score = torch.tensor([float(self.reward_fn(prompts[i], ids[i, P:][mask[i, P:]])) for i in range(ids.shape[0])],
                                 device=ids.device)
            last = (m.cumsum(1) == m.sum(1, keepdim=True)) & (m > 0)          # last response token of every row
            rewards = rewards + last.float() * score.unsqueeze(1)
            adv, ret = gae(rewards, old_v, self.gamma, self.lam)
            adv = adv * m
            adv = (adv - adv.sum() / m.sum().clamp_min(1)) / (adv[m > 0].std(unbiased=False).clamp_min(1e-6)) * m
        self.model.train()
        stats: Dict[str, float] = {}
        for _ in range(self.epochs):
            lp, _, hid = token_logprobs(self.model, ids, mask, return_hidden=True)
            v = self.value_head(hid)[:, :-1]
            ratio = torch.exp(lp - old_lp)
            pg = -(torch.minimum(ratio * adv, ratio.clamp(1 - self.clip, 1 + self.clip) * adv) * m).sum() / m.sum().clamp_min(1)
            v_clip = old_v + (v - old_v).clamp(-self.clip, self.clip)
            vf = 0.5 * (torch.maximum((v - ret) ** 2, (v_clip - ret) ** 2) * m).sum() / m.sum().clamp_min(1)
            loss = pg + self.vf_coef * vf
            self.opt.zero_grad(set_to_none=True)
            loss.backward()
            self.opt.step()
            stats = {"policy_loss": float(pg.detach()), "value_loss": float(vf.detach())}
        kl_mean = float(kl_tok.sum() / m.sum().clamp_min(1))
        self.kl.update(kl_mean, ids.shape[0])
        self.model.train(was_training)
        return {**stats, "reward_mean": float(score.mean()), "kl": kl_mean, "kl_coef": self.kl.coef}


class PiscesLxRewardModelOperator:
    """Bradley-Terry reward model on the final hidden state of the last token: ``-log sigmoid(r_chosen - r_rejected)``."""

    def __init__(self, model: Any, optimizer: torch.optim.Optimizer, head: Optional[YvValueHead] = None):
        self.model, self.opt = model, optimizer
        self.head = head or YvValueHead(model.cfg.hidden_size).to(next(model.parameters()).device)
        nn.init.normal_(self.head.proj.weight, std=0.02)
        optimizer.add_param_group({"params": list(self.head.parameters())})

    def score(self, ids: torch.Tensor, lengths: Optional[torch.Tensor] = None) -> torch.Tensor:
        hid = self.model(input_ids=ids, return_logits=False, return_hidden=True)["hidden_states"]
        idx = (lengths - 1) if lengths is not None else torch.full((ids.shape[0],), ids.shape[1] - 1, device=ids.device)
        return self.head(hid[torch.arange(ids.shape[0], device=ids.device), idx])

    def step(self, chosen: torch.Tensor, rejected: torch.Tensor) -> Dict[str, float]:
        rc, rr = self.score(chosen), self.score(rejected)
        loss = -F.logsigmoid(rc - rr).mean()
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return {"loss": float(loss), "accuracy": float((rc > rr).float().mean()), "margin": float((rc - rr).mean())}


# --------------------------------------------------------------------------------------------------
# KTO / BCO with their running baselines, preference data processing
# --------------------------------------------------------------------------------------------------
class PiscesLxKTOOperator:
    """Kahneman-Tversky optimisation over unpaired (sequence, desirable?) examples.  The reference point is the batch's
    KL estimate taken from MISMATCHED prompt / completion pairs (each prompt with the next example's completion), as the
    method prescribes, and is detached."""

    def __init__(self, model: Any, optimizer: torch.optim.Optimizer, ref_model: Any = None, beta: float = 0.1,
                 w_desirable: float = 1.0, w_undesirable: float = 1.0):
        self.model, self.opt = model, optimizer
        self.ref = ref_model if ref_model is not None else copy.deepcopy(model).eval().requires_grad_(False)
        self.beta, self.wd, self.wu = beta, w_desirable, w_undesirable

    def _seq_lp(self, m: Any, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        return token_logprobs(m, ids, mask)[0].sum(1)

    def step(self, prompts: torch.Tensor, completions: torch.Tensor, desirable: torch.Tensor) -> Dict[str, float]:
        ids = torch.cat([prompts, completions], dim=1)
        mask = torch.zeros_like(ids, dtype=torch.bool)
        mask[:, prompts.shape[1]:] = True
        mism = torch.cat([prompts, completions.roll(1, dims=0)], dim=1)
        with torch.no_grad():
            ref_lp = self._seq_lp(self.ref, ids, mask)
            kl = (self._seq_lp(self.model, mism, mask) - self._seq_lp(self.ref, mism, mask)).mean().clamp_min(0)
        pi_lp = self._seq_lp(self.model, ids, mask)
        loss = kto_loss(pi_lp, ref_lp, desirable.bool(), self.beta, self.wd, self.wu, kl_ref=kl)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        margin = (pi_lp - ref_lp).detach()
        return {"loss": float(loss), "kl_ref": float(kl), "reward_desirable": float(margin[desirable.bool()].mean()) if desirable.any() else 0.0,
                "reward_undesirable": float(margin[~desirable.bool()].mean()) if (~desirable.bool()).any() else 0.0}


class PiscesLxBCOOperator(PiscesLxKTOOperator):
    """Binary classifier optimisation: like KTO with a running mean of the implicit reward as the decision boundary."""

    def __init__(self, *a: Any, momentum: float = 0.9, **k: Any):
        super().__init__(*a, **k)
        self.delta, self.momentum = 0.0, momentum

    def step(self, prompts: torch.Tensor, completions: torch.Tensor, desirable: torch.Tensor) -> Dict[str, float]:
        ids = torch.cat([prompts, completions], dim=1)
        mask = torch.zeros_like(ids, dtype=torch.bool)
        mask[:, prompts.shape[1]:] = True
        with torch.no_grad():
            ref_lp = self._seq_lp(self.ref, ids, mask)
        pi_lp = self._seq_lp(self.model, ids, mask)
        r = self.beta * (pi_lp - ref_lp)
        self.delta = self.momentum * self.delta + (1 - self.momentum) * float(r.detach().mean())
        loss = bco_loss(pi_lp, ref_lp, desirable.bool(), self.beta, delta=self.delta)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return {"loss": float(loss), "delta": self.delta}


class PiscesLxPreferenceDataProcessor:
    """Turns raw preference records into padded tensors: ``{"prompt", "chosen", "rejected"}`` pairs (DPO / ORPO / RM) or
    ``{"prompt", "completion", "label"}`` singles (KTO / BCO); prompt tokens get label -100 (reference
    pref_align.py:881-955)."""

    def __init__(self, tokenizer: Any, max_length: int = 512, pad_token_id: int = 0):
        self.tok, self.max_length, self.pad = tokenizer, max_length, pad_token_id

    def _encode(self, prompt: str, completion: str) -> Tuple[List[int], List[int]]:
        p, c = self.tok.encode(prompt), self.tok.encode(completion)
        ids = (p + c)[: self.max_length]
        labels = ([-100] * len(p) + c)[: self.max_length]
        return ids, labels

    def _pad(self, rows: List[List[int]], fill: int) -> torch.Tensor:
        L = max(len(r) for r in rows)
        return torch.tensor([r + [fill] * (L - len(r)) for r in rows], dtype=torch.long)

    def pairs(self, records: Sequence[Dict[str, str]]) -> Dict[str, torch.Tensor]:
        ch = [self._encode(r["prompt"], r["chosen"]) for r in records]
        rj = [self._encode(r["prompt"], r["rejected"]) for r in records]
        return {"chosen": self._pad([a for a, _ in ch], self.pad), "chosen_labels": self._pad([b for _, b in ch], -100),
                "rejected": self._pad([a for a, _ in rj], self.pad), "rejected_labels": self._pad([b for _, b in rj], -100)}

    def singles(self, records: Sequence[Dict[str, Any]]) -> Dict[str, torch.Tensor]:
        enc = [self._encode(r["prompt"], r["completion"]) for r in records]
        return {"input_ids": self._pad([a for a, _ in enc], self.pad), "labels": self._pad([b for _, b in enc], -100),
                "desirable": torch.tensor([bool(r["label"]) for r in records])}


class PiscesLxRewardNormalizer:
    """Running mean / variance of rewards (Welford, batched) with clipping of the normalised value; what PPO / GRPO
    style trainers put between a reward model and the advantage computation so that the reward scale of one task
    does not set the step size for all (reference opss/train/grpo.py normalises group rewards the same way)."""

    def __init__(self, clip: float = 5.0, eps: float = 1e-8):
        self.clip, self.eps = clip, eps
        self.count, self.mean, self.m2 = 0.0, 0.0, 0.0

    def update(self, rewards: torch.Tensor) -> None:
        r = rewards.detach().double().flatten()
        n = float(r.numel())
        if n == 0:
            return
        b_mean, b_m2 = float(r.mean()), float(((r - r.mean()) ** 2).sum())
        delta = b_mean - self.mean
        tot = self.count + n
        self.mean += delta * n / tot
        self.m2 += b_m2 + delta * delta * self.count * n / tot
        self.count = tot

    @property
    def std(self) -> float:
        return (self.m2 / max(self.count - 1.0, 1.0)) ** 0.5 if self.count > 1 else 1.0

    def __call__(self, rewards: torch.Tensor, update: bool = True) -> torch.Tensor:
        if update:
            self.update(rewards)
        return ((rewards - self.mean) / (self.std + self.eps)).clamp(-self.clip, self.clip)

    def state_dict(self) -> Dict[str, float]:
        return {"count": self.count, "mean": self.mean, "m2": self.m2}

    def load_state_dict(self, sd: Dict[str, float]) -> None:
        self.count, self.mean, self.m2 = float(sd["count"]), float(sd["mean"]), float(sd["m2"])


class PiscesLxGenerativeRewardModel:
    """Reward from a generated judgement: the judge model is prompted with the question and the candidate answer,
    writes a short critique ending in ``Score: n/10`` and the number becomes the reward (reference "GRM": a reward
    model that reasons before it scores).  ``generate(prompt, max_new_tokens) -> text``."""

    PROMPT = ("Question:\n{question}\n\nCandidate answer:\n{answer}\n\n"
              "Critique the answer briefly, then finish with 'Score: n/10'.\n")

    def __init__(self, generate, max_new_tokens: int = 128, default: float = 0.0, normalizer: Optional[PiscesLxRewardNormalizer] = None):
        self.generate, self.max_new_tokens, self.default, self.normalizer = generate, max_new_tokens, default, normalizer

    @staticmethod
    def parse(text: str) -> Optional[float]:
        import re
        m = re.findall(r"score\s*[:=]\s*(\d+(?:\.\d+)?)\s*(?:/\s*10)?", text, re.I)
        return min(10.0, float(m[-1])) / 10.0 if m else None

    def score(self, question: str, answers: List[str]) -> torch.Tensor:
        vals = []
        for a in answers:
            s = self.parse(self.generate(self.PROMPT.format(question=question, answer=a), self.max_new_tokens))
            vals.append(self.default if s is None else s)
        r = torch.tensor(vals, dtype=torch.float32)
        return self.normalizer(r) if self.normalizer is not None else r
