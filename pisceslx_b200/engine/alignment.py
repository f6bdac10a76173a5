"""Post-training objectives: SFT, DPO / IPO, ORPO, KTO, BCO, PPO (clipped surrogate + value loss + GAE), GRPO / DAPO
(group-relative advantages, asymmetric clipping, dynamic sampling), RLVR (verifiable rewards), knowledge
distillation (logit / hidden-state / attention), weak-to-strong confidence loss, and model growth (depth / width /
expert).  They correspond to the reference's stage operators (opss/train/sft.py, dpo.py, pref_align.py, grpo.py,
dapo.py, rlvr.py, distill_loss.py, weak_to_strong.py, growth.py; stage dispatch tools/train/core.py:1951-1984) as
plain loss functions over model outputs plus small trainers that drive ``YvTrainer``-style steps.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------------------
# sequence log-probabilities
# --------------------------------------------------------------------------------------------------
def sequence_logprobs(model: Any, input_ids: torch.Tensor, labels: torch.Tensor, average: bool = False) -> torch.Tensor:
    """Sum (or mean) of token log-probabilities of ``labels`` (shifted inside; -100 positions ignored)."""
    logits = model(input_ids=input_ids, return_logits=True).logits[:, :-1].float()
    tgt = labels[:, 1:]
    mask = tgt != -100
    lp = torch.log_softmax(logits, -1).gather(-1, tgt.clamp_min(0).unsqueeze(-1)).squeeze(-1) * mask
    s = lp.sum(-1)
    return s / mask.sum(-1).clamp_min(1) if average else s


def sft_loss(model: Any, input_ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    return model(input_ids=input_ids, labels=labels).loss


# --------------------------------------------------------------------------------------------------
# preference objectives
# --------------------------------------------------------------------------------------------------
def dpo_loss(pi_chosen: torch.Tensor, pi_rejected: torch.Tensor, ref_chosen: torch.Tensor, ref_rejected: torch.Tensor,
             beta: float = 0.1, label_smoothing: float = 0.0, ipo: bool = False) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    logits = (pi_chosen - pi_rejected) - (ref_chosen - ref_rejected)
    if ipo:
        loss = (logits - 1.0 / (2.0 * beta)).pow(2)
    else:
        loss = -(1 - label_smoothing) * F.logsigmoid(beta * logits) - label_smoothing * F.logsigmoid(-beta * logits)
    stats = {"reward_chosen": beta * (pi_chosen - ref_chosen).detach(), "reward_rejected": beta * (pi_rejected - ref_rejected).detach(),
             "accuracy": (logits > 0).float().mean().detach()}
    return loss.mean(), stats


def orpo_loss(nll_chosen: torch.Tensor, avg_lp_chosen: torch.Tensor, avg_lp_rejected: torch.Tensor, lam: float = 0.1) -> torch.Tensor:
    """SFT loss on the chosen answer + lambda * odds-ratio term (no reference model)."""
    def log_odds(lp):
        return lp - torch.log1p(-torch.exp(lp).clamp(max=1 - 1e-6))
    ratio = log_odds(avg_lp_chosen) - log_odds(avg_lp_rejected)
    return nll_chosen - lam * F.logsigmoid(ratio).mean()


def kto_loss(pi_lp: torch.Tensor, ref_lp: torch.Tensor, desirable: torch.Tensor, beta: float = 0.1,
             lambda_d: float = 1.0, lambda_u: float = 1.0, kl_ref: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``kl_ref``: the reference point (an estimate of KL(policy || reference), detached); by default the batch mean of
    the implicit reward, clamped at zero."""
    r = pi_lp - ref_lp
    z = r.detach().mean().clamp_min(0) if kl_ref is None else kl_ref.detach()
    pos = lambda_d * (1 - torch.sigmoid(beta * (r - z)))
    neg = lambda_u * (1 - torch.sigmoid(beta * (z - r)))
    return torch.where(desirable.bool(), pos, neg).mean()


def bco_loss(pi_lp: torch.Tensor, ref_lp: torch.Tensor, desirable: torch.Tensor, beta: float = 0.1,
             delta: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Binary classifier optimisation: logistic loss on the implicit reward shifted by a running mean."""
    r = beta * (pi_lp - ref_lp)
    d = r.detach().mean() if delta is None else delta
    y = desirable.float()
    return F.binary_cross_entropy_with_logits(r - d, y)


# --------------------------------------------------------------------------------------------------
# policy-gradient objectives
# --------------------------------------------------------------------------------------------------
def gae(rewards: torch.Tensor, values: torch.Tensor, gamma: float = 1.0, lam: float = 0.95) -> Tuple[torch.Tensor, torch.Tensor]:
    """rewards / values [B, T] -> (advantages, returns)."""
    B, T = rewards.shape
    adv = torch.zeros_like(rewards)
    last = torch.zeros(B, device=rewards.device)
    for t in reversed(range(T)):
        nxt = values[:, t + 1] if t + 1 < T else torch.zeros(B, device=rewards.device)
        delta = rewards[:, t] + gamma * nxt - values[:, t]
        last = delta + gamma * lam * last
        adv[:, t] = last
    return adv, adv + values


def ppo_loss(logp: torch.Tensor, old_logp: torch.Tensor, adv: torch.Tensor, values: Optional[torch.Tensor] = None,
             returns: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None, clip: float = 0.2,
             clip_high: Optional[float] = None, vf_coef: float = 0.5, kl_coef: float = 0.0,
             ref_logp: Optional[torch.Tensor] = None) -> torch.Tensor:
    mask = torch.ones_like(logp) if mask is None else mask.float()
    ratio = torch.exp(logp - old_logp)
    hi = clip if clip_high is None else clip_high
    surr = torch.minimum(ratio * adv, ratio.clamp(1 - clip, 1 + hi) * adv)
    loss = -(surr * mask).sum() / mask.sum().clamp_min(1)
    if values is not None and returns is not None:
        loss = loss + vf_coef * (((values - returns) ** 2) * mask).sum() / mask.sum().clamp_min(1)
    if kl_coef and ref_logp is not None:
        d = ref_logp - logp
        kl = torch.exp(d) - d - 1                                   # k3 estimator
        loss = loss + kl_coef * (kl * mask).sum() / mask.sum().clamp_min(1)
    return loss


def group_relative_advantages(rewards: torch.Tensor, group_size: int, eps: float = 1e-6) -> torch.Tensor:
    """GRPO: rewards [N] of N = groups * group_size samples -> advantages normalised inside every group."""
    r = rewards.view(-1, group_size)
    return ((r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True) + eps)).view(-1)


def grpo_loss(logp: torch.Tensor, old_logp: torch.Tensor, rewards: torch.Tensor, group_size: int,
              mask: Optional[torch.Tensor] = None, clip: float = 0.2, clip_high: Optional[float] = None,
              kl_coef: float = 0.0, ref_logp: Optional[torch.Tensor] = None) -> torch.Tensor:
    """logp / old_logp [N, T] token log-probs; rewards [N] sequence rewards."""
    adv = group_relative_advantages(rewards, group_size).unsqueeze(-1).expand_as(logp)
    return ppo_loss(logp, old_logp, adv, mask=mask, clip=clip, clip_high=clip_high, kl_coef=kl_coef, ref_logp=ref_logp)


def dapo_filter_groups(rewards: torch.Tensor, group_size: int) -> torch.Tensor:
    """DAPO dynamic sampling: keep only groups whose rewards are not all equal (zero-advantage groups carry no
    gradient).  Returns a boolean mask over samples."""
    r = rewards.view(-1, group_size)
    keep = (r.max(1).values - r.min(1).values) > 0
    return keep.unsqueeze(1).expand_as(r).reshape(-1)


def dapo_loss(logp, old_logp, rewards, group_size, mask=None, eps_low: float = 0.2, eps_high: float = 0.28):
    """GRPO with decoupled (asymmetric) clipping and token-level normalisation."""
    keep = dapo_filter_groups(rewards, group_size).unsqueeze(-1).float()
    mask = keep if mask is None else mask.float() * keep
    return grpo_loss(logp, old_logp, rewards, group_size, mask=mask, clip=eps_low, clip_high=eps_high)


class PiscesLxRLVRVerifier:
    """Verifiable rewards: exact match, numeric equality within a tolerance, or a user predicate."""

    def __init__(self, kind: str = "exact", tol: float = 1e-6, predicate: Optional[Callable[[str, str], bool]] = None):
        self.kind, self.tol, self.predicate = kind, tol, predicate

    def reward(self, answer: str, truth: str) -> float:
        if self.predicate is not None:
            return float(self.predicate(answer, truth))
        if self.kind == "numeric":
            try:
                return float(abs(float(answer.strip()) - float(truth.strip())) <= self.tol)
            except ValueError:
                return 0.0
        return float(answer.strip() == truth.strip())


# --------------------------------------------------------------------------------------------------
# distillation / weak-to-strong
# --------------------------------------------------------------------------------------------------
def distill_logits_loss(student: torch.Tensor, teacher: torch.Tensor, temperature: float = 2.0,
                        mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    t = temperature
    kl = F.kl_div(torch.log_softmax(student.float() / t, -1), torch.softmax(teacher.float() / t, -1), reduction="none").sum(-1)
    if mask is not None:
        return (kl * mask).sum() / mask.sum().clamp_min(1) * t * t
    return kl.mean() * t * t


def distill_hidden_loss(student_h: torch.Tensor, teacher_h: torch.Tensor, proj: Optional[torch.nn.Module] = None) -> torch.Tensor:
    s = proj(student_h) if proj is not None else student_h
    return F.mse_loss(F.normalize(s.float(), dim=-1), F.normalize(teacher_h.float(), dim=-1))


def distill_attention_loss(student_attn: torch.Tensor, teacher_attn: torch.Tensor) -> torch.Tensor:
    return F.kl_div(torch.log(student_attn.float().clamp_min(1e-9)), teacher_attn.float(), reduction="batchmean")


def weak_to_strong_loss(strong_logits: torch.Tensor, weak_labels: torch.Tensor, alpha: float = 0.5) -> torch.Tensor:
    """Auxiliary-confidence loss: mix the weak supervisor's labels with the strong model's own hardened predictions."""
    own = strong_logits.detach().argmax(-1)
    return (1 - alpha) * F.cross_entropy(strong_logits.float(), weak_labels) + alpha * F.cross_entropy(strong_logits.float(), own)


# --------------------------------------------------------------------------------------------------
# small trainers
# --------------------------------------------------------------------------------------------------
class PiscesLxDPOTrainingOperator:
    def __init__(self, model: Any, optimizer: torch.optim.Optimizer, beta: float = 0.1, ref_model: Any = None):
        self.model, self.opt, self.beta = model, optimizer, beta
        self.ref = ref_model or copy.deepcopy(model).eval().requires_grad_(False)

    def step(self, chosen: torch.Tensor, rejected: torch.Tensor, chosen_labels: torch.Tensor, rejected_labels: torch.Tensor):
        pc, pr = sequence_logprobs(self.model, chosen, chosen_labels), sequence_logprobs(self.model, rejected, rejected_labels)
        with torch.no_grad():
            rc, rr = sequence_logprobs(self.ref, chosen, chosen_labels), sequence_logprobs(self.ref, rejected, rejected_labels)
        loss, stats = dpo_loss(pc, pr, rc, rr, self.beta)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return float(loss), {k: float(v.mean()) for k, v in stats.items()}


class PiscesLxGRPOTrainer:
    """Sample ``group_size`` completions per prompt, score them, update with the group-relative objective."""

    def __init__(self, model: Any, optimizer: torch.optim.Optimizer, reward_fn: Callable[[torch.Tensor], float],
                 group_size: int = 4, max_new_tokens: int = 16, clip: float = 0.2):
        self.model, self.opt, self.reward_fn = model, optimizer, reward_fn
        self.group_size, self.max_new_tokens, self.clip = group_size, max_new_tokens, clip

    def step(self, prompt: torch.Tensor) -> Dict[str, float]:
        from ..models.generation import YvSampler, YvSamplingConfig
        seqs, rewards = [], []
        for g in range(self.group_size):
            out, _ = self.model.generate(prompt, max_new_tokens=self.max_new_tokens, eos_token_id=-1,
                                         sampler=YvSampler(YvSamplingConfig(strategy="top_k_top_p", temperature=1.0, top_k=50,
                                                                             top_p=1.0, seed=1000 + g)))
            seqs.append(out[0])
            rewards.append(self.reward_fn(out[0]))
        ids = torch.stack(seqs)
        labels = ids.clone()
        labels[:, : prompt.shape[1]] = -100
        self.model.train()

        def token_lp(m):
            lg = m(input_ids=ids, return_logits=True).logits[:, :-1].float()
            return torch.log_softmax(lg, -1).gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1)

        with torch.no_grad():
            old = token_lp(self.model)
        lp = token_lp(self.model)
        mask = (labels[:, 1:] != -100).float()
        loss = grpo_loss(lp, old, torch.tensor(rewards, device=ids.device), self.group_size, mask=mask, clip=self.clip)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return {"loss": float(loss), "mean_reward": sum(rewards) / len(rewards)}


# --------------------------------------------------------------------------------------------------
# model growth
# --------------------------------------------------------------------------------------------------
def grow_experts(layer: Any, new_total: int, noise: float = 1e-3) -> None:
    """Expert growth: duplicate existing routed experts (plus small noise) up to ``new_total`` and widen the router."""
    old = layer.experts_w13.shape[0]
    assert new_total >= old
    idx = torch.arange(new_total) % old
    for name in ("experts_w13", "experts_w2"):
        w = getattr(layer, name).data
        grown = w[idx].clone()
        grown[old:] += noise * torch.randn_like(grown[old:])
        setattr(layer, name, torch.nn.Parameter(grown))
    gate = layer.router.gate
    gw = gate.weight.data[idx].clone()
    new_gate = torch.nn.Linear(gate.in_features, new_total, bias=False).to(gw.device, gw.dtype)
    new_gate.weight.data.copy_(gw)
    layer.router.gate = new_gate
    layer.router.num_experts = layer.num_experts = layer.num_local = new_total
    layer.router.expert_bias = torch.zeros(new_total, device=gw.device)
    layer.router.usage_counts = torch.zeros(new_total, dtype=torch.int32, device=gw.device)


def grow_depth(model: Any, positions: Sequence[int]) -> None:
    """Depth growth: insert copies of existing blocks after the given layer indices (function-preserving up to the
    residual contribution of the copied block being small; callers usually zero the copy's output projections)."""
    layers = list(model.model.layers)
    for p in sorted(positions, reverse=True):
        clone = copy.deepcopy(layers[p])
        with torch.no_grad():
            clone.attention.o_proj.zero_()
            if hasattr(clone.mlp, "experts_w2"):
                clone.mlp.experts_w2.zero_()
                if clone.mlp.num_shared:
                    clone.mlp.shared_w2.zero_()
            else:
                clone.mlp.w2.zero_()
        layers.insert(p + 1, clone)
    for i, blk in enumerate(layers):
        blk.layer_idx = i
        blk.attention.layer_idx = i
    model.model.layers = torch.nn.ModuleList(layers)
    model.cfg.n_layer = len(layers)
    model.model.layer_hi = len(layers)


def grow_expert_width(layer: Any, new_ffn: int) -> None:
    """Width growth of the routed experts (function preserving): the FFN dimension grows from F to ``new_ffn``; new
    gate/up rows are small random, the matching new columns of the down projection are zero, so the layer's output is
    unchanged until training moves them."""
    w13, w2 = layer.experts_w13.data, layer.experts_w2.data          # [E, 2F, H], [E, H, F]
    E, twoF, H = w13.shape
    F = twoF // 2
    assert new_ffn >= F
    g13 = torch.zeros(E, 2 * new_ffn, H, dtype=w13.dtype, device=w13.device)
    g13[:, :F], g13[:, new_ffn:new_ffn + F] = w13[:, :F], w13[:, F:]
    g13[:, F:new_ffn].normal_(std=0.02)
    g13[:, new_ffn + F:].normal_(std=0.02)
    g2 = torch.zeros(E, H, new_ffn, dtype=w2.dtype, device=w2.device)
    g2[:, :, :F] = w2
    layer.experts_w13, layer.experts_w2 = torch.nn.Parameter(g13), torch.nn.Parameter(g2)
    layer.ffn = new_ffn


# --------------------------------------------------------------------------------------------------
# self-play and weak-to-strong (reference opss/train: self-play fine-tuning, weak-to-strong generalisation)
# --------------------------------------------------------------------------------------------------
def spin_loss(pi_real: torch.Tensor, pi_synth: torch.Tensor, ref_real: torch.Tensor, ref_synth: torch.Tensor,
              beta: float = 0.1) -> torch.Tensor:
    """Self-play fine-tuning: the current policy must prefer the data's response over the one its previous iterate
    (the opponent, also the reference) generated for the same prompt: logistic loss on the margin of log-ratios."""
    margin = beta * ((pi_real - ref_real) - (pi_synth - ref_synth))
    return -torch.nn.functional.logsigmoid(margin).mean()


class PiscesLxSelfPlayTrainer:
    """Iterated self-play: each round freezes a copy of the policy as opponent, has it answer the prompts
    (``generate_fn(opponent, prompt_ids) -> response_ids``), and trains the policy with ``spin_loss`` to tell the
    data's responses from the opponent's.  ``logprob_fn(model, prompt_ids, response_ids) -> summed log-prob``."""

    def __init__(self, policy: torch.nn.Module, optimizer: torch.optim.Optimizer, generate_fn, logprob_fn,
                 beta: float = 0.1):
        self.policy, self.opt, self.generate_fn, self.logprob_fn, self.beta = policy, optimizer, generate_fn, logprob_fn, beta
        self.opponent: Optional[torch.nn.Module] = None
        self.round = 0

    def start_round(self) -> None:
        self.opponent = copy.deepcopy(self.policy).eval()
        for p in self.opponent.parameters():
            p.requires_grad_(False)
        self.round += 1

    def step(self, prompts: Sequence[torch.Tensor], responses: Sequence[torch.Tensor]) -> Dict[str, float]:
        if self.opponent is None:
            self.start_round()
        with torch.no_grad():
            synth = [self.generate_fn(self.opponent, p) for p in prompts]
            ref_real = torch.stack([self.logprob_fn(self.opponent, p, r) for p, r in zip(prompts, responses)])
            ref_synth = torch.stack([self.logprob_fn(self.opponent, p, s) for p, s in zip(prompts, synth)])
        pi_real = torch.stack([self.logprob_fn(self.policy, p, r) for p, r in zip(prompts, responses)])
        pi_synth = torch.stack([self.logprob_fn(self.policy, p, s) for p, s in zip(prompts, synth)])
        loss = spin_loss(pi_real, pi_synth, ref_real, ref_synth, self.beta)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return {"loss": float(loss.detach()), "margin": float(((pi_real - ref_real) - (pi_synth - ref_synth)).mean().detach()),
                "round": self.round}


class PiscesLxWeakToStrongTrainer:
    """Weak-to-strong generalisation: a strong student is trained on a weak supervisor's labels with the auxiliary
    confidence loss (``weak_to_strong_loss``): as training proceeds the student's own hardened predictions get weight
    ``alpha`` (warmed up linearly), so it can overrule the supervisor's mistakes."""

    def __init__(self, student: torch.nn.Module, optimizer: torch.optim.Optimizer, alpha_max: float = 0.5,
                 warmup_steps: int = 100):
        self.student, self.opt, self.alpha_max, self.warmup = student, optimizer, alpha_max, warmup_steps
        self.steps = 0

    def step(self, inputs: torch.Tensor, weak_labels: torch.Tensor) -> Dict[str, float]:
        alpha = self.alpha_max * min(1.0, self.steps / max(1, self.warmup))
        logits = self.student(inputs)
        loss = weak_to_strong_loss(logits, weak_labels, alpha)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        self.steps += 1
        agree = float((logits.argmax(-1) == weak_labels).float().mean())
        return {"loss": float(loss.detach()), "alpha": alpha, "agreement_with_weak": agree}
