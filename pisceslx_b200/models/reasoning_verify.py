"""Reasoning verification and self-adaptation (reference model/reasoning/verification.py: ``YvCRV`` :42, ``YvOTV``
:136, ``YvARES`` :208, ``YvCRVIntegration`` :264; model/reasoning/self_evolution.py: ``YvSEAL`` :41, ``YvSOLAR``
:237; model/reasoning/ttt_e2e.py:43 ``YvTestTimeTrainer``).  All of it is off the throughput path: the trainer
leaves these switched off and the serving engine never calls them inside a decode step."""
from __future__ import annotations

import copy
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class YvCRV(nn.Module):
    """Step-to-step consistency check over the hidden states of reasoning steps: a bilinear detector scores each
    pair of consecutive steps for contradiction; a chain is consistent when no pair exceeds ``threshold``."""

    def __init__(self, hidden: int, threshold: float = 0.5):
        super().__init__()
        self.detector = nn.Sequential(nn.Linear(3 * hidden, hidden // 2 or 1), nn.GELU(), nn.Linear(hidden // 2 or 1, 1))
        self.threshold = threshold

    def pair_scores(self, steps: torch.Tensor) -> torch.Tensor:
        """steps [N, H] (one pooled hidden state per reasoning step) -> contradiction probability [N-1]."""
        a, b = steps[:-1].float(), steps[1:].float()
        return torch.sigmoid(self.detector(torch.cat([a, b, a * b], -1))).squeeze(-1)

    def forward(self, steps: torch.Tensor) -> Dict[str, Any]:
        if steps.shape[0] < 2:
            return {"consistent": True, "scores": steps.new_zeros(0), "first_bad_step": None}
        s = self.pair_scores(steps)
        bad = (s > self.threshold).nonzero().flatten()
        return {"consistent": bad.numel() == 0, "scores": s, "first_bad_step": int(bad[0]) + 1 if bad.numel() else None}


class YvCRVIntegration(nn.Module):
    """Collects pooled per-layer hidden states as pseudo reasoning steps during a forward and verifies them."""

    def __init__(self, hidden: int, keep: int = 16):
        super().__init__()
        self.crv, self.keep = YvCRV(hidden), keep
        self.checkpoints: List[torch.Tensor] = []

    def record(self, h: torch.Tensor) -> None:
        self.checkpoints.append(h.detach().float().mean(dim=tuple(range(h.dim() - 1))))
        del self.checkpoints[:-self.keep]

    def verify(self) -> Dict[str, Any]:
        out = self.crv(torch.stack(self.checkpoints)) if self.checkpoints else {"consistent": True}
        self.checkpoints.clear()
        return out


class YvOTV(nn.Module):
    """One-token verification: the hidden state of the last token of each step is scored by a linear probe; one
    forward per step, no pairwise analysis."""

    def __init__(self, hidden: int):
        super().__init__()
        self.scorer = nn.Linear(hidden, 1)

    def forward(self, last_hidden: torch.Tensor) -> torch.Tensor:
        return torch.sigmoid(self.scorer(last_hidden.float())).squeeze(-1)

    def filter_steps(self, last_hidden: torch.Tensor, min_quality: float = 0.5) -> torch.Tensor:
        return self.forward(last_hidden) >= min_quality


class YvARES(nn.Module):
    """Entailment stability: the probability that step i is entailed by the steps before it (mean of the earlier
    states as the premise); the chain's score is the product, i.e. the probability that every step holds."""

    def __init__(self, hidden: int):
        super().__init__()
        self.scorer = nn.Sequential(nn.Linear(2 * hidden, hidden), nn.GELU(), nn.Linear(hidden, 1))

    def forward(self, steps: torch.Tensor) -> Dict[str, torch.Tensor]:
        s = steps.float()
        prem = s.cumsum(0)[:-1] / torch.arange(1, s.shape[0], device=s.device)[:, None]
        p = torch.sigmoid(self.scorer(torch.cat([prem, s[1:]], -1))).squeeze(-1)
        return {"step_entailment": p, "chain_soundness": p.prod() if p.numel() else s.new_ones(())}


class YvTestTimeTrainer:
    """Adapts the last ``update_layers`` layers on the prompt itself (next-token loss) for a few small steps, then
    restores the weights: ``with ttt.adapted(input_ids): model.generate(...)``."""

    def __init__(self, model: nn.Module, update_layers: int = 2, lr: float = 1e-5, max_steps: int = 3,
                 min_tokens: int = 32):
        self.model, self.n, self.lr, self.max_steps, self.min_tokens = model, update_layers, lr, max_steps, min_tokens

    def _params(self) -> List[nn.Parameter]:
        layers = list(self.model.model.layers)[-self.n:] if self.n else []
        return [p for l in layers for p in l.parameters() if p.is_floating_point()]

    def adapt(self, input_ids: torch.Tensor) -> Dict[str, Any]:
        ps = self._params()
        if input_ids.shape[1] < self.min_tokens or not ps:
            return {"steps": 0, "snapshot": None}
        snap = [p.detach().clone() for p in ps]
        was_training = self.model.training
        req = [p.requires_grad for p in self.model.parameters()]
        for p in self.model.parameters():
            p.requires_grad_(False)
        for p in ps:
            p.requires_grad_(True)
        self.model.train()
        losses = []
        for _ in range(self.max_steps):
            out = self.model(input_ids=input_ids, labels=input_ids)
            loss = out["loss"]
            grads = torch.autograd.grad(loss, ps, allow_unused=True)
            with torch.no_grad():
                for p, g in zip(ps, grads):
                    if g is not None:
                        p.add_(g.to(p.dtype), alpha=-self.lr)
            losses.append(float(loss.detach()))
        for p, r in zip(self.model.parameters(), req):
            p.requires_grad_(r)
        self.model.train(was_training)
        return {"steps": len(losses), "losses": losses, "snapshot": (ps, snap)}

    @staticmethod
    def restore(state: Dict[str, Any]) -> None:
        if state.get("snapshot"):
            ps, snap = state["snapshot"]
            with torch.no_grad():
                for p, s in zip(ps, snap):
                    p.copy_(s)

    def adapted(self, input_ids: torch.Tensor):
        trainer = self

        class _Ctx:
            def __enter__(self_inner):
                self_inner.state = trainer.adapt(input_ids)
                return self_inner.state

            def __exit__(self_inner, *exc):
                trainer.restore(self_inner.state)
                return False
        return _Ctx()


class YvSEAL:
    """Self-adapting loop: generate -> keep outputs whose mean token confidence passes ``confidence_threshold`` (and
    that an optional verifier accepts) -> fine-tune on them for a step.  ``generate_fn(prompt_ids) -> (ids, conf)``
    and ``train_fn(batch_ids) -> loss`` are supplied by the caller, so that the loop works with any engine."""

    def __init__(self, generate_fn: Callable, train_fn: Callable, confidence_threshold: float = 0.9,
                 max_synthetic_samples: int = 64, verifier: Optional[Callable[[torch.Tensor], bool]] = None):
        self.generate_fn, self.train_fn = generate_fn, train_fn
        self.thr, self.max_n, self.verifier = confidence_threshold, max_synthetic_samples, verifier
        self.buffer: List[torch.Tensor] = []

    def collect(self, prompts: Iterable[torch.Tensor]) -> int:
        kept = 0
        for p in prompts:
            ids, conf = self.generate_fn(p)
            if float(conf) >= self.thr and (self.verifier is None or self.verifier(ids)):
                self.buffer.append(ids)
                kept += 1
            if len(self.buffer) >= self.max_n:
                break
        return kept

    def self_edit(self) -> Optional[float]:
        if not self.buffer:
            return None
        loss = float(self.train_fn(self.buffer))
        self.buffer.clear()
        return loss


class YvSOLAR:
    """Parameter-level meta-optimisation: each parameter tensor keeps its own log step size, raised when successive
    gradients agree in sign and lowered when they disagree (a sign-agreement hypergradient), within bounds."""

    def __init__(self, params: Iterable[nn.Parameter], meta_lr: float = 0.05, lr: float = 1e-3,
                 bounds: Tuple[float, float] = (0.1, 10.0)):
        self.params = [p for p in params if p.requires_grad]
        self.meta_lr, self.lr, self.bounds = meta_lr, lr, bounds
        self.scale = [1.0 for _ in self.params]
        self.prev: List[Optional[torch.Tensor]] = [None for _ in self.params]

    @torch.no_grad()
    def step(self) -> None:
        for i, p in enumerate(self.params):
            if p.grad is None:
                continue
            g = p.grad
            if self.prev[i] is not None:
                agree = float((g * self.prev[i]).sum().sign())
                self.scale[i] = min(self.bounds[1], max(self.bounds[0], self.scale[i] * (1 + self.meta_lr * agree)))
            self.prev[i] = g.detach().clone()
            p.add_(g, alpha=-self.lr * self.scale[i])


# ----------------------------------------------------------------------------------------------------------------------
# VeriCoT on hidden states (reference model/reasoning/vericot.py:42-230).  The text-level checker of arithmetic
# statements is ``models.reasoning.YvVeriCoTVerifier``; the pair below scores a reasoning step's hidden state
# against its context and nudges low-scoring steps, and can call the text checker for a symbolic score.
# ----------------------------------------------------------------------------------------------------------------------
class YvVeriCoTStepVerifier(nn.Module):
    """Step / context projections -> validity in (0, 1).  Without a context the score is the neutral 0.5.  When
    ``step_text`` is given the arithmetic statements in it are checked symbolically and the result is reported (and
    folded into ``combined_score`` with weight ``symbolic_weight``)."""

    def __init__(self, hidden_size: int, proj_dim: Optional[int] = None, ramp_steps: int = 1000,
                 symbolic_weight: float = 0.5):
        super().__init__()
        p = proj_dim or max(8, hidden_size // 2)
        self.questioner_proj = nn.Linear(hidden_size, p)
        self.responder_proj = nn.Linear(hidden_size, p)
        self.quality_estimator = nn.Sequential(nn.Linear(2 * p, p), nn.GELU(), nn.Linear(p, 1), nn.Sigmoid())
        self.ramp_steps, self.symbolic_weight = ramp_steps, symbolic_weight
        self.register_buffer("calls", torch.zeros((), dtype=torch.long))

    @staticmethod
    def _pool(h: torch.Tensor) -> torch.Tensor:
        return h if h.dim() == 2 else h.mean(1)

    def forward(self, step_hidden: torch.Tensor, context_hidden: Optional[torch.Tensor] = None, step_text: str = "",
                return_details: bool = False) -> Dict[str, Any]:
        q = self.questioner_proj(self._pool(step_hidden).float())
        if context_hidden is not None:
            r = self.responder_proj(self._pool(context_hidden).float())
            quality = self.quality_estimator(torch.cat([q, r.expand_as(q)], -1)).squeeze(-1)
        else:
            quality = torch.full((q.shape[0],), 0.5, device=q.device)
        symbolic = None
        if step_text:
            from .reasoning import YvReasoningTrace, YvVeriCoTVerifier
            symbolic = 1.0 if YvVeriCoTVerifier().verify(YvReasoningTrace(steps=[step_text], answer="")) else 0.0
        combined = quality if symbolic is None else (1 - self.symbolic_weight) * quality + self.symbolic_weight * symbolic
        self.calls += 1
        out = {"validity_score": quality, "consistency_score": quality, "combined_score": combined,
               "is_valid": combined > 0.5, "symbolic_score": symbolic if symbolic is not None else 0.0}
        if return_details:
            out["ramp"] = min(1.0, float(self.calls) / max(self.ramp_steps, 1))
        return out

    def verify_chain(self, step_hiddens: Sequence[torch.Tensor], step_texts: Optional[Sequence[str]] = None,
                     context_hidden: Optional[torch.Tensor] = None) -> Dict[str, Any]:
        """Every step against the running context (the given context, then the mean of the steps seen so far)."""
        results, ctx = [], context_hidden
        for i, h in enumerate(step_hiddens):
            results.append(self.forward(h, ctx, step_texts[i] if step_texts else ""))
            pooled = self._pool(h).detach()
            ctx = pooled if ctx is None else 0.5 * (self._pool(ctx) + pooled)
        valid = [bool(r["is_valid"].all()) for r in results]
        score = torch.stack([r["combined_score"].mean() for r in results]).mean() if results else torch.tensor(0.0)
        return {"steps": results, "num_valid": sum(valid), "all_valid": all(valid), "chain_score": score,
                "first_invalid": valid.index(False) if not all(valid) else None}

    def compute_reflection(self, step_hidden: torch.Tensor, result: Dict[str, Any]) -> torch.Tensor:
        """Push a step away from itself in proportion to how invalid it scored (reference :174-190)."""
        q = result["validity_score"].to(step_hidden.dtype)
        q = q.view(-1, *([1] * (step_hidden.dim() - 1)))
        return step_hidden + (1.0 - q) * step_hidden * 0.1


class YvVeriCoTReflector(nn.Module):
    """verify -> reflect loop, at most ``max_reflections`` times (reference :192-230)."""

    def __init__(self, verifier: YvVeriCoTStepVerifier, max_reflections: int = 3):
        super().__init__()
        self.verifier, self.max_reflections = verifier, max_reflections
        self.register_buffer("rounds", torch.zeros((), dtype=torch.long))

    def forward(self, step_hidden: torch.Tensor, context_hidden: Optional[torch.Tensor] = None,
                step_text: str = "") -> Tuple[torch.Tensor, Dict[str, Any]]:
        cur, n = step_hidden, 0
        res = self.verifier(cur, context_hidden, step_text, return_details=True)
        while not bool(res["is_valid"].all()) and n < self.max_reflections:
            cur = self.verifier.compute_reflection(cur, res)
            n += 1
            res = self.verifier(cur, context_hidden, step_text, return_details=True)
        self.rounds += 1
        return cur, {"reflections": n, "final_valid": res["is_valid"], "final_validity": res["validity_score"],
                     "round": int(self.rounds)}


class YvAgenticEvolution(nn.Module):
    """A population of copies of one model under selection and mutation (reference self_evolution.py:151-235):
    score every agent on a task, keep the top fraction, overwrite the others with noisy copies of the survivors."""

    def __init__(self, base_model: nn.Module, num_agents: int = 4, mutation_rate: float = 0.01,
                 selection_pressure: float = 0.5):
        super().__init__()
        self.num_agents, self.mutation_rate, self.selection_pressure = num_agents, mutation_rate, selection_pressure
        self.agents = nn.ModuleList([copy.deepcopy(base_model) for _ in range(num_agents)])
        self.agent_scores = torch.zeros(num_agents)
        self.generation = 0

    @torch.no_grad()
    def evaluate_agents(self, task_inputs: torch.Tensor, task_labels: torch.Tensor,
                        score_fn: Optional[Callable[[torch.Tensor, torch.Tensor], float]] = None) -> torch.Tensor:
        for i, agent in enumerate(self.agents):
            out = agent(task_inputs)
            out = out["logits"] if isinstance(out, dict) else out
            if score_fn is not None:
                self.agent_scores[i] = float(score_fn(out, task_labels))
            elif out.dim() == task_labels.dim() + 1:
                self.agent_scores[i] = float((out.argmax(-1) == task_labels).float().mean())
            else:
                self.agent_scores[i] = -float(F.mse_loss(out.float(), task_labels.float()))
        return self.agent_scores

    @torch.no_grad()
    def evolve_population(self, generator: Optional[torch.Generator] = None) -> List[int]:
        keep = max(1, int(self.num_agents * self.selection_pressure))
        top = torch.topk(self.agent_scores, keep).indices.tolist()
        for i in range(self.num_agents):
            if i in top:
                continue
            parent = self.agents[top[i % keep]]
            for pa, pp in zip(self.agents[i].parameters(), parent.parameters()):
                noise = torch.randn(pp.shape, generator=generator).to(pp) * self.mutation_rate
                pa.copy_(pp + noise)
        self.generation += 1
        return top

    def best(self) -> nn.Module:
        return self.agents[int(self.agent_scores.argmax())]


class YvVerificationFactory:
    """Module-level verification operations behind one class (reference verification.py:306-420)."""

    @staticmethod
    def detect_cot_failure_modes(reasoning_steps: List[str], final_answer: str) -> List[Tuple[str, float]]:
        fails: List[Tuple[str, float]] = []
        steps = [s.strip().lower() for s in reasoning_steps]
        if len(steps) < 3 and len(final_answer.split()) > 5:
            fails.append(("premature_conclusion", 0.7))
        if any(a and b and (a in b or b in a) for i, a in enumerate(steps) for b in steps[i + 1:]):
            fails.append(("circular_reasoning", 0.6))
        if len(steps) > 5 and len(set(steps)) < 0.7 * len(steps):
            fails.append(("hallucination", 0.5))
        from .reasoning import YvReasoningTrace, YvVeriCoTVerifier
        if steps and not YvVeriCoTVerifier().verify(YvReasoningTrace(steps=list(reasoning_steps), answer=final_answer)):
            fails.append(("arithmetic_error", 0.9))
        return fails

    @staticmethod
    def create(kind: str, hidden_size: int, **kw: Any) -> nn.Module:
        kind = kind.lower()
        if kind == "crv":
            return YvCRV(hidden_size, **kw)
        if kind == "otv":
            return YvOTV(hidden_size, **kw)
        if kind == "ares":
            return YvARES(hidden_size, **kw)
        if kind in ("vericot", "vericot_step"):
            return YvVeriCoTStepVerifier(hidden_size, **kw)
        if kind == "vericot_reflector":
            return YvVeriCoTReflector(YvVeriCoTStepVerifier(hidden_size), **kw)
        raise ValueError(f"unknown verifier kind {kind!r}")
