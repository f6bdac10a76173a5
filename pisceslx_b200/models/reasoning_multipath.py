"""The rest of the multi-path reasoning family (reference model/reasoning/reasoner/enhancer.py:100-430,
multipath_infer.py:118-489, multipath_meta.py:110-395):

  * ``YvMultiModalReasoningEnhancer``  a neural module: text features attend to visual / audio features, a pooled
    reasoning state is refined for a few steps with the aggregated evidence and an optional temporal context;
  * ``YvMultiPathInferenceEngine``     prompt level: several sampled reasoning paths per round, scored, deepened until
    the confidence passes a threshold;
  * ``YvMultiPathMetaLearner``         bookkeeping over finished reasoning runs: which depths, strategies and
    confidence curves worked, turned into parameters and priors for the next runs.

The enhancer keeps its diagnostics on the device (the reference copies every attention map to the host and reads a
norm back per step); the inference engine takes plain callables (``generate``, optionally ``embed`` and
``token_logprobs``) instead of a model object plus a downloaded classifier."""
from __future__ import annotations

import math
import re
from collections import Counter
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from .compat import YvCrossAttention
from .reasoning_engine import _x


def _heads(hidden: int, want: int) -> int:
    for h in range(max(1, min(want, hidden)), 0, -1):
        if hidden % h == 0:
            return h
    return 1


class YvMultiModalReasoningEnhancer(nn.Module):
    """forward(text [B, S, H], visual [B, Sv, H]?, audio [B, Sa, H]?, temporal_context [B, St, H]?) ->
    (reasoning_state [B, 1, H], confidence [B, 1]) and, on request, the intermediates.

    Visual evidence enters with weight 0.3 and audio with 0.2 through cross attention from the text; beyond 512 text
    tokens the cross attention is replaced by a linear map of the text modulated by the pooled modality (the reference
    drops the modality altogether on that branch, enhancer.py:268-271).  Each of ``num_reasoning_steps`` steps maps the
    pooled state through a gated MLP, adds a tenth of the aggregated evidence and, with a temporal context, a fifth of
    what the state retrieves from it."""

    VISUAL_WEIGHT, AUDIO_WEIGHT, EVIDENCE_WEIGHT, TEMPORAL_WEIGHT = 0.3, 0.2, 0.1, 0.2

    def __init__(self, cfg: Any):
        super().__init__()
        self.cfg = cfg
        H = self.hidden_size = int(cfg.hidden_size)
        self.num_reasoning_steps = int(_x(cfg, "num_reasoning_steps", 4))
        self.long_sequence_tokens = int(_x(cfg, "enhancer_linear_attention_tokens", 512))
        nh = int(cfg.n_head)
        self.cross_modal_reasoner = nn.ModuleDict({
            "visual_textual": YvCrossAttention(H, H, _heads(H, max(nh // 4, 1))),
            "audio_textual": YvCrossAttention(H, H, _heads(H, max(nh // 4, 1))),
            "temporal_reasoning": YvCrossAttention(H, H, _heads(H, max(nh // 2, 1))),
            "efficient_linear": nn.Sequential(nn.Linear(H, H), nn.LayerNorm(H)),
            "efficient_gate": nn.Linear(H, H)})
        self.reasoning_layers = nn.ModuleList([
            nn.Sequential(nn.Linear(H, 2 * H), nn.SiLU(), nn.Linear(2 * H, H), nn.LayerNorm(H))
            for _ in range(self.num_reasoning_steps)])
        self.evidence_aggregator = nn.Sequential(nn.Linear(3 * H, 2 * H), nn.SiLU(), nn.Linear(2 * H, H), nn.LayerNorm(H))
        self.confidence_estimator = nn.Sequential(nn.Linear(H, max(H // 2, 1)), nn.SiLU(), nn.Linear(max(H // 2, 1), 1),
                                                  nn.Sigmoid())

    def _modal(self, name: str, text: torch.Tensor, feats: torch.Tensor, linear: bool) -> torch.Tensor:
        if linear:
            gate = torch.sigmoid(self.cross_modal_reasoner["efficient_gate"](feats.mean(1, keepdim=True)))
            return self.cross_modal_reasoner["efficient_linear"](text) * gate
        return self.cross_modal_reasoner[name](text, feats)

    def forward(self, text_features: torch.Tensor, visual_features: Optional[torch.Tensor] = None,
                audio_features: Optional[torch.Tensor] = None, temporal_context: Optional[torch.Tensor] = None,
                return_intermediates: bool = False):
        B, S, H = text_features.shape
        linear = S > self.long_sequence_tokens
        state = text_features
        contrib = {"visual": 0.0, "audio": 0.0}
        pooled = [text_features.mean(1)]
        if visual_features is not None:
            state = state + self.VISUAL_WEIGHT * self._modal("visual_textual", text_features, visual_features, linear)
            contrib["visual"] = self.VISUAL_WEIGHT
        pooled.append(visual_features.mean(1) if visual_features is not None else torch.zeros_like(pooled[0]))
        if audio_features is not None:
            state = state + self.AUDIO_WEIGHT * self._modal("audio_textual", text_features, audio_features, linear)
            contrib["audio"] = self.AUDIO_WEIGHT
        pooled.append(audio_features.mean(1) if audio_features is not None else torch.zeros_like(pooled[0]))
        evidence = self.evidence_aggregator(torch.cat(pooled, -1))
        cur = state.mean(1)                                                                  # [B, H]
        steps: List[Dict[str, torch.Tensor]] = []
        for i, layer in enumerate(self.reasoning_layers):
            nxt = layer(cur) + self.EVIDENCE_WEIGHT * evidence
            if temporal_context is not None:
                nxt = nxt + self.TEMPORAL_WEIGHT * self._modal("temporal_reasoning", nxt.unsqueeze(1), temporal_context,
                                                               linear).squeeze(1)
            if return_intermediates:
                steps.append({"step_id": i, "input_state": cur, "output_state": nxt,
                              "state_change": (nxt - cur).float().norm(dim=-1)})
            cur = nxt
        state_out = cur.unsqueeze(1)
        confidence = self.confidence_estimator(cur)
        if not return_intermediates:
            return state_out, confidence
        return state_out, confidence, {"initial_state": text_features, "modal_contributions": contrib,
                                       "step_outputs": steps, "final_confidence": confidence, "final_state": state_out,
                                       "sequence_length": S, "used_linear_attention": linear}


# ---------------------------------------------------------------------------------------------------------------------------
GenerateFn = Callable[..., str]

_LOGIC_PATTERNS = {
    "deductive": (r"if\b.*\bthen", r"given\b.*\btherefore", r"since\b.*\bconclude"),
    "inductive": (r"based on\b.*\bwe can infer", r"evidence suggests", r"observations indicate"),
    "abductive": (r"the best explanation is", r"most likely cause", r"plausible reason"),
}
_NEGATIONS = re.compile(r"\b(not|never|no|cannot|isn't|aren't|doesn't|don't|won't)\b")
_BEFORE_AFTER = re.compile(r"\b(before|after|then|later|earlier|first|finally)\b")
_CAUSAL = re.compile(r"\b(because|therefore|thus|hence|so that|as a result|causes?|leads? to)\b")


def _clauses(text: str) -> List[str]:
    return [c.strip() for c in re.split(r"(?<=[.!?;:])\s+", text) if c.strip()]


class YvMultiPathInferenceEngine:
    """Several sampled reasoning paths per round, the best kept, rounds repeated with a sharper instruction until the
    confidence reaches the threshold or ``max_depth`` rounds are spent.

    ``generate(prompt, temperature=...) -> str`` is the only requirement.  ``embed(text) -> tensor [H]`` makes the
    clause-consistency score semantic (mean pairwise cosine of the clause embeddings; without it a token-overlap
    measure is used), ``token_logprobs(prompt, text) -> tensor [T, V]`` or ``[T]`` makes the uncertainty score the
    entropy (or mean log-probability) of the path instead of a neutral 0.5."""

    TEMPERATURES = (0.3, 0.5, 0.7, 0.9, 1.1)

    def __init__(self, generate: GenerateFn, max_depth: int = 5, confidence_threshold: float = 0.85,
                 embed: Optional[Callable[[str], torch.Tensor]] = None,
                 token_logprobs: Optional[Callable[[str, str], torch.Tensor]] = None, target_chars_per_round: int = 100):
        self.generate, self.embed, self.token_logprobs = generate, embed, token_logprobs
        self.max_depth, self.confidence_threshold = max_depth, confidence_threshold
        self.target_chars = target_chars_per_round
        self.reasoning_cache: Dict[str, Dict[str, Any]] = {}

    # -- scores of a path ----------------------------------------------------------------------------------------------------
    def _estimate_logical_consistency(self, text: str) -> float:
        cl = _clauses(text)
        if len(cl) < 2:
            return 1.0 if cl else 0.0
        if self.embed is not None:
            m = F.normalize(torch.stack([self.embed(c).float().reshape(-1) for c in cl]), dim=-1)
            sim = m @ m.t()
            n = len(cl)
            mean_cos = (sim.sum() - sim.diagonal().sum()) / (n * (n - 1))
            return float(mean_cos.clamp(-1, 1) * 0.5 + 0.5)
        bags = [set(re.findall(r"\w+", c.lower())) for c in cl]
        pairs = [len(a & b) / max(len(a | b), 1) for i, a in enumerate(bags) for b in bags[i + 1:]]
        return float(min(1.0, 0.5 + sum(pairs) / len(pairs)))

    def _measure_uncertainty_reduction(self, prompt: str, text: str) -> float:
        if self.token_logprobs is None or not text:
            return 0.5
        lp = self.token_logprobs(prompt, text).float()
        if lp.dim() == 2:
            ent = -(lp.exp() * lp).sum(-1).mean() / math.log(max(lp.shape[-1], 2))
            return float((1.0 - ent).clamp(0, 1))
        return float(lp.mean().exp().clamp(0, 1))

    @staticmethod
    def _check_self_consistency(text: str) -> float:
        """A statement and its negation in different clauses lower the score."""
        cl = [c.lower() for c in _clauses(text)]
        if len(cl) < 2:
            return 1.0
        clash = 0
        for i, a in enumerate(cl):
            wa = set(re.findall(r"\w+", _NEGATIONS.sub("", a)))
            for b in cl[i + 1:]:
                wb = set(re.findall(r"\w+", _NEGATIONS.sub("", b)))
                same = len(wa & wb) / max(len(wa | wb), 1) > 0.8
                if same and bool(_NEGATIONS.search(a)) != bool(_NEGATIONS.search(b)):
                    clash += 1
        return max(0.0, 1.0 - clash / max(len(cl) - 1, 1))

    @staticmethod
    def _check_temporal_consistency(text: str) -> float:
        t = text.lower()
        first, fin = t.find("first"), t.find("finally")
        if first >= 0 and fin >= 0 and fin < first:
            return 0.3
        return 1.0 if _BEFORE_AFTER.search(t) else 0.7

    @staticmethod
    def _check_causal_consistency(text: str) -> float:
        n = len(_clauses(text))
        links = len(_CAUSAL.findall(text.lower()))
        return min(1.0, 0.5 + 0.5 * links / max(n - 1, 1)) if n > 1 else (1.0 if links else 0.6)

    @staticmethod
    def _check_logical_validity(text: str) -> float:
        t = text.lower()
        scores = [sum(1 for p in pats if re.search(p, t)) / len(pats) for pats in _LOGIC_PATTERNS.values()]
        return sum(scores) / len(scores)

    def _verify_facts(self, text: str) -> Dict[str, float]:
        return {"self_consistency": self._check_self_consistency(text),
                "temporal_consistency": self._check_temporal_consistency(text),
                "causal_consistency": self._check_causal_consistency(text),
                "logical_validity": self._check_logical_validity(text)}

    def _evaluate_reasoning_path(self, prompt: str, path: Dict[str, Any], depth: int) -> float:
        want = self.target_chars * (depth + 1)
        length = 1.0 / (1.0 + abs(len(path["text"]) - want) / self.target_chars)
        # clause similarity alone rewards a statement followed by its own negation, hence the contradiction term
        return 0.25 * length + 0.3 * self._estimate_logical_consistency(path["text"]) + \
            0.2 * self._measure_uncertainty_reduction(prompt, path["text"]) + \
            0.25 * self._check_self_consistency(path["text"])

    @staticmethod
    def _calculate_path_confidence(facts: Dict[str, float]) -> float:
        base = (facts["self_consistency"] + facts["temporal_consistency"] + facts["causal_consistency"]) / 3.0
        return 1.0 / (1.0 + math.exp(-4.0 * (base - 0.5)))           # 0.5 -> 0.5, 1.0 -> 0.88

    # -- the rounds -----------------------------------------------------------------------------------------------------------
    def _generate_reasoning_paths(self, prompt: str, depth: int) -> List[Dict[str, Any]]:
        return [{"text": self.generate(prompt, temperature=t), "temperature": t}
                for t in self.TEMPERATURES[:min(3 + depth, len(self.TEMPERATURES))]]

    def _multi_path_layer_reasoning(self, prompt: str, depth: int) -> Dict[str, Any]:
        paths = self._generate_reasoning_paths(prompt, depth)
        scores = [self._evaluate_reasoning_path(prompt, p, depth) for p in paths]
        best = paths[max(range(len(paths)), key=scores.__getitem__)]
        facts = self._verify_facts(best["text"])
        conf = self._calculate_path_confidence(facts)
        return {"reasoning": best, "confidence": conf, "uncertainty": 1.0 - conf, "facts": facts, "path_scores": scores}

    def multi_path_reason(self, prompt: str, return_metadata: bool = False) -> Union[str, Dict[str, Any]]:
        if prompt in self.reasoning_cache:
            meta = self.reasoning_cache[prompt]
            return meta if return_metadata else meta["answer"]
        layers: List[Dict[str, Any]] = []
        cur = prompt
        for depth in range(self.max_depth):
            layer = self._multi_path_layer_reasoning(cur, depth)
            layers.append(layer)
            if layer["confidence"] >= self.confidence_threshold:
                break
            cur = (f"{prompt}\n\nPrevious attempt (confidence {layer['confidence']:.2f}):\n{layer['reasoning']['text']}\n\n"
                   "Reason again step by step, fixing what is inconsistent.")
        best = max(layers, key=lambda l: l["confidence"])
        meta = {"answer": best["reasoning"]["text"], "confidence": best["confidence"], "reasoning_depth": len(layers),
                "reasoning_chain": [l["reasoning"]["text"] for l in layers],
                "uncertainty_evolution": [l["uncertainty"] for l in layers],
                "fact_verifications": [l["facts"] for l in layers]}
        self.reasoning_cache[prompt] = meta
        return meta if return_metadata else meta["answer"]


# ---------------------------------------------------------------------------------------------------------------------------
class YvMultiPathMetaLearner:
    """Records finished reasoning runs and turns them into parameters for the next ones.

    ``record_reasoning(query, chain, result, metadata)`` stores a run (``metadata``: ``reasoning_depth``, ``confidence``,
    ``uncertainty_evolution``, optionally ``success``).  ``extract_reasoning_patterns`` needs ``min_support`` runs and
    summarises depths, confidence growth and the strategies seen in the chains; ``adapt_reasoning_parameters`` maps that
    to a confidence threshold, a depth bound and preferred strategies; ``create_reasoning_prior(query)`` returns the
    typical uncertainty curve of the most similar stored queries.  Queries are embedded by hashed character trigrams
    (deterministic, no external model) and, when a ``pattern_extractor`` has been trained, projected by it."""

    STRATEGY_CUES = (("analogical", ("analog", "similar to", "just as")),
                     ("decomposition", ("break down", "decompose", "sub-problem", "step by step")),
                     ("assumption_testing", ("assume", "suppose", "hypothes")),
                     ("elimination", ("rule out", "eliminate", "cannot be")))

    def __init__(self, model: Optional[nn.Module] = None, learning_rate: float = 1e-5, hidden_size: Optional[int] = None,
                 min_support: int = 10, capacity: int = 4096):
        self.model, self.learning_rate = model, learning_rate
        cfg = getattr(model, "cfg", None)
        self.hidden_size = int(hidden_size or getattr(cfg, "hidden_size", 256))
        self.min_support, self.capacity = min_support, capacity
        self.reasoning_memory: List[Dict[str, Any]] = []
        self.pattern_extractor = self._build_pattern_extractor()

    def _build_pattern_extractor(self) -> nn.Sequential:
        H = self.hidden_size
        return nn.Sequential(nn.Linear(H, max(H // 2, 1)), nn.ReLU(), nn.Linear(max(H // 2, 1), max(H // 4, 1)), nn.Tanh())

    def _embed_query(self, query: str) -> torch.Tensor:
        v = torch.zeros(self.hidden_size)
        s = f"  {query.lower()}  "
        for i in range(len(s) - 2):
            h = 0
            for ch in s[i:i + 3]:
                h = (h * 16777619 + ord(ch)) & 0xFFFFFFFF
            v[h % self.hidden_size] += 1.0 if (h >> 16) & 1 else -1.0
        return F.normalize(v, dim=0)

    def record_reasoning(self, query: str, reasoning_chain: Sequence[Any], final_result: Any, metadata: Dict[str, Any]) -> None:
        self.reasoning_memory.append({"query": query, "embedding": self._embed_query(query),
                                      "reasoning_chain": list(reasoning_chain), "final_result": final_result,
                                      "metadata": dict(metadata)})
        if len(self.reasoning_memory) > self.capacity:
            del self.reasoning_memory[: len(self.reasoning_memory) - self.capacity]

    # -- analysis -------------------------------------------------------------------------------------------------------------
    @staticmethod
    def _analyze_depth_patterns(experiences: List[Dict[str, Any]]) -> Dict[str, Any]:
        d = torch.tensor([float(e["metadata"].get("reasoning_depth", 1)) for e in experiences])
        q = torch.quantile(d, torch.tensor([0.25, 0.75]))
        return {"mean_depth": float(d.mean()), "depth_variance": float(d.var(unbiased=False)),
                "optimal_depth_range": (float(q[0]), float(q[1]))}

    @staticmethod
    def _calculate_confidence_growth(uncertainty_evolutions: List[List[float]]) -> float:
        """Mean drop of the uncertainty from the first to the last round."""
        g = [u[0] - u[-1] for u in uncertainty_evolutions if len(u) >= 2]
        return sum(g) / len(g) if g else 0.0

    def _analyze_confidence_patterns(self, experiences: List[Dict[str, Any]]) -> Dict[str, float]:
        conf = torch.tensor([float(e["metadata"].get("confidence", 0.5)) for e in experiences])
        evo = [list(e["metadata"].get("uncertainty_evolution", [])) for e in experiences]
        return {"mean_confidence": float(conf.mean()), "stability_threshold": float(torch.quantile(conf, 0.25)),
                "confidence_growth": self._calculate_confidence_growth(evo)}

    def _identify_strategy(self, reasoning_chain: Sequence[Any]) -> str:
        votes = []
        for step in reasoning_chain:
            s = str(step).lower()
            votes.append(next((name for name, cues in self.STRATEGY_CUES if any(c in s for c in cues)), "direct"))
        return Counter(votes).most_common(1)[0][0] if votes else "direct"

    @staticmethod
    def _calculate_strategy_success(strategies: List[str], experiences: List[Dict[str, Any]]) -> Dict[str, float]:
        tot: Dict[str, List[float]] = {}
        for s, e in zip(strategies, experiences):
            m = e["metadata"]
            tot.setdefault(s, []).append(float(m["success"]) if "success" in m else float(m.get("confidence", 0.5)))
        return {s: sum(v) / len(v) for s, v in tot.items()}

    def _analyze_strategy_patterns(self, experiences: List[Dict[str, Any]]) -> Dict[str, Any]:
        strategies = [self._identify_strategy(e["reasoning_chain"]) for e in experiences]
        return {"most_common_strategies": Counter(strategies).most_common(5),
                "strategy_success_rates": self._calculate_strategy_success(strategies, experiences)}

    def extract_reasoning_patterns(self) -> Optional[Dict[str, Any]]:
        if len(self.reasoning_memory) < self.min_support:
            return None
        recent = self.reasoning_memory[-max(self.min_support, 100):]
        return {"optimal_depth_distribution": self._analyze_depth_patterns(recent),
                "confidence_indicators": self._analyze_confidence_patterns(recent),
                "reasoning_strategies": self._analyze_strategy_patterns(recent), "support": len(recent)}

    def adapt_reasoning_parameters(self, patterns: Optional[Dict[str, Any]]) -> Dict[str, Any]:
        if not patterns:
            raise ValueError("adapt_reasoning_parameters needs extracted pattern statistics")
        depth = patterns["optimal_depth_distribution"]["mean_depth"]
        rates = patterns["reasoning_strategies"]["strategy_success_rates"]
        return {"confidence_threshold": max(0.7, patterns["confidence_indicators"]["stability_threshold"]),
                "max_depth": max(3, min(8, int(depth * 1.2))),
                "preferred_strategies": [s for s, _ in sorted(rates.items(), key=lambda kv: -kv[1])[:3]]}

    def apply_to(self, engine: YvMultiPathInferenceEngine) -> Optional[Dict[str, Any]]:
        """Extract, adapt and set the inference engine's threshold and depth; None while the support is too small."""
        pat = self.extract_reasoning_patterns()
        if pat is None:
            return None
        params = self.adapt_reasoning_parameters(pat)
        engine.confidence_threshold, engine.max_depth = params["confidence_threshold"], params["max_depth"]
        return params

    # -- priors ---------------------------------------------------------------------------------------------------------------
    @staticmethod
    def _extract_uncertainty_pattern(experiences: List[Dict[str, Any]]) -> Optional[Dict[str, List[float]]]:
        evo = [list(e["metadata"]["uncertainty_evolution"]) for e in experiences
               if e["metadata"].get("uncertainty_evolution")]
        if not evo:
            return None
        n = max(len(u) for u in evo)
        m = torch.tensor([u + [u[-1]] * (n - len(u)) for u in evo])
        return {"typical_pattern": m.mean(0).tolist(), "variance": m.var(0, unbiased=False).tolist()}

    def create_reasoning_prior(self, query: str, k: int = 5, min_similarity: float = 0.1) -> Optional[Dict[str, Any]]:
        if not self.reasoning_memory:
            return None
        q = self._embed_query(query)
        sims = torch.stack([e["embedding"] for e in self.reasoning_memory]) @ q
        top = sims.topk(min(k, sims.numel()))
        near = [self.reasoning_memory[i] for v, i in zip(top.values.tolist(), top.indices.tolist()) if v >= min_similarity]
        if not near:
            return None
        d = [float(e["metadata"].get("reasoning_depth", 1)) for e in near]
        strategies = [self._identify_strategy(e["reasoning_chain"]) for e in near]
        return {"expected_depth": sum(d) / len(d), "suggested_strategy": Counter(strategies).most_common(1)[0][0],
                "uncertainty_pattern": self._extract_uncertainty_pattern(near), "num_similar": len(near),
                "similarities": [v for v in top.values.tolist() if v >= min_similarity]}
