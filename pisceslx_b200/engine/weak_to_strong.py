"""Weak-to-strong training in full (reference opss/train/weak_to_strong.py:60-647): a frozen weak supervisor labels
the data, a confidence curriculum decides which of its labels are used, the strong student is trained on them with a
confidence-weighted loss and may overrule the supervisor where it is the more confident one (self-correction), and
iterative amplification makes each trained student the supervisor of the next round.

``engine/alignment.py`` has the auxiliary-confidence loss and a minimal trainer; this module is the operator the
training tools call.  Everything in the loss path is per position and stays on the device: the masks enter as weights,
the counts are tensors (the reference branches on ``valid_mask.sum() == 0`` and reads ``.item()`` statistics every
step, weak_to_strong.py:383-420).  Labels and logits are aligned position by position: both models predict the next
token at the same position, so no shift is needed.  Models may return a tensor of logits, an object with ``.logits``
or a mapping with ``"logits"``."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from enum import Enum
from typing import Any, Callable, Dict, Iterable, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..utils.opsc import PiscesLxOperatorInterface


class PiscesLxW2SMode(str, Enum):
    CE = "ce"               # cross-entropy on the weak labels, weighted by the weak confidence
    KL = "kl"               # KL(weak distribution || strong distribution): the full soft supervision
    JS = "js"               # Jensen-Shannon: symmetric and bounded, gentler on confident weak mistakes


@dataclass
class PiscesLxWeakToStrongConfig:
    confidence_threshold: float = 0.7
    final_confidence_threshold: float = 0.5
    use_curriculum: bool = True
    curriculum_steps: int = 1000
    temperature: float = 1.0
    label_smoothing: float = 0.0
    loss_type: str = "ce"
    strong_model_lr: float = 1e-5
    weak_model_frozen: bool = True
    max_grad_norm: float = 1.0
    use_self_correction: bool = True
    correction_weight: float = 0.1
    ignore_index: int = -100

    def __post_init__(self) -> None:
        self.loss_type = PiscesLxW2SMode(getattr(self.loss_type, "value", self.loss_type)).value
        if not 0 < self.temperature:
            raise ValueError("temperature must be positive")
        if not 0 <= self.final_confidence_threshold <= self.confidence_threshold <= 1:
            raise ValueError("need 0 <= final_confidence_threshold <= confidence_threshold <= 1")


def _logits(out: Any) -> torch.Tensor:
    if torch.is_tensor(out):
        return out
    if hasattr(out, "logits") and out.logits is not None:
        return out.logits
    if isinstance(out, dict) and out.get("logits") is not None:
        return out["logits"]
    if isinstance(out, (tuple, list)):
        return out[0]
    raise TypeError("the model's output carries no logits")


def _call(model: nn.Module, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor]) -> torch.Tensor:
    try:
        return _logits(model(input_ids, attention_mask=attention_mask) if attention_mask is not None else model(input_ids))
    except TypeError:
        return _logits(model(input_ids))


class PiscesLxWeakLabelGenerator:
    """argmax labels, their probability as confidence, and the mask of labels above the threshold."""

    def __init__(self, weak_model: nn.Module, config: PiscesLxWeakToStrongConfig):
        self.weak_model, self.config = weak_model, config
        if config.weak_model_frozen:
            weak_model.requires_grad_(False)
            weak_model.eval()

    @torch.no_grad()
    def generate_with_features(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        logits = _call(self.weak_model, input_ids, attention_mask).float()
        probs = torch.softmax(logits / self.config.temperature, -1)
        conf, labels = probs.max(-1)
        valid = conf > self.config.confidence_threshold
        if attention_mask is not None and attention_mask.shape == valid.shape:
            valid = valid & attention_mask.bool()
        return {"weak_labels": labels, "confidence": conf, "valid_mask": valid, "logits": logits, "probs": probs}

    def generate(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        o = self.generate_with_features(input_ids, attention_mask)
        return o["weak_labels"], o["confidence"], o["valid_mask"]


class PiscesLxCurriculumScheduler:
    """The confidence threshold falls linearly from the initial to the final value over ``curriculum_steps`` (easy,
    confident labels first; harder ones later) while the weight of the loss rises from 0.5 to 1."""

    def __init__(self, config: PiscesLxWeakToStrongConfig):
        self.config, self.current_step = config, 0

    def step(self) -> None:
        self.current_step += 1

    @property
    def progress(self) -> float:
        return min(1.0, self.current_step / max(self.config.curriculum_steps, 1)) if self.config.use_curriculum else 1.0

    def get_current_threshold(self) -> float:
        c = self.config
        if not c.use_curriculum:
            return c.confidence_threshold
        return c.confidence_threshold + (c.final_confidence_threshold - c.confidence_threshold) * self.progress

    def get_difficulty_weight(self) -> float:
        return 0.5 + 0.5 * self.progress if self.config.use_curriculum else 1.0

    def state_dict(self) -> Dict[str, int]:
        return {"current_step": self.current_step}

    def load_state_dict(self, sd: Dict[str, int]) -> None:
        self.current_step = int(sd.get("current_step", 0))


class PiscesLxSelfCorrection:
    """Where the student disagrees with the supervisor AND is more confident than it, the student is trained towards its
    own prediction: mean cross-entropy to its hardened labels over those positions (zero when there are none)."""

    def __init__(self, config: PiscesLxWeakToStrongConfig):
        self.config = config

    def correction_mask(self, strong_logits: torch.Tensor, weak_labels: torch.Tensor, confidence: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        sp = torch.softmax(strong_logits.detach().float(), -1)
        sc, sl = sp.max(-1)
        return (sl != weak_labels) & (sc > confidence), sl

    def compute_correction_loss(self, strong_logits: torch.Tensor, weak_labels: torch.Tensor, confidence: torch.Tensor,
                                position_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        mask, own = self.correction_mask(strong_logits, weak_labels, confidence)
        if position_mask is not None:
            mask = mask & position_mask.bool()
        ce = F.cross_entropy(strong_logits.float().reshape(-1, strong_logits.shape[-1]), own.reshape(-1), reduction="none")
        m = mask.reshape(-1).float()
        return (ce * m).sum() / m.sum().clamp_min(1.0)


class PiscesLxWeakToStrongOperator(PiscesLxOperatorInterface):
    """``train_step(input_ids, attention_mask, labels)`` returns the loss (a tensor with a graph) and statistics as
    tensors; the caller runs backward and the optimizer, or uses ``fit`` which does both.  ``labels`` (ground truth) are
    used for the reported accuracies only."""

    name = "training.weak_to_strong"

    def __init__(self, weak_model: nn.Module, strong_model: nn.Module, config: Optional[PiscesLxWeakToStrongConfig] = None):
        self.config = config or PiscesLxWeakToStrongConfig()
        self.weak_model, self.strong_model = weak_model, strong_model
        self.label_generator = PiscesLxWeakLabelGenerator(weak_model, self.config)
        self.curriculum = PiscesLxCurriculumScheduler(self.config)
        self.self_correction = PiscesLxSelfCorrection(self.config) if self.config.use_self_correction else None
        self._stats = {"steps": 0, "total_positions": 0.0, "valid_positions": 0.0, "corrections": 0.0}

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return torch.is_tensor(inputs.get("input_ids"))

    def _compute_loss(self, strong_logits: torch.Tensor, weak: Dict[str, torch.Tensor], valid: torch.Tensor) -> torch.Tensor:
        c = self.config
        V = strong_logits.shape[-1]
        sl = strong_logits.float()
        w = valid.float()
        n = w.sum().clamp_min(1.0)
        if c.loss_type == "ce":
            ce = F.cross_entropy(sl.reshape(-1, V), weak["weak_labels"].reshape(-1), reduction="none",
                                 label_smoothing=c.label_smoothing).view_as(w)
            return (ce * weak["confidence"] * w).sum() / n
        logp = torch.log_softmax(sl, -1)
        q = weak["probs"]
        if c.loss_type == "kl":
            kl = (q * (torch.log(q.clamp_min(1e-12)) - logp)).sum(-1)
            return (kl * w).sum() / n
        p = logp.exp()
        m = 0.5 * (p + q)
        logm = torch.log(m.clamp_min(1e-12))
        js = 0.5 * (q * (torch.log(q.clamp_min(1e-12)) - logm)).sum(-1) + 0.5 * (p * (logp - logm)).sum(-1)
        return (js * w).sum() / n

    def train_step(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                   labels: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        c = self.config
        weak = self.label_generator.generate_with_features(input_ids, attention_mask)
        valid = weak["confidence"] > self.curriculum.get_current_threshold()
        pos = torch.ones_like(valid) if attention_mask is None or attention_mask.shape != valid.shape else attention_mask.bool()
        valid = valid & pos
        strong_logits = _call(self.strong_model, input_ids, attention_mask)
        main = self._compute_loss(strong_logits, weak, valid) * self.curriculum.get_difficulty_weight()
        total, corr, n_corr = main, main.new_zeros(()), main.new_zeros(())
        if self.self_correction is not None:
            corr = self.self_correction.compute_correction_loss(strong_logits, weak["weak_labels"], weak["confidence"], pos)
            n_corr = (self.self_correction.correction_mask(strong_logits, weak["weak_labels"], weak["confidence"])[0] & pos).float().sum()
            total = total + c.correction_weight * corr
        out = {"loss": total, "main_loss": main.detach(), "correction_loss": corr.detach(), "valid_positions": valid.float().sum(),
               "total_positions": pos.float().sum(), "corrections": n_corr,
               "avg_confidence": (weak["confidence"] * valid).sum() / valid.float().sum().clamp_min(1.0),
               "threshold": torch.tensor(self.curriculum.get_current_threshold())}
        if labels is not None:
            keep = (labels != c.ignore_index) & pos
            k = keep.float().sum().clamp_min(1.0)
            out["weak_accuracy"] = ((weak["weak_labels"] == labels) & keep).float().sum() / k
            out["strong_accuracy"] = ((strong_logits.argmax(-1) == labels) & keep).float().sum() / k
        self.curriculum.step()
        s = self._stats
        s["steps"] += 1
        for key in ("total_positions", "valid_positions", "corrections"):
            s[key] = s[key] + out[key].detach()
        return out

    def run(self, inputs: Dict[str, Any]) -> Dict[str, torch.Tensor]:
        return self.train_step(inputs["input_ids"], inputs.get("attention_mask"), inputs.get("labels"))

    def fit(self, batches: Iterable[Any], optimizer: torch.optim.Optimizer, epochs: int = 1) -> Dict[str, float]:
        """Batches are ``input_ids`` tensors, ``(input_ids, labels)`` pairs or dictionaries.  Returns the last step's
        numbers as floats (one read-back at the end)."""
        last: Dict[str, torch.Tensor] = {}
        self.strong_model.train()
        for _ in range(epochs):
            for b in batches:
                if isinstance(b, dict):
                    ids, am, lab = b["input_ids"], b.get("attention_mask"), b.get("labels")
                elif isinstance(b, (tuple, list)):
                    ids, am, lab = b[0], None, (b[1] if len(b) > 1 else None)
                else:
                    ids, am, lab = b, None, None
                last = self.train_step(ids, am, lab)
                optimizer.zero_grad(set_to_none=True)
                last["loss"].backward()
                if self.config.max_grad_norm > 0:
                    torch.nn.utils.clip_grad_norm_(self.strong_model.parameters(), self.config.max_grad_norm)
                optimizer.step()
        return {k: float(v) for k, v in last.items()}

    def get_statistics(self) -> Dict[str, float]:
        return {k: float(v) for k, v in self._stats.items()}


class PiscesLxIterativeAmplification:
    """Round k: the current model supervises a student that starts as its (slightly perturbed) copy, or as a model
    made by ``student_factory`` (a bigger one, for instance); the trained student becomes the supervisor of round
    k + 1."""

    def __init__(self, base_model: nn.Module, config: Optional[PiscesLxWeakToStrongConfig] = None, num_iterations: int = 3,
                 student_factory: Optional[Callable[[nn.Module, int], nn.Module]] = None, init_noise: float = 0.01,
                 optimizer_factory: Optional[Callable[[nn.Module], torch.optim.Optimizer]] = None):
        self.config = config or PiscesLxWeakToStrongConfig()
        self.current_model, self.num_iterations, self.iteration = base_model, num_iterations, 0
        self._student_factory, self._noise = student_factory, init_noise
        self._opt_factory = optimizer_factory or (lambda m: torch.optim.AdamW(m.parameters(), lr=self.config.strong_model_lr))
        self.history: list = []

    def _new_student(self) -> nn.Module:
        if self._student_factory is not None:
            return self._student_factory(self.current_model, self.iteration)
        s = copy.deepcopy(self.current_model)
        s.requires_grad_(True)
        with torch.no_grad():
            for p in s.parameters():
                p.add_(torch.randn_like(p) * self._noise)
        return s

    def step(self, batches: Iterable[Any], epochs: int = 1) -> nn.Module:
        if self.iteration >= self.num_iterations:
            return self.current_model
        student = self._new_student()
        op = PiscesLxWeakToStrongOperator(self.current_model, student, self.config)
        stats = op.fit(batches, self._opt_factory(student), epochs)
        self.history.append({"iteration": self.iteration, **stats, **op.get_statistics()})
        self.current_model = student
        self.iteration += 1
        return student

    def run(self, batches: Iterable[Any], epochs: int = 1) -> nn.Module:
        while self.iteration < self.num_iterations:
            self.step(batches, epochs)
        return self.current_model
