"""Distillation losses (reference opss/train/distillation_losses.py: logits, hidden-state, attention, layer-wise,
contrastive losses and an optimal-transport layer aligner, combined by ``PiscesLxDistillationLoss``).  Inputs are
plain tensors, so the same losses serve a Yv student against any teacher."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class PiscesLxDistillationLossConfig:
    temperature: float = 2.0
    logits_weight: float = 1.0
    hidden_weight: float = 0.0
    attention_weight: float = 0.0
    contrastive_weight: float = 0.0
    hard_label_weight: float = 0.0
    contrastive_temperature: float = 0.1


class PiscesLxLogitsDistillationLoss(nn.Module):
    """KL(teacher || student) at temperature T, scaled by T^2 so that gradients keep their size (Hinton et al.)."""

    def __init__(self, temperature: float = 2.0):
        super().__init__()
        self.T = temperature

    def forward(self, student_logits: torch.Tensor, teacher_logits: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        s = F.log_softmax(student_logits.float() / self.T, -1)
        t = F.softmax(teacher_logits.float() / self.T, -1)
        kl = (t * (torch.log(t.clamp_min(1e-20)) - s)).sum(-1)
        if mask is not None:
            m = mask.to(kl.dtype)
            return (kl * m).sum() / m.sum().clamp_min(1) * self.T ** 2
        return kl.mean() * self.T ** 2


class PiscesLxHiddenStateDistillationLoss(nn.Module):
    """MSE (or cosine) between student states, projected to the teacher's width when they differ, and teacher states."""

    def __init__(self, student_dim: int, teacher_dim: int, kind: str = "mse"):
        super().__init__()
        self.proj = nn.Identity() if student_dim == teacher_dim else nn.Linear(student_dim, teacher_dim, bias=False)
        self.kind = kind

    def forward(self, student_h: torch.Tensor, teacher_h: torch.Tensor) -> torch.Tensor:
        s, t = self.proj(student_h.float()), teacher_h.float()
        if self.kind == "cosine":
            return (1 - F.cosine_similarity(s, t, dim=-1)).mean()
        return F.mse_loss(s, t)


class PiscesLxAttentionDistillationLoss(nn.Module):
    """KL between attention maps [B, h, S, S]; head counts may differ (both are averaged over heads then)."""

    def forward(self, student_attn: torch.Tensor, teacher_attn: torch.Tensor) -> torch.Tensor:
        s, t = student_attn.float(), teacher_attn.float()
        if s.shape[1] != t.shape[1]:
            s, t = s.mean(1, keepdim=True), t.mean(1, keepdim=True)
        return (t * (torch.log(t.clamp_min(1e-12)) - torch.log(s.clamp_min(1e-12)))).sum(-1).mean()


class PiscesLxOptimalTransportAligner:
    """Soft assignment of student layers to teacher layers: entropic optimal transport (Sinkhorn) on the matrix of
    pairwise state distances with uniform marginals; returns the plan [n_student, n_teacher]."""

    def __init__(self, reg: float = 0.1, iters: int = 50):
        self.reg, self.iters = reg, iters

    @torch.no_grad()
    def plan(self, student: Sequence[torch.Tensor], teacher: Sequence[torch.Tensor]) -> torch.Tensor:
        def unit(x):
            x = x.float().flatten(0, -2).mean(0)
            return x / x.norm().clamp_min(1e-12)
        # direction statistics only need equal widths when compared; otherwise compare depth positions
        same = student[0].shape[-1] == teacher[0].shape[-1]
        ns, nt = len(student), len(teacher)
        if same:
            S_, T_ = torch.stack([unit(h) for h in student]), torch.stack([unit(h) for h in teacher])
            cost = 1 - S_ @ T_.t()
        else:
            ps, pt = torch.linspace(0, 1, ns).unsqueeze(1), torch.linspace(0, 1, nt).unsqueeze(0)
            cost = (ps - pt).abs()
        Kmat = torch.exp(-cost / self.reg)
        a, b = torch.full((ns,), 1.0 / ns), torch.full((nt,), 1.0 / nt)
        u, v = torch.ones(ns), torch.ones(nt)
        for _ in range(self.iters):
            u = a / (Kmat @ v).clamp_min(1e-30)
            v = b / (Kmat.t() @ u).clamp_min(1e-30)
        return u.unsqueeze(1) * Kmat * v.unsqueeze(0)


class PiscesLxLayerWiseDistillationLoss(nn.Module):
    """Hidden-state loss over several layers.  ``mapping`` pairs student layer i with teacher layer mapping[i]; without
    one, teacher layers are picked at uniform depth positions, or softly through an optimal-transport plan."""

    def __init__(self, student_dim: int, teacher_dim: int, mapping: Optional[List[int]] = None, use_ot: bool = False):
        super().__init__()
        self.loss = PiscesLxHiddenStateDistillationLoss(student_dim, teacher_dim)
        self.mapping, self.use_ot = mapping, use_ot
        self.aligner = PiscesLxOptimalTransportAligner() if use_ot else None

    def forward(self, student_states: Sequence[torch.Tensor], teacher_states: Sequence[torch.Tensor]) -> torch.Tensor:
        ns, nt = len(student_states), len(teacher_states)
        if self.use_ot:
            plan = self.aligner.plan(student_states, teacher_states).to(student_states[0].device)
            plan = plan / plan.sum(1, keepdim=True)
            return sum(plan[i, j] * self.loss(student_states[i], teacher_states[j])
                       for i in range(ns) for j in range(nt) if float(plan[i, j]) > 1e-3) / ns
        mp = self.mapping or [round((i + 1) * nt / ns) - 1 for i in range(ns)]
        return sum(self.loss(student_states[i], teacher_states[j]) for i, j in enumerate(mp)) / ns


class PiscesLxContrastiveDistillationLoss(nn.Module):
    """InfoNCE between pooled student and teacher representations of the same sample (positives on the diagonal)."""

    def __init__(self, student_dim: int, teacher_dim: int, dim: int = 128, temperature: float = 0.1):
        super().__init__()
        self.ps, self.pt, self.tau = nn.Linear(student_dim, dim, bias=False), nn.Linear(teacher_dim, dim, bias=False), temperature

    def forward(self, student_h: torch.Tensor, teacher_h: torch.Tensor) -> torch.Tensor:
        s = F.normalize(self.ps(student_h.float().mean(1) if student_h.dim() == 3 else student_h.float()), dim=-1)
        t = F.normalize(self.pt(teacher_h.float().mean(1) if teacher_h.dim() == 3 else teacher_h.float()), dim=-1)
        logits = s @ t.t() / self.tau
        tgt = torch.arange(s.shape[0], device=s.device)
        return 0.5 * (F.cross_entropy(logits, tgt) + F.cross_entropy(logits.t(), tgt))


class PiscesLxDistillationLoss(nn.Module):
    """Weighted sum of the parts that are switched on and whose inputs are present; returns (total, parts)."""

    def __init__(self, cfg: Optional[PiscesLxDistillationLossConfig] = None, student_dim: int = 0, teacher_dim: int = 0):
        super().__init__()
        self.cfg = cfg or PiscesLxDistillationLossConfig()
        self.logits = PiscesLxLogitsDistillationLoss(self.cfg.temperature)
        self.hidden = PiscesLxLayerWiseDistillationLoss(student_dim, teacher_dim) if self.cfg.hidden_weight > 0 else None
        self.attn = PiscesLxAttentionDistillationLoss() if self.cfg.attention_weight > 0 else None
        self.contrast = PiscesLxContrastiveDistillationLoss(student_dim, teacher_dim, temperature=self.cfg.contrastive_temperature) \
            if self.cfg.contrastive_weight > 0 else None

    def forward(self, student: Dict[str, torch.Tensor], teacher: Dict[str, torch.Tensor],
                labels: Optional[torch.Tensor] = None):
        c, parts = self.cfg, {}
        if c.logits_weight > 0 and "logits" in student and "logits" in teacher:
            parts["logits"] = c.logits_weight * self.logits(student["logits"], teacher["logits"])
        if self.hidden is not None and "hidden_states" in student and "hidden_states" in teacher:
            parts["hidden"] = c.hidden_weight * self.hidden(student["hidden_states"], teacher["hidden_states"])
        if self.attn is not None and "attentions" in student and "attentions" in teacher:
            parts["attention"] = c.attention_weight * self.attn(student["attentions"], teacher["attentions"])
        if self.contrast is not None and "hidden_states" in student and "hidden_states" in teacher:
            parts["contrastive"] = c.contrastive_weight * self.contrast(student["hidden_states"][-1], teacher["hidden_states"][-1])
        if c.hard_label_weight > 0 and labels is not None and "logits" in student:
            lg = student["logits"].float()
            parts["hard"] = c.hard_label_weight * F.cross_entropy(lg[:, :-1].reshape(-1, lg.shape[-1]), labels[:, 1:].reshape(-1),
                                                                  ignore_index=-100)
        total = sum(parts.values()) if parts else torch.zeros(())
        return total, {k: float(v.detach()) for k, v in parts.items()}
