"""Further cross-modal fusion components (reference model/multimodal/enhanced_fusion.py: ``YvEnhancedModalFusion``,
``YvContrastiveCrossModalAligner``, ``YvTaskAwareModalityImportance``, ``YvOnlineQualityAdaptation``;
rca_fusion.py: ``YvRCACrossCorrelationAttention``, ``YvRecurrentModalRefiner``; fusion.py:
``YvUnifiedMultimodalTokenizer``; vision.py: ``YvHighResolutionTileProcessor``, ``YvVisionPrefixTuning``).
Projections run through the package's GEMM op; the attention here is over a handful of modality tokens, far from the
throughput path."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as F_


def _w(o: int, i: int, std: float = 0.02) -> nn.Parameter:
    return nn.Parameter(torch.empty(o, i).normal_(std=std))


@dataclass
class YvModalFusionConfig:
    hidden_size: int = 512
    modalities: Tuple[str, ...] = ("text", "image", "audio", "video")
    n_head: int = 8
    n_output_tokens: int = 8
    n_tasks: int = 4
    temperature: float = 0.07


class YvContrastiveCrossModalAligner(nn.Module):
    """Projects two modalities into a shared space and scores them with a symmetric InfoNCE loss; ``hard_k`` keeps
    only the k hardest negatives per row in the denominator (hard negative mining)."""

    def __init__(self, dim_a: int, dim_b: int, embed: int = 256, temperature: float = 0.07, hard_k: int = 0):
        super().__init__()
        self.pa, self.pb = _w(embed, dim_a), _w(embed, dim_b)
        self.log_t = nn.Parameter(torch.tensor(math.log(1.0 / temperature)))
        self.hard_k = hard_k

    def embed(self, a: torch.Tensor, b: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return (F.normalize(F_.linear(a, self.pa.to(a.dtype)).float(), dim=-1),
                F.normalize(F_.linear(b, self.pb.to(b.dtype)).float(), dim=-1))

    def _nce(self, logits: torch.Tensor) -> torch.Tensor:
        n = logits.shape[0]
        if self.hard_k and n - 1 > self.hard_k:
            eye = torch.eye(n, dtype=torch.bool, device=logits.device)
            neg = logits.masked_fill(eye, float("-inf")).topk(self.hard_k, -1).values
            all_ = torch.cat([logits.diagonal()[:, None], neg], 1)
            return -torch.log_softmax(all_, -1)[:, 0].mean()
        return F.cross_entropy(logits, torch.arange(n, device=logits.device))

    def forward(self, a: torch.Tensor, b: torch.Tensor) -> Dict[str, torch.Tensor]:
        ea, eb = self.embed(a, b)
        logits = ea @ eb.t() * self.log_t.exp().clamp(max=100.0)
        loss = 0.5 * (self._nce(logits) + self._nce(logits.t()))
        return {"loss": loss, "accuracy": (logits.argmax(-1) == torch.arange(len(a), device=a.device)).float().mean(),
                "logits": logits}


class YvTaskAwareModalityImportance(nn.Module):
    """Modality weights from the pooled modality features, modulated by a task embedding (reasoning, generation,
    understanding, ...): softmax over modalities that are present."""

    def __init__(self, hidden: int, n_modalities: int, n_tasks: int = 4):
        super().__init__()
        self.score = _w(1, hidden)
        self.task = nn.Embedding(n_tasks, n_modalities)
        nn.init.zeros_(self.task.weight)

    def forward(self, pooled: torch.Tensor, task_id: torch.Tensor, present: Optional[torch.Tensor] = None) -> torch.Tensor:
        """pooled [B, M, H]; task_id [B]; present [B, M] bool -> weights [B, M]."""
        s = F_.linear(pooled, self.score.to(pooled.dtype)).float().squeeze(-1) + self.task(task_id)
        if present is not None:
            s = s.masked_fill(~present, float("-inf"))
        return torch.softmax(s, -1)


class YvOnlineQualityAdaptation:
    """Per-modality quality weights adapted online from task rewards: an exponentiated-gradient (bandit) update on
    the weights of the modalities that took part, with a small replay of past (usage, reward) pairs for stability."""

    def __init__(self, n_modalities: int, lr: float = 0.1, replay: int = 64):
        self.logw = torch.zeros(n_modalities)
        self.lr, self.replay_size = lr, replay
        self.buffer: List[Tuple[torch.Tensor, float]] = []
        self.baseline = 0.0

    def weights(self) -> torch.Tensor:
        return torch.softmax(self.logw, 0)

    def update(self, usage: torch.Tensor, reward: float) -> torch.Tensor:
        """usage [M] in [0, 1]: how much each modality contributed to the answer that earned ``reward``."""
        self.buffer.append((usage.float().clone(), float(reward)))
        del self.buffer[:-self.replay_size]
        self.baseline = 0.9 * self.baseline + 0.1 * reward
        for u, r in self.buffer[-8:]:
            self.logw += self.lr / 8 * (r - self.baseline) * (u - self.weights())
        return self.weights()


class YvRCACrossCorrelationAttention(nn.Module):
    """Cross-correlation attention between two token sets: the affinity matrix A = Q_a K_b^T is used in both
    directions (a attends to b with softmax over b, b attends to a with softmax over a), so that one correlation
    computation refines both sides."""

    def __init__(self, hidden: int, n_head: int = 8):
        super().__init__()
        self.h, self.d = n_head, hidden // n_head
        self.qa, self.kb, self.va, self.vb = _w(hidden, hidden), _w(hidden, hidden), _w(hidden, hidden), _w(hidden, hidden)
        self.oa, self.ob = nn.Parameter(torch.zeros(hidden, hidden)), nn.Parameter(torch.zeros(hidden, hidden))

    def forward(self, a: torch.Tensor, b: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        B, Sa, H = a.shape
        Sb = b.shape[1]
        sp = lambda t, w, S: F_.linear(t, w.to(t.dtype)).view(B, S, self.h, self.d).transpose(1, 2).float()
        q, k = sp(a, self.qa, Sa), sp(b, self.kb, Sb)
        A = torch.matmul(q, k.transpose(-1, -2)) * self.d ** -0.5                      # [B, h, Sa, Sb]
        ra = torch.matmul(torch.softmax(A, -1), sp(b, self.vb, Sb))
        rb = torch.matmul(torch.softmax(A.transpose(-1, -2), -1), sp(a, self.va, Sa))
        merge = lambda r, S: r.transpose(1, 2).reshape(B, S, H)
        return (a + F_.linear(merge(ra, Sa).to(a.dtype), self.oa.to(a.dtype)),
                b + F_.linear(merge(rb, Sb).to(b.dtype), self.ob.to(b.dtype)))


class YvRecurrentModalRefiner(nn.Module):
    """Applies one shared cross-correlation block ``rounds`` times with a GRU-style gate on each side, so that extra
    rounds refine rather than overwrite."""

    def __init__(self, hidden: int, rounds: int = 3, n_head: int = 8):
        super().__init__()
        self.rounds, self.rca = rounds, YvRCACrossCorrelationAttention(hidden, n_head)
        self.gate_a, self.gate_b = _w(hidden, 2 * hidden), _w(hidden, 2 * hidden)

    def forward(self, a: torch.Tensor, b: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        for _ in range(self.rounds):
            na, nb = self.rca(a, b)
            za = torch.sigmoid(F_.linear(torch.cat([a, na], -1), self.gate_a.to(a.dtype)).float()).to(a.dtype)
            zb = torch.sigmoid(F_.linear(torch.cat([b, nb], -1), self.gate_b.to(b.dtype)).float()).to(b.dtype)
            a, b = (1 - za) * a + za * na, (1 - zb) * b + zb * nb
        return a, b


class YvUnifiedMultimodalTokenizer(nn.Module):
    """Maps every modality's features into the text embedding space: a projection per modality plus a learned
    modality embedding, then concatenation in a fixed modality order with begin / end marker embeddings."""

    def __init__(self, hidden: int, feature_dims: Dict[str, int]):
        super().__init__()
        self.order = list(feature_dims)
        self.proj = nn.ParameterDict({m: _w(hidden, d) for m, d in feature_dims.items()})
        self.mod_emb = nn.ParameterDict({m: nn.Parameter(torch.zeros(hidden)) for m in feature_dims})
        self.markers = nn.ParameterDict({m: nn.Parameter(torch.randn(2, hidden) * 0.02) for m in feature_dims})

    def forward(self, features: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, List[Tuple[str, int, int]]]:
        """features[m] [B, N_m, D_m] -> (tokens [B, sum(N_m + 2), H], spans [(modality, start, end)])."""
        parts, spans, pos = [], [], 0
        for m in self.order:
            if m not in features:
                continue
            x = features[m]
            t = F_.linear(x, self.proj[m].to(x.dtype)) + self.mod_emb[m].to(x.dtype)
            B = t.shape[0]
            mk = self.markers[m].to(x.dtype)
            seq = torch.cat([mk[0].expand(B, 1, -1), t, mk[1].expand(B, 1, -1)], 1)
            parts.append(seq)
            spans.append((m, pos, pos + seq.shape[1]))
            pos += seq.shape[1]
        return torch.cat(parts, 1), spans


class YvEnhancedModalFusion(nn.Module):
    """Fusion pipeline: per-modality pooled features -> task-aware importance weights -> weighted modality tokens ->
    learned output queries cross-attend to all modality tokens -> ``n_output_tokens`` fused tokens (prepended to the
    text embeddings by the trunk)."""

    def __init__(self, config: Optional[YvModalFusionConfig] = None):
        super().__init__()
        self.config = c = config or YvModalFusionConfig()
        self.importance = YvTaskAwareModalityImportance(c.hidden_size, len(c.modalities), c.n_tasks)
        self.queries = nn.Parameter(torch.randn(c.n_output_tokens, c.hidden_size) * 0.02)
        self.kv = _w(2 * c.hidden_size, c.hidden_size)
        self.o = _w(c.hidden_size, c.hidden_size)
        self.h, self.d = c.n_head, c.hidden_size // c.n_head

    def forward(self, features: Dict[str, torch.Tensor], task_id: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        """features[m] [B, N_m, H] for the modalities present."""
        c = self.config
        mods = [m for m in c.modalities if m in features]
        B = features[mods[0]].shape[0]
        dev = features[mods[0]].device
        pooled = torch.stack([features[m].mean(1) if m in features else torch.zeros(B, c.hidden_size, device=dev)
                              for m in c.modalities], 1)
        present = torch.tensor([m in features for m in c.modalities], device=dev).expand(B, -1)
        task_id = task_id if task_id is not None else torch.zeros(B, dtype=torch.long, device=dev)
        w = self.importance(pooled, task_id, present)                                  # [B, M]
        toks = torch.cat([features[m] * w[:, c.modalities.index(m), None, None].to(features[m].dtype) * len(mods) for m in mods], 1)
        N = toks.shape[1]
        k, v = F_.linear(toks, self.kv.to(toks.dtype)).view(B, N, 2, self.h, self.d).unbind(2)
        q = self.queries.to(toks.dtype).view(1, -1, self.h, self.d).expand(B, -1, -1, -1)
        a = torch.softmax(torch.einsum("bqhd,bnhd->bhqn", q.float(), k.float()) * self.d ** -0.5, -1)
        fused = torch.einsum("bhqn,bnhd->bqhd", a, v.float()).reshape(B, -1, c.hidden_size).to(toks.dtype)
        return {"tokens": F_.linear(fused, self.o.to(toks.dtype)) + self.queries.to(toks.dtype), "modality_weights": w}


class YvHighResolutionTileProcessor:
    """Splits a large image into overlapping tiles plus a down-scaled global view, and merges per-tile feature maps
    back with linear blending in the overlaps."""

    def __init__(self, tile: int = 448, overlap: int = 32):
        assert 0 <= overlap < tile
        self.tile, self.overlap = tile, overlap

    def grid(self, H: int, W: int) -> List[Tuple[int, int]]:
        step = self.tile - self.overlap
        ys = list(range(0, max(H - self.tile, 0) + 1, step))
        xs = list(range(0, max(W - self.tile, 0) + 1, step))
        if ys[-1] + self.tile < H:
            ys.append(H - self.tile)
        if xs[-1] + self.tile < W:
            xs.append(W - self.tile)
        return [(y, x) for y in ys for x in xs]

    def split(self, img: torch.Tensor) -> Dict[str, Any]:
        """img [C, H, W] with H, W >= tile -> tiles [n, C, tile, tile], their origins, and a global view."""
        C, H, W = img.shape
        origins = self.grid(H, W)
        tiles = torch.stack([img[:, y:y + self.tile, x:x + self.tile] for y, x in origins])
        glob = F.interpolate(img[None].float(), size=(self.tile, self.tile), mode="bilinear", align_corners=False)[0].to(img.dtype)
        return {"tiles": tiles, "origins": origins, "global": glob, "size": (H, W)}

    def merge(self, tile_maps: torch.Tensor, origins: Sequence[Tuple[int, int]], size: Tuple[int, int]) -> torch.Tensor:
        """tile_maps [n, C, tile, tile] (same resolution as the tiles) -> [C, H, W] with blended overlaps."""
        H, W = size
        C, t = tile_maps.shape[1], self.tile
        out = torch.zeros(C, H, W, dtype=torch.float32, device=tile_maps.device)
        wt = torch.zeros(H, W, dtype=torch.float32, device=tile_maps.device)
        ramp = torch.ones(t, device=tile_maps.device)
        if self.overlap:
            r = torch.linspace(0, 1, self.overlap + 2, device=tile_maps.device)[1:-1]
            ramp[: self.overlap], ramp[-self.overlap:] = r, r.flip(0)
        w2 = ramp[:, None] * ramp[None, :]
        for m, (y, x) in zip(tile_maps, origins):
            out[:, y:y + t, x:x + t] += m.float() * w2
            wt[y:y + t, x:x + t] += w2
        return (out / wt.clamp_min(1e-6)).to(tile_maps.dtype)


class YvVisionPrefixTuning(nn.Module):
    """Soft prefix: ``n_prefix`` learned tokens are prepended to the vision tokens as extra keys / values of an
    attention layer (the vision tokens themselves are returned refined, the prefix is not part of the output)."""

    def __init__(self, dim: int, n_prefix: int = 16, n_head: int = 8):
        super().__init__()
        self.prefix = nn.Parameter(torch.randn(n_prefix, dim) * 0.02)
        self.h, self.d = n_head, dim // n_head
        self.q, self.kv = _w(dim, dim), _w(2 * dim, dim)
        self.o = nn.Parameter(torch.zeros(dim, dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, N, D = x.shape
        ctx = torch.cat([self.prefix.to(x.dtype).expand(B, -1, -1), x], 1)
        M = ctx.shape[1]
        q = F_.linear(x, self.q.to(x.dtype)).view(B, N, self.h, self.d).transpose(1, 2).float()
        k, v = F_.linear(ctx, self.kv.to(x.dtype)).view(B, M, 2, self.h, self.d).unbind(2)
        a = torch.softmax(torch.matmul(q, k.transpose(1, 2).transpose(-1, -2).float()) * self.d ** -0.5, -1)
        r = torch.matmul(a, v.transpose(1, 2).float()).transpose(1, 2).reshape(B, N, D).to(x.dtype)
        return x + F_.linear(r, self.o.to(x.dtype))
