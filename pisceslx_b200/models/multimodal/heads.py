"""Multimodal output side: image tokenizer, vision task heads, speech generation, deep cross-modal injection.

Reference components covered: ``YvLFQTokenizer`` (lookup-free quantisation of patch features, model/multimodal/vision.py),
detection / segmentation / VQA heads (model/multimodal/vision.py task heads), ``YvNeuralVocoder`` and ``YvTalker``
(model/multimodal/audio.py: codec-token language head and a transposed-convolution vocoder),
``YvRecursiveCrossModalFusion`` / ``YvDeepCrossLayerInjector`` (model/multimodal/fusion.py: modality features injected at
several depths through gated cross attention).  All projections run through the package's GEMM ops."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as F_


def _w(o: int, i: int, std: float = 0.02) -> nn.Parameter:
    return nn.Parameter(torch.empty(o, i).normal_(std=std))


class YvLFQTokenizer(nn.Module):
    """Lookup-free quantiser: features are projected to ``bits`` dimensions, each dimension is quantised to its sign,
    and the token id is the integer those bits spell (codebook of 2**bits entries with no embedding table).  The
    backward pass is straight-through; ``aux`` holds the commitment and the entropy terms."""

    def __init__(self, dim: int, bits: int = 12, commitment: float = 0.25):
        super().__init__()
        self.bits, self.commitment = bits, commitment
        self.proj_in, self.proj_out = _w(bits, dim), _w(dim, bits)
        self.register_buffer("pow2", 2 ** torch.arange(bits), persistent=False)

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, Dict[str, torch.Tensor]]:
        z = F_.linear(x, self.proj_in.to(x.dtype))
        q = torch.where(z >= 0, torch.ones_like(z), -torch.ones_like(z))
        ids = ((q > 0).long() * self.pow2).sum(-1)
        commit = (z.float() - q.float()).pow(2).mean()
        p = torch.sigmoid(4.0 * z.float())
        per_sample = -(p * torch.log(p + 1e-6) + (1 - p) * torch.log(1 - p + 1e-6)).mean()
        pm = p.reshape(-1, self.bits).mean(0)
        codebook = -(pm * torch.log(pm + 1e-6) + (1 - pm) * torch.log(1 - pm + 1e-6)).mean()
        zq = z + (q - z).detach()
        out = F_.linear(zq, self.proj_out.to(x.dtype))
        return out, ids, {"commit": self.commitment * commit, "entropy": per_sample - codebook}

    def decode(self, ids: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        bits = ((ids[..., None] // self.pow2) % 2).to(dtype) * 2 - 1
        return F_.linear(bits, self.proj_out.to(dtype))


class YvDetectionHead(nn.Module):
    """Query-based detection: ``n_queries`` learned queries cross-attend to patch features and predict class logits
    and (cx, cy, w, h) boxes in [0, 1]."""

    def __init__(self, dim: int, n_classes: int, n_queries: int = 32):
        super().__init__()
        self.queries = nn.Parameter(torch.randn(n_queries, dim) * 0.02)
        self.kv = _w(2 * dim, dim)
        self.cls, self.box = _w(n_classes + 1, dim), _w(4, dim)

    def forward(self, feats: torch.Tensor) -> Dict[str, torch.Tensor]:
        k, v = F_.linear(feats, self.kv.to(feats.dtype)).chunk(2, -1)
        a = torch.softmax(torch.einsum("qd,bnd->bqn", self.queries.to(feats.dtype), k).float() * feats.shape[-1] ** -0.5, -1)
        h = torch.einsum("bqn,bnd->bqd", a.to(feats.dtype), v) + self.queries.to(feats.dtype)
        return {"logits": F_.linear(h, self.cls.to(h.dtype)), "boxes": torch.sigmoid(F_.linear(h, self.box.to(h.dtype)).float())}


class YvSegmentationHead(nn.Module):
    """Per-patch class logits upsampled to pixels: [B, N, D] with N = gh*gw -> [B, classes, gh*patch, gw*patch]."""

    def __init__(self, dim: int, n_classes: int, patch: int = 16):
        super().__init__()
        self.cls, self.patch = _w(n_classes, dim), patch

    def forward(self, feats: torch.Tensor, grid: Tuple[int, int]) -> torch.Tensor:
        B, N, _ = feats.shape
        gh, gw = grid
        lg = F_.linear(feats, self.cls.to(feats.dtype)).float().transpose(1, 2).reshape(B, -1, gh, gw)
        return F.interpolate(lg, scale_factor=self.patch, mode="bilinear", align_corners=False)


class YvVQAHead(nn.Module):
    """Answer classification from pooled image features and a pooled question state."""

    def __init__(self, dim: int, text_dim: int, n_answers: int):
        super().__init__()
        self.wi, self.wt, self.out = _w(dim, dim), _w(dim, text_dim), _w(n_answers, dim)

    def forward(self, feats: torch.Tensor, question: torch.Tensor) -> torch.Tensor:
        h = F_.linear(feats.mean(1), self.wi.to(feats.dtype)) * torch.tanh(F_.linear(question, self.wt.to(question.dtype)))
        return F_.linear(h, self.out.to(h.dtype))


class YvTalker(nn.Module):
    """Speech-token head: from the language model's hidden states, predicts ``n_codebooks`` parallel streams of codec
    tokens (one classifier per codebook, later codebooks conditioned on the embeddings of the earlier ones)."""

    def __init__(self, hidden: int, codebook_size: int = 1024, n_codebooks: int = 4, dim: int = 512):
        super().__init__()
        self.inp = _w(dim, hidden)
        self.emb = nn.ParameterList([nn.Parameter(torch.randn(codebook_size, dim) * 0.02) for _ in range(n_codebooks)])
        self.cls = nn.ParameterList([_w(codebook_size, dim) for _ in range(n_codebooks)])

    def forward(self, hidden: torch.Tensor, codes: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        """hidden [B, T, H]; codes [B, T, n_codebooks] teacher tokens (training) or None (greedy)."""
        h = F_.linear(hidden, self.inp.to(hidden.dtype))
        logits, picked = [], []
        for i, (e, c) in enumerate(zip(self.emb, self.cls)):
            lg = F_.linear(h, c.to(h.dtype))
            tok = codes[..., i] if codes is not None else lg.argmax(-1)
            logits.append(lg)
            picked.append(tok)
            h = h + F.embedding(tok, e.to(h.dtype))
        out = {"logits": torch.stack(logits, 2), "codes": torch.stack(picked, -1)}
        if codes is not None:
            out["loss"] = F.cross_entropy(out["logits"].float().flatten(0, 2), codes.flatten())
        return out


class YvNeuralVocoder(nn.Module):
    """Codec tokens -> waveform: summed codebook embeddings, then transposed-convolution upsampling stages with
    residual dilated convolutions (the HiFi-GAN generator shape)."""

    def __init__(self, codebook_size: int = 1024, n_codebooks: int = 4, dim: int = 128, rates: Sequence[int] = (8, 5, 4, 2)):
        super().__init__()
        self.emb = nn.ModuleList([nn.Embedding(codebook_size, dim) for _ in range(n_codebooks)])
        ups, res, c = [], [], dim
        for r in rates:
            ups.append(nn.ConvTranspose1d(c, c // 2, 2 * r, stride=r, padding=r // 2 + r % 2, output_padding=r % 2))
            c //= 2
            res.append(nn.ModuleList([nn.Conv1d(c, c, 3, dilation=d, padding=d) for d in (1, 3, 9)]))
        self.ups, self.res = nn.ModuleList(ups), nn.ModuleList(res)
        self.out = nn.Conv1d(c, 1, 7, padding=3)
        self.hop = 1
        for r in rates:
            self.hop *= r

    def forward(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, T, n_codebooks] -> waveform [B, T * hop]."""
        x = sum(e(codes[..., i]) for i, e in enumerate(self.emb)).transpose(1, 2)
        for up, rs in zip(self.ups, self.res):
            x = up(F.leaky_relu(x, 0.1))
            for conv in rs:
                x = x + conv(F.leaky_relu(x, 0.1))
        return torch.tanh(self.out(F.leaky_relu(x, 0.1))).squeeze(1)


class YvDeepCrossLayerInjector(nn.Module):
    """Gated cross attention from the text stream to modality features, one instance per injection depth; the gate
    starts at zero so that an untrained injector leaves the language model unchanged."""

    def __init__(self, hidden: int, mod_dim: int, n_head: int = 8):
        super().__init__()
        self.h, self.d = n_head, hidden // n_head
        self.q, self.kv, self.o = _w(hidden, hidden), _w(2 * hidden, mod_dim), _w(hidden, hidden)
        self.gate = nn.Parameter(torch.zeros(1))

    def forward(self, x: torch.Tensor, mod: torch.Tensor) -> torch.Tensor:
        B, S, H = x.shape
        M = mod.shape[1]
        q = F_.linear(x, self.q.to(x.dtype)).view(B, S, self.h, self.d).transpose(1, 2)
        k, v = F_.linear(mod.to(x.dtype), self.kv.to(x.dtype)).chunk(2, -1)
        k, v = k.view(B, M, self.h, self.d).transpose(1, 2), v.view(B, M, self.h, self.d).transpose(1, 2)
        a = torch.softmax(torch.matmul(q.float(), k.float().transpose(-1, -2)) * self.d ** -0.5, -1)
        r = torch.matmul(a, v.float()).to(x.dtype).transpose(1, 2).reshape(B, S, H)
        return x + torch.tanh(self.gate).to(x.dtype) * F_.linear(r, self.o.to(x.dtype))


class YvRecursiveCrossModalFusion(nn.Module):
    """Runs ``rounds`` of mutual refinement: text attends to the modality, the modality attends back to the refined
    text; injectors are shared across rounds (the recursion)."""

    def __init__(self, hidden: int, mod_dim: int, rounds: int = 2, n_head: int = 8):
        super().__init__()
        self.rounds = rounds
        self.t_from_m = YvDeepCrossLayerInjector(hidden, mod_dim, n_head)
        self.m_from_t = YvDeepCrossLayerInjector(mod_dim, hidden, max(1, min(n_head, mod_dim // 16)))

    def forward(self, text: torch.Tensor, mod: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        for _ in range(self.rounds):
            text = self.t_from_m(text, mod)
            mod = self.m_from_t(mod, text)
        return text, mod
