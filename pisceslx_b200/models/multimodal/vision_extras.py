"""Vision-side extras (reference model/multimodal/vision.py: ``YvImageDecoder`` :1109, ``YvDiffusionImageEnhancer``
:1283, ``YvSigLIPVisionEncoder`` :1671, ``YvDynamicResolutionProcessor`` :1979, ``YvMoVEVisionEncoder`` :2252,
``YvSparseCutRouter`` :2350) and the remaining normalisation / rotary variants (model/core/norms.py
``YvAdaptiveLayerNorm`` / ``YvGroupNorm``; model/core/mr_rope.py ``YvMrRoPERotaryEmbedding``; model/utils/rope.py:115
``YvLinearScalingRoPE``).

The ViT trunk itself (patchify kernel + GEMM patch embed + flash attention blocks) is ``multimodal.vision``; the
classes here wrap or post-process it."""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as F_


# ------------------------------------------------------------------------------------------------ norms / rotary
class YvAdaptiveLayerNorm(nn.Module):
    """LayerNorm whose scale and shift are predicted from a conditioning vector (zero-initialised: starts as a plain
    parameter-free LayerNorm)."""

    def __init__(self, dim: int, cond_dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.mod = nn.Linear(cond_dim, 2 * dim)
        nn.init.zeros_(self.mod.weight)
        nn.init.zeros_(self.mod.bias)

    def forward(self, x: torch.Tensor, cond: torch.Tensor) -> torch.Tensor:
        scale, shift = self.mod(cond.float()).chunk(2, -1)
        while scale.dim() < x.dim():
            scale, shift = scale.unsqueeze(-2), shift.unsqueeze(-2)
        return (F.layer_norm(x.float(), x.shape[-1:], eps=self.eps) * (1 + scale) + shift).to(x.dtype)


class YvGroupNorm(nn.GroupNorm):
    """GroupNorm over the channel (last) dimension of [B, ..., C] token tensors (fp32 statistics)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        shp = x.shape
        y = super().forward(x.float().reshape(shp[0], -1, shp[-1]).transpose(1, 2))
        return y.transpose(1, 2).reshape(shp).to(x.dtype)


class YvLinearScalingRoPE(nn.Module):
    """Position interpolation: positions are divided by ``scale`` before the rotary angles are formed."""

    def __init__(self, rot_dim: int, theta: float = 1e4, scale: float = 1.0):
        super().__init__()
        self.scale = scale
        self.register_buffer("inv_freq", theta ** (-torch.arange(0, rot_dim, 2).float() / rot_dim), persistent=False)

    def forward(self, positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        ang = (positions.float() / self.scale)[..., None] * self.inv_freq
        ang = torch.cat([ang, ang], -1)
        return ang.cos(), ang.sin()


class YvMrRoPERotaryEmbedding(nn.Module):
    """Mixed-radix rotary embedding: the frequency ladder is built from two bases.  ``uni`` interleaves them pair by
    pair; ``pro`` moves progressively from the small base (fast, local pairs) to the large one (slow pairs that
    carry long-range position), which is what allows extrapolation by raising only the large base."""

    def __init__(self, rot_dim: int, base_small: float = 1e4, base_large: float = 1e6, mode: str = "pro"):
        super().__init__()
        n = rot_dim // 2
        d = torch.arange(n).float() / n
        if mode == "uni":
            base = torch.where(torch.arange(n) % 2 == 0, torch.tensor(base_small), torch.tensor(base_large))
        elif mode == "pro":
            base = torch.exp(torch.lerp(torch.tensor(math.log(base_small)), torch.tensor(math.log(base_large)), d))
        else:
            raise ValueError(mode)
        self.register_buffer("inv_freq", base ** (-d), persistent=False)

    def forward(self, positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        ang = positions.float()[..., None] * self.inv_freq
        ang = torch.cat([ang, ang], -1)
        return ang.cos(), ang.sin()


# ------------------------------------------------------------------------------------------------ resolution / routing
class YvDynamicResolutionProcessor:
    """Native-resolution preprocessing: each image keeps its aspect ratio, is scaled so that its patch count stays
    within [min_patches, max_patches], and is padded up to a multiple of the patch size."""

    def __init__(self, patch: int = 14, min_patches: int = 16, max_patches: int = 4096):
        self.patch, self.min_p, self.max_p = patch, min_patches, max_patches

    def target_size(self, h: int, w: int) -> Tuple[int, int]:
        p = self.patch
        n = (h / p) * (w / p)
        s = 1.0
        if n > self.max_p:
            s = math.sqrt(self.max_p / n)
        elif n < self.min_p:
            s = math.sqrt(self.min_p / n)
        gh, gw = max(1, round(h * s / p)), max(1, round(w * s / p))
        while gh * gw > self.max_p:
            if gh >= gw:
                gh -= 1
            else:
                gw -= 1
        return gh * p, gw * p

    def __call__(self, img: torch.Tensor) -> Dict[str, object]:
        """img [C, H, W] -> {"image": [C, H', W'], "grid": (gh, gw)} with H', W' multiples of the patch."""
        C, H, W = img.shape
        th, tw = self.target_size(H, W)
        out = F.interpolate(img[None].float(), size=(th, tw), mode="bilinear", align_corners=False, antialias=True)[0]
        return {"image": out.to(img.dtype) if img.is_floating_point() else out, "grid": (th // self.patch, tw // self.patch)}


class YvSparseCutRouter(nn.Module):
    """Keeps the ``ratio`` highest-scoring visual tokens (learned scalar score per token); kept tokens stay in their
    original order and are scaled by a straight-through gate so that the scorer trains."""

    def __init__(self, dim: int, ratio: float = 0.5, min_tokens: int = 1):
        super().__init__()
        self.score = nn.Linear(dim, 1)
        self.ratio, self.min_tokens = ratio, min_tokens

    def forward(self, tokens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        B, N, D = tokens.shape
        k = max(self.min_tokens, min(N, int(round(N * self.ratio))))
        s = self.score(tokens.float()).squeeze(-1)
        idx = s.topk(k, -1).indices.sort(-1).values
        g = torch.sigmoid(torch.gather(s, 1, idx))
        kept = torch.gather(tokens, 1, idx[..., None].expand(-1, -1, D))
        return kept * (1 + g - g.detach())[..., None].to(tokens.dtype), idx


class YvMoVEVisionEncoder(nn.Module):
    """Mixture of vision encoders: every encoder maps images to [B, N, D] tokens on the same grid; a gate on the mean
    token mixes the top-``k`` encoders per token.  With one encoder it is a pass-through."""

    def __init__(self, encoders: Dict[str, nn.Module], dim: int, top_k: int = 1):
        super().__init__()
        self.encoders = nn.ModuleDict(encoders)
        self.top_k = min(top_k, len(encoders))
        self.gate = nn.Linear(dim, len(encoders)) if len(encoders) > 1 else None

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        outs = [enc(images) for enc in self.encoders.values()]
        if self.gate is None:
            return outs[0]
        stack = torch.stack(outs, 2)                                           # [B, N, E, D]
        probs = torch.softmax(self.gate(stack.float().mean(2)), -1)            # [B, N, E]
        w, idx = probs.topk(self.top_k, -1)
        w = w / w.sum(-1, keepdim=True)
        mix = torch.zeros_like(probs).scatter_(-1, idx, w)
        return (stack * mix[..., None].to(stack.dtype)).sum(2)


class _GRN(nn.Module):
    """Global response normalisation over tokens (ConvNeXt-V2): x + gamma * (x * ||x||_token / mean) + beta."""

    def __init__(self, dim: int):
        super().__init__()
        self.gamma, self.beta = nn.Parameter(torch.zeros(dim)), nn.Parameter(torch.zeros(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        g = x.float().norm(dim=1, keepdim=True)
        n = g / g.mean(-1, keepdim=True).clamp_min(1e-6)
        return (x.float() + self.gamma * (x.float() * n) + self.beta).to(x.dtype)


class YvSigLIPVisionEncoder(nn.Module):
    """SigLIP-style tower around a ViT trunk: LayerScale'd residual refinement with GRN, multi-scale token features
    (taps after given fractions of the trunk are not needed here: the trunk returns its final tokens), an attention
    pooling head (one learned probe) and the pairwise sigmoid loss with learnable temperature and bias."""

    def __init__(self, trunk: nn.Module, dim: int, embed_dim: int = 512, n_head: int = 8, layer_scale: float = 1e-5):
        super().__init__()
        self.trunk, self.h, self.d = trunk, n_head, dim // n_head
        self.grn = _GRN(dim)
        self.ls = nn.Parameter(torch.full((dim,), layer_scale))
        self.probe = nn.Parameter(torch.randn(1, dim) * 0.02)
        self.kv = nn.Parameter(torch.empty(2 * dim, dim).normal_(std=0.02))
        self.proj = nn.Parameter(torch.empty(embed_dim, dim).normal_(std=0.02))
        self.logit_scale = nn.Parameter(torch.tensor(math.log(10.0)))
        self.logit_bias = nn.Parameter(torch.tensor(-10.0))

    def tokens(self, images: torch.Tensor) -> torch.Tensor:
        t = self.trunk(images)
        return t + self.ls.to(t.dtype) * self.grn(t)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        t = self.tokens(images)
        B, N, D = t.shape
        k, v = F_.linear(t, self.kv.to(t.dtype)).view(B, N, 2, self.h, self.d).unbind(2)
        q = self.probe.to(t.dtype).view(1, 1, self.h, self.d).expand(B, -1, -1, -1)
        a = torch.softmax(torch.einsum("bqhd,bnhd->bhqn", q.float(), k.float()) * self.d ** -0.5, -1)
        pooled = torch.einsum("bhqn,bnhd->bqhd", a, v.float()).reshape(B, D).to(t.dtype)
        return F.normalize(F_.linear(pooled, self.proj.to(t.dtype)).float(), dim=-1)

    def sigmoid_loss(self, img_emb: torch.Tensor, txt_emb: torch.Tensor) -> torch.Tensor:
        logits = img_emb @ txt_emb.t() * self.logit_scale.exp() + self.logit_bias
        labels = 2 * torch.eye(logits.shape[0], device=logits.device) - 1
        return -F.logsigmoid(labels * logits).sum() / logits.shape[0]


# ------------------------------------------------------------------------------------------------ image generation
class _ResBlock(nn.Module):
    def __init__(self, c: int, groups: int = 8):
        super().__init__()
        g = math.gcd(groups, c)
        self.n1, self.c1 = nn.GroupNorm(g, c), nn.Conv2d(c, c, 3, padding=1)
        self.n2, self.c2 = nn.GroupNorm(g, c), nn.Conv2d(c, c, 3, padding=1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.c1(F.silu(self.n1(x)))
        return x + self.c2(F.silu(self.n2(h)))


class YvImageDecoder(nn.Module):
    """Latent -> RGB by progressive 2x upsampling: the latent is projected to a ``base`` x ``base`` map, then each
    stage doubles the resolution (nearest + conv) and halves the channels, with a residual block per stage."""

    def __init__(self, latent_dim: int, base: int = 8, stages: int = 3, channels: int = 128):
        super().__init__()
        self.base, self.c0 = base, channels
        self.inp = nn.Linear(latent_dim, channels * base * base)
        ups, c = [], channels
        for _ in range(stages):
            ups += [nn.Upsample(scale_factor=2, mode="nearest"), nn.Conv2d(c, max(8, c // 2), 3, padding=1), _ResBlock(max(8, c // 2))]
            c = max(8, c // 2)
        self.ups = nn.Sequential(*ups)
        self.out = nn.Conv2d(c, 3, 3, padding=1)

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        x = self.inp(z.float()).view(-1, self.c0, self.base, self.base)
        return torch.tanh(self.out(F.silu(self.ups(x))))


class YvDiffusionImageEnhancer(nn.Module):
    """A small DDPM refiner: a two-level U-Net predicts the noise in an image at step t (sinusoidal time embedding
    added per level); ``enhance`` noises the decoder's image to ``t_start`` and denoises it back deterministically
    (DDIM, eta 0)."""

    def __init__(self, channels: int = 32, steps: int = 1000):
        super().__init__()
        self.steps, self.c = steps, channels
        beta = torch.linspace(1e-4, 0.02, steps)
        self.register_buffer("abar", torch.cumprod(1 - beta, 0), persistent=False)
        self.t_mlp = nn.Sequential(nn.Linear(channels, channels), nn.SiLU(), nn.Linear(channels, 2 * channels))
        self.inp = nn.Conv2d(3, channels, 3, padding=1)
        self.d1, self.down = _ResBlock(channels), nn.Conv2d(channels, 2 * channels, 3, stride=2, padding=1)
        self.mid = _ResBlock(2 * channels)
        self.up = nn.ConvTranspose2d(2 * channels, channels, 4, stride=2, padding=1)
        self.u1, self.out = _ResBlock(channels), nn.Conv2d(channels, 3, 3, padding=1)
        nn.init.zeros_(self.out.weight)
        nn.init.zeros_(self.out.bias)

    def time_embedding(self, t: torch.Tensor) -> torch.Tensor:
        half = self.c // 2
        f = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device) / half)
        a = t.float()[:, None] * f
        return torch.cat([a.sin(), a.cos()], -1)

    def predict_noise(self, x: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        e1, e2 = self.t_mlp(self.time_embedding(t)).split([self.c, self.c], -1)
        h1 = self.d1(self.inp(x) + e1[..., None, None])
        h2 = self.mid(self.down(h1) + torch.cat([e2, e2], -1)[..., None, None])
        return self.out(self.u1(self.up(h2) + h1))

    def training_loss(self, x0: torch.Tensor) -> torch.Tensor:
        t = torch.randint(0, self.steps, (x0.shape[0],), device=x0.device)
        n = torch.randn_like(x0)
        a = self.abar[t].view(-1, 1, 1, 1)
        return F.mse_loss(self.predict_noise(a.sqrt() * x0 + (1 - a).sqrt() * n, t), n)

    @torch.no_grad()
    def enhance(self, img: torch.Tensor, t_start: int = 200, n_steps: int = 10) -> torch.Tensor:
        ts = torch.linspace(t_start, 0, n_steps + 1).long().tolist()
        a0 = self.abar[ts[0]]
        x = a0.sqrt() * img + (1 - a0).sqrt() * torch.randn_like(img)
        for t, t_next in zip(ts[:-1], ts[1:]):
            a, an = self.abar[t], self.abar[t_next] if t_next > 0 else torch.tensor(1.0, device=img.device)
            eps = self.predict_noise(x, torch.full((img.shape[0],), t, device=img.device))
            x0 = ((x - (1 - a).sqrt() * eps) / a.sqrt()).clamp(-1, 1)
            x = an.sqrt() * x0 + (1 - an).sqrt() * eps
        return x
