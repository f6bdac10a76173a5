"""SigLIP building blocks (reference model/multimodal/vision.py:1490-1930): attention, MLP, transformer layer, multi-scale
feature extractor, global response normalisation and vision-to-text cross attention, plus a tower assembled from them.

For the device: the attention projects q, k and v with ONE GEMM and runs through ``scaled_dot_product_attention`` (the
flash kernel); the multi-scale extractor normalises and projects its four taps as one batched GEMM over a [scales, ...]
stack instead of four separate small layers (the taps have one shape, so stacking costs a copy and saves three launches
of each of norm, GEMM and activation)."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class YvSigLIPAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, dropout: float = 0.0):
        super().__init__()
        if hidden_size % num_heads:
            raise ValueError("hidden_size must be a multiple of num_heads")
        self.hidden_size, self.num_heads, self.head_dim, self.dropout = hidden_size, num_heads, hidden_size // num_heads, dropout
        self.qkv = nn.Linear(hidden_size, 3 * hidden_size)
        self.out_proj = nn.Linear(hidden_size, hidden_size)

    def forward(self, x: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, N, D = x.shape
        q, k, v = self.qkv(x).view(B, N, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=attention_mask, dropout_p=self.dropout if self.training else 0.0)
        return self.out_proj(a.transpose(1, 2).reshape(B, N, D))


class YvSigLIPMLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: Optional[int] = None):
        super().__init__()
        self.fc1 = nn.Linear(hidden_size, intermediate_size or 4 * hidden_size)
        self.fc2 = nn.Linear(intermediate_size or 4 * hidden_size, hidden_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.fc2(F.gelu(self.fc1(x), approximate="tanh"))


class YvSigLIPTransformerLayer(nn.Module):
    """Pre-norm block with LayerScale on both branches."""

    def __init__(self, hidden_size: int, num_heads: int, intermediate_size: Optional[int] = None, layer_scale: float = 1.0, dropout: float = 0.0):
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(hidden_size), nn.LayerNorm(hidden_size)
        self.attn, self.mlp = YvSigLIPAttention(hidden_size, num_heads, dropout), YvSigLIPMLP(hidden_size, intermediate_size)
        self.ls1, self.ls2 = nn.Parameter(torch.full((hidden_size,), layer_scale)), nn.Parameter(torch.full((hidden_size,), layer_scale))

    def forward(self, x: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = x + self.ls1 * self.attn(self.norm1(x), attention_mask)
        return x + self.ls2 * self.mlp(self.norm2(x))


class YvSigLIPGRN(nn.Module):
    """Global response normalisation over the tokens: x + gamma (x n) + beta with n the per-channel token norm over its mean."""

    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.gamma, self.beta, self.eps = nn.Parameter(torch.zeros(hidden_size)), nn.Parameter(torch.zeros(hidden_size)), eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        g = xf.norm(dim=-2, keepdim=True)
        n = g / g.mean(-1, keepdim=True).clamp_min(self.eps)
        return (xf + self.gamma * (xf * n) + self.beta).to(x.dtype)


class YvSigLIPMultiScaleFeatureExtractor(nn.Module):
    """Taps after 1/4, 1/2, 3/4 and all of the layers; each is normalised, projected and activated, and the results are
    mixed with softmax weights."""

    def __init__(self, hidden_size: int, num_layers: int, num_scales: int = 4):
        super().__init__()
        self.hidden_size, self.num_scales = hidden_size, num_scales
        self.scale_indices = [min(num_layers - 1, max(0, (i + 1) * num_layers // num_scales - 1)) for i in range(num_scales)]
        self.norm_weight, self.norm_bias = nn.Parameter(torch.ones(num_scales, 1, 1, hidden_size)), nn.Parameter(torch.zeros(num_scales, 1, 1, hidden_size))
        self.proj_weight = nn.Parameter(torch.empty(num_scales, hidden_size, hidden_size))
        self.proj_bias = nn.Parameter(torch.zeros(num_scales, 1, hidden_size))
        for w in self.proj_weight:
            nn.init.kaiming_uniform_(w, a=math.sqrt(5))
        self.scale_weights = nn.Parameter(torch.ones(num_scales) / num_scales)

    def forward(self, all_hidden_states: Sequence[torch.Tensor]) -> torch.Tensor:
        x = torch.stack([all_hidden_states[i] for i in self.scale_indices])                # [S, B, N, D]
        S, B, N, D = x.shape
        x = F.layer_norm(x, (D,)) * self.norm_weight + self.norm_bias
        y = F.gelu(torch.baddbmm(self.proj_bias, x.reshape(S, B * N, D), self.proj_weight.transpose(1, 2))).view(S, B, N, D)
        return (torch.softmax(self.scale_weights, 0).view(S, 1, 1, 1).to(y.dtype) * y).sum(0)


class YvSigLIPCrossModalAttention(nn.Module):
    """Vision tokens attend to text tokens (residual on the vision stream); ``text_mask`` [B, Tt] marks the real text."""

    def __init__(self, hidden_size: int, num_heads: int):
        super().__init__()
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, hidden_size // num_heads
        self.vision_norm, self.text_norm = nn.LayerNorm(hidden_size), nn.LayerNorm(hidden_size)
        self.q, self.kv, self.o = nn.Linear(hidden_size, hidden_size), nn.Linear(hidden_size, 2 * hidden_size), nn.Linear(hidden_size, hidden_size)

    def forward(self, vision_features: torch.Tensor, text_features: torch.Tensor, text_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, Tv, D = vision_features.shape
        Tt = text_features.shape[1]
        q = self.q(self.vision_norm(vision_features)).view(B, Tv, self.num_heads, self.head_dim).transpose(1, 2)
        k, v = self.kv(self.text_norm(text_features)).view(B, Tt, 2, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        m = text_mask.bool().view(B, 1, 1, Tt) if text_mask is not None else None
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=m)
        return vision_features + self.o(a.transpose(1, 2).reshape(B, Tv, D))


class YvSigLIPTower(nn.Module):
    """Patch embedding -> layers -> multi-scale mix -> GRN -> attention pooling -> normalised embedding; ``forward`` returns
    (embedding [B, E], tokens [B, N, D])."""

    def __init__(self, image_size: int = 224, patch_size: int = 16, hidden_size: int = 768, num_layers: int = 12, num_heads: int = 12,
                 embed_dim: int = 512, layer_scale: float = 1.0):
        super().__init__()
        if image_size % patch_size:
            raise ValueError("image_size must be a multiple of patch_size")
        self.patch = nn.Conv2d(3, hidden_size, patch_size, patch_size)
        self.pos = nn.Parameter(torch.zeros(1, (image_size // patch_size) ** 2, hidden_size))
        nn.init.trunc_normal_(self.pos, std=0.02)
        self.layers = nn.ModuleList([YvSigLIPTransformerLayer(hidden_size, num_heads, layer_scale=layer_scale) for _ in range(num_layers)])
        self.multi_scale = YvSigLIPMultiScaleFeatureExtractor(hidden_size, num_layers)
        self.grn, self.norm = YvSigLIPGRN(hidden_size), nn.LayerNorm(hidden_size)
        self.probe = nn.Parameter(torch.randn(1, 1, hidden_size) * 0.02)
        self.pool = nn.MultiheadAttention(hidden_size, num_heads, batch_first=True)
        self.proj = nn.Linear(hidden_size, embed_dim, bias=False)
        self.logit_scale, self.logit_bias = nn.Parameter(torch.tensor(math.log(10.0))), nn.Parameter(torch.tensor(-10.0))

    def forward(self, images: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        x = self.patch(images).flatten(2).transpose(1, 2) + self.pos
        hs: List[torch.Tensor] = []
        for layer in self.layers:
            x = layer(x)
            hs.append(x)
        t = self.norm(self.grn(self.multi_scale(hs)))
        pooled = self.pool(self.probe.expand(t.shape[0], -1, -1), t, t, need_weights=False)[0][:, 0]
        return F.normalize(self.proj(pooled).float(), dim=-1), t

    def sigmoid_loss(self, img_emb: torch.Tensor, txt_emb: torch.Tensor) -> torch.Tensor:
        logits = img_emb @ txt_emb.t() * self.logit_scale.exp() + self.logit_bias
        labels = 2 * torch.eye(logits.shape[0], device=logits.device) - 1
        return -F.logsigmoid(labels * logits).sum() / logits.shape[0]
