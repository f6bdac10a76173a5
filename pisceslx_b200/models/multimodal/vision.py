"""Vision and video encoders.

``YvVisionEncoder``: ViT with a patch-embed GEMM (the reference uses ``Conv2d(3, hidden, 14, stride 14)``,
model/multimodal/vision.py:492-497), ImageNet mean/std normalisation, learned position embedding interpolated to
the image's patch grid (:824-849), pre-LN blocks with non-causal attention and a GELU MLP x4 (:932-982), a
projection to the language width.  Width / depth / heads are independent of the LM here (the reference ties them
to it, :483-485).  With ``native_resolution`` images of different sizes are *packed*: every image contributes its
own number of patches to one token stream and attention runs per image through the variable-length kernel.

``YvVideoEncoder`` (reference multimodal/video.py:84-351): frame patches -> ViT blocks whose attention uses the
3-D (t, h, w) rotary embedding (``YvSpatioTemporalRoPE3D``) -> pooled tokens.

On GPU the patch extraction is the ``patchify`` kernel (im2col-free: it writes rows that the tcgen05 GEMM
consumes), attention is the flash-attention kernel, projections are the tcgen05 GEMM.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...config import YvConfig
from ...ops import functional as F_
from ...ops import kernels, reference as ref
from ..norms import YvLayerNorm, YvSpatioTemporalRoPE3D

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)


class YvPatchEmbed(nn.Module):
    def __init__(self, patch: int, in_ch: int, dim: int):
        super().__init__()
        self.patch, self.in_ch, self.dim = patch, in_ch, dim
        k = in_ch * patch * patch
        self.k, self.k_pad = k, (k + 63) // 64 * 64
        self.weight = nn.Parameter(torch.empty(dim, self.k_pad))
        nn.init.normal_(self.weight, std=0.02)
        with torch.no_grad():
            self.weight[:, k:].zero_()
        self.bias = nn.Parameter(torch.zeros(dim))
        self.register_buffer("mean", torch.tensor(IMAGENET_MEAN[:in_ch] if in_ch <= 3 else [0.5] * in_ch))
        self.register_buffer("std", torch.tensor(IMAGENET_STD[:in_ch] if in_ch <= 3 else [0.5] * in_ch))

    def forward(self, img: torch.Tensor) -> torch.Tensor:
        """img [B, C, H, W] (H, W multiples of the patch) -> [B * gh * gw, dim]"""
        B, C, H, W = img.shape
        if img.is_cuda:
            rows = torch.empty(B * (H // self.patch) * (W // self.patch), self.k_pad, dtype=torch.bfloat16,
                               device=img.device)
            src = img.contiguous() if img.dtype in (torch.float32, torch.bfloat16) else img.float().contiguous()
            kernels().patchify(src, rows, self.patch, self.mean.float(), self.std.float())
        else:
            rows = ref.patchify(img, self.patch, self.mean, self.std, self.k_pad).to(self.weight.dtype)
        return F_.linear(rows, self.weight, self.bias)

    def conv_weight(self) -> torch.Tensor:
        """The equivalent Conv2d weight [dim, C, P, P] (checkpoint interchange with the reference layout)."""
        return self.weight[:, : self.k].reshape(self.dim, self.in_ch, self.patch, self.patch)


class YvViTBlock(nn.Module):
    def __init__(self, dim: int, heads: int, mlp_ratio: float = 4.0, rope3d: Optional[YvSpatioTemporalRoPE3D] = None):
        super().__init__()
        self.dim, self.heads, self.hd = dim, heads, dim // heads
        self.norm1, self.norm2 = YvLayerNorm(dim), YvLayerNorm(dim)
        self.qkv = nn.Parameter(torch.empty(3 * dim, dim).normal_(std=0.02))
        self.qkv_bias = nn.Parameter(torch.zeros(3 * dim))
        self.proj = nn.Parameter(torch.empty(dim, dim).normal_(std=0.02))
        self.proj_bias = nn.Parameter(torch.zeros(dim))
        hid = int(dim * mlp_ratio)
        self.fc1 = nn.Parameter(torch.empty(hid, dim).normal_(std=0.02))
        self.fc1_bias = nn.Parameter(torch.zeros(hid))
        self.fc2 = nn.Parameter(torch.empty(dim, hid).normal_(std=0.02))
        self.fc2_bias = nn.Parameter(torch.zeros(dim))
        self.rope3d = rope3d

    def forward(self, x: torch.Tensor, cu: torch.Tensor, max_len: int,
                pos_thw: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [T, dim] packed tokens of several images / clips; cu int32 [n+1] their offsets."""
        T = x.shape[0]
        qkv = F_.linear(self.norm1(x), self.qkv, self.qkv_bias)
        d = self.dim
        if self.rope3d is not None and pos_thw is not None:
            q, k = self.rope3d(qkv[:, :d].reshape(T, self.heads, self.hd), qkv[:, d:2 * d].reshape(T, self.heads, self.hd),
                               pos_thw)
            q, k = q.reshape(T, d), k.reshape(T, d)
        else:
            q, k = qkv[:, :d], qkv[:, d:2 * d]
        o = F_.attention(q, k, qkv[:, 2 * d:], cu, cu, max_len, max_len, self.heads, self.heads, self.hd, causal=False)
        x = x + F_.linear(o, self.proj, self.proj_bias)
        h = F.gelu(F_.linear(self.norm2(x), self.fc1, self.fc1_bias))
        return x + F_.linear(h, self.fc2, self.fc2_bias)


class YvVisionEncoder(nn.Module):
    def __init__(self, cfg: YvConfig, dim: Optional[int] = None, depth: Optional[int] = None,
                 heads: Optional[int] = None, base_grid: int = 16):
        super().__init__()
        self.cfg = cfg
        self.dim = dim or cfg.vision_hidden_size or cfg.hidden_size
        self.depth = depth or cfg.vision_n_layer or cfg.n_layer
        self.heads = heads or cfg.vision_n_head or cfg.n_head
        self.patch = cfg.image_patch
        self.patch_embed = YvPatchEmbed(self.patch, 3, self.dim)
        self.base_grid = base_grid
        self.pos_embed = nn.Parameter(torch.zeros(1, self.dim, base_grid, base_grid).normal_(std=0.02))
        self.cls_token = nn.Parameter(torch.zeros(1, self.dim).normal_(std=0.02))
        self.blocks = nn.ModuleList([YvViTBlock(self.dim, self.heads) for _ in range(self.depth)])
        self.norm = YvLayerNorm(self.dim)
        self.proj = nn.Parameter(torch.empty(cfg.hidden_size, self.dim).normal_(std=0.02))

    def _pos(self, gh: int, gw: int, dtype: torch.dtype) -> torch.Tensor:
        p = self.pos_embed.float()
        if (gh, gw) != (self.base_grid, self.base_grid):
            p = F.interpolate(p, size=(gh, gw), mode="bicubic", align_corners=False)
        return p.flatten(2).transpose(1, 2).squeeze(0).to(dtype)        # [gh*gw, dim]

    def encode_packed(self, images: Sequence[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        """images: list of [C, H, W] tensors of possibly different sizes (native resolution).  Returns
        (tokens [T, hidden_lm], cu_seqlens) with one CLS + gh*gw patch tokens per image."""
        toks: List[torch.Tensor] = []
        lens: List[int] = []
        for img in images:
            C, H, W = img.shape
            Hc, Wc = H // self.patch * self.patch, W // self.patch * self.patch
            x = self.patch_embed(img[:, :Hc, :Wc].unsqueeze(0))
            x = x + self._pos(Hc // self.patch, Wc // self.patch, x.dtype)
            toks += [self.cls_token.to(x.dtype), x]
            lens.append(1 + x.shape[0])
        x = torch.cat(toks, 0)
        dev = x.device
        cu = torch.zeros(len(lens) + 1, dtype=torch.int32, device=dev)
        cu[1:] = torch.tensor(lens, dtype=torch.int32, device=dev).cumsum(0)
        mx = max(lens)
        for blk in self.blocks:
            x = blk(x, cu, mx)
        return F_.linear(self.norm(x), self.proj), cu

    def forward(self, images: torch.Tensor, pool: bool = True) -> torch.Tensor:
        """images [B, C, H, W] -> pooled features [B, 1, hidden_lm] (reference vision.py:1005-1013) or all patch
        tokens [B, 1 + gh*gw, hidden_lm] when ``pool`` is False."""
        B, C, H, W = images.shape
        gh, gw = H // self.patch, W // self.patch
        x = self.patch_embed(images[:, :, : gh * self.patch, : gw * self.patch])
        x = x.view(B, gh * gw, self.dim) + self._pos(gh, gw, x.dtype).unsqueeze(0)
        x = torch.cat([self.cls_token.to(x.dtype).expand(B, 1, self.dim), x], 1)
        L = x.shape[1]
        cu = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=x.device)
        x = x.reshape(B * L, self.dim)
        for blk in self.blocks:
            x = blk(x, cu, L)
        x = F_.linear(self.norm(x), self.proj).view(B, L, -1)
        return x.mean(1, keepdim=True) if pool else x


class YvVideoEncoder(nn.Module):
    def __init__(self, cfg: YvConfig, dim: Optional[int] = None, depth: int = 4, heads: Optional[int] = None,
                 out_tokens: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        self.dim = dim or cfg.vision_hidden_size or cfg.hidden_size
        self.heads = heads or cfg.vision_n_head or cfg.n_head
        self.patch = cfg.image_patch
        self.patch_embed = YvPatchEmbed(self.patch, 3, self.dim)
        rope = YvSpatioTemporalRoPE3D(self.dim // self.heads)
        self.blocks = nn.ModuleList([YvViTBlock(self.dim, self.heads, rope3d=rope) for _ in range(depth)])
        self.norm = YvLayerNorm(self.dim)
        self.proj = nn.Parameter(torch.empty(cfg.hidden_size, self.dim).normal_(std=0.02))
        self.out_tokens = out_tokens or cfg.video_tokens

    def forward(self, video: torch.Tensor) -> torch.Tensor:
        """video [B, T, C, H, W] -> [B, out_tokens, hidden_lm] (tokens average-pooled along the sequence)."""
        B, T, C, H, W = video.shape
        gh, gw = H // self.patch, W // self.patch
        x = self.patch_embed(video.reshape(B * T, C, H, W)[:, :, : gh * self.patch, : gw * self.patch])
        L = T * gh * gw
        pos = YvSpatioTemporalRoPE3D.grid_positions(T, gh, gw, x.device).repeat(B, 1)
        cu = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=x.device)
        for blk in self.blocks:
            x = blk(x, cu, L, pos)
        x = F_.linear(self.norm(x), self.proj).view(B, L, -1)
        n = min(self.out_tokens, L)
        return F.adaptive_avg_pool1d(x.float().transpose(1, 2), n).transpose(1, 2).to(x.dtype)
