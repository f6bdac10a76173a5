"""Processors around a vision encoder (reference model/multimodal/vision.py:306-360, :2038-2300):

  * ``YvVisualTextProcessor``          rendered-text images (dark glyphs on a light page) -> compressed patch tokens;
  * ``YvHighResolutionProcessor``      up-scale, cut into overlapping tiles, encode, fuse a global and a local view;
  * ``YvVideoUnderstandingProcessor``  per-frame features -> key frames by motion + learned score -> temporal attention.

``encoder`` is any callable ``images [N, 3, H, W] -> patch features [N, P, D]`` (``YvVisionEncoder(...)(x, pool=False)``
fits).  The tiles of all images go through the encoder as ONE batch and the frames of all clips as ONE batch; the
reference encodes tile by tile in a Python loop (vision.py:2093-2096).  Key frames are picked with a batched gather;
the reference loops over frames for the differences and over the batch for the gather (vision.py:2163-2175)."""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..compat import YvFlashAttention

Encoder = Callable[[torch.Tensor], torch.Tensor]


class YvVisualTextProcessor(nn.Module):
    """Normalises with statistics of text pages (mean 0.95, std 0.1: mostly white), clamps the dark glyph pixels to
    +-5 sigma, embeds ``patch_size`` patches and passes them through a bottleneck MLP + LayerNorm."""

    def __init__(self, hidden_size: int, patch_size: int = 14):
        super().__init__()
        self.hidden_size, self.patch_size = hidden_size, patch_size
        self.register_buffer("text_mean", torch.full((1, 3, 1, 1), 0.95))
        self.register_buffer("text_std", torch.full((1, 3, 1, 1), 0.1))
        self.text_patch_embed = nn.Conv2d(3, hidden_size, patch_size, patch_size)
        self.text_compressor = nn.Sequential(nn.Linear(hidden_size, max(hidden_size // 2, 1)), nn.GELU(),
                                             nn.Linear(max(hidden_size // 2, 1), hidden_size), nn.LayerNorm(hidden_size))

    def forward(self, text_images: torch.Tensor) -> torch.Tensor:
        """[B, 3, H, W] in [0, 1] -> [B, (H // p) * (W // p), hidden]."""
        x = ((text_images - self.text_mean.to(text_images.dtype)) / self.text_std.to(text_images.dtype)).clamp(-5.0, 5.0)
        return self.text_compressor(self.text_patch_embed(x).flatten(2).transpose(1, 2))


class YvHighResolutionProcessor(nn.Module):
    """Image -> 2x bicubic up-scale -> overlapping ``tile_size`` tiles (stride = tile x (1 - overlap); one resized tile
    when the image is smaller than a tile) -> encoder on all tiles at once -> + tile position embedding ->
    global view (mean over tiles and patches) and local view (per-tile mean through an MLP) -> fused vector."""

    def __init__(self, hidden_size: int, patch_size: int, tile_size: int = 512, overlap: float = 0.25, max_tiles: int = 49):
        super().__init__()
        assert 0.0 <= overlap < 1.0
        self.hidden_size, self.patch_size, self.tile_size, self.overlap, self.max_tiles = hidden_size, patch_size, tile_size, overlap, max_tiles
        self.tile_pos_embed = nn.Parameter(torch.randn(1, max_tiles, hidden_size) * 0.02)
        self.local_enhance = nn.Sequential(nn.Linear(hidden_size, hidden_size), nn.GELU(), nn.Linear(hidden_size, hidden_size))
        self.aggregate = nn.Sequential(nn.Linear(2 * hidden_size, hidden_size), nn.LayerNorm(hidden_size), nn.GELU(),
                                       nn.Linear(hidden_size, hidden_size))

    def _extract_tiles(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """[B, C, H, W] -> tiles [B, n, C, t, t] and their (row, column) origins [n, 2].  ``unfold`` cuts every tile
        in one call; at most ``max_tiles`` (evenly thinned) are kept."""
        B, C, H, W = x.shape
        t = self.tile_size
        if H < t or W < t:
            tile = F.interpolate(x.float(), size=(t, t), mode="bicubic", align_corners=False).to(x.dtype)
            return tile.unsqueeze(1), torch.zeros(1, 2, dtype=torch.long, device=x.device)
        stride = max(1, int(t * (1.0 - self.overlap)))
        tiles = x.unfold(2, t, stride).unfold(3, t, stride)                         # [B, C, ny, nx, t, t]
        ny, nx = tiles.shape[2], tiles.shape[3]
        tiles = tiles.permute(0, 2, 3, 1, 4, 5).reshape(B, ny * nx, C, t, t)
        ys, xs = torch.meshgrid(torch.arange(ny, device=x.device) * stride, torch.arange(nx, device=x.device) * stride, indexing="ij")
        origins = torch.stack([ys.flatten(), xs.flatten()], -1)
        if ny * nx > self.max_tiles:
            keep = torch.linspace(0, ny * nx - 1, self.max_tiles, device=x.device).round().long()
            tiles, origins = tiles[:, keep], origins[keep]
        return tiles.contiguous(), origins

    def forward(self, x: torch.Tensor, encoder: Encoder, text_features: Optional[torch.Tensor] = None) -> Dict[str, Any]:
        up = F.interpolate(x.float(), scale_factor=2.0, mode="bicubic", align_corners=False).to(x.dtype)
        tiles, origins = self._extract_tiles(up)
        B, n, C, t, _ = tiles.shape
        feats = encoder(tiles.reshape(B * n, C, t, t))                              # one batch for every tile
        feats = feats.reshape(B, n, feats.shape[-2], feats.shape[-1])
        feats = feats + self.tile_pos_embed[:, :n].to(feats.dtype).unsqueeze(2)
        global_vec = feats.mean(dim=(1, 2)).unsqueeze(1)                            # [B, 1, D]
        local_feat = self.local_enhance(feats.mean(2))                              # [B, n, D]
        fused = self.aggregate(torch.cat([global_vec, local_feat.mean(1, keepdim=True)], -1))
        return {"features": fused, "patch_features": local_feat, "tile_features": feats, "tile_origins": origins,
                "spatial_shape": (t // self.patch_size, t // self.patch_size)}


class YvVideoUnderstandingProcessor(nn.Module):
    """Frames -> encoder (all frames of all clips in one batch) -> per-frame vectors -> ``num_key_frames`` key frames
    (learned score + half the motion, motion = distance to the previous frame's vector; kept in temporal order) ->
    pooling MLP -> temporal self-attention + LayerNorm -> compressor -> one clip vector (cross-attended to text
    features when given)."""

    def __init__(self, hidden_size: int, num_heads: int, max_frames: int = 128, num_key_frames: int = 32):
        super().__init__()
        H = hidden_size
        self.hidden_size, self.num_heads, self.max_frames, self.num_key_frames = H, num_heads, max_frames, num_key_frames
        self.temporal_attn = YvFlashAttention(H, num_heads, causal=False)
        self.temporal_norm = nn.LayerNorm(H)
        self.motion_estimator = nn.Sequential(nn.Linear(H, 128), nn.GELU(), nn.Linear(128, 1))
        self.temporal_pool = nn.Sequential(nn.Linear(H, H), nn.GELU(), nn.Linear(H, H))
        self.frame_compressor = nn.Sequential(nn.Linear(H, max(H // 2, 1)), nn.GELU(), nn.Linear(max(H // 2, 1), H))
        self.text_query = nn.Linear(H, H, bias=False)

    def _extract_key_frames(self, frame_features: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """[B, T, D] -> (key frames [B, K, D], their frame indices [B, K], ascending)."""
        B, T, D = frame_features.shape
        if T <= self.num_key_frames:
            return frame_features, torch.arange(T, device=frame_features.device).expand(B, T)
        motion = F.pad((frame_features[:, 1:] - frame_features[:, :-1]).float().norm(dim=-1), (1, 0))
        scores = self.motion_estimator(frame_features).squeeze(-1).float() + 0.5 * motion
        idx = scores.topk(self.num_key_frames, 1).indices.sort(1).values
        return frame_features.gather(1, idx.unsqueeze(-1).expand(-1, -1, D)), idx

    def forward(self, x: torch.Tensor, encoder: Encoder, video_shape: Optional[Tuple[int, int, int]] = None,
                text_features: Optional[torch.Tensor] = None) -> Dict[str, Any]:
        """x [B, T, 3, H, W], or [B * T, 3, H, W] with ``video_shape = (T, H, W)``."""
        if x.dim() == 5:
            B, T, C, H, W = x.shape
            flat = x.reshape(B * T, C, H, W)
        else:
            T, H, W = video_shape
            B, flat = x.shape[0] // T, x
        patches = encoder(flat)                                                      # [B*T, P, D]
        frames = patches.reshape(B, T, patches.shape[-2], patches.shape[-1]).mean(2)
        keys, idx = self._extract_key_frames(frames)
        pooled = self.temporal_pool(keys) if keys.shape[1] > 1 else keys
        temporal = self.temporal_norm(pooled + self.temporal_attn(pooled))
        clip = self.frame_compressor(temporal).mean(1, keepdim=True)                 # [B, 1, D]
        if text_features is not None:
            a = torch.softmax((self.text_query(clip) @ text_features.transpose(1, 2)).float() / self.hidden_size ** 0.5, -1)
            clip = clip + a.to(text_features.dtype) @ text_features
        return {"features": clip, "temporal_features": temporal, "key_frame_indices": idx, "frame_features": frames}
