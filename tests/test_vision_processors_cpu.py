"""Visual-text, high-resolution and video-understanding processors around a patch encoder."""
import torch
from torch import nn

from pisceslx_b200.models.multimodal.vision_processors import (YvHighResolutionProcessor, YvVideoUnderstandingProcessor,
                                                               YvVisualTextProcessor)

D = 32


class PatchEncoder(nn.Module):
    """images [N, 3, H, W] -> [N, (H // 8) * (W // 8), D]; counts its calls."""

    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(3, D, 8, 8)
        self.calls = 0

    def forward(self, x):
        self.calls += 1
        return self.conv(x).flatten(2).transpose(1, 2)


def test_visual_text_tokens():
    torch.manual_seed(0)
    p = YvVisualTextProcessor(D, patch_size=7)
    page = torch.ones(2, 3, 28, 42) * 0.97
    page[:, :, 5:9, 5:30] = 0.05                                   # a line of dark glyphs
    out = p(page)
    assert tuple(out.shape) == (2, 4 * 6, D) and bool(torch.isfinite(out).all())
    assert not torch.allclose(out[0, 0], out[0, 7])                # glyph patches differ from blank ones


def test_high_resolution_tiles_in_one_encoder_call():
    torch.manual_seed(0)
    enc = PatchEncoder()
    p = YvHighResolutionProcessor(D, patch_size=8, tile_size=32, overlap=0.25)
    x = torch.rand(2, 3, 40, 40)                                   # up-scaled to 80: tiles at 0, 24, 48 in each axis
    tiles, origins = p._extract_tiles(torch.rand(2, 3, 80, 80))
    assert tuple(tiles.shape) == (2, 9, 3, 32, 32) and origins[:, 0].unique().tolist() == [0, 24, 48]
    up = torch.rand(1, 3, 80, 80)
    t, o = p._extract_tiles(up)
    assert torch.equal(t[0, 4], up[0, :, 24:56, 24:56])
    out = p(x, enc)
    assert enc.calls == 1
    assert tuple(out["features"].shape) == (2, 1, D) and tuple(out["patch_features"].shape) == (2, 9, D)
    assert tuple(out["tile_features"].shape) == (2, 9, 16, D) and out["spatial_shape"] == (4, 4)
    small = p(torch.rand(1, 3, 8, 8), enc)                         # smaller than a tile even after the up-scale
    assert tuple(small["tile_features"].shape) == (1, 1, 16, D)
    capped = YvHighResolutionProcessor(D, 8, tile_size=16, overlap=0.5, max_tiles=5)
    assert capped._extract_tiles(torch.rand(1, 3, 64, 64))[0].shape[1] == 5
    out["features"].sum().backward()
    assert p.tile_pos_embed.grad is not None


def test_video_key_frames_follow_motion_and_stay_ordered():
    torch.manual_seed(0)
    enc = PatchEncoder()
    v = YvVideoUnderstandingProcessor(D, 4, num_key_frames=4)
    with torch.no_grad():
        for m in v.motion_estimator:
            if isinstance(m, nn.Linear):
                m.weight.zero_()
                m.bias.zero_()                                      # scores = motion only
    frames = torch.zeros(1, 10, D)
    frames[0, 3:] += 5.0                                           # cuts at frames 3, 6, 8 (and a small one at 9)
    frames[0, 6:] += 5.0
    frames[0, 8:] += 5.0
    frames[0, 9:] += 1.0
    keys, idx = v._extract_key_frames(frames)
    assert idx.tolist() == [[3, 6, 8, 9]] and torch.equal(keys[0, 0], frames[0, 3])
    video = torch.rand(2, 6, 3, 16, 16)
    out = v(video, enc)
    assert enc.calls == 1
    assert tuple(out["features"].shape) == (2, 1, D) and tuple(out["temporal_features"].shape) == (2, 4, D)
    assert bool((out["key_frame_indices"][:, 1:] > out["key_frame_indices"][:, :-1]).all())
    flat = v(video.reshape(12, 3, 16, 16), enc, video_shape=(6, 16, 16))
    assert torch.allclose(flat["features"], out["features"], atol=1e-6)
    with_text = v(video, enc, text_features=torch.randn(2, 5, D))
    assert not torch.allclose(with_text["features"], out["features"])
    short = v(torch.rand(1, 3, 3, 16, 16), enc)                     # fewer frames than key frames: all are kept
    assert tuple(short["temporal_features"].shape) == (1, 3, D)
    with_text["features"].sum().backward()
    assert v.text_query.weight.grad is not None and enc.conv.weight.grad is not None
