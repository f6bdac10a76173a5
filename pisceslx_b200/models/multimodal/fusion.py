"""Audio encoder, cross-modal attention and modal fusion.

``YvAudioEncoder``       log-mel front end (STFT n_fft 1024 / hop 512 / 128 mels at 16 kHz as in the reference's
                         config fields) -> 2x strided Conv1d subsampling -> transformer blocks -> audio tokens
                         (reference multimodal/audio.py).
``YvCrossModalAttention`` LN(q), LN(kv) -> multi-head attention of text queries over modal keys -> o_proj
                         (reference multimodal/attention.py:79-239); on GPU the packed flash-attention kernel with
                         separate query / key lengths.
``YvDynamicModalFusion`` gathers the tokens of all present modalities, refines them with self-attention blocks and
                         reads them out through learned queries into ``native_fusion_output_tokens`` fusion tokens
                         [B, n, H] that the trunk prepends to the text embeddings (reference multimodal/fusion.py:348-858,
                         model/core/model.py:2139-2144).
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...config import YvConfig
from ...ops import functional as F_
from ..norms import YvLayerNorm
from .vision import YvViTBlock, YvVideoEncoder, YvVisionEncoder


def mel_filterbank(n_mels: int, n_fft: int, sr: int) -> torch.Tensor:
    def hz2mel(f):
        return 2595.0 * math.log10(1.0 + f / 700.0)

    def mel2hz(m):
        return 700.0 * (10 ** (m / 2595.0) - 1.0)

    pts = torch.linspace(hz2mel(0.0), hz2mel(sr / 2), n_mels + 2).apply_(mel2hz)
    bins = torch.floor((n_fft + 1) * pts / sr).long()
    fb = torch.zeros(n_mels, n_fft // 2 + 1)
    for m in range(1, n_mels + 1):
        l, c, r = int(bins[m - 1]), int(bins[m]), int(bins[m + 1])
        for k in range(l, c):
            fb[m - 1, k] = (k - l) / max(c - l, 1)
        for k in range(c, r):
            fb[m - 1, k] = (r - k) / max(r - c, 1)
    return fb


class YvAudioEncoder(nn.Module):
    def __init__(self, cfg: YvConfig, dim: int = 512, depth: int = 4, heads: int = 8):
        super().__init__()
        self.cfg, self.dim = cfg, dim
        self.n_fft, self.hop, self.n_mels = cfg.audio_n_fft, cfg.audio_hop_length, cfg.audio_n_mels
        self.register_buffer("fb", mel_filterbank(self.n_mels, self.n_fft, cfg.audio_sampling_rate), persistent=False)
        self.register_buffer("window", torch.hann_window(self.n_fft), persistent=False)
        self.conv1 = nn.Conv1d(self.n_mels, dim, 3, padding=1)
        self.conv2 = nn.Conv1d(dim, dim, 3, stride=2, padding=1)
        self.blocks = nn.ModuleList([YvViTBlock(dim, heads) for _ in range(depth)])
        self.norm = YvLayerNorm(dim)
        self.proj = nn.Parameter(torch.empty(cfg.hidden_size, dim).normal_(std=0.02))
        self.max_tokens = cfg.audio_tokens

    def log_mel(self, wav: torch.Tensor) -> torch.Tensor:
        """wav [B, samples] -> [B, n_mels, frames]"""
        spec = torch.stft(wav.float(), self.n_fft, self.hop, window=self.window.float().to(wav.device),
                          return_complex=True).abs().pow(2)
        mel = self.fb.float().to(wav.device) @ spec
        return torch.log(mel.clamp_min(1e-10))

    def forward(self, audio: torch.Tensor) -> torch.Tensor:
        """audio [B, samples] waveform or [B, n_mels, frames] features -> [B, tokens, hidden_lm]"""
        mel = self.log_mel(audio) if audio.dim() == 2 else audio.float()
        dt = self.conv1.weight.dtype
        x = F.gelu(self.conv2(F.gelu(self.conv1(mel.to(dt)))))             # [B, dim, frames/2]
        x = x.transpose(1, 2)
        B, L, _ = x.shape
        pos = torch.arange(L, device=x.device, dtype=torch.float32).unsqueeze(1)
        div = torch.exp(torch.arange(0, self.dim, 2, device=x.device, dtype=torch.float32) * (-math.log(1e4) / self.dim))
        pe = torch.zeros(L, self.dim, device=x.device)
        pe[:, 0::2], pe[:, 1::2] = torch.sin(pos * div), torch.cos(pos * div)
        x = (x + pe.to(x.dtype)).reshape(B * L, self.dim)
        cu = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=x.device)
        for blk in self.blocks:
            x = blk(x, cu, L)
        x = F_.linear(self.norm(x), self.proj).view(B, L, -1)
        if L > self.max_tokens:
            x = F.adaptive_avg_pool1d(x.float().transpose(1, 2), self.max_tokens).transpose(1, 2).to(x.dtype)
        return x


class YvCrossModalAttention(nn.Module):
    def __init__(self, hidden: int, heads: int, dropout: float = 0.0):
        super().__init__()
        self.hidden, self.heads, self.hd = hidden, heads, hidden // heads
        self.norm_q, self.norm_kv = YvLayerNorm(hidden), YvLayerNorm(hidden)
        self.q_proj = nn.Parameter(torch.empty(hidden, hidden).normal_(std=0.02))
        self.kv_proj = nn.Parameter(torch.empty(2 * hidden, hidden).normal_(std=0.02))
        self.o_proj = nn.Parameter(torch.empty(hidden, hidden).normal_(std=0.02))

    def forward(self, query: torch.Tensor, context: torch.Tensor) -> torch.Tensor:
        """query [B, Sq, H], context [B, Sk, H] -> [B, Sq, H] (residual added by the caller)."""
        B, Sq, H = query.shape
        Sk = context.shape[1]
        q = F_.linear(self.norm_q(query).reshape(B * Sq, H), self.q_proj)
        kv = F_.linear(self.norm_kv(context).reshape(B * Sk, H), self.kv_proj)
        dev = query.device
        cq = torch.arange(0, (B + 1) * Sq, Sq, dtype=torch.int32, device=dev)
        ck = torch.arange(0, (B + 1) * Sk, Sk, dtype=torch.int32, device=dev)
        o = F_.attention(q, kv[:, :H], kv[:, H:], cq, ck, Sq, Sk, self.heads, self.heads, self.hd, causal=False)
        return F_.linear(o, self.o_proj).view(B, Sq, H)


class YvDynamicModalFusion(nn.Module):
    def __init__(self, cfg: YvConfig, heads: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        H = cfg.hidden_size
        heads = heads or max(1, H // 128 if H % 128 == 0 else H // 64)
        self.n_out = cfg.native_fusion_output_tokens
        self.modal_embed = nn.Parameter(torch.zeros(4, H).normal_(std=0.02))       # image, video, audio, other
        self.blocks = nn.ModuleList([YvViTBlock(H, heads) for _ in range(cfg.native_fusion_num_layers)])
        self.queries = nn.Parameter(torch.zeros(self.n_out, H).normal_(std=0.02))
        self.readout = YvCrossModalAttention(H, heads)
        self.norm = YvLayerNorm(H)

    def forward(self, modal_tokens: Dict[str, torch.Tensor]) -> torch.Tensor:
        """modal_tokens: name -> [B, n_i, H].  Returns fusion tokens [B, n_out, H]."""
        order = {"image": 0, "video": 1, "audio": 2}
        parts = []
        for name, t in modal_tokens.items():
            parts.append(t + self.modal_embed[order.get(name, 3)].to(t.dtype))
        x = torch.cat(parts, 1)
        B, L, H = x.shape
        cu = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=x.device)
        flat = x.reshape(B * L, H)
        for blk in self.blocks:
            flat = blk(flat, cu, L)
        x = flat.view(B, L, H)
        q = self.queries.to(x.dtype).unsqueeze(0).expand(B, self.n_out, H)
        return self.norm(q + self.readout(q, x))

    def encode_modalities(self, trunk: Any, images: Optional[torch.Tensor] = None, video: Optional[torch.Tensor] = None,
                          audio: Optional[torch.Tensor] = None, **_: Any) -> Optional[torch.Tensor]:
        """Run the trunk's encoders on whatever modalities are present and fuse them into prefix tokens."""
        toks: Dict[str, torch.Tensor] = {}
        if images is not None and trunk.vision_encoder is not None:
            if images.dim() == 5:                                        # [B, n_img, C, H, W]
                B, n = images.shape[:2]
                f = trunk.vision_encoder(images.flatten(0, 1), pool=False)
                toks["image"] = f.reshape(B, n * f.shape[1], f.shape[2])
            else:
                toks["image"] = trunk.vision_encoder(images, pool=False)
        if video is not None and trunk.video_encoder is not None:
            toks["video"] = trunk.video_encoder(video)
        if audio is not None and trunk.audio_encoder is not None:
            toks["audio"] = trunk.audio_encoder(audio)
        if not toks:
            return None
        return self.forward(toks)


def attach_multimodal(model: Any, vision: bool = True, video: bool = False, audio: bool = False) -> None:
    """Materialise the multimodal components on a ``YvModelForCausalLM`` (lazy like the reference's
    ``LAZY_COMPONENTS``, model/core/model.py:1458-1478)."""
    trunk = model.model
    cfg = model.cfg
    p = next(model.parameters())
    kw = dict(device=p.device, dtype=p.dtype)
    if vision and trunk.vision_encoder is None:
        trunk.attach("vision_encoder", YvVisionEncoder(cfg).to(**kw))
    if video and trunk.video_encoder is None:
        trunk.attach("video_encoder", YvVideoEncoder(cfg).to(**kw))
    if audio and trunk.audio_encoder is None:
        trunk.attach("audio_encoder", YvAudioEncoder(cfg).to(**kw))
    if trunk.modal_fusion is None:
        trunk.attach("modal_fusion", YvDynamicModalFusion(cfg).to(**kw))
