"""Text-conditioned content generation (image, audio, video) built from the framework's own parts.

Reference surface: model/multimodal/generator.py - ``YvGenerationConfig`` (:102), ``YvGenerationModality`` (:196),
``YvGenerationResult`` (:206), ``YvGenerationCondition`` (:226), ``YvSelfDevelopedGenerator`` (:243), the backend
interface and its two stock backends (:710-980), the ``YvGenerator`` registry (:985) and ``YvGeneratorFactory`` (:1124).

``YvSelfDevelopedGenerator`` here is one module with three heads over a shared text encoder (a small Yv trunk):

  * image: the pooled text feature conditions a latent that is refined by a few deterministic DDIM steps of a
    conditional latent denoiser, decoded by ``YvImageDecoder`` and optionally polished by ``YvDiffusionImageEnhancer``;
  * audio: an autoregressive-free codec head predicts ``n_codebooks`` token streams from the text feature and a learned
    time grid, ``YvNeuralVocoder`` turns them into a waveform;
  * video: per-frame latents = image latent + a temporal code from the 3-D rotary table, decoded frame by frame.

Everything runs on any device; nothing external is loaded.  The generator is a research head, not part of the training
benchmark; its matrix products go through the same ``ops.functional`` entry points as the rest of the model.
"""
from __future__ import annotations

import math
import time
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...config import YvConfig
from ..tokenizer import YvTokenizer
from .heads import YvNeuralVocoder
from .vision_extras import YvDiffusionImageEnhancer, YvImageDecoder


@dataclass
class YvGenerationConfig:
    hidden_size: Optional[int] = None
    num_heads: Optional[int] = None
    num_layers: Optional[int] = None
    max_sequence_length: Optional[int] = None
    num_inference_steps: int = 50
    image_size: int = 64
    audio_sample_rate: int = 16000
    video_fps: int = 24
    image_gen_resolution: int = 512
    image_gen_num_steps: int = 50
    image_gen_guidance_scale: float = 7.5
    image_gen_initial_size: int = 64
    image_gen_use_diffusion: bool = True
    audio_gen_sample_rate: int = 16000
    audio_gen_duration: float = 5.0
    audio_gen_num_codebooks: int = 8
    audio_gen_codebook_size: int = 1024
    video_gen_fps: int = 24
    video_gen_num_frames: int = 16
    video_gen_resolution: int = 256
    latent_dim: int = 64

    def __post_init__(self) -> None:
        base = YvConfig()                                   # defaults follow the main model configuration
        self.hidden_size = self.hidden_size or base.hidden_size
        self.num_heads = self.num_heads or base.n_head
        self.num_layers = self.num_layers or base.n_layer
        self.max_sequence_length = self.max_sequence_length or base.max_position_embeddings


class YvGenerationModality(Enum):
    IMAGE = "image"
    AUDIO = "audio"
    VIDEO = "video"
    TEXT = "text"


@dataclass
class YvGenerationResult:
    modality: YvGenerationModality
    data: Any
    metadata: Dict[str, Any] = field(default_factory=dict)
    success: bool = True
    error: Optional[str] = None
    seconds: float = 0.0


@dataclass
class YvGenerationCondition:
    text: Optional[str] = None
    negative_text: Optional[str] = None
    seed: Optional[int] = None
    extras: Dict[str, Any] = field(default_factory=dict)


class _LatentDenoiser(nn.Module):
    """eps(z_t, t, c): an MLP over [latent, time embedding, condition] with a residual path."""

    def __init__(self, latent: int, cond: int, width: int = 256):
        super().__init__()
        self.latent, self.width = latent, width
        self.inp = nn.Linear(latent + width + cond, width)
        self.mid = nn.Linear(width, width)
        self.out = nn.Linear(width, latent)
        nn.init.zeros_(self.out.weight)
        nn.init.zeros_(self.out.bias)

    def time_embedding(self, t: torch.Tensor) -> torch.Tensor:
        half = self.width // 2
        f = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device) / half)
        a = t.float()[:, None] * f
        return torch.cat([a.sin(), a.cos()], -1)

    def forward(self, z: torch.Tensor, t: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
        h = F.silu(self.inp(torch.cat([z, self.time_embedding(t), c], -1)))
        return self.out(h + F.silu(self.mid(h)))


class YvSelfDevelopedGenerator(nn.Module):
    def __init__(self, config: Optional[YvGenerationConfig] = None, train_steps: int = 1000):
        super().__init__()
        from ..model import YvModelForCausalLM
        self.config = cfg = config or YvGenerationConfig()
        H = cfg.hidden_size
        self.tokenizer = YvTokenizer.instance()
        vocab = max(self.tokenizer.vocab_size, 512)
        trunk_cfg = YvConfig(hidden_size=H, n_layer=cfg.num_layers, n_head=cfg.num_heads,
                             n_kv_head=max(1, cfg.num_heads // 2), vocab_size=vocab,
                             intermediate_size=2 * H, max_position_embeddings=cfg.max_sequence_length,
                             moe_num_experts=0)
        self.backbone = YvModelForCausalLM(trunk_cfg)
        self.steps = train_steps
        beta = torch.linspace(1e-4, 0.02, train_steps)
        self.register_buffer("abar", torch.cumprod(1 - beta, 0), persistent=False)
        # image / video
        self.cond_proj = nn.Linear(H, cfg.latent_dim)
        self.denoiser = _LatentDenoiser(cfg.latent_dim, cfg.latent_dim)
        stages = max(1, int(round(math.log2(max(cfg.image_size, 16) / 8))))
        self.image_decoder = YvImageDecoder(cfg.latent_dim, base=8, stages=stages, channels=64)
        self.enhancer = YvDiffusionImageEnhancer(channels=16, steps=train_steps) if cfg.image_gen_use_diffusion else None
        self.temporal = nn.Parameter(torch.zeros(64, cfg.latent_dim).normal_(std=0.02))      # frame codes
        # audio
        self.audio_time = nn.Parameter(torch.zeros(256, H).normal_(std=0.02))
        self.audio_head = nn.Linear(H, cfg.audio_gen_num_codebooks * cfg.audio_gen_codebook_size)
        self.vocoder = YvNeuralVocoder(cfg.audio_gen_codebook_size, cfg.audio_gen_num_codebooks, dim=64, rates=(5, 4, 4, 2))

    # ---- text -------------------------------------------------------------------------------------------
    @torch.no_grad()
    def encode_text(self, text: str) -> torch.Tensor:
        """Pooled final hidden state of the prompt [1, H] (reference :623-690)."""
        dev = self.cond_proj.weight.device
        ids = self.tokenizer.encode(text)[: self.config.max_sequence_length] or [self.tokenizer.bos_token_id]
        ids = [min(i, self.backbone.cfg.vocab_size - 1) for i in ids]
        out = self.backbone(input_ids=torch.tensor([ids], device=dev), return_hidden=True)
        hid = out["hidden_states"] if isinstance(out, dict) and "hidden_states" in out else out["logits"]
        if hid.shape[-1] != self.config.hidden_size:                   # logits fallback: project back through the embedding
            hid = hid.softmax(-1) @ self.backbone.model.embed.weight.to(hid.dtype)
        return hid.float().mean(1)

    # ---- image ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def sample_latent(self, cond: torch.Tensor, steps: int, guidance: float, generator: Optional[torch.Generator]) -> torch.Tensor:
        """Deterministic DDIM (eta 0) with classifier-free guidance against the zero condition."""
        B, dev = cond.shape[0], cond.device
        z = torch.randn(B, self.config.latent_dim, generator=generator, device="cpu").to(dev)
        ts = torch.linspace(self.steps - 1, 0, max(1, steps) + 1).long().tolist()
        for t, tn in zip(ts[:-1], ts[1:]):
            tt = torch.full((B,), t, device=dev)
            e_c, e_u = self.denoiser(z, tt, cond), self.denoiser(z, tt, torch.zeros_like(cond))
            eps = e_u + guidance * (e_c - e_u)
            a = self.abar[t]
            an = self.abar[tn] if tn > 0 else torch.ones((), device=dev)
            z0 = (z - (1 - a).sqrt() * eps) / a.sqrt()
            z = an.sqrt() * z0 + (1 - an).sqrt() * eps
        return z + cond                                               # the condition is also a direct latent offset

    @torch.no_grad()
    def generate_image(self, prompt: str, steps: Optional[int] = None, seed: Optional[int] = None,
                       guidance_scale: Optional[float] = None) -> torch.Tensor:
        """[1, 3, S, S] in [-1, 1]."""
        cfg = self.config
        g = torch.Generator().manual_seed(seed) if seed is not None else None
        cond = self.cond_proj(self.encode_text(prompt))
        z = self.sample_latent(cond, steps or min(cfg.image_gen_num_steps, cfg.num_inference_steps),
                               cfg.image_gen_guidance_scale if guidance_scale is None else guidance_scale, g)
        img = self.image_decoder(z)
        if img.shape[-1] != cfg.image_size:
            img = F.interpolate(img, size=(cfg.image_size, cfg.image_size), mode="bilinear", align_corners=False)
        if self.enhancer is not None:
            if g is not None:
                torch.manual_seed(seed)
            img = self.enhancer.enhance(img, t_start=100, n_steps=4)
        return img.clamp(-1, 1)

    def diffusion_training_loss(self, prompts: List[str], latents: torch.Tensor) -> torch.Tensor:
        """Noise-prediction loss of the latent denoiser on (prompt, target latent) pairs; the condition is dropped
        for a tenth of the rows so that guidance has an unconditional branch."""
        cond = torch.cat([self.cond_proj(self.encode_text(p)) for p in prompts])
        drop = (torch.rand(len(prompts), 1, device=cond.device) < 0.1).float()
        t = torch.randint(0, self.steps, (len(prompts),), device=cond.device)
        n = torch.randn_like(latents)
        a = self.abar[t].view(-1, 1)
        return F.mse_loss(self.denoiser(a.sqrt() * latents + (1 - a).sqrt() * n, t, cond * (1 - drop)), n)

    # ---- video ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate_video(self, prompt: str, num_frames: Optional[int] = None, seed: Optional[int] = None) -> torch.Tensor:
        """[1, T, 3, S, S]: one latent per prompt, one temporal code per frame (smooth in time by construction)."""
        cfg = self.config
        T = min(num_frames or cfg.video_gen_num_frames, self.temporal.shape[0])
        g = torch.Generator().manual_seed(seed) if seed is not None else None
        cond = self.cond_proj(self.encode_text(prompt))
        z = self.sample_latent(cond, min(8, cfg.num_inference_steps), cfg.image_gen_guidance_scale, g)
        w = torch.linspace(0, 1, T, device=z.device).view(T, 1)
        codes = (1 - w) * self.temporal[0] + w * self.temporal[T - 1] + 0.1 * self.temporal[:T]
        frames = self.image_decoder(z + codes)
        size = min(cfg.video_gen_resolution, cfg.image_size)
        if frames.shape[-1] != size:
            frames = F.interpolate(frames, size=(size, size), mode="bilinear", align_corners=False)
        return frames.unsqueeze(0).clamp(-1, 1)

    # ---- audio ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate_audio(self, prompt: str, duration: Optional[float] = None) -> torch.Tensor:
        """[1, samples] in [-1, 1] at ``audio_gen_sample_rate``."""
        cfg = self.config
        want = int((duration or cfg.audio_gen_duration) * cfg.audio_gen_sample_rate)
        n_tok = min(self.audio_time.shape[0], max(1, math.ceil(want / self.vocoder.hop)))
        feat = self.encode_text(prompt).unsqueeze(1) + self.audio_time[:n_tok].unsqueeze(0)
        logits = self.audio_head(feat).view(1, n_tok, cfg.audio_gen_num_codebooks, cfg.audio_gen_codebook_size)
        wav = self.vocoder(logits.argmax(-1))
        if wav.shape[-1] < want:                                       # the time grid is finite: tile to the length asked
            wav = wav.repeat(1, math.ceil(want / wav.shape[-1]))
        return wav[:, :want]


class YvGenerationBackend(ABC):
    """One way of producing one modality (reference :710-760)."""

    @property
    @abstractmethod
    def modality(self) -> YvGenerationModality: ...

    @property
    @abstractmethod
    def name(self) -> str: ...

    @abstractmethod
    def generate(self, condition: YvGenerationCondition, **kw: Any) -> YvGenerationResult: ...

    def is_available(self) -> bool:
        return True

    def get_capabilities(self) -> Dict[str, Any]:
        return {"name": self.name, "modality": self.modality.value, "available": self.is_available()}


class _SharedGeneratorBackend(YvGenerationBackend):
    def __init__(self, generator: YvSelfDevelopedGenerator):
        self.generator = generator

    def _run(self, fn, condition: YvGenerationCondition, **meta: Any) -> YvGenerationResult:
        t0 = time.perf_counter()
        try:
            data = fn()
            return YvGenerationResult(self.modality, data, {"prompt": condition.text, "backend": self.name, **meta},
                                      seconds=time.perf_counter() - t0)
        except Exception as e:                                         # a backend failure is a result, not a crash
            return YvGenerationResult(self.modality, None, {"backend": self.name}, False, f"{type(e).__name__}: {e}",
                                      time.perf_counter() - t0)


class YvTextToImageBackend(_SharedGeneratorBackend):
    modality = YvGenerationModality.IMAGE
    name = "yv-text-to-image"

    def generate(self, condition: YvGenerationCondition, **kw: Any) -> YvGenerationResult:
        g = self.generator
        return self._run(lambda: g.generate_image(condition.text or "", kw.get("steps"), condition.seed,
                                                  kw.get("guidance_scale")), condition, size=g.config.image_size)


class YvTextToAudioBackend(_SharedGeneratorBackend):
    modality = YvGenerationModality.AUDIO
    name = "yv-text-to-audio"

    def generate(self, condition: YvGenerationCondition, **kw: Any) -> YvGenerationResult:
        g = self.generator
        return self._run(lambda: g.generate_audio(condition.text or "", kw.get("duration")), condition,
                         sample_rate=g.config.audio_gen_sample_rate)


class YvTextToVideoBackend(_SharedGeneratorBackend):
    modality = YvGenerationModality.VIDEO
    name = "yv-text-to-video"

    def generate(self, condition: YvGenerationCondition, **kw: Any) -> YvGenerationResult:
        g = self.generator
        return self._run(lambda: g.generate_video(condition.text or "", kw.get("num_frames"), condition.seed), condition,
                         fps=g.config.video_gen_fps)


class YvGenerator:
    """Registry of generation backends keyed by modality (reference :985-1122)."""

    def __init__(self, config: Optional[YvGenerationConfig] = None, generator: Optional[YvSelfDevelopedGenerator] = None):
        self.config = config or YvGenerationConfig()
        self._shared = generator
        self._backends: Dict[YvGenerationModality, YvGenerationBackend] = {}
        self._register_default_backends()

    def _model(self) -> YvSelfDevelopedGenerator:
        if self._shared is None:                                       # built on first use: the registry itself is cheap
            self._shared = YvSelfDevelopedGenerator(self.config).eval()
        return self._shared

    def _register_default_backends(self) -> None:
        outer = self

        class _Lazy:                                                   # backends share one lazily built model
            def __getattr__(self, item):
                return getattr(outer._model(), item)
        lazy = _Lazy()
        for cls in (YvTextToImageBackend, YvTextToAudioBackend, YvTextToVideoBackend):
            self.register_backend(cls(lazy))                           # type: ignore[arg-type]

    def register_backend(self, backend: YvGenerationBackend) -> None:
        self._backends[backend.modality] = backend

    def get_available_modalities(self) -> List[str]:
        return [m.value for m, b in self._backends.items() if b.is_available()]

    def get_backend(self, modality: Union[str, YvGenerationModality]) -> Optional[YvGenerationBackend]:
        if isinstance(modality, str):
            try:
                modality = YvGenerationModality(modality.lower())
            except ValueError:
                return None
        return self._backends.get(modality)

    def generate_from_text(self, text: str, modality: Union[str, YvGenerationModality] = "image",
                           **kw: Any) -> YvGenerationResult:
        b = self.get_backend(modality)
        if b is None:
            m = modality if isinstance(modality, YvGenerationModality) else YvGenerationModality.TEXT
            return YvGenerationResult(m, None, {}, False, f"no backend for modality {modality!r}")
        return b.generate(YvGenerationCondition(text=text, seed=kw.pop("seed", None)), **kw)

    def get_capabilities(self) -> Dict[str, Any]:
        return {"modalities": self.get_available_modalities(),
                "backends": {m.value: b.get_capabilities() for m, b in self._backends.items()}}


class YvGeneratorFactory:
    @staticmethod
    def create_generator(config: Optional[YvGenerationConfig] = None) -> YvGenerator:
        return YvGenerator(config)
