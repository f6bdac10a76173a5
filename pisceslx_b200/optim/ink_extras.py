"""The rest of the Ink memory-saving package around ``YvInkOptimizer`` (reference opss/optim/ink/: config.py,
gradient.py, checkpoint.py, kv_cache.py, moe.py, integrator.py, operator.py):

  * ``PiscesLxInkConfig``               one validated configuration for every component, with a memory estimate;
  * ``PiscesLxInkGradientCompressor``   block int8 / int4 gradient compression (stochastic rounding), dense or top-k,
                                        with ERROR FEEDBACK so that what a round loses is sent with the next one;
  * ``PiscesLxInkCheckpointSelector``   picks which blocks to recompute from a byte / FLOP cost model of each block
                                        and wraps their forwards; 8-bit activation compression for the others;
  * ``PiscesLxInkKVCacheQuantizer``     int8 / int4 KV cache: keys per channel group, values per token, packed nibbles;
  * ``PiscesLxInkMoEManager``           which experts stay on the GPU: LRU residency under a slot budget;
  * ``PiscesLxInkIntegrator``           GaLore projection, FP4 weight emulation and ROOT orthogonalisation as
                                        transforms on a gradient, each switchable;
  * ``PiscesLxInkOperator``             operator front (initialize / execute / step / state_dict) for the run tools.

What differs from the reference: the gradient compressor keeps a residual per tensor (the reference drops the rounding
and sparsification error, gradient.py:87-260); 4-bit values are stored two per byte (the reference stores one int4 per
uint8 and so saves nothing over int8, gradient.py:113-116, kv_cache.py:215-257); the checkpoint selector scores whole
transformer blocks from measured parameter bytes and an activation estimate and skips blocks whose recomputation
costs more than it frees (the reference classifies leaf modules by name, checkpoint.py:172-192, and wraps EVERY other
module in a forward that compresses its output and throws the result away, :335-383)."""
from __future__ import annotations

import math
import time
from collections import OrderedDict
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Set, Tuple

import torch
import torch.nn as nn
import torch.utils.checkpoint as tcp

from .ink import PiscesLxGaLoreProjector, PiscesLxInkBlockQuantizer, YvInkOptimizer


# ---------------------------------------------------------------------------------------------------------------- config
@dataclass
class PiscesLxInkConfig:
    name: str = "ink"
    lr: float = 1e-4
    weight_decay: float = 0.01
    betas: Tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    max_grad_norm: float = 1.0
    momentum_bits: int = 8
    momentum_block_size: int = 128
    variance_bits: int = 8
    variance_block_size: int = 256
    sparse_ratio: float = 1.0
    use_galore: bool = False
    galore_rank: int = 128
    galore_update_proj_gap: int = 200
    use_fp4: bool = False
    fp4_block_size: int = 16
    fp4_stochastic_rounding: bool = True
    use_root_ortho: bool = False
    root_ortho_steps: int = 5
    root_soft_threshold: float = 0.1
    root_spectral_norm_clip: float = 1.0
    root_min_dim_for_ortho: int = 16
    gradient_bits: int = 8
    gradient_block_size: int = 128
    gradient_sparse_ratio: float = 0.01
    kv_cache_bits: int = 8
    kv_cache_block_size: int = 64
    max_experts_on_gpu: int = 4
    moe_offload_threshold: float = 0.8
    checkpoint_ratio: float = 0.5
    num_update_blocks: int = 1

    def __post_init__(self) -> None:
        self.betas = tuple(self.betas)
        self._validate_config()

    def _validate_config(self) -> None:
        if self.lr < 0:
            raise ValueError(f"invalid learning rate: {self.lr}")
        for i, b in enumerate(self.betas):
            if not 0 <= b < 1:
                raise ValueError(f"invalid beta{i + 1}: {b}")
        for nm in ("momentum_bits", "variance_bits", "gradient_bits", "kv_cache_bits"):
            if getattr(self, nm) not in (4, 8):
                raise ValueError(f"{nm} must be 4 or 8, got {getattr(self, nm)}")
        for nm in ("sparse_ratio", "gradient_sparse_ratio", "checkpoint_ratio"):
            if not 0 < getattr(self, nm) <= 1:
                raise ValueError(f"{nm} must be in (0, 1], got {getattr(self, nm)}")
        for nm in ("momentum_block_size", "variance_block_size", "gradient_block_size", "kv_cache_block_size", "fp4_block_size"):
            if getattr(self, nm) < 1:
                raise ValueError(f"{nm} must be positive, got {getattr(self, nm)}")

    @classmethod
    def from_optimizer_config(cls, opt_config: Any) -> "PiscesLxInkConfig":
        """Take every field this class knows from an object or dictionary of optimizer settings."""
        get = (lambda k: opt_config.get(k)) if isinstance(opt_config, dict) else (lambda k: getattr(opt_config, k, None))
        kw = {k: get(k) for k in cls.__dataclass_fields__ if get(k) is not None}
        return cls(**kw)

    def get_memory_savings_ratio(self) -> float:
        """Optimizer-state bytes per parameter relative to fp32 Adam (8 bytes): quantised moments plus one fp32 scale
        per block."""
        m = self.momentum_bits / 8 + 4 / self.momentum_block_size
        v = self.variance_bits / 8 + 4 / self.variance_block_size
        return 1.0 - (m + v) / 8.0

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["betas"] = list(self.betas)
        return d


# ---------------------------------------------------------------------------------------------------------------- packing
def pack_nibbles(q: torch.Tensor) -> torch.Tensor:
    """int8 values in [-8, 7], last dimension even -> uint8 of half the length (low nibble first)."""
    u = (q.to(torch.int16) & 0xF).to(torch.uint8)
    return u[..., 0::2] | (u[..., 1::2] << 4)


def unpack_nibbles(p: torch.Tensor) -> torch.Tensor:
    lo, hi = (p & 0xF).to(torch.int8), (p >> 4).to(torch.int8)
    sign = lambda t: torch.where(t > 7, t - 16, t)
    return torch.stack([sign(lo), sign(hi)], -1).flatten(-2)


def _stochastic_round(x: torch.Tensor, lo: float, hi: float, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    noise = torch.rand(x.shape, device=x.device, dtype=x.dtype, generator=generator)
    return torch.floor(x + noise).clamp(lo, hi)


# ---------------------------------------------------------------------------------------------------------------- gradients
class PiscesLxInkGradientCompressor:
    """compress(gradient, key) -> a dictionary holding the quantised blocks and what is needed to restore them;
    decompress(payload) -> the gradient.  With a ``key`` the rounding (and, for the sparse form, the dropped entries)
    is remembered and added to the next gradient of the same key, so the sum over steps is preserved."""

    def __init__(self, gradient_bits: int = 8, block_size: int = 128, stochastic_rounding: bool = True,
                 error_feedback: bool = True, generator: Optional[torch.Generator] = None):
        assert gradient_bits in (4, 8) and block_size % 2 == 0
        self.gradient_bits, self.block_size, self.stochastic_rounding = gradient_bits, block_size, stochastic_rounding
        self.error_feedback, self._gen = error_feedback, generator
        self.qmax = 127.0 if gradient_bits == 8 else 7.0
        self._residual: Dict[Any, torch.Tensor] = {}
        self.reset_statistics()

    def _quantize_blocks(self, flat: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        pad = (-flat.numel()) % self.block_size
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        blocks = flat.view(-1, self.block_size)
        scale = blocks.abs().amax(1, keepdim=True).clamp_min(1e-12) / self.qmax
        x = blocks / scale
        q = _stochastic_round(x, -self.qmax, self.qmax, self._gen) if self.stochastic_rounding else torch.round(x).clamp(-self.qmax, self.qmax)
        return q.to(torch.int8), scale.squeeze(1)

    def _dequantize_blocks(self, q: torch.Tensor, scale: torch.Tensor, n: int) -> torch.Tensor:
        return (q.float() * scale.unsqueeze(1)).flatten()[:n]

    def _store(self, q: torch.Tensor) -> torch.Tensor:
        return pack_nibbles(q) if self.gradient_bits == 4 else q

    def _load(self, stored: torch.Tensor) -> torch.Tensor:
        return unpack_nibbles(stored) if self.gradient_bits == 4 else stored

    def compress(self, gradient: torch.Tensor, key: Any = None) -> Dict[str, Any]:
        g = gradient.detach().float().flatten()
        if self.error_feedback and key is not None and key in self._residual:
            g = g + self._residual[key]
        q, scale = self._quantize_blocks(g)
        if self.error_feedback and key is not None:
            self._residual[key] = g - self._dequantize_blocks(q, scale, g.numel())
        payload = {"kind": "dense", "q": self._store(q), "scale": scale, "shape": tuple(gradient.shape), "dtype": gradient.dtype}
        self._account(gradient, payload)
        return payload

    def compress_sparse(self, gradient: torch.Tensor, sparse_ratio: float = 0.01, key: Any = None) -> Dict[str, Any]:
        g = gradient.detach().float().flatten()
        if self.error_feedback and key is not None and key in self._residual:
            g = g + self._residual[key]
        k = max(1, min(g.numel(), int(math.ceil(g.numel() * sparse_ratio))))
        idx = g.abs().topk(k).indices.sort().values
        vals = g[idx]
        q, scale = self._quantize_blocks(vals)
        if self.error_feedback and key is not None:
            sent = torch.zeros_like(g)
            sent[idx] = self._dequantize_blocks(q, scale, k)
            self._residual[key] = g - sent
        payload = {"kind": "sparse", "q": self._store(q), "scale": scale, "index": idx.to(torch.int32 if g.numel() < 2 ** 31 else torch.int64),
                   "count": k, "shape": tuple(gradient.shape), "dtype": gradient.dtype}
        self._account(gradient, payload)
        return payload

    def decompress(self, payload: Dict[str, Any]) -> torch.Tensor:
        n = int(math.prod(payload["shape"]))
        q = self._load(payload["q"])
        self._stats["total_decompressions"] += 1
        if payload["kind"] == "dense":
            return self._dequantize_blocks(q, payload["scale"], n).view(payload["shape"]).to(payload["dtype"])
        out = torch.zeros(n, device=q.device, dtype=torch.float32)
        out[payload["index"].long()] = self._dequantize_blocks(q, payload["scale"], payload["count"])
        return out.view(payload["shape"]).to(payload["dtype"])

    decompress_sparse = decompress

    @staticmethod
    def payload_bytes(payload: Dict[str, Any]) -> int:
        return sum(v.numel() * v.element_size() for v in payload.values() if torch.is_tensor(v))

    def _account(self, gradient: torch.Tensor, payload: Dict[str, Any]) -> None:
        s = self._stats
        s["total_compressions"] += 1
        s["bytes_in"] += gradient.numel() * 4
        s["bytes_out"] += self.payload_bytes(payload)

    def residual_norm(self, key: Any) -> float:
        r = self._residual.get(key)
        return float(r.norm()) if r is not None else 0.0

    def get_statistics(self) -> Dict[str, Any]:
        s = dict(self._stats)
        s["avg_compression_ratio"] = s["bytes_in"] / s["bytes_out"] if s["bytes_out"] else 0.0
        return s

    def reset_statistics(self) -> None:
        self._stats = {"total_compressions": 0, "total_decompressions": 0, "bytes_in": 0, "bytes_out": 0}

    def state_dict(self) -> Dict[str, Any]:
        return {"gradient_bits": self.gradient_bits, "block_size": self.block_size, "stochastic_rounding": self.stochastic_rounding,
                "error_feedback": self.error_feedback, "residual": {k: v.clone() for k, v in self._residual.items()},
                "compression_stats": dict(self._stats)}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.gradient_bits, self.block_size = sd["gradient_bits"], sd["block_size"]
        self.stochastic_rounding, self.error_feedback = sd["stochastic_rounding"], sd.get("error_feedback", True)
        self.qmax = 127.0 if self.gradient_bits == 8 else 7.0
        self._residual = {k: v.clone() for k, v in sd.get("residual", {}).items()}
        self._stats = dict(sd.get("compression_stats", self._stats))


# ---------------------------------------------------------------------------------------------------------------- checkpoints
class PiscesLxInkCheckpointSelector:
    """Chooses the blocks whose activations are dropped and recomputed in the backward.

    ``analyze_model(model, tokens)`` finds the repeated blocks (children of the largest ``nn.ModuleList``; pass
    ``block_filter`` to choose differently) and estimates for each: parameter bytes, activation bytes kept without
    recomputation (``activation_factor`` x tokens x width x 2 bytes; the width is read from the block's largest linear
    weight) and recomputation cost (2 x parameters x tokens FLOPs).  ``get_checkpoint_layers`` keeps the
    ``checkpoint_ratio`` share of blocks with the most activation bytes freed per recomputed FLOP, never a block whose
    activations are smaller than ``activation_size_threshold``.  ``apply_checkpoint`` wraps exactly those."""

    def __init__(self, checkpoint_ratio: float = 0.5, activation_factor: float = 16.0, activation_size_threshold: int = 1 << 20,
                 block_filter: Optional[Callable[[str, nn.Module], bool]] = None):
        self.checkpoint_ratio, self.activation_factor = checkpoint_ratio, activation_factor
        self.activation_size_threshold, self.block_filter = activation_size_threshold, block_filter
        self.reset()

    def reset(self) -> None:
        self._layer_info: Dict[str, Dict[str, Any]] = {}
        self._checkpoint_layers: Set[str] = set()
        self._wrapped: Dict[str, Callable] = {}
        self._analyzed = False
        self._stats = {"total_layers": 0, "checkpoint_layers": 0, "memory_saved_mb": 0.0, "analyze_time_ms": 0.0}

    @staticmethod
    def _find_blocks(model: nn.Module) -> List[Tuple[str, nn.Module]]:
        best: List[Tuple[str, nn.Module]] = []
        best_params = -1
        for name, m in model.named_modules():
            if isinstance(m, nn.ModuleList) and len(m) > 1:
                n = sum(p.numel() for p in m.parameters())
                if n > best_params:
                    best_params, best = n, [(f"{name}.{i}" if name else str(i), b) for i, b in enumerate(m)]
        return best

    def analyze_model(self, model: nn.Module, tokens: int = 4096) -> Dict[str, Any]:
        t0 = time.perf_counter()
        wrapped = self._wrapped                               # blocks already wrapped stay wrapped across a re-analysis
        self.reset()
        self._wrapped = wrapped
        blocks = [(n, m) for n, m in model.named_modules() if self.block_filter(n, m)] if self.block_filter else self._find_blocks(model)
        for i, (name, blk) in enumerate(blocks):
            ps = list(blk.parameters())
            n_params = sum(p.numel() for p in ps)
            width = max((min(p.shape) for p in ps if p.dim() == 2), default=0)
            self._layer_info[name] = {"name": name, "type": type(blk).__name__, "layer_id": i, "param_count": n_params,
                                      "param_bytes": sum(p.numel() * p.element_size() for p in ps), "width": width,
                                      "activation_bytes": int(self.activation_factor * tokens * width * 2),
                                      "recompute_flops": 2.0 * n_params * tokens}
        self._analyzed = True
        self._stats.update(total_layers=len(blocks), analyze_time_ms=(time.perf_counter() - t0) * 1e3)
        return {"total_layers": len(blocks), "total_params": sum(i["param_count"] for i in self._layer_info.values()),
                "layer_info": self._layer_info}

    def get_checkpoint_layers(self) -> Set[str]:
        if not self._analyzed:
            return set()
        cands = [i for i in self._layer_info.values() if i["activation_bytes"] >= self.activation_size_threshold]
        cands.sort(key=lambda i: (-i["activation_bytes"] / max(i["recompute_flops"], 1.0), i["layer_id"]))
        want = int(round(len(self._layer_info) * self.checkpoint_ratio))
        self._checkpoint_layers = {i["name"] for i in cands[:want]}
        self._stats["checkpoint_layers"] = len(self._checkpoint_layers)
        self._stats["memory_saved_mb"] = sum(self._layer_info[n]["activation_bytes"] for n in self._checkpoint_layers) / 2 ** 20
        return set(self._checkpoint_layers)

    def apply_checkpoint(self, model: nn.Module, checkpoint_fn: Optional[Callable] = None) -> int:
        """Wrap the forward of every selected block (idempotent); returns how many blocks are wrapped.  Recomputation
        happens only while gradients are enabled and the module is in training mode."""
        if not self._analyzed:
            self.analyze_model(model)
        if not self._checkpoint_layers:
            self.get_checkpoint_layers()
        fn = checkpoint_fn or (lambda f, *a, **k: tcp.checkpoint(f, *a, use_reentrant=False, **k))
        mods = dict(model.named_modules())
        for name in self._checkpoint_layers:
            m = mods.get(name)
            if m is None or name in self._wrapped:
                continue
            orig = m.forward
            self._wrapped[name] = orig

            def wrapped(*a, __o=orig, __m=m, **k):
                if __m.training and torch.is_grad_enabled():
                    return fn(__o, *a, **k)
                return __o(*a, **k)
            m.forward = wrapped
        return len(self._wrapped)

    def remove_checkpoint(self, model: nn.Module) -> int:
        mods = dict(model.named_modules())
        n = 0
        for name, orig in list(self._wrapped.items()):
            if name in mods:
                mods[name].forward = orig
                n += 1
            del self._wrapped[name]
        return n

    # -- 8-bit activation round trip --------------------------------------------------------------------------------------
    @staticmethod
    def compress_activation(activation: torch.Tensor, block_size: int = 256) -> Dict[str, Any]:
        q, scale, shape, n = PiscesLxInkBlockQuantizer(8, block_size).quantize(activation)
        return {"q": q, "scale": scale, "shape": shape, "n": n, "dtype": activation.dtype, "block_size": block_size}

    @staticmethod
    def recompute_activation(c: Dict[str, Any]) -> torch.Tensor:
        return PiscesLxInkBlockQuantizer(8, c["block_size"]).dequantize(c["q"], c["scale"], c["shape"], c["n"]).to(c["dtype"])

    def estimate_memory_savings(self, model: nn.Module, batch_size: int = 1, seq_len: int = 512) -> Dict[str, float]:
        self.analyze_model(model, batch_size * seq_len)
        self.get_checkpoint_layers()
        every = sum(i["activation_bytes"] for i in self._layer_info.values()) / 2 ** 20
        saved = self._stats["memory_saved_mb"]
        boundary = sum(batch_size * seq_len * self._layer_info[n]["width"] * 2 for n in self._checkpoint_layers) / 2 ** 20
        return {"no_checkpoint_mb": every, "selective_checkpoint_mb": every - saved + boundary, "savings_mb": saved - boundary,
                "savings_percent": 100.0 * (saved - boundary) / every if every else 0.0,
                "checkpoint_layers": len(self._checkpoint_layers), "total_layers": len(self._layer_info),
                "extra_flops": sum(self._layer_info[n]["recompute_flops"] for n in self._checkpoint_layers)}

    def get_statistics(self) -> Dict[str, Any]:
        return dict(self._stats)

    def state_dict(self) -> Dict[str, Any]:
        return {"checkpoint_ratio": self.checkpoint_ratio, "activation_factor": self.activation_factor,
                "activation_size_threshold": self.activation_size_threshold, "checkpoint_layers": sorted(self._checkpoint_layers)}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.checkpoint_ratio, self.activation_factor = sd["checkpoint_ratio"], sd["activation_factor"]
        self.activation_size_threshold = sd["activation_size_threshold"]
        self._checkpoint_layers = set(sd.get("checkpoint_layers", ()))


# ---------------------------------------------------------------------------------------------------------------- KV cache
class PiscesLxInkKVCacheQuantizer:
    """Keys are quantised per channel group along the sequence (key outliers live in fixed channels), values per token
    (one scale per token and head).  Inputs ``[..., S, D]``.  4-bit codes are packed two per byte."""

    def __init__(self, bits: int = 8, block_size: int = 64):
        assert bits in (4, 8)
        self.bits, self.block_size = bits, block_size
        self.qmax = 127.0 if bits == 8 else 7.0
        self._cache: Dict[str, Dict[str, Any]] = {}

    def _pack(self, q: torch.Tensor) -> torch.Tensor:
        return pack_nibbles(q) if self.bits == 4 else q

    def _unpack(self, q: torch.Tensor) -> torch.Tensor:
        return unpack_nibbles(q) if self.bits == 4 else q

    def quantize_k(self, k: torch.Tensor) -> Dict[str, Any]:
        """Per channel, per block of ``block_size`` positions: scale [..., ceil(S / block), D]."""
        *lead, S, D = k.shape
        assert D % 2 == 0
        pad = (-S) % self.block_size
        x = torch.cat([k.float(), k.new_zeros(*lead, pad, D, dtype=torch.float32)], -2) if pad else k.float()
        blocks = x.view(*lead, -1, self.block_size, D)
        scale = blocks.abs().amax(-2, keepdim=True).clamp_min(1e-12) / self.qmax
        q = torch.round(blocks / scale).clamp(-self.qmax, self.qmax).to(torch.int8).view(*lead, S + pad, D)
        return {"q": self._pack(q), "scale": scale.squeeze(-2).to(torch.float16), "seq": S, "dtype": k.dtype, "axis": "channel"}

    def quantize_v(self, v: torch.Tensor) -> Dict[str, Any]:
        """Per token: scale [..., S, 1]."""
        assert v.shape[-1] % 2 == 0
        scale = v.float().abs().amax(-1, keepdim=True).clamp_min(1e-12) / self.qmax
        q = torch.round(v.float() / scale).clamp(-self.qmax, self.qmax).to(torch.int8)
        return {"q": self._pack(q), "scale": scale.to(torch.float16), "seq": v.shape[-2], "dtype": v.dtype, "axis": "token"}

    def dequantize_k(self, c: Dict[str, Any]) -> torch.Tensor:
        q = self._unpack(c["q"]).float()
        *lead, Sp, D = q.shape
        x = q.view(*lead, -1, self.block_size, D) * c["scale"].float().unsqueeze(-2)
        return x.view(*lead, Sp, D)[..., : c["seq"], :].to(c["dtype"])

    def dequantize_v(self, c: Dict[str, Any]) -> torch.Tensor:
        return (self._unpack(c["q"]).float() * c["scale"].float()).to(c["dtype"])

    # -- a small store keyed by layer ---------------------------------------------------------------------------------------
    def store(self, layer_name: str, k: torch.Tensor, v: torch.Tensor) -> None:
        self._cache[layer_name] = {"k": self.quantize_k(k), "v": self.quantize_v(v),
                                   "original_bytes": (k.numel() + v.numel()) * k.element_size()}

    def load(self, layer_name: str) -> Tuple[torch.Tensor, torch.Tensor]:
        c = self._cache[layer_name]
        return self.dequantize_k(c["k"]), self.dequantize_v(c["v"])

    def get_cache_size(self, layer_name: Optional[str] = None) -> Dict[str, int]:
        names = [layer_name] if layer_name is not None else list(self._cache)
        stored = orig = 0
        for n in names:
            c = self._cache.get(n)
            if c is None:
                continue
            orig += c["original_bytes"]
            for part in (c["k"], c["v"]):
                stored += sum(t.numel() * t.element_size() for t in part.values() if torch.is_tensor(t))
        return {"stored_bytes": stored, "original_bytes": orig}

    def clear_cache(self, layer_name: Optional[str] = None) -> None:
        if layer_name is None:
            self._cache.clear()
        else:
            self._cache.pop(layer_name, None)

    def get_memory_savings(self, original_bytes: Optional[int] = None) -> Dict[str, Any]:
        s = self.get_cache_size()
        orig = original_bytes if original_bytes is not None else s["original_bytes"]
        return {"original_bytes": orig, "stored_bytes": s["stored_bytes"], "savings_bytes": orig - s["stored_bytes"],
                "compression_ratio": orig / s["stored_bytes"] if s["stored_bytes"] else 0.0}

    def state_dict(self) -> Dict[str, Any]:
        return {"bits": self.bits, "block_size": self.block_size}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.bits, self.block_size = sd["bits"], sd["block_size"]
        self.qmax = 127.0 if self.bits == 8 else 7.0


# ---------------------------------------------------------------------------------------------------------------- MoE residency
class PiscesLxInkMoEManager:
    """Keeps at most ``max_experts_on_gpu`` experts on the compute device; the least recently used one moves to the
    host when room is needed.  ``record_access(e)`` is called where the router picks expert ``e``; ``load_expert`` makes
    it resident.  ``mover(module, device)`` does the move (``module.to(device)`` by default), so tests can run on CPU
    with a recorder and production can use pinned buffers."""

    def __init__(self, max_experts_on_gpu: int = 4, offload_threshold: float = 0.8, device: Any = "cuda", host: Any = "cpu",
                 mover: Optional[Callable[[nn.Module, Any], None]] = None, window: int = 1024):
        self.max_experts_on_gpu, self.offload_threshold = max_experts_on_gpu, offload_threshold
        self.device, self.host = device, host
        self._move = mover or (lambda m, d: m.to(d))
        self._experts: Dict[int, nn.Module] = {}
        self._resident: "OrderedDict[int, None]" = OrderedDict()
        self._access: Dict[int, int] = {}
        self._recent: List[int] = []
        self._window = window
        self.reset_statistics()

    def register_expert(self, expert_id: int, module: nn.Module, resident: bool = False) -> None:
        self._experts[expert_id] = module
        self._access.setdefault(expert_id, 0)
        if resident:
            self.load_expert(expert_id)

    def record_access(self, expert_id: int) -> None:
        self._access[expert_id] = self._access.get(expert_id, 0) + 1
        self._recent.append(expert_id)
        if len(self._recent) > self._window:
            del self._recent[: len(self._recent) - self._window]
        if expert_id in self._resident:
            self._resident.move_to_end(expert_id)
            self._stats["hits"] += 1
        else:
            self._stats["misses"] += 1

    def get_active_experts(self) -> Set[int]:
        return set(self._resident)

    def should_offload(self, expert_id: int) -> bool:
        """Resident, the device is over ``offload_threshold`` of its slots, and the expert is the least recently used."""
        if expert_id not in self._resident or len(self._resident) < self.offload_threshold * self.max_experts_on_gpu:
            return False
        return next(iter(self._resident)) == expert_id

    def offload_least_used(self) -> Optional[int]:
        if not self._resident:
            return None
        eid, _ = self._resident.popitem(last=False)
        self._move(self._experts[eid], self.host)
        self._stats["offloads"] += 1
        return eid

    def load_expert(self, expert_id: int) -> bool:
        if expert_id not in self._experts:
            return False
        if expert_id in self._resident:
            self._resident.move_to_end(expert_id)
            return True
        while len(self._resident) >= self.max_experts_on_gpu:
            self.offload_least_used()
        self._move(self._experts[expert_id], self.device)
        self._resident[expert_id] = None
        self._stats["loads"] += 1
        return True

    def get_utilization(self) -> Dict[int, float]:
        n = max(len(self._recent), 1)
        return {e: self._recent.count(e) / n for e in self._experts}

    def get_overutilized_experts(self, factor: float = 2.0) -> List[int]:
        fair = 1.0 / max(len(self._experts), 1)
        return sorted(e for e, u in self.get_utilization().items() if u > factor * fair)

    def get_underutilized_experts(self, factor: float = 0.5) -> List[int]:
        fair = 1.0 / max(len(self._experts), 1)
        return sorted(e for e, u in self.get_utilization().items() if u < factor * fair)

    def dynamic_manage(self) -> Dict[str, List[int]]:
        """Make the most used experts of the recent window resident (up to the budget), offloading what they displace."""
        util = self.get_utilization()
        want = [e for e, _ in sorted(util.items(), key=lambda kv: (-kv[1], kv[0]))[: self.max_experts_on_gpu] if util[e] > 0]
        before = set(self._resident)
        for e in list(self._resident):
            if e not in want and len(self._resident) + len([w for w in want if w not in self._resident]) > self.max_experts_on_gpu:
                self._resident.pop(e)
                self._move(self._experts[e], self.host)
                self._stats["offloads"] += 1
        for e in want:
            self.load_expert(e)
        after = set(self._resident)
        return {"loaded": sorted(after - before), "offloaded": sorted(before - after)}

    def get_memory_footprint(self) -> Dict[str, float]:
        size = lambda m: sum(p.numel() * p.element_size() for p in m.parameters()) / 2 ** 20
        on = sum(size(self._experts[e]) for e in self._resident)
        tot = sum(size(m) for m in self._experts.values())
        return {"gpu_mb": on, "host_mb": tot - on, "total_mb": tot, "resident_experts": len(self._resident)}

    def get_statistics(self) -> Dict[str, Any]:
        s = dict(self._stats)
        n = s["hits"] + s["misses"]
        s["hit_rate"] = s["hits"] / n if n else 0.0
        return s

    def reset_statistics(self) -> None:
        self._stats = {"hits": 0, "misses": 0, "loads": 0, "offloads": 0}

    def state_dict(self) -> Dict[str, Any]:
        return {"max_experts_on_gpu": self.max_experts_on_gpu, "offload_threshold": self.offload_threshold,
                "resident": list(self._resident), "access": dict(self._access), "stats": dict(self._stats)}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.max_experts_on_gpu, self.offload_threshold = sd["max_experts_on_gpu"], sd["offload_threshold"]
        self._access, self._stats = dict(sd.get("access", {})), dict(sd.get("stats", self._stats))
        for e in sd.get("resident", ()):
            self.load_expert(e)


# ---------------------------------------------------------------------------------------------------------------- integrator
class PiscesLxInkIntegrator:
    """The optional transforms of the Ink step as separate calls, each a no-op when switched off in the configuration:
    ``apply_galore`` (project a 2-D gradient to rank r / back), ``apply_fp4_forward`` (weights as the FP4 grid sees
    them, straight-through), ``apply_root_denoise`` (soft-threshold gradient spikes), ``apply_root_ortho``
    (Newton-Schulz orthogonalisation of a 2-D update), ``apply_root_spectral_clip`` (bound the largest singular value,
    estimated by power iteration)."""

    def __init__(self, config: Optional[PiscesLxInkConfig] = None):
        self.config = config or PiscesLxInkConfig()
        self._galore: Dict[str, PiscesLxGaLoreProjector] = {}
        self._fp4_state: Dict[str, Dict[str, Any]] = {}
        self._fp4 = None
        self._step = 0
        self._counts = {"galore": 0, "fp4": 0, "ortho": 0, "denoise": 0, "clip": 0}
        self._initialized = False

    def initialize(self) -> None:
        if self.config.use_fp4:
            from ..quant.fp4 import PiscesLxFP4Quantizer
            self._fp4 = PiscesLxFP4Quantizer(self.config.fp4_block_size, self.config.fp4_stochastic_rounding)
        self._initialized = True

    def advance(self) -> int:
        self._step += 1
        return self._step

    def apply_galore(self, name: str, grad: torch.Tensor) -> Tuple[torch.Tensor, Optional[Callable[[torch.Tensor], torch.Tensor]]]:
        """Returns (projected gradient, function that maps an update back) or (grad, None) when not applicable."""
        c = self.config
        if not c.use_galore or grad.dim() != 2 or min(grad.shape) <= c.galore_rank:
            return grad, None
        pr = self._galore.setdefault(name, PiscesLxGaLoreProjector(c.galore_rank, c.galore_update_proj_gap))
        self._counts["galore"] += 1
        return pr.project(grad, self._step), pr.project_back

    def apply_fp4_forward(self, name: str, weight: torch.Tensor) -> torch.Tensor:
        if not self.config.use_fp4 or weight.dim() != 2 or weight.numel() % self.config.fp4_block_size:
            return weight
        if self._fp4 is None:
            self.initialize()
        q = self._fp4.fake_quant(weight.detach())
        self._counts["fp4"] += 1
        self._fp4_state[name] = {"error": float((q.detach().float() - weight.detach().float()).norm() / weight.detach().float().norm().clamp_min(1e-12))}
        return weight + (q - weight).detach()

    def apply_fp4_backward(self, name: str, grad: torch.Tensor) -> torch.Tensor:
        """The straight-through estimator passes the gradient unchanged."""
        return grad

    def should_orthogonalize(self, param: torch.Tensor) -> bool:
        return self.config.use_root_ortho and param.dim() == 2 and min(param.shape) >= self.config.root_min_dim_for_ortho

    def apply_root_denoise(self, grad: torch.Tensor) -> torch.Tensor:
        """Soft threshold at ``root_soft_threshold`` x the largest magnitude: sign(g) max(|g| - t, 0) for the entries
        ABOVE the robust scale (median x 10), identity below - isolated spikes shrink, ordinary entries stay."""
        if not self.config.use_root_ortho:
            return grad
        a = grad.abs()
        robust = a.flatten().median() * 10.0
        t = self.config.root_soft_threshold * a.max()
        self._counts["denoise"] += 1
        return torch.where(a > robust, torch.sign(grad) * (a - t).clamp_min(robust), grad)

    def apply_root_ortho(self, update: torch.Tensor) -> torch.Tensor:
        if not self.should_orthogonalize(update):
            return update
        from ..ops.reference import MUON_NS_COEFFS, newton_schulz
        self._counts["ortho"] += 1
        return newton_schulz(update.float(), MUON_NS_COEFFS[-self.config.root_ortho_steps:]).to(update.dtype)

    def apply_root_spectral_clip(self, update: torch.Tensor, iters: int = 8) -> torch.Tensor:
        if not self.config.use_root_ortho or update.dim() != 2:
            return update
        u = update.float()
        v = torch.ones(u.shape[1], device=u.device) / math.sqrt(u.shape[1])
        for _ in range(iters):
            v = torch.nn.functional.normalize(u.t() @ (u @ v), dim=0)
        sigma = (u @ v).norm()
        self._counts["clip"] += 1
        return (u * (self.config.root_spectral_norm_clip / sigma).clamp(max=1.0)).to(update.dtype)

    def get_galore_state(self, name: str) -> Dict[str, Any]:
        p = self._galore.get(name)
        return {} if p is None else {"P": p.P, "left": p.left}

    def set_galore_state(self, name: str, state: Dict[str, Any]) -> None:
        pr = self._galore.setdefault(name, PiscesLxGaLoreProjector(self.config.galore_rank, self.config.galore_update_proj_gap))
        pr.P, pr.left = state.get("P"), state.get("left", True)

    def get_fp4_state(self, name: str) -> Dict[str, Any]:
        return dict(self._fp4_state.get(name, {}))

    def get_component_status(self) -> Dict[str, bool]:
        c = self.config
        return {"galore": c.use_galore, "fp4": c.use_fp4, "root_ortho": c.use_root_ortho, "initialized": self._initialized}

    def get_statistics(self) -> Dict[str, Any]:
        return {"step": self._step, "calls": dict(self._counts), "galore_params": len(self._galore), "fp4_params": len(self._fp4_state)}

    def reset_states(self) -> None:
        self._galore.clear()
        self._fp4_state.clear()

    def state_dict(self) -> Dict[str, Any]:
        return {"step": self._step, "galore": {n: self.get_galore_state(n) for n in self._galore}, "config": self.config.to_dict()}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self._step = int(sd.get("step", 0))
        for n, st in sd.get("galore", {}).items():
            self.set_galore_state(n, st)


# ---------------------------------------------------------------------------------------------------------------- operator
class PiscesLxInkOperator:
    """Operator front of the Ink optimizer for the run tools: ``initialize(model)`` builds the optimizer (and, when the
    configuration asks, selects checkpoint blocks); ``execute({"action": ...})`` with ``step`` / ``zero_grad`` /
    ``memory`` / ``statistics``; gradient clipping to ``max_grad_norm`` happens inside ``step``."""

    name, version = "ink", "1.0"
    description = "memory-saving optimizer: quantised moments, sparse / low-rank gradients, selective recomputation"

    def __init__(self, config: Optional[PiscesLxInkConfig] = None):
        self.config = config or PiscesLxInkConfig()
        self.integrator = PiscesLxInkIntegrator(self.config)
        self.optimizer: Optional[YvInkOptimizer] = None
        self.checkpoint_selector: Optional[PiscesLxInkCheckpointSelector] = None
        self._model: Optional[nn.Module] = None
        self._steps = 0
        self._last_norm = 0.0

    input_schema = {"action": "step | zero_grad | memory | statistics"}
    output_schema = {"success": "bool", "output": "dict", "error": "str | None"}

    @staticmethod
    def validate_inputs(inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs, dict) and inputs.get("action", "step") in ("step", "zero_grad", "memory", "statistics")

    def initialize(self, model: nn.Module, config: Optional[PiscesLxInkConfig] = None, apply_checkpoint: bool = False) -> None:
        if config is not None:
            self.config = config
            self.integrator = PiscesLxInkIntegrator(config)
        c = self.config
        self._model = model
        self.integrator.initialize()
        self.optimizer = YvInkOptimizer([p for p in model.parameters() if p.requires_grad], lr=c.lr, betas=c.betas, eps=c.eps,
                                        weight_decay=c.weight_decay, momentum_bits=c.momentum_bits, variance_bits=c.variance_bits,
                                        block_size=c.momentum_block_size, sparse_ratio=c.sparse_ratio,
                                        galore_rank=c.galore_rank if c.use_galore else 0,
                                        galore_update_interval=c.galore_update_proj_gap, cyclic_blocks=c.num_update_blocks)
        if apply_checkpoint:
            self.checkpoint_selector = PiscesLxInkCheckpointSelector(c.checkpoint_ratio, activation_size_threshold=0)
            self.checkpoint_selector.apply_checkpoint(model)

    def _need(self) -> YvInkOptimizer:
        if self.optimizer is None:
            raise RuntimeError("initialize(model) first")
        return self.optimizer

    def step(self) -> float:
        opt = self._need()
        params = [p for g in opt.param_groups for p in g["params"] if p.grad is not None]
        if self.config.max_grad_norm > 0 and params:
            self._last_norm = float(torch.nn.utils.clip_grad_norm_(params, self.config.max_grad_norm))
        opt.step()
        self.integrator.advance()
        self._steps += 1
        return self._last_norm

    def zero_grad(self, set_to_none: bool = True) -> None:
        self._need().zero_grad(set_to_none=set_to_none)

    def get_memory_info(self) -> Dict[str, Any]:
        opt = self._need()
        n = sum(p.numel() for g in opt.param_groups for p in g["params"])
        return {"parameters": n, "state_bytes": opt.state_bytes(), "fp32_adam_state_bytes": 8 * n,
                "expected_savings_ratio": self.config.get_memory_savings_ratio()}

    def get_statistics(self) -> Dict[str, Any]:
        return {"steps": self._steps, "last_grad_norm": self._last_norm, "integrator": self.integrator.get_statistics(),
                "checkpoint": self.checkpoint_selector.get_statistics() if self.checkpoint_selector else None}

    def execute(self, inputs: Dict[str, Any], **kwargs: Any) -> Dict[str, Any]:
        if not self.validate_inputs(inputs):
            return {"success": False, "output": {}, "error": f"invalid inputs: {inputs!r}"}
        try:
            a = inputs.get("action", "step")
            if a == "step":
                out: Dict[str, Any] = {"grad_norm": self.step(), "steps": self._steps}
            elif a == "zero_grad":
                self.zero_grad(inputs.get("set_to_none", True))
                out = {}
            elif a == "memory":
                out = self.get_memory_info()
            else:
                out = self.get_statistics()
            return {"success": True, "output": out, "error": None}
        except Exception as e:
            return {"success": False, "output": {}, "error": f"{type(e).__name__}: {e}"}

    def state_dict(self) -> Dict[str, Any]:
        return {"config": self.config.to_dict(), "steps": self._steps, "optimizer": self._need().state_dict(),
                "integrator": self.integrator.state_dict()}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self._steps = int(sd.get("steps", 0))
        self._need().load_state_dict(sd["optimizer"])
        self.integrator.load_state_dict(sd.get("integrator", {}))
