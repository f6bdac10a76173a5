"""Small platform utilities (reference utils/device.py ``PiscesLxDeviceResolver``, utils/vram_controller.py
``PiscesLxVramController`` / ``PiscesLxVRAMMonitor``, utils/dtype_safe.py ``PiscesLxDtypeSafe``, utils/log_bridge.py
``PiscesLxThirdPartyLogBridge``, utils/modality_scanner.py ``PiscesLxModalityScanner``, utils/console.py
``PiscesLxConsoleEncoding``).

The memory controller works per process (allocator statistics and the per-process memory fraction); it never touches
a setting of the GPU itself."""
from __future__ import annotations

import logging
import os
import sys
from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Optional, Set, Tuple

import torch


# ------------------------------------------------------------------------------------------------ device
class PiscesLxDeviceResolver:
    @staticmethod
    def _env_int(name: str) -> Optional[int]:
        try:
            return int(os.environ[name])
        except (KeyError, ValueError):
            return None

    @classmethod
    def rank(cls, local_rank: Optional[int], device_count: int) -> int:
        lr = local_rank if local_rank is not None else (cls._env_int("LOCAL_RANK") or 0)
        return lr % device_count if device_count > 0 else 0

    @classmethod
    def default(cls, local_rank: Optional[int] = None) -> torch.device:
        if torch.cuda.is_available():
            return torch.device("cuda", cls.rank(local_rank, torch.cuda.device_count()))
        return torch.device("cpu")

    @classmethod
    def resolve(cls, device: Any = None, tensor_hint: Optional[torch.Tensor] = None,
                local_rank: Optional[int] = None) -> torch.device:
        if device is not None:
            d = torch.device(device) if not isinstance(device, torch.device) else device
            if d.type == "cuda" and d.index is None and torch.cuda.is_available():
                d = torch.device("cuda", cls.rank(local_rank, torch.cuda.device_count()))
            return d
        if tensor_hint is not None:
            return tensor_hint.device
        return cls.default(local_rank)

    @classmethod
    def probe(cls, device: torch.device) -> bool:
        """True when a tiny allocation on the device works."""
        try:
            torch.empty(1, device=device)
            return True
        except Exception:
            return False


# ------------------------------------------------------------------------------------------------ memory
@dataclass
class PiscesLxVRAMProfile:
    total_gb: float
    free_gb: float
    name: str = "cpu"
    reserve_gb: float = 6.0

    def safe_budget_gb(self) -> float:
        return max(0.0, self.total_gb * 0.86 - self.reserve_gb)


class PiscesLxVramController:
    """Estimates what a configuration needs and proposes the cheapest set of memory savers that makes it fit a
    180 GB part: (1) recompute activations, (2) bf16 optimizer state, (3) smaller micro-batch, (4) more sharding."""

    @staticmethod
    def profile_gpu(device: Optional[torch.device] = None) -> PiscesLxVRAMProfile:
        if torch.cuda.is_available():
            d = device or torch.device("cuda", torch.cuda.current_device())
            free, total = torch.cuda.mem_get_info(d)
            return PiscesLxVRAMProfile(total / 2 ** 30, free / 2 ** 30, torch.cuda.get_device_name(d))
        return PiscesLxVRAMProfile(0.0, 0.0)

    @staticmethod
    def estimate_model_vram(cfg: Any, micro_batch: int, seq_len: int, world: int = 1, state_bytes: float = 2.0,
                            recompute: bool = True) -> Dict[str, float]:
        p = cfg.count_parameters()["total"]
        g = 2 ** 30
        weights, grads, opt = p * 2 / g, p * 2 / g, p * state_bytes / g / world
        tokens = micro_batch * seq_len
        per_layer = tokens * cfg.hidden_size * 2 * (1 if recompute else 34) / g
        act = per_layer * cfg.n_layer + tokens * cfg.vocab_size * 4 / g / 8
        return {"weights_gb": weights, "grads_gb": grads, "optimizer_gb": opt, "activations_gb": act,
                "total_gb": weights + grads + opt + act}

    @classmethod
    def optimize_for_vram(cls, cfg: Any, budget_gb: float, micro_batch: int, seq_len: int, world: int = 1) -> Dict[str, Any]:
        plan = {"recompute": False, "state_bytes": 4.0, "micro_batch": micro_batch, "streaming_optimizer": False}
        steps: List[str] = []

        def total() -> float:
            est = cls.estimate_model_vram(cfg, plan["micro_batch"], seq_len, world, plan["state_bytes"], plan["recompute"])
            return est["total_gb"] - (est["grads_gb"] * 0.9 if plan["streaming_optimizer"] else 0.0)
        for name, change in (("recompute activations", {"recompute": True}),
                             ("bf16 optimizer state", {"state_bytes": 2.0}),
                             ("fold gradients into the optimizer as they arrive", {"streaming_optimizer": True})):
            if total() <= budget_gb:
                break
            plan.update(change)
            steps.append(name)
        while total() > budget_gb and plan["micro_batch"] > 1:
            plan["micro_batch"] //= 2
            steps.append(f"micro-batch {plan['micro_batch']}")
        plan["fits"], plan["estimated_gb"], plan["steps"] = total() <= budget_gb, total(), steps
        return plan


class PiscesLxVRAMMonitor:
    """Checks allocator pressure every ``check_interval`` steps and moves between tiers: 0 normal, 1 empty the cache
    between steps, 2 ask the trainer to halve the micro-batch.  De-escalates after ``calm_checks`` quiet checks."""

    def __init__(self, high: float = 0.94, low: float = 0.80, check_interval: int = 50, calm_checks: int = 4,
                 stats_fn=None):
        self.high, self.low, self.interval, self.calm_needed = high, low, check_interval, calm_checks
        self.tier, self.step, self.calm = 0, 0, 0
        self.stats_fn = stats_fn or self._cuda_stats

    @staticmethod
    def _cuda_stats() -> Tuple[float, float]:
        if not torch.cuda.is_available():
            return 0.0, 1.0
        free, total = torch.cuda.mem_get_info()
        return float(total - free), float(total)

    def check_and_adjust(self) -> bool:
        """Returns True when the tier changed."""
        self.step += 1
        if self.step % self.interval:
            return False
        used, total = self.stats_fn()
        frac = used / max(total, 1.0)
        if frac > self.high and self.tier < 2:
            self.tier, self.calm = self.tier + 1, 0
            if self.tier >= 1 and torch.cuda.is_available():
                torch.cuda.empty_cache()
            return True
        if frac < self.low and self.tier > 0:
            self.calm += 1
            if self.calm >= self.calm_needed:
                self.tier, self.calm = self.tier - 1, 0
                return True
        else:
            self.calm = 0
        return False


# ------------------------------------------------------------------------------------------------ dtype safety
class PiscesLxDtypeSafe:
    """Linear-algebra routines that have no bf16 / fp16 kernels run in fp32 and return the caller's dtype."""

    @staticmethod
    def qr_safe(m: torch.Tensor) -> torch.Tensor:
        q, _ = torch.linalg.qr(m.float())
        return q.to(m.dtype)

    @staticmethod
    def svd_safe(m: torch.Tensor, full_matrices: bool = False):
        u, s, vh = torch.linalg.svd(m.float(), full_matrices=full_matrices)
        return u.to(m.dtype), s.to(m.dtype), vh.to(m.dtype)

    @staticmethod
    def finite_or_zero(t: torch.Tensor) -> torch.Tensor:
        return torch.nan_to_num(t, nan=0.0, posinf=0.0, neginf=0.0)


# ------------------------------------------------------------------------------------------------ logging / console
class PiscesLxThirdPartyLogBridge:
    NOISY = {"urllib3": "WARNING", "filelock": "WARNING", "transformers": "ERROR", "torch.distributed": "WARNING",
             "uvicorn.access": "WARNING"}

    @classmethod
    def quiet(cls, levels: Optional[Dict[str, str]] = None) -> int:
        levels = levels if levels is not None else cls.NOISY
        for name, lvl in levels.items():
            logging.getLogger(name).setLevel(getattr(logging, lvl))
        return len(levels)

    @staticmethod
    def capture(logger_name: Optional[str], sink: logging.Handler) -> bool:
        lg = logging.getLogger(logger_name)
        if sink in lg.handlers:
            return False
        lg.addHandler(sink)
        return True

    @staticmethod
    def release(logger_name: Optional[str], sink: logging.Handler) -> bool:
        lg = logging.getLogger(logger_name)
        if sink not in lg.handlers:
            return False
        lg.removeHandler(sink)
        return True


class PiscesLxConsoleEncoding:
    @staticmethod
    def ensure_utf8() -> bool:
        ok = True
        for s in (sys.stdout, sys.stderr):
            try:
                if hasattr(s, "reconfigure") and (s.encoding or "").lower().replace("-", "") != "utf8":
                    s.reconfigure(encoding="utf-8", errors="replace")
            except Exception:
                ok = False
        return ok

    @staticmethod
    def child_environment(environment: Dict[str, str]) -> Dict[str, str]:
        env = dict(environment)
        env.setdefault("PYTHONIOENCODING", "utf-8")
        env.setdefault("PYTHONUTF8", "1")
        return env


# ------------------------------------------------------------------------------------------------ modality scanner
class PiscesLxModalityScanner:
    """Finds which modalities a dataset carries from the keys / values of a few samples, so that the trainer builds
    only the encoders it needs."""

    KEYS = {"image": ("image", "images", "pixel_values", "img"), "audio": ("audio", "waveform", "mel", "speech"),
            "video": ("video", "frames", "clip"), "text": ("text", "input_ids", "prompt", "messages", "content")}
    EXT = {"image": (".png", ".jpg", ".jpeg", ".webp", ".bmp"), "audio": (".wav", ".flac", ".mp3", ".ogg"),
           "video": (".mp4", ".mkv", ".webm", ".avi")}

    @classmethod
    def scan_sample(cls, sample: Any) -> Set[str]:
        found: Set[str] = set()
        if isinstance(sample, dict):
            for k, v in sample.items():
                kl = str(k).lower()
                for mod, names in cls.KEYS.items():
                    if any(kl == n or kl.startswith(n + "_") or kl.endswith("_" + n) for n in names) and v is not None:
                        found.add(mod)
                if isinstance(v, str):
                    for mod, exts in cls.EXT.items():
                        if v.lower().endswith(exts):
                            found.add(mod)
                elif isinstance(v, (dict, list, tuple)):
                    found |= cls.scan_sample(v)
        elif isinstance(sample, (list, tuple)):
            for v in sample:
                found |= cls.scan_sample(v)
        return found

    @classmethod
    def scan_dataset(cls, dataset: Iterable[Any], num_samples: int = 3) -> Set[str]:
        found: Set[str] = set()
        for i, s in enumerate(dataset):
            if i >= num_samples:
                break
            found |= cls.scan_sample(s)
        return found or {"text"}
