"""Operator layer.

``ops.functional`` is the API the models call.  For CUDA bf16 tensors every function runs the
hand-written sm_100a kernels of ``ops/csrc`` (through ``torch.ops.yv``); for CPU tensors (tests, the
fp32 oracle, Gloo runs) it runs the plain PyTorch math in ``ops.reference``.  There is no silent GPU
fallback: a CUDA call without the built extension raises.
"""
from __future__ import annotations

import os
import threading
from pathlib import Path
from typing import Dict, Optional

import torch

_SO = Path(__file__).resolve().parent / "_yv_ops.so"
_lock = threading.Lock()
_loaded = False
_status: Dict[int, torch.Tensor] = {}


class KernelStatusError(RuntimeError):
    """A device-side bounded wait ran out or a kernel rejected an index; see ``status_bits``."""

    def __init__(self, bits: int):
        self.status_bits = bits
        names = [n for b, n in ((1, "wait-timeout"), (2, "bad-argument"), (4, "peer-timeout"),
                                (8, "index-out-of-range")) if bits & b]
        super().__init__(f"sm_100a kernel reported status {bits:#x} ({', '.join(names) or 'unknown'})")


def extension_path() -> Path:
    return _SO


def extension_built() -> bool:
    return _SO.exists()


def load_extension(build_if_missing: bool = False) -> None:
    """Load ``_yv_ops.so`` (idempotent).  Raises ``RuntimeError`` when it has not been built."""
    global _loaded
    if _loaded:
        return
    with _lock:
        if _loaded:
            return
        if not _SO.exists():
            if build_if_missing or os.environ.get("YV_BUILD_ON_IMPORT") == "1":
                from .build import build
                build()
            else:
                raise RuntimeError(
                    f"{_SO} is missing: run `python -m pisceslx_b200.ops.build` (or __graft_entry__.build()) first")
        torch.ops.load_library(str(_SO))
        _loaded = True


def kernels():
    """The ``torch.ops.yv`` namespace (loads the extension on first use)."""
    load_extension()
    return torch.ops.yv


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] status buffer that kernels OR their error bits into."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device: Optional[torch.device] = None, reset: bool = True) -> None:
    """Read the status word (synchronises the device) and raise ``KernelStatusError`` if it is set."""
    if not _status:
        return
    for idx, t in list(_status.items()):
        if device is not None and device.index not in (None, idx):
            continue
        bits = int(t[0].item())
        if bits != 0:
            if reset:
                t.zero_()
            raise KernelStatusError(bits)


def use_kernels(*tensors: torch.Tensor) -> bool:
    """True when the arguments live on a GPU (then the CUDA kernels are mandatory)."""
    return any(t is not None and t.is_cuda for t in tensors)
