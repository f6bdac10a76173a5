"""Checkpoint verifier (reference tools/dev/verify_checkpoint.py:93-233): is the file strictly loadable, do the
weights differ from a fresh initialisation, and is the held-out cross-entropy below ln(vocab)?"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch

from .checkpoint import extract_state_dict
from .loader import resolve_model_config


class PiscesLxCheckpointVerifier:
    def verify(self, ckpt: str, model_size: str = "0.01B", model_config: Optional[str] = None, tokens: int = 256,
               seed: int = 0) -> Dict[str, Any]:
        from ..models import build_model
        cfg = resolve_model_config(model_size, model_config)
        rep: Dict[str, Any] = {"ok": False, "checkpoint": ckpt}
        model = build_model(cfg, "cpu", torch.float32, seed=seed + 1)
        fresh = {k: v.clone() for k, v in model.to_reference_state_dict().items()}
        try:
            sd = extract_state_dict(torch.load(ckpt, map_location="cpu", weights_only=False))
            leftover = model.load_reference_state_dict(sd, strict=True)
            rep["strict_loadable"] = not leftover
            rep["unexpected_keys"] = leftover[:8]
        except Exception as e:
            rep["strict_loadable"] = False
            rep["error"] = str(e)
            return rep
        now = model.to_reference_state_dict()
        changed = sum(1 for k in fresh if not torch.equal(fresh[k], now[k]))
        rep["tensors_differing_from_fresh_init"] = changed
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(0, cfg.vocab_size, (1, tokens), generator=g)
        model.eval()
        with torch.no_grad():
            ce = float(model(input_ids=ids, labels=ids).loss)
        rep["held_out_ce"], rep["uniform_ce"] = ce, math.log(cfg.vocab_size)
        rep["ok"] = bool(rep["strict_loadable"] and changed > 0 and math.isfinite(ce))
        return rep
