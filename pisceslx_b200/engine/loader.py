"""Model construction from presets and checkpoints (shared by ``manage.py train / infer / serve``).

Follows the reference's loading contract: ``YvConfig.from_yaml(configs/model/<size>.yaml)`` -> model ->
``torch.load(ckpt)`` accepting ``model_state_dict | model | state_dict | raw`` (tools/infer/core.py:209-226,
opss/infer/native_ruchbah.py:77-84); ``save_pretrained`` writes ``pytorch_model.bin`` + ``config.json``
(model/core/model.py:1240-1253)."""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Any, Optional

import torch

from ..config import YvConfig
from ..models import build_model
from .checkpoint import extract_state_dict

REPO_ROOT = Path(__file__).resolve().parents[2]


def resolve_model_config(model_size: str = "0.01B", model_config: Optional[str] = None) -> YvConfig:
    if model_config:
        p = Path(model_config)
        return YvConfig.from_json(p) if p.suffix == ".json" else YvConfig.from_yaml(p)
    p = REPO_ROOT / "configs" / "model" / f"{model_size}.yaml"
    if not p.exists():
        raise FileNotFoundError(f"no preset {p}; available: {sorted(x.stem for x in p.parent.glob('*.yaml'))}")
    return YvConfig.from_yaml(p)


def attach_optional_components(model: Any, cfg: YvConfig, parallel: Any = None) -> None:
    trunk = model.model
    p = next(model.parameters())
    if cfg.use_pq_field and trunk.subconscious is None:
        from ..models.subconscious import YvPQKnowledgeField
        grp = parallel.world_group if (parallel is not None and parallel.world_size > 1) else None
        field = YvPQKnowledgeField(cfg, grp).to(device=p.device, dtype=p.dtype)
        trunk.attach("subconscious", field)
        field.materialise_shards()
    elif cfg.use_subconscious and trunk.subconscious is None:
        from ..models.subconscious import YvSubconsciousSystem
        trunk.attach("subconscious", YvSubconsciousSystem(cfg).to(p.device))
    if getattr(cfg, "use_subconscious_blocks", False) and trunk.block_field is None:
        from ..models.block_field import YvSubconsciousBlockField
        trunk.attach("block_field", YvSubconsciousBlockField.from_config(cfg).to(p.device))
    if cfg.vision_hidden_size and trunk.vision_encoder is None:
        from ..models.multimodal import attach_multimodal
        attach_multimodal(model, vision=True)


def load_model_for_inference(model_size: str = "0.01B", ckpt: Optional[str] = None, device: Optional[str] = None,
                             model_config: Optional[str] = None, dtype: Optional[torch.dtype] = None) -> Any:
    cfg = resolve_model_config(model_size, model_config)
    dev = torch.device(device) if device else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model = build_model(cfg, dev, dtype)
    attach_optional_components(model, cfg)
    if ckpt:
        path = Path(ckpt)
        if path.is_dir() and (path / "pytorch_model.bin").exists():
            path = path / "pytorch_model.bin"
        sd = extract_state_dict(torch.load(path, map_location="cpu", weights_only=False))
        model.load_reference_state_dict(sd, strict=False)
    return model.eval()


def save_pretrained(model: Any, directory: str) -> None:
    os.makedirs(directory, exist_ok=True)
    torch.save({k: v.cpu() for k, v in model.to_reference_state_dict().items()},
               os.path.join(directory, "pytorch_model.bin"))
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(model.cfg.to_dict(), f, indent=2, default=str)


def from_pretrained(directory: str, device: Optional[str] = None) -> Any:
    cfg = YvConfig.from_json(os.path.join(directory, "config.json"))
    dev = torch.device(device) if device else torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model = build_model(cfg, dev)
    attach_optional_components(model, cfg)
    sd = torch.load(os.path.join(directory, "pytorch_model.bin"), map_location="cpu", weights_only=False)
    model.load_reference_state_dict(sd, strict=False)
    return model
