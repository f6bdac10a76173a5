"""Export and packaging (reference tools/publish: safetensors export, Docker context, hub layout) and the model-cache
bookkeeping of tools/cache.

``export_safetensors`` writes the model in the reference's parameter naming (per-expert ``gate_proj`` / ``up_proj`` /
``down_proj`` keys), sharded by size with an ``index.json`` weight map, plus ``config.json``; ``load_safetensors``
reads it back into a model."""
from __future__ import annotations

import hashlib
import json
import os
import time
from typing import Any, Dict, List, Optional

import torch


def export_safetensors(model: Any, directory: str, max_shard_bytes: int = 4 << 30) -> Dict[str, Any]:
    from safetensors.torch import save_file
    os.makedirs(directory, exist_ok=True)
    sd = {k: v.detach().cpu().contiguous() for k, v in model.to_reference_state_dict().items()}
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for k, v in sd.items():
        b = v.numel() * v.element_size()
        if size + b > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][k] = v
        size += b
    weight_map: Dict[str, str] = {}
    for i, sh in enumerate(shards):
        name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(directory, name), metadata={"format": "pt"})
        weight_map.update({k: name for k in sh})
    total = sum(v.numel() * v.element_size() for v in sd.values())
    index = {"metadata": {"total_size": total}, "weight_map": weight_map}
    json.dump(index, open(os.path.join(directory, "model.safetensors.index.json"), "w"), indent=1)
    model.cfg.to_json(os.path.join(directory, "config.json"))
    return index


def load_safetensors(model: Any, directory: str, strict: bool = True) -> List[str]:
    from safetensors.torch import load_file
    index = json.load(open(os.path.join(directory, "model.safetensors.index.json")))
    sd: Dict[str, torch.Tensor] = {}
    for name in sorted(set(index["weight_map"].values())):
        sd.update(load_file(os.path.join(directory, name)))
    return model.load_reference_state_dict(sd, strict=strict)


def write_docker_context(directory: str, image_base: str = "nvcr.io/nvidia/pytorch:25.03-py3", port: int = 8000) -> str:
    """A Dockerfile that builds the sm_100a extension in the image and starts the OpenAI-compatible server."""
    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, "Dockerfile")
    with open(path, "w") as f:
        f.write(f"FROM {image_base}\nWORKDIR /app\nCOPY . /app\n"
                "RUN python -c \"import __graft_entry__ as g; g.build()\"\n"
                f"EXPOSE {port}\nCMD [\"python\", \"manage.py\", \"serve\", \"--port\", \"{port}\"]\n")
    return path


def model_card(model: Any, metrics: Optional[Dict[str, Any]] = None) -> str:
    c = model.cfg
    n = c.count_parameters()
    lines = [f"# Yv model ({n['total'] / 1e9:.2f} B parameters, {n.get('active', n['total']) / 1e9:.2f} B active)", "",
             f"* layers {c.n_layer}, hidden {c.hidden_size}, heads {c.n_head}/{c.n_kv_head}, vocab {c.vocab_size}",
             f"* experts {c.moe_num_experts} (top-{c.moe_top_k}), shared {c.moe_shared_experts}", ""]
    for k, v in (metrics or {}).items():
        lines.append(f"* {k}: {v}")
    return "\n".join(lines) + "\n"


class PiscesLxCacheManager:
    """Directory of downloaded / exported artefacts with size accounting and least-recently-used clean-up."""

    def __init__(self, root: str, max_bytes: int = 200 << 30):
        self.root, self.max_bytes = root, max_bytes
        os.makedirs(root, exist_ok=True)
        self.manifest_path = os.path.join(root, "manifest.json")
        self.manifest: Dict[str, Dict[str, Any]] = json.load(open(self.manifest_path)) if os.path.exists(self.manifest_path) else {}

    def _save(self) -> None:
        json.dump(self.manifest, open(self.manifest_path, "w"), indent=1)

    def path_for(self, key: str) -> str:
        return os.path.join(self.root, hashlib.sha256(key.encode()).hexdigest()[:16])

    def register(self, key: str, nbytes: int) -> str:
        self.manifest[key] = {"path": self.path_for(key), "bytes": nbytes, "last_use": time.time()}
        self._save()
        return self.manifest[key]["path"]

    def touch(self, key: str) -> Optional[str]:
        e = self.manifest.get(key)
        if e is None:
            return None
        e["last_use"] = time.time()
        self._save()
        return e["path"]

    def total_bytes(self) -> int:
        return sum(e["bytes"] for e in self.manifest.values())

    def cleanup(self) -> List[str]:
        removed = []
        for key, e in sorted(self.manifest.items(), key=lambda kv: kv[1]["last_use"]):
            if self.total_bytes() <= self.max_bytes:
                break
            removed.append(key)
            del self.manifest[key]
        self._save()
        return removed
