"""Publishing pipeline (reference tools/publish: exporter, Docker builder, registry, hub publisher, orchestrator,
runner, CLI and their config classes) on top of ``tools.publish``: export -> checksums -> metadata / model card ->
Docker context -> local registry entry.  Uploading to a hub needs a network, which this runtime does not have: the hub
publisher prepares the folder and returns what would be uploaded."""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import time
from dataclasses import asdict, dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional

from .publish import export_safetensors, model_card, write_docker_context


class PiscesLxExportFormat(str, Enum):
    SAFETENSORS = "safetensors"
    TORCH = "torch"


class PiscesLxExportAction(str, Enum):
    EXPORT = "export"
    DOCKER = "docker"
    REGISTER = "register"
    HUB = "hub"


@dataclass
class PiscesLxPublishModelExportConfig:
    format: PiscesLxExportFormat = PiscesLxExportFormat.SAFETENSORS
    max_shard_gb: float = 4.0


@dataclass
class PiscesLxPublishChecksumConfig:
    algorithm: str = "sha256"
    enabled: bool = True


@dataclass
class PiscesLxPublishMetadataConfig:
    name: str = "yv-model"
    version: str = "0.1.0"
    license: str = "apache-2.0"
    tags: List[str] = field(default_factory=list)


@dataclass
class PiscesLxPublishDockerConfig:
    enabled: bool = False
    image_base: str = "nvcr.io/nvidia/pytorch:25.03-py3"
    port: int = 8000


@dataclass
class PiscesLxPublishRegistryConfig:
    root: Optional[str] = None


@dataclass
class PiscesLxHubConfig:
    repo_id: str = ""
    private: bool = True


@dataclass
class PiscesLxPublishConfig:
    output_dir: str = "publish_out"
    export: PiscesLxPublishModelExportConfig = field(default_factory=PiscesLxPublishModelExportConfig)
    checksum: PiscesLxPublishChecksumConfig = field(default_factory=PiscesLxPublishChecksumConfig)
    metadata: PiscesLxPublishMetadataConfig = field(default_factory=PiscesLxPublishMetadataConfig)
    docker: PiscesLxPublishDockerConfig = field(default_factory=PiscesLxPublishDockerConfig)
    registry: PiscesLxPublishRegistryConfig = field(default_factory=PiscesLxPublishRegistryConfig)
    hub: PiscesLxHubConfig = field(default_factory=PiscesLxHubConfig)


def file_checksums(directory: str, algorithm: str = "sha256") -> Dict[str, str]:
    out = {}
    for n in sorted(os.listdir(directory)):
        p = os.path.join(directory, n)
        if os.path.isfile(p) and n != "checksums.json":
            h = hashlib.new(algorithm)
            with open(p, "rb") as f:
                for chunk in iter(lambda: f.read(1 << 20), b""):
                    h.update(chunk)
            out[n] = h.hexdigest()
    return out


class PiscesLxPublishExporter:
    def __init__(self, config: PiscesLxPublishConfig):
        self.config = config

    def export(self, model: Any, metrics: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        c, d = self.config, self.config.output_dir
        os.makedirs(d, exist_ok=True)
        if c.export.format == PiscesLxExportFormat.SAFETENSORS:
            index = export_safetensors(model, d, int(c.export.max_shard_gb * 2 ** 30))
            files = sorted(set(index["weight_map"].values()))
        else:
            import torch
            torch.save(model.to_reference_state_dict(), os.path.join(d, "pytorch_model.bin"))
            model.cfg.to_json(os.path.join(d, "config.json"))
            files = ["pytorch_model.bin"]
        with open(os.path.join(d, "README.md"), "w") as f:
            f.write(model_card(model, metrics))
        meta = {**asdict(c.metadata), "format": c.export.format.value, "created": time.time(), "weight_files": files}
        json.dump(meta, open(os.path.join(d, "metadata.json"), "w"), indent=1)
        if c.checksum.enabled:
            json.dump({"algorithm": c.checksum.algorithm, "files": file_checksums(d, c.checksum.algorithm)},
                      open(os.path.join(d, "checksums.json"), "w"), indent=1)
        return meta

    @staticmethod
    def verify(directory: str) -> List[str]:
        """File names whose checksum no longer matches (empty = intact)."""
        rec = json.load(open(os.path.join(directory, "checksums.json")))
        now = file_checksums(directory, rec["algorithm"])
        return sorted(n for n, h in rec["files"].items() if now.get(n) != h)


class PiscesLxPublishDockerBuilder:
    def __init__(self, config: PiscesLxPublishDockerConfig):
        self.config = config

    def write_context(self, directory: str) -> str:
        return write_docker_context(directory, self.config.image_base, self.config.port)


class PiscesLxPublishRegistry:
    """Local registry: ``<root>/<name>/<version>/`` holds a copy of the published folder; ``index.json`` lists them."""

    def __init__(self, root: str):
        self.root = root
        os.makedirs(root, exist_ok=True)

    def _index_path(self) -> str:
        return os.path.join(self.root, "index.json")

    def entries(self) -> List[Dict[str, Any]]:
        return json.load(open(self._index_path())) if os.path.exists(self._index_path()) else []

    def register(self, directory: str, name: str, version: str) -> str:
        dst = os.path.join(self.root, name, version)
        if os.path.exists(dst):
            raise FileExistsError(f"{name} {version} is already registered")
        shutil.copytree(directory, dst)
        idx = self.entries() + [{"name": name, "version": version, "path": dst, "registered": time.time()}]
        json.dump(idx, open(self._index_path(), "w"), indent=1)
        return dst

    def resolve(self, name: str, version: Optional[str] = None) -> Optional[str]:
        cands = [e for e in self.entries() if e["name"] == name and (version is None or e["version"] == version)]
        return max(cands, key=lambda e: e["registered"])["path"] if cands else None


class PiscesLxModelHubPublisher:
    def __init__(self, config: PiscesLxHubConfig):
        self.config = config

    def prepare(self, directory: str) -> Dict[str, Any]:
        files = sorted(n for n in os.listdir(directory) if os.path.isfile(os.path.join(directory, n)))
        return {"repo_id": self.config.repo_id, "private": self.config.private, "files": files,
                "bytes": sum(os.path.getsize(os.path.join(directory, n)) for n in files), "uploaded": False,
                "reason": "offline runtime: nothing was uploaded; push this folder from a machine with network access"}


class PiscesLxPublishOrchestrator:
    """export -> (docker) -> (register) -> (hub), as the config enables them; returns one report."""

    def __init__(self, config: Optional[PiscesLxPublishConfig] = None):
        self.config = config or PiscesLxPublishConfig()

    def run(self, model: Any, metrics: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        c = self.config
        report: Dict[str, Any] = {"actions": [PiscesLxExportAction.EXPORT.value]}
        report["metadata"] = PiscesLxPublishExporter(c).export(model, metrics)
        if c.docker.enabled:
            report["dockerfile"] = PiscesLxPublishDockerBuilder(c.docker).write_context(c.output_dir)
            report["actions"].append(PiscesLxExportAction.DOCKER.value)
        if c.registry.root:
            report["registered"] = PiscesLxPublishRegistry(c.registry.root).register(c.output_dir, c.metadata.name, c.metadata.version)
            report["actions"].append(PiscesLxExportAction.REGISTER.value)
        if c.hub.repo_id:
            report["hub"] = PiscesLxModelHubPublisher(c.hub).prepare(c.output_dir)
            report["actions"].append(PiscesLxExportAction.HUB.value)
        return report


PiscesLxPublishRunner = PiscesLxToolsPublish = PiscesLxPublishOrchestrator


class PiscesLxPublishCli:
    """``manage.py publish --ckpt … --out … [--docker] [--registry DIR] [--name N --version V]``."""

    def run(self, args: Any, load_model) -> int:
        cfg = PiscesLxPublishConfig(output_dir=getattr(args, "out", None) or "publish_out")
        cfg.docker.enabled = bool(getattr(args, "docker", False))
        cfg.registry.root = getattr(args, "registry", None)
        cfg.metadata.name = getattr(args, "name", None) or cfg.metadata.name
        cfg.metadata.version = getattr(args, "version", None) or cfg.metadata.version
        print(json.dumps(PiscesLxPublishOrchestrator(cfg).run(load_model()), indent=1, default=str))
        return 0
