"""CPU test of the publishing pipeline: export, checksums, Docker context, local registry, hub preparation."""
from __future__ import annotations

import json
import os

import pytest
import torch

from pisceslx_b200 import YvConfig
from pisceslx_b200.models import build_model
from pisceslx_b200.tools.publish import load_safetensors
from pisceslx_b200.tools.publish_pipeline import (PiscesLxExportFormat, PiscesLxPublishConfig, PiscesLxPublishExporter,
                                                  PiscesLxPublishOrchestrator, PiscesLxPublishRegistry)


def test_publish_orchestrator_end_to_end(tmp_path):
    cfg = YvConfig.tiny_text_moe(vocab_size=128)
    cfg.n_layer = 1
    m = build_model(cfg)
    pc = PiscesLxPublishConfig(output_dir=str(tmp_path / "out"))
    pc.docker.enabled, pc.registry.root, pc.hub.repo_id = True, str(tmp_path / "registry"), "org/yv-tiny"
    pc.metadata.name, pc.metadata.version = "yv-tiny", "1.0.0"
    rep = PiscesLxPublishOrchestrator(pc).run(m, {"loss": 1.23})
    assert rep["actions"] == ["export", "docker", "register", "hub"]
    out = tmp_path / "out"
    for n in ("config.json", "metadata.json", "checksums.json", "README.md", "Dockerfile", "model.safetensors.index.json"):
        assert (out / n).exists(), n
    assert "loss: 1.23" in (out / "README.md").read_text() and rep["hub"]["uploaded"] is False
    assert PiscesLxPublishExporter.verify(str(out)) == ["Dockerfile"] or PiscesLxPublishExporter.verify(str(out)) == []
    # the registered copy loads back into a fresh model, bit for bit
    reg = PiscesLxPublishRegistry(pc.registry.root)
    path = reg.resolve("yv-tiny")
    assert path and path.endswith(os.path.join("yv-tiny", "1.0.0")) and reg.resolve("other") is None
    m2 = build_model(cfg, seed=99)
    load_safetensors(m2, path)
    ids = torch.randint(0, 128, (1, 8))
    assert torch.equal(m(input_ids=ids).logits, m2(input_ids=ids).logits)
    with pytest.raises(FileExistsError):
        reg.register(str(out), "yv-tiny", "1.0.0")
    # tampering is detected
    weight = next(n for n in os.listdir(out) if n.endswith(".safetensors"))
    with open(out / weight, "ab") as f:
        f.write(b"x")
    assert weight in PiscesLxPublishExporter.verify(str(out))
    pt = PiscesLxPublishConfig(output_dir=str(tmp_path / "pt"))
    pt.export.format = PiscesLxExportFormat.TORCH
    meta = PiscesLxPublishExporter(pt).export(m)
    assert meta["weight_files"] == ["pytorch_model.bin"] and json.load(open(tmp_path / "pt" / "metadata.json"))["format"] == "torch"
