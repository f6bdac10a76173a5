"""Directory layout of a working tree: ``$PISCESLX_HOME`` (default ``.pisceslx``) with ``ckpt/``, ``runs/``,
``logs/`` and ``cache/`` below it (reference utils/paths.py: ``PiscesLxPaths``)."""
from __future__ import annotations

import os
import shutil
from pathlib import Path
from typing import Dict, Optional


def _home() -> Path:
    return Path(os.environ.get("PISCESLX_HOME", ".pisceslx"))


class PiscesLxPaths:
    def __init__(self, home: Optional[Path] = None):
        self.home = Path(home) if home else _home()

    def logs(self, name: str = "default") -> Path:
        p = self.home / "logs" / name
        p.mkdir(parents=True, exist_ok=True)
        return p

    def ckpt(self) -> Path:
        return self.home / "ckpt"

    def runs(self) -> Path:
        return self.home / "runs"

    def cache(self) -> Path:
        p = self.home / "cache"
        p.mkdir(parents=True, exist_ok=True)
        return p

    def describe(self) -> Dict[str, str]:
        return {"home": str(self.home), "ckpt": str(self.ckpt()), "runs": str(self.runs()), "cache": str(self.cache())}

    def clear_cache(self) -> int:
        c = self.cache()
        n = sum(1 for _ in c.rglob("*") if _.is_file())
        shutil.rmtree(c, ignore_errors=True)
        return n
