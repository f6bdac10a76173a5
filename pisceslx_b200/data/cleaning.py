"""Text cleaning, quality scoring and de-duplication (reference ``tools/data/clean``, ``tools/data/dedup``,
``tools/data/lineage``): rule-based cleaner, heuristic quality metrics, exact (hash) and MinHash near-duplicate
removal, and a lineage tracker that records which transformation produced which file."""
from __future__ import annotations

import hashlib
import json
import re
import time
import unicodedata
from dataclasses import asdict, dataclass, field
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Set, Tuple

_WS = re.compile(r"[ \t ]+")
_CTRL = re.compile(r"[\x00-\x08\x0b\x0c\x0e-\x1f\x7f]")
_URL = re.compile(r"https?://\S+")


class PiscesLxDatasetCleaner:
    def __init__(self, min_chars: int = 20, max_chars: int = 200_000, strip_urls: bool = False,
                 max_symbol_ratio: float = 0.4, max_repeat_line_ratio: float = 0.5):
        self.min_chars, self.max_chars, self.strip_urls = min_chars, max_chars, strip_urls
        self.max_symbol_ratio, self.max_repeat_line_ratio = max_symbol_ratio, max_repeat_line_ratio

    def normalise(self, text: str) -> str:
        text = unicodedata.normalize("NFC", text)
        text = _CTRL.sub("", text)
        if self.strip_urls:
            text = _URL.sub("", text)
        return "\n".join(_WS.sub(" ", ln).strip() for ln in text.splitlines()).strip()

    def keep(self, text: str) -> bool:
        n = len(text)
        if n < self.min_chars or n > self.max_chars:
            return False
        sym = sum(1 for c in text if not (c.isalnum() or c.isspace()))
        if sym / n > self.max_symbol_ratio:
            return False
        lines = [l for l in text.splitlines() if l]
        if len(lines) >= 4 and 1 - len(set(lines)) / len(lines) > self.max_repeat_line_ratio:
            return False
        return True

    def clean(self, texts: Iterable[str]) -> Iterator[str]:
        for t in texts:
            t = self.normalise(t)
            if self.keep(t):
                yield t


@dataclass
class PiscesLxDataQualityMetrics:
    chars: int
    words: int
    mean_word_len: float
    alpha_ratio: float
    unique_word_ratio: float
    score: float


class PiscesLxToolsDataQualityController:
    def score(self, text: str) -> PiscesLxDataQualityMetrics:
        words = text.split()
        n = max(len(text), 1)
        alpha = sum(c.isalpha() for c in text) / n
        uniq = len(set(words)) / max(len(words), 1)
        mwl = sum(map(len, words)) / max(len(words), 1)
        score = 0.4 * min(alpha / 0.8, 1.0) + 0.4 * min(uniq / 0.5, 1.0) + 0.2 * (1.0 if 3 <= mwl <= 10 else 0.3)
        return PiscesLxDataQualityMetrics(len(text), len(words), mwl, alpha, uniq, score)

    def filter(self, texts: Iterable[str], threshold: float = 0.5) -> Iterator[str]:
        return (t for t in texts if self.score(t).score >= threshold)


class PiscesLxDataExactDeduplicator:
    def __init__(self):
        self.seen: Set[str] = set()

    def is_new(self, text: str) -> bool:
        h = hashlib.sha1(text.encode("utf-8")).hexdigest()
        if h in self.seen:
            return False
        self.seen.add(h)
        return True

    def dedup(self, texts: Iterable[str]) -> Iterator[str]:
        return (t for t in texts if self.is_new(t))


class PiscesLxDataMinHashDeduplicator:
    """MinHash over word shingles with LSH banding."""

    def __init__(self, num_perm: int = 64, bands: int = 16, shingle: int = 5, threshold: float = 0.8):
        assert num_perm % bands == 0
        self.num_perm, self.bands, self.rows, self.shingle, self.threshold = num_perm, bands, num_perm // bands, shingle, threshold
        self.buckets: List[Dict[Tuple[int, ...], List[int]]] = [dict() for _ in range(bands)]
        self.sigs: List[Tuple[int, ...]] = []
        self._salts = [int(hashlib.md5(str(i).encode()).hexdigest()[:8], 16) for i in range(num_perm)]

    def signature(self, text: str) -> Tuple[int, ...]:
        w = text.split()
        sh = {" ".join(w[i:i + self.shingle]) for i in range(max(1, len(w) - self.shingle + 1))}
        hs = [int(hashlib.md5(s.encode()).hexdigest()[:8], 16) for s in sh] or [0]
        return tuple(min((h ^ salt) * 2654435761 % (1 << 32) for h in hs) for salt in self._salts)

    def is_new(self, text: str) -> bool:
        sig = self.signature(text)
        cands: Set[int] = set()
        for b in range(self.bands):
            cands.update(self.buckets[b].get(sig[b * self.rows:(b + 1) * self.rows], []))
        for c in cands:
            if sum(a == b for a, b in zip(sig, self.sigs[c])) / self.num_perm >= self.threshold:
                return False
        idx = len(self.sigs)
        self.sigs.append(sig)
        for b in range(self.bands):
            self.buckets[b].setdefault(sig[b * self.rows:(b + 1) * self.rows], []).append(idx)
        return True

    def dedup(self, texts: Iterable[str]) -> Iterator[str]:
        return (t for t in texts if self.is_new(t))


@dataclass
class PiscesLxDataLineageRecord:
    output: str
    inputs: List[str]
    operation: str
    params: Dict[str, object] = field(default_factory=dict)
    ts: float = field(default_factory=time.time)


class PiscesLxDataLineageTracker:
    def __init__(self, path: Optional[str] = None):
        self.path, self.records = path, []

    def record(self, output: str, inputs: Sequence[str], operation: str, **params: object) -> None:
        rec = PiscesLxDataLineageRecord(output, list(inputs), operation, dict(params))
        self.records.append(rec)
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(asdict(rec)) + "\n")

    def ancestors(self, output: str) -> List[str]:
        out, todo = [], [output]
        while todo:
            cur = todo.pop()
            for r in self.records:
                if r.output == cur:
                    for i in r.inputs:
                        if i not in out:
                            out.append(i)
                            todo.append(i)
        return out
