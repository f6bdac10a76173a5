"""Data augmentation, sample caches, offline teacher records and dataset resolution (reference tools/data/augment,
tools/data/cache (mmap / LRU caches), tools/data/distill (offline teacher providers), tools/data/download (hub
clients)).  There is no network access at run time in this framework's target deployment: ``resolve_dataset`` maps
a hub-style name to a local directory and says exactly what is missing instead of trying to fetch it."""
from __future__ import annotations

import hashlib
import json
import os
import random
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch


# ------------------------------------------------------------------------------------------------ augmentation
class PiscesLxTokenAugmenter:
    """Token-level augmentation for language-model pre-training batches; labels of touched positions can be masked
    out (-100) so that the model is not trained to predict noise."""

    def __init__(self, vocab_size: int, mask_token_id: Optional[int] = None, seed: int = 0):
        self.vocab, self.mask_id, self.rng = vocab_size, mask_token_id, random.Random(seed)

    def token_dropout(self, ids: List[int], p: float) -> List[int]:
        out = [t for t in ids if self.rng.random() >= p]
        return out or ids[:1]

    def random_replace(self, ids: List[int], p: float) -> Tuple[List[int], List[int]]:
        out, labels = list(ids), list(ids)
        for i in range(len(out)):
            if self.rng.random() < p:
                out[i] = self.rng.randrange(self.vocab)
                labels[i] = -100
        return out, labels

    def span_mask(self, ids: List[int], ratio: float = 0.15, mean_span: int = 3) -> Tuple[List[int], List[int]]:
        """T5-style span corruption in place: spans are replaced by the mask token; labels keep the originals there
        and -100 elsewhere."""
        assert self.mask_id is not None
        n, out, labels = len(ids), list(ids), [-100] * len(ids)
        budget, i = int(round(n * ratio)), 0
        while budget > 0 and i < n:
            if self.rng.random() < ratio / max(mean_span, 1) * 2:
                span = min(budget, max(1, int(self.rng.expovariate(1.0 / mean_span))), n - i)
                for j in range(i, i + span):
                    labels[j], out[j] = ids[j], self.mask_id
                budget -= span
                i += span
            i += 1
        return out, labels

    def swap_adjacent(self, ids: List[int], p: float) -> List[int]:
        out, i = list(ids), 0
        while i < len(out) - 1:
            if self.rng.random() < p:
                out[i], out[i + 1] = out[i + 1], out[i]
                i += 1
            i += 1
        return out


class PiscesLxTextAugmenter:
    """Character / word level text augmentation used for robustness fine-tuning sets."""

    def __init__(self, seed: int = 0):
        self.rng = random.Random(seed)

    def word_dropout(self, text: str, p: float) -> str:
        w = text.split()
        kept = [x for x in w if self.rng.random() >= p]
        return " ".join(kept or w[:1])

    def typo(self, text: str, p: float) -> str:
        c = list(text)
        for i in range(len(c) - 1):
            if c[i].isalpha() and c[i + 1].isalpha() and self.rng.random() < p:
                c[i], c[i + 1] = c[i + 1], c[i]
        return "".join(c)

    def template(self, sample: Dict[str, str], templates: Sequence[str]) -> str:
        return self.rng.choice(list(templates)).format(**sample)


# ------------------------------------------------------------------------------------------------ caches
class PiscesLxDataLRUCache:
    """Byte-bounded LRU cache of tokenised samples."""

    def __init__(self, max_bytes: int = 1 << 30):
        self.max_bytes, self.bytes = max_bytes, 0
        self.d: "OrderedDict[Any, np.ndarray]" = OrderedDict()
        self.hits = self.misses = 0

    def get(self, key: Any, make: Callable[[], np.ndarray]) -> np.ndarray:
        if key in self.d:
            self.d.move_to_end(key)
            self.hits += 1
            return self.d[key]
        self.misses += 1
        v = np.asarray(make())
        self.d[key] = v
        self.bytes += v.nbytes
        while self.bytes > self.max_bytes and len(self.d) > 1:
            _, old = self.d.popitem(last=False)
            self.bytes -= old.nbytes
        return v


class PiscesLxDataTokenCache:
    """On-disk cache of tokenised corpora: one flat ``.bin`` of token ids plus an ``.idx.json`` with document
    offsets, keyed by a hash of (source file identity, tokenizer name); reopened with ``np.memmap``."""

    def __init__(self, root: str):
        self.root = root
        os.makedirs(root, exist_ok=True)

    @staticmethod
    def key(path: str, tokenizer_name: str) -> str:
        st = os.stat(path)
        return hashlib.sha1(f"{os.path.abspath(path)}|{st.st_size}|{int(st.st_mtime)}|{tokenizer_name}".encode()).hexdigest()[:20]

    def build(self, key: str, docs: Iterable[Sequence[int]], dtype=np.int32) -> Tuple[np.memmap, List[int]]:
        binp, idxp = os.path.join(self.root, key + ".bin"), os.path.join(self.root, key + ".idx.json")
        offsets = [0]
        with open(binp + ".tmp", "wb") as f:
            for d in docs:
                a = np.asarray(d, dtype=dtype)
                a.tofile(f)
                offsets.append(offsets[-1] + len(a))
        os.replace(binp + ".tmp", binp)
        with open(idxp, "w") as f:
            json.dump({"dtype": np.dtype(dtype).name, "offsets": offsets}, f)
        return self.open(key)

    def open(self, key: str) -> Optional[Tuple[np.memmap, List[int]]]:
        binp, idxp = os.path.join(self.root, key + ".bin"), os.path.join(self.root, key + ".idx.json")
        if not (os.path.exists(binp) and os.path.exists(idxp)):
            return None
        with open(idxp) as f:
            meta = json.load(f)
        if meta["offsets"][-1] == 0:
            return np.zeros(0, dtype=meta["dtype"]), meta["offsets"]          # type: ignore[return-value]
        return np.memmap(binp, dtype=meta["dtype"], mode="r"), meta["offsets"]


# ------------------------------------------------------------------------------------------------ offline teachers
@dataclass
class PiscesLxTeacherRecord:
    input_ids: List[int]
    topk_ids: List[List[int]]        # per position, the teacher's k most likely next tokens
    topk_logprobs: List[List[float]]


class PiscesLxOfflineTeacherProvider:
    """Distillation targets computed once and stored: JSONL of per-position top-k teacher log-probabilities.
    ``record`` writes them from a teacher model; ``sparse_kl`` is the student's loss against a stored record."""

    def __init__(self, path: str, k: int = 8):
        self.path, self.k = path, k

    @torch.no_grad()
    def record(self, teacher: Any, batches: Iterable[torch.Tensor]) -> int:
        n = 0
        with open(self.path, "a") as f:
            for ids in batches:
                lp = torch.log_softmax(teacher(input_ids=ids).logits.float(), -1)
                v, i = lp.topk(self.k, -1)
                for b in range(ids.shape[0]):
                    f.write(json.dumps({"input_ids": ids[b].tolist(), "topk_ids": i[b].tolist(),
                                        "topk_logprobs": [[round(x, 5) for x in row] for row in v[b].tolist()]}) + "\n")
                    n += 1
        return n

    def __iter__(self) -> Iterator[PiscesLxTeacherRecord]:
        with open(self.path) as f:
            for line in f:
                yield PiscesLxTeacherRecord(**json.loads(line))

    @staticmethod
    def sparse_kl(student_logits: torch.Tensor, rec: PiscesLxTeacherRecord) -> torch.Tensor:
        """KL(teacher_topk || student) with the teacher's mass renormalised over its stored top-k."""
        ids = torch.tensor(rec.topk_ids, device=student_logits.device)
        t = torch.softmax(torch.tensor(rec.topk_logprobs, device=student_logits.device), -1)
        s = torch.log_softmax(student_logits.float(), -1).gather(-1, ids)
        s = s - torch.logsumexp(s, -1, keepdim=True)
        return (t * (torch.log(t.clamp_min(1e-12)) - s)).sum(-1).mean()


# ------------------------------------------------------------------------------------------------ dataset resolution
class PiscesLxDatasetUnavailable(FileNotFoundError):
    pass


def resolve_dataset(name: str, roots: Optional[Sequence[str]] = None) -> str:
    """Maps ``org/name`` (hub style) or a plain name to a local directory under one of ``roots`` (default:
    ``$PISCESLX_DATA``, ``./data``).  Raises with the list of places searched; nothing is downloaded."""
    roots = list(roots) if roots else [r for r in (os.environ.get("PISCESLX_DATA"), "data") if r]
    tried = []
    for r in roots:
        for cand in (name, name.replace("/", "__"), name.split("/")[-1]):
            p = os.path.join(r, cand)
            tried.append(p)
            if os.path.isdir(p) or os.path.isfile(p):
                return p
    raise PiscesLxDatasetUnavailable(
        f"dataset {name!r} is not available offline; looked in: {', '.join(tried)}. Copy it there (any of jsonl / txt / "
        f"parquet / bin+idx) and re-run.")


PiscesLxDataTextAugmenter = PiscesLxTextAugmenter                         # the reference names it by its folder (tools/data/augment/text_aug.py)
