"""Datasets, collation and loaders.

``PiscesLxToolsDataTextCollator`` reproduces the reference batch format (tools/data/dataset/raw_text.py:220-356):
``{input_ids, attention_mask, labels}`` with label ``-100`` on padding; *pack* mode concatenates all ids, cuts
fixed ``seq_len`` rows and pads the tail; SFT pairs mask the prompt.  Datasets: synthetic uniform token ids (the
benchmark data), raw text / JSONL files, memory-mapped token arrays, a streaming iterable over sharded files, and a
preference-pair dataset for DPO-style stages.  Samplers: distributed (rank-strided), dynamic-length batching and a
curriculum sampler (easy -> hard by length)."""
from __future__ import annotations

import json
import math
import os
import random
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, IterableDataset, Sampler

from ..models.tokenizer import YvTokenizer


class SyntheticTokenDataset(IterableDataset):
    """Endless stream of uniform-random token ids of shape [batch, seq_len]."""

    def __init__(self, vocab_size: int, seq_len: int, batch: int, seed: int = 0, pin: bool = False):
        self.vocab, self.seq_len, self.batch, self.seed, self.pin = vocab_size, seq_len, batch, seed, pin

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        g = torch.Generator().manual_seed(self.seed)
        while True:
            ids = torch.randint(0, self.vocab, (self.batch, self.seq_len), generator=g, dtype=torch.int64)
            if self.pin and torch.cuda.is_available():
                ids = ids.pin_memory()
            yield {"input_ids": ids, "labels": ids}


class PiscesLxToolsDataRawTextDataset(Dataset):
    """One sample per line (``.txt``) or per JSON object with a text field (``.jsonl``)."""

    def __init__(self, path: str, text_field: str = "text", tokenizer: Optional[YvTokenizer] = None):
        self.tok = tokenizer or YvTokenizer.instance()
        self.samples: List[str] = []
        p = Path(path)
        files = sorted(p.glob("*")) if p.is_dir() else [p]
        for f in files:
            if f.suffix == ".jsonl":
                for line in f.read_text().splitlines():
                    if line.strip():
                        self.samples.append(str(json.loads(line).get(text_field, "")))
            elif f.suffix in (".txt", ".md"):
                self.samples += [l for l in f.read_text().splitlines() if l.strip()]

    def __len__(self) -> int:
        return len(self.samples)

    def __getitem__(self, i: int) -> Dict[str, List[int]]:
        return {"input_ids": self.tok.encode(self.samples[i], add_eos=True)}


class PiscesLxToolsDataSupervisedDataset(Dataset):
    """Prompt / response pairs; the collator masks the prompt tokens out of the loss."""

    def __init__(self, records: Sequence[Dict[str, str]], tokenizer: Optional[YvTokenizer] = None):
        self.records, self.tok = list(records), tokenizer or YvTokenizer.instance()

    def __len__(self) -> int:
        return len(self.records)

    def __getitem__(self, i: int) -> Dict[str, Any]:
        r = self.records[i]
        p = self.tok.encode(r.get("prompt", ""))
        a = self.tok.encode(r.get("response", ""), add_eos=True)
        return {"input_ids": p + a, "prompt_len": len(p)}


class PiscesLxToolsDataPreferenceDataset(Dataset):
    def __init__(self, records: Sequence[Dict[str, str]], tokenizer: Optional[YvTokenizer] = None):
        self.records, self.tok = list(records), tokenizer or YvTokenizer.instance()

    def __len__(self) -> int:
        return len(self.records)

    def __getitem__(self, i: int) -> Dict[str, Any]:
        r = self.records[i]
        p = self.tok.encode(r["prompt"])
        return {"prompt_len": len(p), "chosen": p + self.tok.encode(r["chosen"], add_eos=True),
                "rejected": p + self.tok.encode(r["rejected"], add_eos=True)}


class PiscesLxDataMemoryMappedArray(Dataset):
    """Token ids stored as one flat ``uint32`` file; sample i = ids[i*seq_len : (i+1)*seq_len]."""

    def __init__(self, path: str, seq_len: int):
        self.arr = np.memmap(path, dtype=np.uint32, mode="r")
        self.seq_len = seq_len

    @staticmethod
    def write(path: str, ids: Iterable[int]) -> None:
        np.asarray(list(ids), dtype=np.uint32).tofile(path)

    def __len__(self) -> int:
        return len(self.arr) // self.seq_len

    def __getitem__(self, i: int) -> Dict[str, List[int]]:
        return {"input_ids": self.arr[i * self.seq_len:(i + 1) * self.seq_len].astype(np.int64).tolist()}


class PiscesLxToolsDataLargeScaleStreamingDataset(IterableDataset):
    """Round-robins over shard files, keeping one shard in memory at a time."""

    def __init__(self, shards: Sequence[str], text_field: str = "text", tokenizer: Optional[YvTokenizer] = None,
                 rank: int = 0, world: int = 1):
        self.shards, self.field, self.tok = list(shards)[rank::world], text_field, tokenizer or YvTokenizer.instance()

    def __iter__(self) -> Iterator[Dict[str, List[int]]]:
        for s in self.shards:
            for rec in PiscesLxToolsDataRawTextDataset(s, self.field, self.tok).samples:
                yield {"input_ids": self.tok.encode(rec, add_eos=True)}


class PiscesLxToolsDataTextCollator:
    def __init__(self, seq_len: int, pad_id: int = 0, pack: bool = False, mask_prompt: bool = True):
        self.seq_len, self.pad_id, self.pack, self.mask_prompt = seq_len, pad_id, pack, mask_prompt

    def __call__(self, samples: List[Dict[str, Any]]) -> Dict[str, torch.Tensor]:
        if self.pack:
            flat: List[int] = []
            for s in samples:
                flat += list(s["input_ids"])
            rows = [flat[i:i + self.seq_len] for i in range(0, max(len(flat), 1), self.seq_len)]
        else:
            rows = [list(s["input_ids"])[: self.seq_len] for s in samples]
        L = self.seq_len if self.pack else max(len(r) for r in rows)
        ids = torch.full((len(rows), L), self.pad_id, dtype=torch.long)
        mask = torch.zeros(len(rows), L, dtype=torch.long)
        labels = torch.full((len(rows), L), -100, dtype=torch.long)
        for i, r in enumerate(rows):
            n = len(r)
            ids[i, :n] = torch.tensor(r, dtype=torch.long)
            mask[i, :n] = 1
            labels[i, :n] = ids[i, :n]
            if not self.pack and self.mask_prompt and "prompt_len" in samples[i]:
                labels[i, : min(samples[i]["prompt_len"], n)] = -100
        return {"input_ids": ids, "attention_mask": mask, "labels": labels}


class PiscesLxToolsDataDistributedSampler(Sampler):
    def __init__(self, n: int, rank: int = 0, world: int = 1, shuffle: bool = True, seed: int = 0):
        self.n, self.rank, self.world, self.shuffle, self.seed, self.epoch = n, rank, world, shuffle, seed, 0

    def set_epoch(self, e: int) -> None:
        self.epoch = e

    def __iter__(self) -> Iterator[int]:
        idx = list(range(self.n))
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(idx)
        per = math.ceil(self.n / self.world)
        idx += idx[: per * self.world - self.n]
        return iter(idx[self.rank::self.world])

    def __len__(self) -> int:
        return math.ceil(self.n / self.world)


class PiscesLxDynamicBatchSampler(Sampler):
    """Batches of similar length bounded by a token budget."""

    def __init__(self, lengths: Sequence[int], max_tokens: int, shuffle: bool = True, seed: int = 0):
        self.lengths, self.max_tokens, self.shuffle, self.seed = list(lengths), max_tokens, shuffle, seed

    def __iter__(self) -> Iterator[List[int]]:
        order = sorted(range(len(self.lengths)), key=lambda i: self.lengths[i])
        batches, cur, mx = [], [], 0
        for i in order:
            mx2 = max(mx, self.lengths[i])
            if cur and mx2 * (len(cur) + 1) > self.max_tokens:
                batches.append(cur)
                cur, mx2 = [], self.lengths[i]
            cur.append(i)
            mx = mx2
        if cur:
            batches.append(cur)
        if self.shuffle:
            random.Random(self.seed).shuffle(batches)
        return iter(batches)

    def __len__(self) -> int:
        return sum(1 for _ in self.__iter__())


class PiscesLxCurriculumSampler(Sampler):
    """Feeds the shortest fraction of the data first; the admitted fraction grows linearly with the epoch."""

    def __init__(self, lengths: Sequence[int], epochs_to_full: int = 4, seed: int = 0):
        self.order = sorted(range(len(lengths)), key=lambda i: lengths[i])
        self.epochs_to_full, self.seed, self.epoch = max(1, epochs_to_full), seed, 0

    def set_epoch(self, e: int) -> None:
        self.epoch = e

    def __iter__(self) -> Iterator[int]:
        frac = min(1.0, (self.epoch + 1) / self.epochs_to_full)
        idx = self.order[: max(1, int(len(self.order) * frac))]
        random.Random(self.seed + self.epoch).shuffle(idx)
        return iter(idx)

    def __len__(self) -> int:
        return len(self.order)


def build_dataloader(dataset: str, vocab_size: int, seq_len: int, batch: int, seed: int = 0, rank: int = 0,
                     world: int = 1, pack: bool = True) -> Iterable[Dict[str, torch.Tensor]]:
    if dataset in ("synthetic", None, ""):
        return SyntheticTokenDataset(vocab_size, seq_len, batch, seed)
    ds = PiscesLxToolsDataRawTextDataset(dataset)
    if len(ds) == 0:
        raise FileNotFoundError(f"no samples found under {dataset!r}")
    sampler = PiscesLxToolsDataDistributedSampler(len(ds), rank, world, seed=seed)
    col = PiscesLxToolsDataTextCollator(seq_len, pack=pack)

    def clamp(b: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        b["input_ids"].clamp_(0, vocab_size - 1)
        b["labels"] = torch.where(b["labels"] >= vocab_size, torch.full_like(b["labels"], -100), b["labels"])
        return b

    def gen() -> Iterator[Dict[str, torch.Tensor]]:
        epoch = 0
        while True:
            sampler.set_epoch(epoch)
            for b in DataLoader(ds, batch_size=batch, sampler=sampler, collate_fn=col):
                yield clamp(b)
            epoch += 1

    return gen()
