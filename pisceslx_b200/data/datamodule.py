"""Data module layer: source configuration, datasets over mixed sources (text, image-text, conversation, preference),
streaming, loaders with dynamic / curriculum / distributed sampling and prefetch, bounded buffers and memory monitors
(reference tools/data/datamodule.py:63-800, tools/data/dataset/loader.py:36-460, core.py:73-490, memory.py:33-180,
raw_text.py:71-460).

What is shaped by the device: batches are padded to a multiple of 64 tokens; a prefetched loader stages every batch in
pinned memory and copies it on a side stream (``data.prefetch.PiscesLxPrefetchLoader``), so the step that consumes it only
waits on an event; image tensors are produced in channels-first float16 already normalised, so that no per-step
conversion kernel runs on the training stream."""
from __future__ import annotations

import json
import math
import os
import queue
import random
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple, Union

import torch
from torch.utils.data import DataLoader, Dataset, IterableDataset, Sampler

from .datasets import PiscesLxToolsDataDistributedSampler
from .prefetch import PiscesLxPrefetchLoader

PAD_MULTIPLE = 64
TEXT_KEYS = ("text", "content", "body", "document", "passage", "output", "response", "answer")


# ---- records --------------------------------------------------------------------------------------------------------------------
class PiscesLxToolsDataJsonSampleReader:
    """Samples from ``.jsonl`` / ``.json`` / ``.txt`` files and folders of them.  A file that cannot be read is recorded in
    ``failures`` (path, error) and skipped; it does not end the scan."""

    failures: List[Tuple[str, str]] = []

    @staticmethod
    def extract_text(item: Any) -> str:
        if isinstance(item, str):
            return item
        if not isinstance(item, dict):
            return ""
        if "instruction" in item:
            return "\n".join(str(item[k]) for k in ("instruction", "input", "output") if item.get(k))
        if "prompt" in item:
            return "\n".join(str(item[k]) for k in ("prompt", "response", "completion", "chosen") if item.get(k))
        msgs = item.get("messages") or item.get("conversations")
        if isinstance(msgs, list):
            return "\n".join(str(m.get("content", m.get("value", ""))) for m in msgs if isinstance(m, dict))
        for k in TEXT_KEYS:
            v = item.get(k)
            if isinstance(v, str) and v.strip():
                return v
        return ""

    @classmethod
    def load_samples(cls, file_path: str) -> List[Dict[str, Any]]:
        p = Path(file_path)
        try:
            if p.suffix == ".jsonl":
                return [json.loads(l) for l in p.read_text(encoding="utf-8").splitlines() if l.strip()]
            if p.suffix == ".json":
                d = json.loads(p.read_text(encoding="utf-8"))
                if isinstance(d, dict):
                    d = d.get("data") or d.get("train") or d.get("samples") or [d]
                return [x if isinstance(x, dict) else {"text": str(x)} for x in d]
            if p.suffix in (".txt", ".md"):
                return [{"text": t} for t in p.read_text(encoding="utf-8").split("\n\n") if t.strip()]
        except (OSError, ValueError) as e:
            cls.failures.append((str(p), f"{type(e).__name__}: {e}"))
        return []

    @classmethod
    def scan_directory(cls, directory: str) -> List[Dict[str, Any]]:
        out: List[Dict[str, Any]] = []
        for f in sorted(Path(directory).rglob("*")):
            if f.is_file() and f.suffix in (".jsonl", ".json", ".txt", ".md"):
                out += cls.load_samples(str(f))
        return out

    @classmethod
    def resolve(cls, data_spec: str) -> List[Dict[str, Any]]:
        p = Path(data_spec)
        if p.is_dir():
            return cls.scan_directory(data_spec)
        if p.exists():
            return cls.load_samples(data_spec)
        raise FileNotFoundError(f"no data at {data_spec}")


class PiscesLxToolsDataSampleRecord:
    @staticmethod
    def encode_ids(tokenizer: Any, text: str, max_len: int, add_eos: bool = False) -> torch.Tensor:
        try:
            ids = tokenizer.encode(text, add_eos=add_eos)
        except TypeError:
            ids = list(tokenizer.encode(text))
        return torch.tensor(list(ids)[:max_len], dtype=torch.long)

    @classmethod
    def field(cls, sample: Dict[str, Any], names: Sequence[str]) -> str:
        for n in names:
            v = sample.get(n)
            if v is not None and str(v).strip():
                return str(v)
        return ""

    @classmethod
    def encode_pair(cls, tokenizer: Any, prompt: str, response: str, max_len: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """(ids, labels) with the prompt masked out; an over-long pair loses the beginning of its prompt."""
        r = cls.encode_ids(tokenizer, response, max_len, add_eos=True)
        p = cls.encode_ids(tokenizer, prompt, 10 ** 9) if prompt else torch.empty(0, dtype=torch.long)
        p = p[max(0, len(p) - (max_len - len(r))):]
        ids = torch.cat([p, r])
        labels = ids.clone()
        labels[: len(p)] = -100
        return ids, labels


def pad_collate(samples: List[Dict[str, Any]], pad_id: int = 0, multiple: int = PAD_MULTIPLE) -> Dict[str, Any]:
    """Pads every 1-D integer tensor field to the longest in the batch rounded up to ``multiple`` (labels with -100,
    masks with 0, ids with ``pad_id``), stacks equal-shaped tensors, keeps the rest as lists."""
    out: Dict[str, Any] = {}
    for k in samples[0]:
        vals = [s[k] for s in samples]
        if all(torch.is_tensor(v) and v.dim() == 1 and not v.is_floating_point() for v in vals):
            n = max(int(v.shape[0]) for v in vals)
            n = ((n + multiple - 1) // multiple) * multiple
            fill = -100 if "label" in k and "class" not in k else (0 if "mask" in k else pad_id)
            t = torch.full((len(vals), n), fill, dtype=torch.long)
            for i, v in enumerate(vals):
                t[i, : v.shape[0]] = v
            out[k] = t
        elif all(torch.is_tensor(v) for v in vals) and len({tuple(v.shape) for v in vals}) == 1:
            out[k] = torch.stack(vals)
        elif all(isinstance(v, (int, float)) for v in vals):
            out[k] = torch.tensor(vals)
        else:
            out[k] = vals
    return out


class PiscesLxToolsDataClassificationDataset(Dataset):
    """``{"text", "label"}`` samples; labels may be strings (mapped to indices in order of first appearance)."""

    def __init__(self, samples: List[Dict[str, Any]], tokenizer: Any, max_len: int):
        self.tok, self.max_len = tokenizer, max_len
        self.samples = [s for s in samples if PiscesLxToolsDataJsonSampleReader.extract_text(s) and ("label" in s or "class" in s)]
        self.label_map: Dict[Any, int] = {}
        for s in self.samples:
            self.label_map.setdefault(s.get("label", s.get("class")), len(self.label_map))

    def __len__(self) -> int:
        return len(self.samples)

    def __getitem__(self, idx: int) -> Dict[str, torch.Tensor]:
        s = self.samples[idx]
        ids = PiscesLxToolsDataSampleRecord.encode_ids(self.tok, PiscesLxToolsDataJsonSampleReader.extract_text(s), self.max_len)
        return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "class_label": self.label_map[s.get("label", s.get("class"))]}


# ---- source configuration and datasets -------------------------------------------------------------------------------------
@dataclass
class PiscesLxDataSourcesConfig:
    """The sources of a data module (the reference's data-module ``PiscesLxDataConfig``, datamodule.py:63-150; the training
    configuration's data section is ``engine.train_config.PiscesLxDataConfig``)."""
    batch_size: int = 8
    max_seq_length: int = 2048
    num_workers: int = 0
    pin_memory: bool = True
    shuffle: bool = True
    seed: int = 0
    image_size: int = 224
    val_fraction: float = 0.0
    sources: List[Dict[str, Any]] = field(default_factory=list)

    def _add(self, kind: str, path: str, weight: float, **kw: Any) -> "PiscesLxDataSourcesConfig":
        self.sources.append({"type": kind, "path": path, "weight": float(weight), **kw})
        return self

    def add_text_data(self, path: str, weight: float = 1.0, text_field: Optional[str] = None) -> "PiscesLxDataSourcesConfig":
        return self._add("text", path, weight, text_field=text_field)

    def add_image_text_data(self, path: str, image_dir: Optional[str] = None, weight: float = 1.0, image_field: str = "image",
                            text_field: str = "caption") -> "PiscesLxDataSourcesConfig":
        return self._add("image_text", path, weight, image_dir=image_dir, image_field=image_field, text_field=text_field)

    def add_conversation_data(self, path: str, weight: float = 1.0) -> "PiscesLxDataSourcesConfig":
        return self._add("conversation", path, weight)

    def add_preference_data(self, path: str, weight: float = 1.0) -> "PiscesLxDataSourcesConfig":
        return self._add("preference", path, weight)


class PiscesLxBaseDataset(Dataset):
    """Loads every source of the configuration into ``self.samples`` (each tagged with ``_type`` and ``_source``).  A source
    weight above 1 repeats the source's samples (the fraction by a seeded draw), below 1 keeps that share."""

    def __init__(self, config: PiscesLxDataSourcesConfig, tokenizer: Any = None, split: str = "train"):
        self.config, self.split = config, split
        if tokenizer is None:
            from ..models.tokenizer import YvTokenizer
            tokenizer = YvTokenizer.instance()
        self.tok = tokenizer
        self.pad_id = int(getattr(tokenizer, "pad_token_id", 0) or 0)
        self.samples: List[Dict[str, Any]] = []
        self._load_data_sources()

    def _load_data_sources(self) -> None:
        rng = random.Random(self.config.seed)
        for si, src in enumerate(self.config.sources):
            loader = getattr(self, f"_load_{src['type']}_source", None)
            if loader is None:
                raise ValueError(f"unknown source type {src['type']}")
            rows = loader(src)
            for r in rows:
                r["_type"], r["_source"] = src["type"], si
            w = float(src.get("weight", 1.0))
            whole, frac = int(w), w - int(w)
            picked = rows * whole + [r for r in rows if rng.random() < frac]
            self.samples += picked
        if self.config.val_fraction > 0:
            order = list(range(len(self.samples)))
            random.Random(self.config.seed + 1).shuffle(order)
            n_val = int(len(order) * self.config.val_fraction)
            keep = set(order[:n_val]) if self.split in ("val", "validation", "test") else set(order[n_val:])
            self.samples = [s for i, s in enumerate(self.samples) if i in keep]

    @staticmethod
    def _read_text_file(file_path: str) -> List[Dict[str, Any]]:
        return PiscesLxToolsDataJsonSampleReader.resolve(file_path)

    def _load_text_source(self, source: Dict[str, Any]) -> List[Dict[str, Any]]:
        tf = source.get("text_field")
        out = []
        for s in self._read_text_file(source["path"]):
            t = str(s.get(tf, "")) if tf else PiscesLxToolsDataJsonSampleReader.extract_text(s)
            if t.strip():
                out.append({"text": t})
        return out

    def _load_image_text_source(self, source: Dict[str, Any]) -> List[Dict[str, Any]]:
        base = source.get("image_dir") or str(Path(source["path"]).parent if Path(source["path"]).is_file() else source["path"])
        out = []
        for s in self._read_text_file(source["path"]):
            img, txt = s.get(source.get("image_field", "image")), s.get(source.get("text_field", "caption"), s.get("text", ""))
            if img and txt:
                out.append({"image": img if os.path.isabs(str(img)) else os.path.join(base, str(img)), "text": str(txt)})
        return out

    def _load_conversation_source(self, source: Dict[str, Any]) -> List[Dict[str, Any]]:
        out = []
        for s in self._read_text_file(source["path"]):
            msgs = s.get("messages") or s.get("conversations")
            if isinstance(msgs, list) and msgs:
                out.append({"messages": [{"role": m.get("role", {"human": "user", "gpt": "assistant"}.get(m.get("from"), m.get("from", "user"))),
                                          "content": m.get("content", m.get("value", ""))} for m in msgs if isinstance(m, dict)]})
        return out

    def _load_preference_source(self, source: Dict[str, Any]) -> List[Dict[str, Any]]:
        out = []
        for s in self._read_text_file(source["path"]):
            if s.get("chosen") is not None and s.get("rejected") is not None:
                out.append({"prompt": str(s.get("prompt", s.get("question", ""))), "chosen": str(s["chosen"]), "rejected": str(s["rejected"])})
        return out

    def __len__(self) -> int:
        return len(self.samples)

    def __getitem__(self, idx: int) -> Dict[str, Any]:
        return self.samples[idx]

    def collate(self, samples: List[Dict[str, Any]]) -> Dict[str, Any]:
        return pad_collate(samples, self.pad_id)


class PiscesLxTextDataset(PiscesLxBaseDataset):
    def __getitem__(self, idx: int) -> Dict[str, Any]:
        s = self.samples[idx]
        text = s.get("text") or PiscesLxToolsDataJsonSampleReader.extract_text(s)
        ids = PiscesLxToolsDataSampleRecord.encode_ids(self.tok, text, self.config.max_seq_length, add_eos=True)
        return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids.clone()}


def load_image_tensor(path: str, size: int) -> torch.Tensor:
    """[3, size, size] float16, ImageNet-normalised; ``.pt`` / ``.npy`` arrays, or an image file through PIL when PIL is there.
    A file that cannot be read gives zeros (the sample's text still trains)."""
    mean, std = torch.tensor([0.485, 0.456, 0.406]).view(3, 1, 1), torch.tensor([0.229, 0.224, 0.225]).view(3, 1, 1)
    try:
        if path.endswith(".pt"):
            x = torch.load(path, map_location="cpu", weights_only=True).float()
        elif path.endswith(".npy"):
            import numpy as np
            x = torch.from_numpy(np.load(path)).float()
        else:
            import numpy as np
            from PIL import Image
            x = torch.from_numpy(np.asarray(Image.open(path).convert("RGB"))).float()
        if x.dim() == 3 and x.shape[-1] == 3:
            x = x.permute(2, 0, 1)
        if x.max() > 2.0:
            x = x / 255.0
        x = torch.nn.functional.interpolate(x.unsqueeze(0), size=(size, size), mode="bilinear", align_corners=False)[0]
        return ((x - mean) / std).half()
    except Exception:
        return torch.zeros(3, size, size, dtype=torch.float16)


class PiscesLxMultimodalDataset(PiscesLxBaseDataset):
    """Every sample type becomes ``input_ids`` / ``attention_mask`` / ``labels`` (plus ``images`` for image-text samples and
    the rejected row for preference samples); the ``sample_type`` field tells them apart."""

    def __init__(self, config: PiscesLxDataSourcesConfig, tokenizer: Any = None, split: str = "train", image_loader: Optional[Callable[[str, int], torch.Tensor]] = None):
        super().__init__(config, tokenizer, split)
        self.image_loader = image_loader or load_image_tensor

    def __getitem__(self, idx: int) -> Dict[str, Any]:
        s = self.samples[idx]
        return getattr(self, f"_get_{s['_type']}_sample")(s)

    def _get_text_sample(self, s: Dict[str, Any]) -> Dict[str, Any]:
        ids = PiscesLxToolsDataSampleRecord.encode_ids(self.tok, s["text"], self.config.max_seq_length, add_eos=True)
        return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids.clone(), "sample_type": "text"}

    def _get_image_text_sample(self, s: Dict[str, Any]) -> Dict[str, Any]:
        out = self._get_text_sample(s)
        out["images"], out["sample_type"] = self.image_loader(s["image"], self.config.image_size), "image_text"
        return out

    def _get_conversation_sample(self, s: Dict[str, Any]) -> Dict[str, Any]:
        """Only assistant turns carry labels."""
        ids: List[int] = []
        labels: List[int] = []
        for m in s["messages"]:
            head = PiscesLxToolsDataSampleRecord.encode_ids(self.tok, f"<|{m['role']}|>\n", 64).tolist()
            body = PiscesLxToolsDataSampleRecord.encode_ids(self.tok, str(m["content"]) + "\n", self.config.max_seq_length, add_eos=m["role"] == "assistant").tolist()
            ids += head + body
            labels += [-100] * len(head) + (body if m["role"] == "assistant" else [-100] * len(body))
        ids, labels = ids[-self.config.max_seq_length:], labels[-self.config.max_seq_length:]
        t = torch.tensor(ids, dtype=torch.long)
        return {"input_ids": t, "attention_mask": torch.ones_like(t), "labels": torch.tensor(labels, dtype=torch.long), "sample_type": "conversation"}

    def _get_preference_sample(self, s: Dict[str, Any]) -> Dict[str, Any]:
        L = self.config.max_seq_length
        ci, cl = PiscesLxToolsDataSampleRecord.encode_pair(self.tok, s["prompt"], s["chosen"], L)
        ri, rl = PiscesLxToolsDataSampleRecord.encode_pair(self.tok, s["prompt"], s["rejected"], L)
        return {"input_ids": ci, "attention_mask": torch.ones_like(ci), "labels": cl, "rejected_input_ids": ri, "rejected_labels": rl, "sample_type": "preference"}


class PiscesLxStreamingDataset(IterableDataset):
    """Reads the files one at a time; ranks and loader workers take strided files; a shuffle buffer mixes neighbours."""

    def __init__(self, paths: Union[str, Sequence[str]], tokenizer: Any = None, max_seq_length: int = 2048, shuffle_buffer: int = 0, seed: int = 0,
                 rank: int = 0, world: int = 1, process: Optional[Callable[[Dict[str, Any]], Optional[Dict[str, Any]]]] = None):
        ps = [paths] if isinstance(paths, str) else list(paths)
        files: List[str] = []
        for p in ps:
            files += sorted(str(f) for f in Path(p).rglob("*") if f.suffix in (".jsonl", ".json", ".txt")) if Path(p).is_dir() else [p]
        self.files, self.max_seq_length, self.shuffle_buffer, self.seed, self.rank, self.world = files, max_seq_length, shuffle_buffer, seed, rank, world
        if tokenizer is None:
            from ..models.tokenizer import YvTokenizer
            tokenizer = YvTokenizer.instance()
        self.tok, self.process = tokenizer, process

    def _process_sample(self, sample: Dict[str, Any]) -> Optional[Dict[str, Any]]:
        if self.process is not None:
            return self.process(sample)
        text = PiscesLxToolsDataJsonSampleReader.extract_text(sample)
        if not text.strip():
            return None
        ids = PiscesLxToolsDataSampleRecord.encode_ids(self.tok, text, self.max_seq_length, add_eos=True)
        return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids.clone()}

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        info = torch.utils.data.get_worker_info()
        wid, nw = (info.id, info.num_workers) if info is not None else (0, 1)
        files = self.files[self.rank * nw + wid:: self.world * nw]
        rng, buf = random.Random(self.seed + self.rank * 1000 + wid), []
        for f in files:
            for s in PiscesLxToolsDataJsonSampleReader.load_samples(f):
                out = self._process_sample(s)
                if out is None:
                    continue
                if self.shuffle_buffer <= 1:
                    yield out
                    continue
                buf.append(out)
                if len(buf) >= self.shuffle_buffer:
                    yield buf.pop(rng.randrange(len(buf)))
        rng.shuffle(buf)
        yield from buf


# ---- samplers and loaders ---------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxToolsDataBatchConfig:
    batch_size: int = 8
    max_tokens: Optional[int] = None              # a token budget makes the batches dynamic
    shuffle: bool = True
    drop_last: bool = False
    num_workers: int = 0
    pin_memory: bool = True
    prefetch_factor: int = 2
    persistent_workers: bool = False
    seed: int = 0
    bucket_multiple: int = PAD_MULTIPLE


class PiscesLxToolsDataDynamicBatchSampler(Sampler):
    """Batches under a token budget: samples are sorted by length, cut where padded length x rows would pass ``max_tokens``
    (padded length = the batch's longest rounded up to ``bucket_multiple``), and the batches are shuffled per epoch."""

    def __init__(self, dataset: Any, max_tokens: int, length_fn: Optional[Callable[[int], int]] = None, max_batch_size: Optional[int] = None,
                 shuffle: bool = True, seed: int = 0, bucket_multiple: int = PAD_MULTIPLE, lengths: Optional[Sequence[int]] = None):
        self.dataset, self.max_tokens, self.max_batch_size = dataset, max_tokens, max_batch_size
        self.length_fn, self.shuffle, self.seed, self.epoch, self.bucket = length_fn or self._default_length_fn, shuffle, seed, 0, max(bucket_multiple, 1)
        self.lengths = list(lengths) if lengths is not None else self._compute_lengths()
        self.batches = self._create_batches()

    def _default_length_fn(self, idx: int) -> int:
        s = self.dataset[idx]
        v = s.get("input_ids") if isinstance(s, dict) else s
        return int(len(v)) if v is not None else 1

    def _compute_lengths(self) -> List[int]:
        return [self.length_fn(i) for i in range(len(self.dataset))]

    def _padded(self, n: int) -> int:
        return ((n + self.bucket - 1) // self.bucket) * self.bucket

    def _create_batches(self) -> List[List[int]]:
        order = sorted(range(len(self.lengths)), key=lambda i: self.lengths[i])
        out, cur = [], []
        for i in order:
            rows = len(cur) + 1
            if cur and (self._padded(self.lengths[i]) * rows > self.max_tokens or (self.max_batch_size and rows > self.max_batch_size)):
                out.append(cur)
                cur = []
            cur.append(i)
        if cur:
            out.append(cur)
        return out

    def __iter__(self) -> Iterator[List[int]]:
        b = list(self.batches)
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(b)
        return iter(b)

    def __len__(self) -> int:
        return len(self.batches)

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def reset(self) -> None:
        self.lengths = self._compute_lengths()
        self.batches = self._create_batches()

    def padding_waste(self) -> float:
        """Share of the padded token slots that hold padding."""
        real = sum(self.lengths)
        slots = sum(self._padded(max(self.lengths[i] for i in b)) * len(b) for b in self.batches)
        return 1.0 - real / max(slots, 1)


class PiscesLxToolsDataCurriculumSampler(Sampler):
    """Admits the samples whose difficulty is under a threshold that rises from ``start_fraction`` of the difficulty range to
    all of it over ``total_steps`` calls of ``step()``; difficulty defaults to the sample's length."""

    def __init__(self, dataset: Any, difficulty_fn: Optional[Callable[[int], float]] = None, total_steps: int = 1000, start_fraction: float = 0.2,
                 shuffle: bool = True, seed: int = 0, difficulties: Optional[Sequence[float]] = None):
        self.dataset, self.total_steps, self.start_fraction, self.shuffle, self.seed = dataset, max(total_steps, 1), start_fraction, shuffle, seed
        self.difficulty_fn = difficulty_fn or self._default_difficulty_fn
        self.difficulties = list(difficulties) if difficulties is not None else self._compute_difficulties()
        self.order = sorted(range(len(self.difficulties)), key=lambda i: self.difficulties[i])
        self.current_step = 0

    def _default_difficulty_fn(self, idx: int) -> float:
        s = self.dataset[idx]
        v = s.get("input_ids") if isinstance(s, dict) else s
        return float(len(v)) if v is not None else 0.0

    def _compute_difficulties(self) -> List[float]:
        return [self.difficulty_fn(i) for i in range(len(self.dataset))]

    def _get_current_threshold(self) -> float:
        """The admitted share of the samples (by rank of difficulty), in [start_fraction, 1]."""
        return min(1.0, self.start_fraction + (1.0 - self.start_fraction) * self.current_step / self.total_steps)

    def admitted(self) -> List[int]:
        return self.order[: max(1, int(math.ceil(len(self.order) * self._get_current_threshold())))]

    def __iter__(self) -> Iterator[int]:
        idx = list(self.admitted())
        if self.shuffle:
            random.Random(self.seed + self.current_step).shuffle(idx)
        return iter(idx)

    def __len__(self) -> int:
        return len(self.admitted())

    def step(self) -> None:
        self.current_step += 1

    def set_step(self, step: int) -> None:
        self.current_step = max(int(step), 0)


class PiscesLxToolsDataPrefetchDataLoader:
    """A loader whose batches are staged in pinned memory and copied to the device on a side stream ahead of use."""

    def __init__(self, dataloader: Iterable, prefetch_batches: int = 2, device: Optional[torch.device] = None):
        self.dataloader, self.prefetch_batches, self.device = dataloader, prefetch_batches, device

    def _prefetch_batch(self, batch: Dict[str, Any]) -> Dict[str, Any]:
        return PiscesLxPrefetchLoader([batch], 1, self.device)._stage(batch)

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        return iter(PiscesLxPrefetchLoader(self.dataloader, self.prefetch_batches, self.device))

    def __len__(self) -> int:
        return len(self.dataloader)


class PiscesLxToolsDataOptimizedDataLoader:
    """Chooses the loader for a dataset and a batch configuration: iterable datasets get a plain loader, a token budget a
    dynamic batch sampler, ``world > 1`` a distributed sampler, otherwise a shuffled loader."""

    def __init__(self, dataset: Any, config: Optional[PiscesLxToolsDataBatchConfig] = None, collate_fn: Optional[Callable] = None, rank: int = 0, world: int = 1):
        self.dataset, self.config, self.rank, self.world = dataset, config or PiscesLxToolsDataBatchConfig(), rank, world
        self.collate_fn = collate_fn or getattr(dataset, "collate", None) or pad_collate

    def _kw(self) -> Dict[str, Any]:
        c = self.config
        kw: Dict[str, Any] = {"num_workers": c.num_workers, "pin_memory": c.pin_memory and torch.cuda.is_available(), "collate_fn": self.collate_fn}
        if c.num_workers > 0:
            kw.update(prefetch_factor=c.prefetch_factor, persistent_workers=c.persistent_workers)
        return kw

    def _get_standard_dataloader(self) -> DataLoader:
        c = self.config
        g = torch.Generator().manual_seed(c.seed)
        return DataLoader(self.dataset, batch_size=c.batch_size, shuffle=c.shuffle, drop_last=c.drop_last, generator=g, **self._kw())

    def _get_iterable_dataloader(self) -> DataLoader:
        return DataLoader(self.dataset, batch_size=self.config.batch_size, drop_last=self.config.drop_last, **self._kw())

    def _get_dynamic_dataloader(self) -> DataLoader:
        c = self.config
        s = PiscesLxToolsDataDynamicBatchSampler(self.dataset, c.max_tokens, max_batch_size=None, shuffle=c.shuffle, seed=c.seed, bucket_multiple=c.bucket_multiple)
        return DataLoader(self.dataset, batch_sampler=s, **self._kw())

    def _get_distributed_dataloader(self) -> DataLoader:
        c = self.config
        s = PiscesLxToolsDataDistributedSampler(len(self.dataset), self.rank, self.world, shuffle=c.shuffle, seed=c.seed)
        return DataLoader(self.dataset, batch_size=c.batch_size, sampler=s, drop_last=c.drop_last, **self._kw())

    def get(self) -> DataLoader:
        if isinstance(self.dataset, IterableDataset):
            return self._get_iterable_dataloader()
        if self.config.max_tokens:
            return self._get_dynamic_dataloader()
        if self.world > 1:
            return self._get_distributed_dataloader()
        return self._get_standard_dataloader()

    def get_prefetched(self, prefetch_batches: int = 2, device: Optional[torch.device] = None) -> PiscesLxToolsDataPrefetchDataLoader:
        return PiscesLxToolsDataPrefetchDataLoader(self.get(), prefetch_batches, device)

    def get_curriculum(self, difficulty_fn: Optional[Callable[[int], float]] = None, total_steps: int = 1000, start_fraction: float = 0.2):
        s = PiscesLxToolsDataCurriculumSampler(self.dataset, difficulty_fn, total_steps, start_fraction, self.config.shuffle, self.config.seed)
        return DataLoader(self.dataset, batch_size=self.config.batch_size, sampler=s, drop_last=self.config.drop_last, **self._kw()), s

    @classmethod
    def create_dataloader(cls, dataset: Any, batch_size: int = 8, **kw: Any) -> DataLoader:
        names = set(PiscesLxToolsDataBatchConfig.__dataclass_fields__)
        cfg = PiscesLxToolsDataBatchConfig(batch_size=batch_size, **{k: v for k, v in kw.items() if k in names})
        return cls(dataset, cfg, **{k: v for k, v in kw.items() if k not in names}).get()


class PiscesLxDataModule:
    """``setup()`` builds the train / val / test datasets from the sources, ``*_dataloader()`` returns their loaders."""

    def __init__(self, config: PiscesLxDataSourcesConfig, tokenizer: Any = None, multimodal: Optional[bool] = None, rank: int = 0, world: int = 1,
                 max_tokens: Optional[int] = None):
        self.config, self.tok, self.rank, self.world, self.max_tokens = config, tokenizer, rank, world, max_tokens
        self.multimodal = any(s["type"] != "text" for s in config.sources) if multimodal is None else multimodal
        self.datasets: Dict[str, Dataset] = {}

    def _create_dataset(self, split: str) -> Dataset:
        cls = PiscesLxMultimodalDataset if self.multimodal else PiscesLxTextDataset
        return cls(self.config, self.tok, split)

    def setup(self, stage: str = "fit") -> None:
        if stage in ("fit", "train"):
            self.datasets["train"] = self._create_dataset("train")
            if self.config.val_fraction > 0:
                self.datasets["val"] = self._create_dataset("val")
        elif stage in ("validate", "val"):
            self.datasets["val"] = self._create_dataset("val")
        elif stage == "test":
            self.datasets["test"] = self._create_dataset("test")
        else:
            raise ValueError(f"unknown stage {stage}")

    def _loader(self, split: str, shuffle: bool) -> DataLoader:
        if split not in self.datasets:
            raise RuntimeError(f"setup() has not built the {split} dataset")
        c = self.config
        bc = PiscesLxToolsDataBatchConfig(batch_size=c.batch_size, max_tokens=self.max_tokens if split == "train" else None, shuffle=shuffle and c.shuffle,
                                          num_workers=c.num_workers, pin_memory=c.pin_memory, seed=c.seed)
        return PiscesLxToolsDataOptimizedDataLoader(self.datasets[split], bc, rank=self.rank, world=self.world).get()

    def train_dataloader(self) -> DataLoader:
        return self._loader("train", True)

    def val_dataloader(self) -> DataLoader:
        return self._loader("val", False)

    def test_dataloader(self) -> DataLoader:
        return self._loader("test", False)

    def teardown(self, stage: str = "fit") -> None:
        self.datasets.clear()

    @staticmethod
    def create_datamodule(text: Optional[str] = None, conversations: Optional[str] = None, preferences: Optional[str] = None, image_text: Optional[str] = None,
                          tokenizer: Any = None, **kw: Any) -> "PiscesLxDataModule":
        names = set(PiscesLxDataSourcesConfig.__dataclass_fields__)
        cfg = PiscesLxDataSourcesConfig(**{k: v for k, v in kw.items() if k in names})
        for path, add in ((text, cfg.add_text_data), (conversations, cfg.add_conversation_data), (preferences, cfg.add_preference_data), (image_text, cfg.add_image_text_data)):
            if path:
                add(path)
        return PiscesLxDataModule(cfg, tokenizer, **{k: v for k, v in kw.items() if k not in names})


# ---- buffers and memory ----------------------------------------------------------------------------------------------------------
class PiscesLxToolsDataStreamingDataBuffer:
    """A bounded buffer between a producer and a consumer thread; ``stop()`` wakes both sides."""

    def __init__(self, max_size: int = 1000):
        self._q: "queue.Queue" = queue.Queue(max_size)
        self._stopped = threading.Event()
        self.max_size = max_size

    def put(self, item: Any, timeout: float = 0.1) -> bool:
        while not self._stopped.is_set():
            try:
                self._q.put(item, timeout=timeout)
                return True
            except queue.Full:
                continue
        return False

    def get(self, timeout: Optional[float] = None) -> Optional[Any]:
        end = None if timeout is None else time.monotonic() + timeout
        while True:
            try:
                return self._q.get(timeout=0.05)
            except queue.Empty:
                if self._stopped.is_set() or (end is not None and time.monotonic() >= end):
                    return None

    def stop(self) -> None:
        self._stopped.set()

    def is_stopped(self) -> bool:
        return self._stopped.is_set()

    def size(self) -> int:
        return self._q.qsize()

    def is_empty(self) -> bool:
        return self._q.empty()

    def is_full(self) -> bool:
        return self._q.full()


class PiscesLxDataPrefetcher:
    """Worker threads that call ``dataset[i]`` ahead of the consumer, in order (``get`` / iteration return samples in index
    order whatever thread finished first)."""

    def __init__(self, dataset: Any, queue_size: int = 100, num_workers: int = 2, indices: Optional[Sequence[int]] = None):
        self.dataset, self.queue_size, self.num_workers = dataset, queue_size, max(num_workers, 1)
        self.indices = list(indices) if indices is not None else list(range(len(dataset)))
        self._results: Dict[int, Any] = {}
        self._cv = threading.Condition()
        self._next_job = self._next_out = 0
        self._threads: List[threading.Thread] = []
        self._stop = False

    def start(self) -> "PiscesLxDataPrefetcher":
        if not self._threads:
            self._stop = False
            self._threads = [threading.Thread(target=self._worker_loop, daemon=True) for _ in range(self.num_workers)]
            for t in self._threads:
                t.start()
        return self

    def stop(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify_all()
        for t in self._threads:
            t.join(timeout=2)
        self._threads = []

    def _worker_loop(self) -> None:
        while True:
            with self._cv:
                while not self._stop and (self._next_job >= len(self.indices) or self._next_job - self._next_out >= self.queue_size):
                    if self._next_job >= len(self.indices):
                        return
                    self._cv.wait(0.05)
                if self._stop:
                    return
                job = self._next_job
                self._next_job += 1
            try:
                val = self.dataset[self.indices[job]]
            except Exception as e:
                val = e
            with self._cv:
                self._results[job] = val
                self._cv.notify_all()

    def get(self, timeout: float = 10.0) -> Optional[Dict[str, Any]]:
        end = time.monotonic() + timeout
        with self._cv:
            if self._next_out >= len(self.indices):
                return None
            while self._next_out not in self._results:
                left = end - time.monotonic()
                if left <= 0 or self._stop:
                    return None
                self._cv.wait(min(left, 0.05))
            val = self._results.pop(self._next_out)
            self._next_out += 1
            self._cv.notify_all()
        if isinstance(val, Exception):
            raise val
        return val

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        self.start()
        try:
            while True:
                v = self.get()
                if v is None:
                    return
                yield v
        finally:
            self.stop()


class PiscesLxToolsDataMemoryMonitor:
    """Resident memory of this process in GB (psutil, else ``resource``), with the peak seen."""

    def __init__(self) -> None:
        self.peak = 0.0
        self.samples = 0

    def check_memory(self) -> float:
        try:
            import psutil
            gb = psutil.Process().memory_info().rss / 2 ** 30
        except Exception:
            import resource
            gb = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 2 ** 20
        self.peak, self.samples = max(self.peak, gb), self.samples + 1
        return gb

    def get_peak_memory(self) -> float:
        return self.peak

    def get_memory_stats(self) -> Dict[str, float]:
        cur = self.check_memory()
        return {"current_gb": cur, "peak_gb": self.peak, "samples": float(self.samples)}


class PiscesLxToolsMemoryMonitor(PiscesLxToolsDataMemoryMonitor):
    def __init__(self, threshold_gb: float = 8.0):
        super().__init__()
        self.threshold_gb = threshold_gb

    def check_memory(self) -> Dict[str, float]:                                      # type: ignore[override]
        gb = super().check_memory()
        return {"used_gb": gb, "threshold_gb": self.threshold_gb, "over_threshold": float(gb > self.threshold_gb), "peak_gb": self.peak}


# ---- the cached single-source dataset ------------------------------------------------------------------------------------------
@dataclass
class PiscesLxDatasetConfig:
    cache_enabled: bool = True
    custom_image_keys: Optional[Any] = None
    custom_audio_keys: Optional[Any] = None
    custom_video_keys: Optional[Any] = None
    force_enable_vision: bool = False
    force_enable_audio: bool = False
    force_enable_video: bool = False
    cache_size: int = 10000
    prefetch_enabled: bool = True
    prefetch_workers: int = 2
    prefetch_queue_size: int = 100
    augmentation_enabled: bool = False
    text_augmentation_prob: float = 0.1
    image_augmentation_prob: float = 0.1
    max_text_length: int = 8192
    truncate_mode: str = "tail"                   # which end is cut: "tail" keeps the beginning, "head" keeps the end, "middle" keeps both ends
    return_quality_score: bool = False


class PiscesLxDataAugmentationPipeline:
    """Text augmentation with probability ``text_prob`` (``data.augment.PiscesLxTextAugmenter``); image augmentation is applied to
    tensors (flip / brightness) with probability ``image_prob``."""

    def __init__(self, text_prob: float = 0.1, image_prob: float = 0.1, seed: int = 0):
        self.text_prob, self.image_prob, self.rng = text_prob, image_prob, random.Random(seed)
        self._text = None

    def _lazy_init_text_augmenter(self):
        if self._text is None:
            from .augment import PiscesLxTextAugmenter
            self._text = PiscesLxTextAugmenter(seed=self.rng.randrange(1 << 30))
        return self._text

    def augment_text(self, text: str) -> str:
        if self.rng.random() >= self.text_prob or not text.strip():
            return text
        aug = self._lazy_init_text_augmenter()
        out = aug.word_dropout(text, 0.05) if self.rng.random() < 0.5 else aug.typo(text, 0.02)
        return out if isinstance(out, str) and out.strip() else text

    def augment_image(self, image: torch.Tensor) -> torch.Tensor:
        if self.rng.random() >= self.image_prob or not torch.is_tensor(image):
            return image
        if self.rng.random() < 0.5:
            image = image.flip(-1)
        return image * (0.8 + 0.4 * self.rng.random())


class PiscesLxDataset(Dataset):
    """Samples of one source with an LRU of processed items, optional augmentation and modality keys."""

    _global_cache: Dict[str, Any] = {}
    IMAGE_KEYS, AUDIO_KEYS, VIDEO_KEYS = ("image", "image_path", "img"), ("audio", "audio_path"), ("video", "video_path")

    def __init__(self, data: Union[str, Sequence[Dict[str, Any]]], config: Optional[PiscesLxDatasetConfig] = None, tokenizer: Any = None):
        self.config = config or PiscesLxDatasetConfig()
        self.items = PiscesLxToolsDataJsonSampleReader.resolve(data) if isinstance(data, str) else list(data)
        if tokenizer is None:
            from ..models.tokenizer import YvTokenizer
            tokenizer = YvTokenizer.instance()
        self.tok = tokenizer
        from collections import OrderedDict
        self._cache: "OrderedDict[int, Dict[str, Any]]" = OrderedDict()
        self.cache_hits = 0
        c = self.config
        self.aug = PiscesLxDataAugmentationPipeline(c.text_augmentation_prob, c.image_augmentation_prob) if c.augmentation_enabled else None

    def __len__(self) -> int:
        return len(self.items)

    def _extract_text(self, item: Dict[str, Any]) -> str:
        return PiscesLxToolsDataJsonSampleReader.extract_text(item)

    def _truncate(self, ids: List[int]) -> List[int]:
        n, mode = self.config.max_text_length, self.config.truncate_mode
        if len(ids) <= n:
            return ids
        if mode == "head":
            return ids[-n:]
        if mode == "middle":
            return ids[: n // 2] + ids[len(ids) - (n - n // 2):]
        return ids[:n]

    def _keys(self, custom: Optional[Any], default: Tuple[str, ...]) -> Tuple[str, ...]:
        return tuple([custom] if isinstance(custom, str) else custom) if custom else default

    def _process_mm_lazy(self, item: Dict[str, Any]) -> Dict[str, Any]:
        """Paths of the modalities present; decoding happens where the batch is assembled."""
        out = {}
        c = self.config
        for name, keys in (("image", self._keys(c.custom_image_keys, self.IMAGE_KEYS)), ("audio", self._keys(c.custom_audio_keys, self.AUDIO_KEYS)),
                           ("video", self._keys(c.custom_video_keys, self.VIDEO_KEYS))):
            for k in keys:
                if item.get(k):
                    out[f"{name}_path"] = item[k]
                    break
        return out

    def __getitem__(self, idx: int) -> Dict[str, Any]:
        c = self.config
        if c.cache_enabled and self.aug is None and idx in self._cache:
            self._cache.move_to_end(idx)
            self.cache_hits += 1
            return self._cache[idx]
        item = self.items[idx]
        text = self._extract_text(item)
        if self.aug is not None:
            text = self.aug.augment_text(text)
        try:
            ids = list(self.tok.encode(text, add_eos=True))
        except TypeError:
            ids = list(self.tok.encode(text))
        t = torch.tensor(self._truncate(ids), dtype=torch.long)
        out: Dict[str, Any] = {"input_ids": t, "attention_mask": torch.ones_like(t), "labels": t.clone(), **self._process_mm_lazy(item)}
        if c.return_quality_score:
            words = text.split()
            out["quality_score"] = min(1.0, len(set(words)) / max(len(words), 1) + 0.1) if words else 0.0
        if c.cache_enabled and self.aug is None:
            self._cache[idx] = out
            while len(self._cache) > c.cache_size:
                self._cache.popitem(last=False)
        return out

    def get_prefetcher(self, queue_size: int = 100, num_workers: int = 2) -> PiscesLxDataPrefetcher:
        return PiscesLxDataPrefetcher(self, queue_size, num_workers)

    def clear_cache(self) -> None:
        self._cache.clear()

    @classmethod
    def get_global_cache(cls, key: str) -> Optional[Any]:
        return cls._global_cache.get(key)

    @classmethod
    def set_global_cache(cls, key: str, value: Any) -> None:
        cls._global_cache[key] = value

    @classmethod
    def clear_global_cache(cls) -> None:
        cls._global_cache.clear()


class PiscesLxDataIterableDataset(IterableDataset):
    """A map-style dataset as a stream: optional shuffle per pass, strided over loader workers, endless when ``repeat``."""

    def __init__(self, dataset: Any, shuffle: bool = False, seed: int = 0, repeat: bool = False):
        self.dataset, self.shuffle, self.seed, self.repeat = dataset, shuffle, seed, repeat

    def __iter__(self) -> Iterator[Any]:
        info = torch.utils.data.get_worker_info()
        wid, nw = (info.id, info.num_workers) if info is not None else (0, 1)
        epoch = 0
        while True:
            order = list(range(len(self.dataset)))
            if self.shuffle:
                random.Random(self.seed + epoch).shuffle(order)
            for i in order[wid::nw]:
                yield self.dataset[i]
            epoch += 1
            if not self.repeat:
                return

    def __len__(self) -> int:
        return len(self.dataset)
