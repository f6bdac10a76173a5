"""Dataset acquisition and large-corpus plumbing: source routing with retry and resume, a parquet corpus, and
process-parallel cleaning / loading of sharded corpora.

Reference surface: ``tools/data/download`` (``PiscesLxToolsDataSourceRouter`` picks ModelScope / Hugging Face / Kaggle
by preference and connectivity, ``PiscesLxDataRetryStrategy``, ``PiscesLxDataResumeManager`` with a JSON state file per
dataset, ``PiscesLxToolsDataDatasetDownload`` driven by ``configs/dataset.yaml``), ``tools/data/dataset/parquet.py``
(``PiscesLxToolsDataParquetCorpus``) and ``tools/data/distributed`` (Dask loader, Ray cleaner).

What differs: a *source* here is an object with ``available()`` and ``fetch(item, dest)``; the hub back ends import
their client library lazily and report themselves unavailable when it, or the network, is missing, and a ``local``
source (a directory or ``file://`` mirror) is always present, so the same download plan works on an air-gapped
cluster from a staged mirror.  The distributed loader / cleaner partition shards over a process pool of the host (the
node's CPU cores feed 8 GPUs; no cluster scheduler is required) and fall back to Dask / Ray only if asked for and
importable.
"""
from __future__ import annotations

import glob
import hashlib
import json
import os
import random
import shutil
import time
from concurrent.futures import ProcessPoolExecutor
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple


# --------------------------------------------------------------------------------------------------
# plan
# --------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxToolsDatasetItem:
    name: str                                  # hub id or mirror-relative path
    save_name: str = ""
    source_preference: List[str] = field(default_factory=list)
    split: str = "train"
    max_samples: Optional[int] = None
    text_field: str = "text"

    def __post_init__(self):
        self.save_name = self.save_name or self.name.replace("/", "__")

    def normalize_source_preference(self, default: Sequence[str]) -> List[str]:
        seen, out = set(), []
        for s in list(self.source_preference) + list(default):
            s = {"hf": "huggingface", "ms": "modelscope"}.get(s.lower(), s.lower())
            if s not in seen:
                seen.add(s)
                out.append(s)
        return out


@dataclass
class PiscesLxToolsDataDownloadConfig:
    datasets: List[PiscesLxToolsDatasetItem] = field(default_factory=list)
    data_dir: str = "data"
    source_preference: List[str] = field(default_factory=lambda: ["local", "modelscope", "huggingface", "kaggle"])
    max_samples: Optional[int] = None
    retries: int = 3
    mirror: Optional[str] = None               # directory or file:// URL of a staged mirror


class PiscesLxToolsDataConfigLoader:
    """``configs/dataset.yaml``: a list under ``datasets`` of names or ``{name, save_name, sources, split, max_samples}``."""

    def __init__(self, path: str = "configs/dataset.yaml"):
        self.path = path

    def load(self) -> PiscesLxToolsDataDownloadConfig:
        import yaml
        raw = yaml.safe_load(Path(self.path).read_text()) or {}
        items = []
        for d in raw.get("datasets", []):
            if isinstance(d, str):
                items.append(PiscesLxToolsDatasetItem(d))
            else:
                items.append(PiscesLxToolsDatasetItem(d["name"], d.get("save_name", ""), list(d.get("sources", [])),
                                                      d.get("split", "train"), d.get("max_samples"), d.get("text_field", "text")))
        cfg = PiscesLxToolsDataDownloadConfig(items)
        for k in ("data_dir", "max_samples", "retries", "mirror"):
            if raw.get(k) is not None:
                setattr(cfg, k, raw[k])
        if raw.get("source_preference"):
            cfg.source_preference = list(raw["source_preference"])
        return cfg


# --------------------------------------------------------------------------------------------------
# sources
# --------------------------------------------------------------------------------------------------
class PiscesLxDataSource:
    name = "base"

    def available(self) -> bool:
        return False

    def fetch(self, item: PiscesLxToolsDatasetItem, dest: Path) -> int:
        """Write ``dest/<save_name>.jsonl``; returns the number of records."""
        raise NotImplementedError


def _write_jsonl(records: Iterable[Dict[str, Any]], path: Path, limit: Optional[int]) -> int:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".part")
    n = 0
    with open(tmp, "w", encoding="utf-8") as f:
        for r in records:
            if limit is not None and n >= limit:
                break
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
            n += 1
    os.replace(tmp, path)
    return n


class PiscesLxLocalMirrorSource(PiscesLxDataSource):
    """A directory (or ``file://`` URL) laid out ``<root>/<name>/...`` or ``<root>/<save_name>.{jsonl,txt,parquet}``."""
    name = "local"

    def __init__(self, root: Optional[str]):
        self.root = Path(root[7:] if root and root.startswith("file://") else root) if root else None

    def available(self) -> bool:
        return self.root is not None and self.root.is_dir()

    def _candidates(self, item: PiscesLxToolsDatasetItem) -> List[Path]:
        out: List[Path] = []
        for stem in dict.fromkeys((item.name, item.save_name)):
            base = self.root / stem
            if base.is_dir():
                out += sorted(p for p in base.rglob("*") if p.suffix in (".jsonl", ".json", ".txt", ".parquet"))
            for ext in (".jsonl", ".json", ".txt", ".parquet"):
                if (self.root / (stem + ext)).exists():
                    out.append(self.root / (stem + ext))
        return list(dict.fromkeys(out))

    def fetch(self, item: PiscesLxToolsDatasetItem, dest: Path) -> int:
        files = self._candidates(item)
        if not files:
            raise FileNotFoundError(f"{item.name} is not in the mirror {self.root}")

        def records():
            for p in files:
                if p.suffix == ".parquet":
                    yield from PiscesLxToolsDataParquetCorpus(str(p), item.text_field).records()
                elif p.suffix == ".txt":
                    for line in open(p, encoding="utf-8", errors="replace"):
                        if line.strip():
                            yield {item.text_field: line.rstrip("\n")}
                else:
                    for line in open(p, encoding="utf-8", errors="replace"):
                        line = line.strip()
                        if line:
                            try:
                                yield json.loads(line)
                            except json.JSONDecodeError:
                                continue
        return _write_jsonl(records(), dest / f"{item.save_name}.jsonl", item.max_samples)


class _HubSource(PiscesLxDataSource):
    module = ""
    probe_host = ""

    def available(self) -> bool:
        try:
            __import__(self.module)
        except Exception:
            return False
        import socket
        try:
            socket.create_connection((self.probe_host, 443), timeout=2).close()
            return True
        except OSError:
            return False


class PiscesLxHuggingFaceSource(_HubSource):
    name, module, probe_host = "huggingface", "datasets", "huggingface.co"

    def fetch(self, item, dest):
        import datasets
        ds = datasets.load_dataset(item.name, split=item.split, streaming=True)
        return _write_jsonl(iter(ds), dest / f"{item.save_name}.jsonl", item.max_samples)


class PiscesLxModelScopeSource(_HubSource):
    name, module, probe_host = "modelscope", "modelscope", "modelscope.cn"

    def fetch(self, item, dest):
        from modelscope.msdatasets import MsDataset
        ds = MsDataset.load(item.name, split=item.split)
        return _write_jsonl(iter(ds), dest / f"{item.save_name}.jsonl", item.max_samples)


class PiscesLxKaggleSource(_HubSource):
    name, module, probe_host = "kaggle", "kaggle", "www.kaggle.com"

    def fetch(self, item, dest):
        import kaggle
        tmp = dest / f".kaggle_{item.save_name}"
        kaggle.api.dataset_download_files(item.name, path=str(tmp), unzip=True)
        n = PiscesLxLocalMirrorSource(str(tmp.parent)).fetch(
            PiscesLxToolsDatasetItem(tmp.name, item.save_name, max_samples=item.max_samples, text_field=item.text_field), dest)
        shutil.rmtree(tmp, ignore_errors=True)
        return n


class PiscesLxToolsDataSourceRouter:
    def __init__(self, mirror: Optional[str] = None, extra: Optional[Dict[str, PiscesLxDataSource]] = None):
        self.sources: Dict[str, PiscesLxDataSource] = {
            "local": PiscesLxLocalMirrorSource(mirror or os.environ.get("PISCESLX_DATA_MIRROR")),
            "huggingface": PiscesLxHuggingFaceSource(), "modelscope": PiscesLxModelScopeSource(),
            "kaggle": PiscesLxKaggleSource()}
        self.sources.update(extra or {})
        self._avail: Dict[str, bool] = {}

    def available(self, name: str) -> bool:
        if name not in self._avail:
            self._avail[name] = name in self.sources and self.sources[name].available()
        return self._avail[name]

    def route(self, item: PiscesLxToolsDatasetItem, default: Sequence[str]) -> List[PiscesLxDataSource]:
        return [self.sources[s] for s in item.normalize_source_preference(default) if self.available(s)]


# --------------------------------------------------------------------------------------------------
# retry / resume / runner
# --------------------------------------------------------------------------------------------------
class PiscesLxDataRetryStrategy:
    def __init__(self, max_attempts: int = 3, base_delay: float = 1.0, max_delay: float = 60.0, jitter: float = 0.1,
                 sleep: Callable[[float], None] = time.sleep):
        self.max_attempts, self.base, self.cap, self.jitter, self.sleep = max_attempts, base_delay, max_delay, jitter, sleep

    def get_delay(self, attempt: int) -> float:
        d = min(self.cap, self.base * (2 ** max(attempt - 1, 0)))
        return d * (1.0 + random.uniform(-self.jitter, self.jitter))

    def should_retry(self, attempt: int, error: Optional[BaseException] = None) -> bool:
        if isinstance(error, (FileNotFoundError, PermissionError, KeyboardInterrupt)):
            return False                                           # retrying cannot change these
        return attempt < self.max_attempts


@dataclass
class PiscesLxDataDownloadState:
    save_name: str
    status: str = "pending"                    # pending | running | completed | failed
    source: Optional[str] = None
    attempts: int = 0
    records: int = 0
    error: Optional[str] = None
    updated: float = 0.0


class PiscesLxDataResumeManager:
    def __init__(self, state_dir: str):
        self.dir = Path(state_dir)
        self.dir.mkdir(parents=True, exist_ok=True)

    def _path(self, save_name: str) -> Path:
        return self.dir / f"{save_name}.state.json"

    def load_state(self, save_name: str) -> Optional[PiscesLxDataDownloadState]:
        try:
            return PiscesLxDataDownloadState(**json.loads(self._path(save_name).read_text()))
        except (OSError, ValueError, TypeError):
            return None

    def save_state(self, st: PiscesLxDataDownloadState) -> None:
        st.updated = time.time()
        tmp = self._path(st.save_name).with_suffix(".tmp")
        tmp.write_text(json.dumps(asdict(st)))
        os.replace(tmp, self._path(st.save_name))

    def is_completed(self, save_name: str) -> bool:
        st = self.load_state(save_name)
        return st is not None and st.status == "completed"

    def clear_state(self, save_name: str) -> None:
        self._path(save_name).unlink(missing_ok=True)


class PiscesLxToolsDataDatasetDownload:
    def __init__(self, router: Optional[PiscesLxToolsDataSourceRouter] = None,
                 retry: Optional[PiscesLxDataRetryStrategy] = None):
        self.router, self.retry = router, retry

    def download(self, config: Any = "configs/dataset.yaml", max_samples_per_dataset: Optional[int] = None) -> Dict[str, Any]:
        cfg = config if isinstance(config, PiscesLxToolsDataDownloadConfig) else PiscesLxToolsDataConfigLoader(str(config)).load()
        router = self.router or PiscesLxToolsDataSourceRouter(cfg.mirror)
        retry = self.retry or PiscesLxDataRetryStrategy(cfg.retries)
        dest = Path(cfg.data_dir)
        resume = PiscesLxDataResumeManager(str(dest / ".download_state"))
        report: Dict[str, Any] = {"completed": [], "skipped": [], "failed": {}}
        for item in cfg.datasets:
            item.max_samples = max_samples_per_dataset or item.max_samples or cfg.max_samples
            if resume.is_completed(item.save_name) and (dest / f"{item.save_name}.jsonl").exists():
                report["skipped"].append(item.save_name)
                continue
            st = resume.load_state(item.save_name) or PiscesLxDataDownloadState(item.save_name)
            sources = router.route(item, cfg.source_preference)
            if not sources:
                st.status, st.error = "failed", "no source available (no network, no client library, no mirror)"
                resume.save_state(st)
                report["failed"][item.save_name] = st.error
                continue
            done = False
            for src in sources:
                attempt = 0
                while not done:
                    attempt += 1
                    st.status, st.source, st.attempts = "running", src.name, st.attempts + 1
                    resume.save_state(st)
                    try:
                        st.records = src.fetch(item, dest)
                        st.status, st.error, done = "completed", None, True
                    except BaseException as e:
                        st.error = f"{src.name}: {type(e).__name__}: {e}"
                        if isinstance(e, KeyboardInterrupt) or not retry.should_retry(attempt, e):
                            break
                        retry.sleep(retry.get_delay(attempt))
                if done:
                    break
            if not done:
                st.status = "failed"
                report["failed"][item.save_name] = st.error
            else:
                report["completed"].append(item.save_name)
            resume.save_state(st)
        return report


# --------------------------------------------------------------------------------------------------
# parquet corpus
# --------------------------------------------------------------------------------------------------
class PiscesLxToolsDataParquetCorpus:
    """Row-group streaming over one parquet file or a directory of them; rank-sharded by row group."""

    def __init__(self, path: str, text_field: str = "text", rank: int = 0, world: int = 1, batch_rows: int = 4096):
        self.files = sorted(glob.glob(os.path.join(path, "**", "*.parquet"), recursive=True)) if os.path.isdir(path) else [path]
        self.text_field, self.rank, self.world, self.batch_rows = text_field, rank, world, batch_rows

    def _groups(self) -> List[Tuple[str, int]]:
        import pyarrow.parquet as pq
        out = []
        for f in self.files:
            out += [(f, g) for g in range(pq.ParquetFile(f).num_row_groups)]
        return out[self.rank::self.world]

    def __len__(self) -> int:
        import pyarrow.parquet as pq
        return sum(pq.ParquetFile(f).metadata.row_group(g).num_rows for f, g in self._groups())

    def records(self) -> Iterator[Dict[str, Any]]:
        import pyarrow.parquet as pq
        for f, g in self._groups():
            tbl = pq.ParquetFile(f).read_row_group(g)
            yield from tbl.to_pylist()

    def texts(self) -> Iterator[str]:
        for r in self.records():
            t = r.get(self.text_field)
            if t:
                yield str(t)

    @staticmethod
    def write(records: Iterable[Dict[str, Any]], path: str, rows_per_group: int = 4096) -> int:
        import pyarrow as pa
        import pyarrow.parquet as pq
        rows = list(records)
        if not rows:
            return 0
        pq.write_table(pa.Table.from_pylist(rows), path, row_group_size=rows_per_group)
        return len(rows)


# --------------------------------------------------------------------------------------------------
# process-parallel loading / cleaning of sharded corpora
# --------------------------------------------------------------------------------------------------
def _read_shard(args: Tuple[str, str]) -> List[str]:
    path, field_name = args
    if path.endswith(".parquet"):
        return list(PiscesLxToolsDataParquetCorpus(path, field_name).texts())
    out = []
    for line in open(path, encoding="utf-8", errors="replace"):
        line = line.strip()
        if not line:
            continue
        if path.endswith((".jsonl", ".json")):
            try:
                t = json.loads(line).get(field_name)
            except json.JSONDecodeError:
                continue
            if t:
                out.append(str(t))
        else:
            out.append(line)
    return out


def _clean_shard(args: Tuple[str, str, str, int]) -> Dict[str, Any]:
    path, field_name, out_dir, min_chars = args
    from .cleaning import PiscesLxDatasetCleaner
    cleaner = PiscesLxDatasetCleaner(min_chars=min_chars)
    kept, hashes, n_in = [], set(), 0
    for t in _read_shard((path, field_name)):
        n_in += 1
        c = cleaner.normalise(t)
        if not cleaner.keep(c):
            continue
        h = hashlib.sha1(c.encode("utf-8")).hexdigest()
        if h in hashes:
            continue
        hashes.add(h)
        kept.append((h, c))
    out = Path(out_dir) / (Path(path).stem + ".clean.jsonl")
    _write_jsonl(({"text": c, "sha1": h} for h, c in kept), out, None)
    return {"shard": path, "out": str(out), "in": n_in, "kept": len(kept), "hashes": [h for h, _ in kept]}


class PiscesLxDataDistributedLoader:
    """Reads the shards of a corpus in parallel worker processes (``backend='process'``) or through Dask bags when
    ``backend='dask'`` is requested and importable (reference: PiscesLxDataDaskDistributedLoader)."""

    def __init__(self, pattern: str, text_field: str = "text", workers: int = 0, backend: str = "process"):
        self.shards = sorted(glob.glob(pattern, recursive=True))
        self.text_field, self.workers, self.backend = text_field, workers or min(8, os.cpu_count() or 1), backend

    def load(self) -> List[str]:
        jobs = [(s, self.text_field) for s in self.shards]
        if self.backend == "dask":
            try:
                import dask.bag as db
                return db.from_sequence(jobs, npartitions=max(len(jobs), 1)).map(_read_shard).flatten().compute()
            except ImportError:
                pass
        if len(jobs) <= 1 or self.workers <= 1:
            return [t for j in jobs for t in _read_shard(j)]
        with ProcessPoolExecutor(self.workers) as ex:
            return [t for part in ex.map(_read_shard, jobs) for t in part]


class PiscesLxDataDistributedCleaner:
    """Cleans and exact-deduplicates every shard in a worker process, then removes duplicates ACROSS shards in one
    pass over the content hashes (first shard wins).  ``backend='ray'`` uses Ray tasks when importable (reference:
    PiscesLxDataRayDistributedCleaner)."""

    def __init__(self, pattern: str, out_dir: str, text_field: str = "text", workers: int = 0, min_chars: int = 1,
                 backend: str = "process"):
        self.shards = sorted(glob.glob(pattern, recursive=True))
        self.out_dir, self.text_field, self.min_chars, self.backend = out_dir, text_field, min_chars, backend
        self.workers = workers or min(8, os.cpu_count() or 1)

    def run(self) -> Dict[str, Any]:
        Path(self.out_dir).mkdir(parents=True, exist_ok=True)
        jobs = [(s, self.text_field, self.out_dir, self.min_chars) for s in self.shards]
        results: List[Dict[str, Any]]
        if self.backend == "ray":
            try:
                import ray
                ray.init(ignore_reinit_error=True, log_to_driver=False)
                results = ray.get([ray.remote(_clean_shard).remote(j) for j in jobs])
            except ImportError:
                results = []
        else:
            results = []
        if not results:
            if len(jobs) <= 1 or self.workers <= 1:
                results = [_clean_shard(j) for j in jobs]
            else:
                with ProcessPoolExecutor(self.workers) as ex:
                    results = list(ex.map(_clean_shard, jobs))
        seen, cross = set(), 0
        for r in results:                                              # shard order = priority
            dup = [h for h in r["hashes"] if h in seen]
            if dup:
                dset = set(dup)
                rows = [json.loads(l) for l in open(r["out"], encoding="utf-8")]
                _write_jsonl((x for x in rows if x["sha1"] not in dset), Path(r["out"]), None)
                cross += len(dup)
                r["kept"] -= len(dup)
            seen.update(r["hashes"])
        return {"shards": len(results), "in": sum(r["in"] for r in results), "kept": sum(r["kept"] for r in results),
                "cross_shard_duplicates": cross, "outputs": [r["out"] for r in results]}
