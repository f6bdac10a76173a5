"""Data module layer: readers, datasets over mixed sources, samplers, loaders, buffers, prefetcher, cached dataset."""
import json
import threading

import pytest
import torch

from pisceslx_b200.data.datamodule import (
    PAD_MULTIPLE, PiscesLxDataIterableDataset, PiscesLxDataModule, PiscesLxDataPrefetcher, PiscesLxDataSourcesConfig, PiscesLxDataset, PiscesLxDatasetConfig,
    PiscesLxMultimodalDataset, PiscesLxStreamingDataset, PiscesLxTextDataset, PiscesLxToolsDataBatchConfig, PiscesLxToolsDataClassificationDataset,
    PiscesLxToolsDataCurriculumSampler, PiscesLxToolsDataDynamicBatchSampler, PiscesLxToolsDataJsonSampleReader, PiscesLxToolsDataMemoryMonitor,
    PiscesLxToolsDataOptimizedDataLoader, PiscesLxToolsDataPrefetchDataLoader, PiscesLxToolsDataSampleRecord, PiscesLxToolsDataStreamingDataBuffer,
    PiscesLxToolsMemoryMonitor, pad_collate)
from pisceslx_b200.models.tokenizer import YvTokenizer


@pytest.fixture
def tok():
    return YvTokenizer(use_files=False)


@pytest.fixture
def files(tmp_path):
    (tmp_path / "t.jsonl").write_text("\n".join(json.dumps({"text": "word " * (3 + 5 * i)}) for i in range(8)))
    (tmp_path / "c.jsonl").write_text(json.dumps({"conversations": [{"from": "human", "value": "hi"}, {"from": "gpt", "value": "hello there"}]}) + "\n")
    (tmp_path / "p.jsonl").write_text(json.dumps({"prompt": "q: ", "chosen": "good", "rejected": "bad bad"}) + "\n" + json.dumps({"prompt": "x"}) + "\n")
    torch.save(torch.rand(3, 10, 12), tmp_path / "img.pt")
    (tmp_path / "i.jsonl").write_text(json.dumps({"image": "img.pt", "caption": "a picture"}) + "\n")
    (tmp_path / "broken.json").write_text("{not json")
    return tmp_path


def test_reader_and_records(files, tok):
    R = PiscesLxToolsDataJsonSampleReader
    R.failures.clear()
    assert R.extract_text({"instruction": "a", "output": "b"}) == "a\nb" and R.extract_text({"messages": [{"content": "x"}, {"content": "y"}]}) == "x\ny"
    assert R.extract_text(5) == "" and len(R.resolve(str(files / "t.jsonl"))) == 8
    allrows = R.scan_directory(str(files))
    assert len(allrows) == 8 + 1 + 2 + 1 and R.failures and "broken.json" in R.failures[0][0]
    with pytest.raises(FileNotFoundError):
        R.resolve(str(files / "none"))
    ids, lab = PiscesLxToolsDataSampleRecord.encode_pair(tok, "abcdefgh", "XY", 6)
    assert len(ids) == 6 and (lab[:3] == -100).all() and lab[3:].tolist() == tok.encode("XY", add_eos=True)
    assert PiscesLxToolsDataSampleRecord.field({"a": "", "b": "v"}, ["a", "b"]) == "v"
    b = pad_collate([{"input_ids": torch.ones(3, dtype=torch.long), "labels": torch.ones(3, dtype=torch.long), "k": "s", "n": 1},
                     {"input_ids": torch.ones(70, dtype=torch.long), "labels": torch.ones(70, dtype=torch.long), "k": "t", "n": 2}], pad_id=9)
    assert b["input_ids"].shape == (2, 128) and b["input_ids"][0, 3] == 9 and b["labels"][0, 3] == -100 and b["k"] == ["s", "t"] and b["n"].tolist() == [1, 2]
    c = PiscesLxToolsDataClassificationDataset([{"text": "a", "label": "pos"}, {"text": "b", "label": "neg"}, {"text": "c", "label": "pos"}, {"text": "d"}], tok, 8)
    assert len(c) == 3 and c.label_map == {"pos": 0, "neg": 1} and c[2]["class_label"] == 0


def test_mixed_sources_weights_and_split(files, tok):
    cfg = PiscesLxDataSourcesConfig(max_seq_length=32, batch_size=2, image_size=8)
    cfg.add_text_data(str(files / "t.jsonl"), weight=2.0).add_conversation_data(str(files / "c.jsonl")).add_preference_data(str(files / "p.jsonl")) \
       .add_image_text_data(str(files / "i.jsonl"))
    ds = PiscesLxMultimodalDataset(cfg, tok)
    kinds = [s["_type"] for s in ds.samples]
    assert kinds.count("text") == 16 and kinds.count("conversation") == 1 and kinds.count("preference") == 1 and kinds.count("image_text") == 1
    conv = ds[kinds.index("conversation")]
    n_lab = int((conv["labels"] != -100).sum())
    assert conv["sample_type"] == "conversation" and 0 < n_lab < len(conv["labels"])
    assert n_lab == len(tok.encode("hello there\n", add_eos=True))
    pref = ds[kinds.index("preference")]
    assert pref["rejected_input_ids"].shape[0] > pref["input_ids"].shape[0] - 5 and (pref["labels"][:3] == -100).all()
    img = ds[kinds.index("image_text")]
    assert img["images"].shape == (3, 8, 8) and img["images"].dtype == torch.float16
    half = PiscesLxDataSourcesConfig(max_seq_length=32, val_fraction=0.25).add_text_data(str(files / "t.jsonl"))
    tr, va = PiscesLxTextDataset(half, tok, "train"), PiscesLxTextDataset(half, tok, "val")
    assert len(tr) == 6 and len(va) == 2 and not {s["text"] for s in tr.samples} & {s["text"] for s in va.samples}
    part = PiscesLxDataSourcesConfig().add_text_data(str(files / "t.jsonl"), weight=0.5)
    assert 0 < len(PiscesLxTextDataset(part, tok)) < 8
    with pytest.raises(ValueError):
        PiscesLxTextDataset(PiscesLxDataSourcesConfig(sources=[{"type": "nope", "path": "x"}]), tok)


def test_dynamic_sampler_budget_and_curriculum(files, tok):
    ds = PiscesLxTextDataset(PiscesLxDataSourcesConfig(max_seq_length=512).add_text_data(str(files / "t.jsonl")), tok)
    s = PiscesLxToolsDataDynamicBatchSampler(ds, max_tokens=256, seed=1)
    batches = list(s)
    assert sorted(i for b in batches for i in b) == list(range(8)) and len(s) == len(batches)
    for b in batches:
        longest = max(s.lengths[i] for i in b)
        assert s._padded(longest) * len(b) <= 256 or len(b) == 1
    assert 0.0 <= s.padding_waste() < 0.8
    s.set_epoch(1)
    assert list(s) != batches or len(batches) == 1
    c = PiscesLxToolsDataCurriculumSampler(ds, total_steps=4, start_fraction=0.25, shuffle=False)
    assert len(c) == 2 and list(c) == c.order[:2] and c.difficulties[c.order[0]] <= c.difficulties[c.order[-1]]
    c.step(); c.step()
    assert len(c) == 5
    c.set_step(100)
    assert len(c) == 8


def test_optimized_loader_module_and_prefetch(files, tok):
    cfg = PiscesLxDataSourcesConfig(max_seq_length=64, batch_size=3, val_fraction=0.25).add_text_data(str(files / "t.jsonl"))
    dm = PiscesLxDataModule(cfg, tok)
    with pytest.raises(RuntimeError):
        dm.train_dataloader()
    dm.setup("fit")
    tb = list(dm.train_dataloader())
    assert sum(b["input_ids"].shape[0] for b in tb) == 6 and all(b["input_ids"].shape[1] % PAD_MULTIPLE == 0 for b in tb)
    assert sum(b["input_ids"].shape[0] for b in dm.val_dataloader()) == 2
    dyn = PiscesLxDataModule(cfg, tok, max_tokens=128)
    dyn.setup()
    assert all(b["input_ids"].numel() <= 128 or b["input_ids"].shape[0] == 1 for b in dyn.train_dataloader())
    ds = dm.datasets["train"]
    dist = [PiscesLxToolsDataOptimizedDataLoader(ds, PiscesLxToolsDataBatchConfig(batch_size=2, shuffle=False), rank=r, world=2).get() for r in range(2)]
    assert sum(b["input_ids"].shape[0] for d in dist for b in d) == 6
    pre = PiscesLxToolsDataOptimizedDataLoader(ds, PiscesLxToolsDataBatchConfig(batch_size=2)).get_prefetched(2, torch.device("cpu"))
    assert isinstance(pre, PiscesLxToolsDataPrefetchDataLoader) and len(pre) == 3 and sum(b["input_ids"].shape[0] for b in pre) == 6
    dl, samp = PiscesLxToolsDataOptimizedDataLoader(ds, PiscesLxToolsDataBatchConfig(batch_size=2)).get_curriculum(total_steps=2, start_fraction=0.5)
    assert sum(b["input_ids"].shape[0] for b in dl) == 3
    samp.set_step(2)
    assert sum(b["input_ids"].shape[0] for b in dl) == 6
    assert len(PiscesLxToolsDataOptimizedDataLoader.create_dataloader(ds, batch_size=4, shuffle=False)) == 2
    m2 = PiscesLxDataModule.create_datamodule(text=str(files / "t.jsonl"), preferences=str(files / "p.jsonl"), tokenizer=tok, batch_size=2, max_seq_length=16)
    assert m2.multimodal and len(m2.config.sources) == 2
    dm.teardown()
    assert dm.datasets == {}


def test_streaming_dataset(files, tok):
    st = PiscesLxStreamingDataset(str(files), tok, max_seq_length=16, shuffle_buffer=4, seed=0)
    rows = list(st)
    assert len(rows) >= 11 and all(len(r["input_ids"]) <= 16 for r in rows)
    a = list(PiscesLxStreamingDataset(str(files), tok, rank=0, world=2))
    b = list(PiscesLxStreamingDataset(str(files), tok, rank=1, world=2))
    assert len(a) + len(b) == len(rows)
    it = PiscesLxDataIterableDataset(list(range(5)), shuffle=True, seed=1, repeat=True)
    g = iter(it)
    first = [next(g) for _ in range(5)]
    second = [next(g) for _ in range(5)]
    assert sorted(first) == sorted(second) == list(range(5)) and len(it) == 5


def test_buffer_prefetcher_and_memory():
    buf = PiscesLxToolsDataStreamingDataBuffer(2)
    assert buf.put(1) and buf.put(2) and buf.is_full() and buf.size() == 2
    t = threading.Thread(target=lambda: buf.put(3))
    t.start()
    assert buf.get() == 1
    t.join(2)
    assert buf.get() == 2 and buf.get() == 3 and buf.get(timeout=0.05) is None and buf.is_empty()
    buf.stop()
    assert not buf.put(4) and buf.is_stopped() and buf.get() is None

    class Slow:
        def __len__(self):
            return 20

        def __getitem__(self, i):
            if i == 13:
                raise KeyError("bad row")
            return {"i": i}
    assert [r["i"] for r in PiscesLxDataPrefetcher(Slow(), queue_size=4, num_workers=3, indices=range(10))] == list(range(10))
    with pytest.raises(KeyError):
        list(PiscesLxDataPrefetcher(Slow(), queue_size=4, num_workers=2))
    m = PiscesLxToolsDataMemoryMonitor()
    assert m.check_memory() > 0 and m.get_peak_memory() > 0 and m.get_memory_stats()["samples"] == 2.0
    assert PiscesLxToolsMemoryMonitor(1e6).check_memory()["over_threshold"] == 0.0


def test_cached_dataset(tok):
    items = [{"text": "alpha beta gamma delta " * 4, "image": "a.png"}, {"content": "short", "snd": "x.wav"}]
    cfg = PiscesLxDatasetConfig(max_text_length=10, truncate_mode="middle", custom_audio_keys="snd", return_quality_score=True, cache_size=1)
    ds = PiscesLxDataset(items, cfg, tok)
    a = ds[0]
    full = tok.encode(items[0]["text"], add_eos=True)
    assert a["input_ids"].tolist() == full[:5] + full[-5:] and a["image_path"] == "a.png" and 0 < a["quality_score"] <= 1.0
    assert ds[0] is a and ds.cache_hits == 1
    assert ds[1]["audio_path"] == "x.wav" and len(ds._cache) == 1
    assert [r["input_ids"].shape[0] for r in ds.get_prefetcher(2, 1)] == [10, len(tok.encode("short", add_eos=True))]
    PiscesLxDataset.set_global_cache("k", 1)
    assert PiscesLxDataset.get_global_cache("k") == 1
    PiscesLxDataset.clear_global_cache()
    assert PiscesLxDataset.get_global_cache("k") is None
    aug = PiscesLxDataset(items, PiscesLxDatasetConfig(augmentation_enabled=True, text_augmentation_prob=1.0), tok)
    assert aug[0]["input_ids"].numel() > 0 and len(aug._cache) == 0
    assert PiscesLxDataset(items, PiscesLxDatasetConfig(max_text_length=4, truncate_mode="head"), tok)[0]["input_ids"].tolist() == full[-4:]
