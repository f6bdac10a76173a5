"""Dataset acquisition: source routing with a local mirror, retry, resume; parquet corpus; shard-parallel cleaning."""
import json

from pisceslx_b200.data import acquire as aq


def _mirror(tmp_path):
    root = tmp_path / "mirror"
    (root / "org__corpus").mkdir(parents=True)
    with open(root / "org__corpus" / "part0.jsonl", "w") as f:
        for i in range(10):
            f.write(json.dumps({"text": f"document number {i} with enough characters"}) + "\n")
    (root / "plain.txt").write_text("first line of plain text\n\nsecond line of plain text\n")
    return root


def test_download_from_mirror_with_resume_and_failure_report(tmp_path):
    root = _mirror(tmp_path)
    cfg = aq.PiscesLxToolsDataDownloadConfig(
        [aq.PiscesLxToolsDatasetItem("org/corpus", source_preference=["hf"], max_samples=4),
         aq.PiscesLxToolsDatasetItem("plain"), aq.PiscesLxToolsDatasetItem("missing/dataset")],
        data_dir=str(tmp_path / "data"), mirror=f"file://{root}")
    dl = aq.PiscesLxToolsDataDatasetDownload(retry=aq.PiscesLxDataRetryStrategy(2, sleep=lambda s: None))
    rep = dl.download(cfg)
    assert rep["completed"] == ["org__corpus", "plain"] and "missing__dataset" in rep["failed"]
    assert "FileNotFoundError" in rep["failed"]["missing__dataset"]          # no hub reachable, not in the mirror
    rows = [json.loads(l) for l in open(tmp_path / "data" / "org__corpus.jsonl")]
    assert len(rows) == 4 and rows[0]["text"].startswith("document number 0")
    assert len(open(tmp_path / "data" / "plain.jsonl").readlines()) == 2
    resume = aq.PiscesLxDataResumeManager(str(tmp_path / "data" / ".download_state"))
    st = resume.load_state("org__corpus")
    assert st.status == "completed" and st.source == "local" and st.records == 4
    rep2 = dl.download(cfg)                                                   # second run: nothing to redo
    assert rep2["skipped"] == ["org__corpus", "plain"] and rep2["completed"] == []
    item = aq.PiscesLxToolsDatasetItem("x", source_preference=["HF", "ms", "hf"])
    assert item.normalize_source_preference(["local", "kaggle"]) == ["huggingface", "modelscope", "local", "kaggle"]


def test_retry_strategy_and_flaky_source(tmp_path):
    delays = []
    retry = aq.PiscesLxDataRetryStrategy(max_attempts=3, base_delay=1.0, jitter=0.0, sleep=delays.append)
    assert [retry.get_delay(a) for a in (1, 2, 3)] == [1.0, 2.0, 4.0]
    assert retry.should_retry(1, TimeoutError()) and not retry.should_retry(3, TimeoutError())
    assert not retry.should_retry(1, FileNotFoundError())

    class Flaky(aq.PiscesLxDataSource):
        name, calls = "flaky", 0

        def available(self):
            return True

        def fetch(self, item, dest):
            Flaky.calls += 1
            if Flaky.calls < 3:
                raise ConnectionError("reset by peer")
            return aq._write_jsonl(({"text": str(i)} for i in range(3)), dest / f"{item.save_name}.jsonl", None)

    router = aq.PiscesLxToolsDataSourceRouter(extra={"flaky": Flaky()})
    cfg = aq.PiscesLxToolsDataDownloadConfig([aq.PiscesLxToolsDatasetItem("d", source_preference=["flaky"])],
                                             data_dir=str(tmp_path / "out"), source_preference=[])
    rep = aq.PiscesLxToolsDataDatasetDownload(router, retry).download(cfg)
    assert rep["completed"] == ["d"] and Flaky.calls == 3 and delays == [1.0, 2.0]


def test_parquet_corpus_and_distributed_cleaning(tmp_path):
    recs = [{"text": f"parquet row {i} padded to a useful length", "id": i} for i in range(25)]
    path = str(tmp_path / "c.parquet")
    assert aq.PiscesLxToolsDataParquetCorpus.write(recs, path, rows_per_group=10) == 25
    full = aq.PiscesLxToolsDataParquetCorpus(path)
    assert len(full) == 25 and next(full.texts()).startswith("parquet row 0")
    r0, r1 = aq.PiscesLxToolsDataParquetCorpus(path, rank=0, world=2), aq.PiscesLxToolsDataParquetCorpus(path, rank=1, world=2)
    assert len(r0) + len(r1) == 25 and len(r0) == 15                        # row groups 0 and 2 / row group 1
    shards = tmp_path / "shards"
    shards.mkdir()
    for s in range(3):
        with open(shards / f"s{s}.jsonl", "w") as f:
            for i in range(6):
                f.write(json.dumps({"text": f"a sentence that is long enough to keep, number {i + 2 * s}"}) + "\n")
            f.write(json.dumps({"text": "short"}) + "\n")
    texts = aq.PiscesLxDataDistributedLoader(str(shards / "*.jsonl"), workers=2).load()
    assert len(texts) == 21
    rep = aq.PiscesLxDataDistributedCleaner(str(shards / "*.jsonl"), str(tmp_path / "clean"), workers=2, min_chars=20).run()
    # numbers 0..9 are distinct; shards overlap by four sentences each
    assert rep["in"] == 21 and rep["kept"] == 10 and rep["cross_shard_duplicates"] == 8 and rep["shards"] == 3
    kept = [json.loads(l)["text"] for p in rep["outputs"] for l in open(p)]
    assert len(kept) == len(set(kept)) == 10
