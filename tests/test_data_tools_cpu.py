"""CPU tests of augmentation, sample caches, offline teacher records, dataset resolution, and monitor alerts."""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch


def test_token_and_text_augmenters():
    from pisceslx_b200.data.augment import PiscesLxTextAugmenter, PiscesLxTokenAugmenter
    aug = PiscesLxTokenAugmenter(1000, mask_token_id=999, seed=0)
    ids = list(range(200))
    d = aug.token_dropout(ids, 0.2)
    assert 120 < len(d) < 190 and d == sorted(d)
    r, lab = aug.random_replace(ids, 0.1)
    changed = [i for i in range(200) if lab[i] == -100]
    assert 5 < len(changed) < 45 and all(r[i] == ids[i] for i in range(200) if lab[i] != -100)
    m, ml = aug.span_mask(ids, 0.15, 3)
    masked = [i for i in range(200) if m[i] == 999]
    assert 0 < len(masked) <= 30 and all(ml[i] == ids[i] for i in masked) and all(ml[i] == -100 for i in range(200) if i not in masked)
    s = aug.swap_adjacent(ids, 0.3)
    assert sorted(s) == ids and s != ids
    t = PiscesLxTextAugmenter(1)
    assert len(t.word_dropout("a b c d e f g h", 0.5).split()) < 8
    assert sorted(t.typo("hello world example", 0.5)) == sorted("hello world example")
    assert t.template({"q": "2+2", "a": "4"}, ["Q: {q} A: {a}"]) == "Q: 2+2 A: 4"


def test_lru_and_token_caches(tmp_path):
    from pisceslx_b200.data.augment import PiscesLxDataLRUCache, PiscesLxDataTokenCache
    c = PiscesLxDataLRUCache(max_bytes=3 * 400)
    made = []
    for k in [0, 1, 2, 0, 3, 1]:
        c.get(k, lambda k=k: made.append(k) or np.full(100, k, dtype=np.int32))
    assert made == [0, 1, 2, 3, 1] and c.hits == 1 and list(c.d) == [0, 3, 1]
    src = tmp_path / "corpus.txt"
    src.write_text("x")
    tc = PiscesLxDataTokenCache(str(tmp_path / "cache"))
    key = tc.key(str(src), "tok-a")
    assert key != tc.key(str(src), "tok-b") and tc.open(key) is None
    arr, off = tc.build(key, [[1, 2, 3], [4, 5], []])
    assert off == [0, 3, 5, 5] and arr[off[1]:off[2]].tolist() == [4, 5]
    arr2, off2 = tc.open(key)
    assert arr2.tolist() == [1, 2, 3, 4, 5] and off2 == off


def test_offline_teacher_and_dataset_resolution(tmp_path, monkeypatch):
    from pisceslx_b200.data.augment import (PiscesLxDatasetUnavailable, PiscesLxOfflineTeacherProvider, resolve_dataset)

    class Teacher:
        def __call__(self, input_ids):
            torch.manual_seed(int(input_ids.sum()))
            return type("O", (), {"logits": torch.randn(*input_ids.shape, 50)})()
    prov = PiscesLxOfflineTeacherProvider(str(tmp_path / "teacher.jsonl"), k=4)
    n = prov.record(Teacher(), [torch.randint(0, 50, (2, 6))])
    recs = list(prov)
    assert n == 2 and len(recs) == 2 and len(recs[0].topk_ids) == 6 and len(recs[0].topk_ids[0]) == 4
    # a student equal to the teacher (on the stored support) has zero loss; a different one has more
    lp = torch.full((6, 50), -30.0)
    for t, (ids, v) in enumerate(zip(recs[0].topk_ids, recs[0].topk_logprobs)):
        lp[t, ids] = torch.tensor(v)
    assert float(prov.sparse_kl(lp, recs[0])) < 1e-4
    assert float(prov.sparse_kl(torch.randn(6, 50), recs[0])) > 0.01
    (tmp_path / "data" / "org__set").mkdir(parents=True)
    assert resolve_dataset("org/set", [str(tmp_path / "data")]).endswith("org__set")
    with pytest.raises(PiscesLxDatasetUnavailable) as e:
        resolve_dataset("org/missing", [str(tmp_path / "data")])
    assert "not available offline" in str(e.value)


def test_alert_manager_and_stats():
    from pisceslx_b200.utils.alerts import PiscesLxAlertManager, PiscesLxAlertRule, PiscesLxStatsCollector
    now = [0.0]
    got = []
    am = PiscesLxAlertManager([PiscesLxAlertRule("mem", "gpus.0.memory_used_frac", ">", 0.9, hold_s=10, cooldown_s=100)],
                              sinks=[got.append], clock=lambda: now[0])
    snap = {"gpus": [{"memory_used_frac": 0.95}]}
    assert am.evaluate(snap) == []                   # not held long enough
    now[0] = 5
    assert am.evaluate({"gpus": [{"memory_used_frac": 0.5}]}) == []     # condition cleared: hold restarts
    now[0] = 6
    am.evaluate(snap)
    now[0] = 17
    fired = am.evaluate(snap)
    assert len(fired) == 1 and fired[0].rule == "mem" and got == fired
    now[0] = 50
    assert am.evaluate(snap) == []                   # cooling down
    now[0] = 120
    assert len(am.evaluate(snap)) == 1
    assert am.evaluate({"gpus": []}) == [] and len(PiscesLxAlertManager.default_rules()) >= 4
    st = PiscesLxStatsCollector(window=4)
    for v in [10, 10, 10, 10, 10, 5]:
        st.add("tps", v)
    s = st.summary("tps")
    assert s["n"] == 4 and s["min"] == 5 and abs(s["last_over_mean"] - 5 / 8.75) < 1e-9 and st.summary("none") == {}
