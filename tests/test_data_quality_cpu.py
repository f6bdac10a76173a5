"""Language / domain / perplexity / readability signals, the incremental ledger and the quality-aware cleaner."""
import json
import math

import pytest

from pisceslx_b200.data.quality import (PiscesLxDataCleaningConfig, PiscesLxDataDomainClassifier,
                                        PiscesLxDataIncrementalState, PiscesLxDataLanguageDetector,
                                        PiscesLxDataPerplexityCalculator, PiscesLxDataQualityAwareCleaner,
                                        PiscesLxDataReadabilityScorer, PiscesLxLanguageType as L)

EN = "The committee reviewed the proposal carefully and decided that the bridge should be rebuilt before winter arrives."


def test_language_detection():
    d = PiscesLxDataLanguageDetector.detect
    assert d(EN) == L.ENGLISH and d("") == L.UNKNOWN and d(None) == L.UNKNOWN and d("12345 !!!") == L.UNKNOWN
    assert d("今天天气很好，我们一起去公园散步吧。") == L.CHINESE
    assert d("今日はとても良い天気ですので、公園へ散歩に行きましょう。") == L.JAPANESE
    assert d("오늘은 날씨가 정말 좋아서 공원에 산책하러 갑니다.") == L.KOREAN
    assert d("Сегодня очень хорошая погода, и мы идём гулять в парк.") == L.RUSSIAN
    assert d("اليوم الطقس جميل جدا ونذهب إلى الحديقة") == L.ARABIC
    assert d("Le chat est dans la maison et il dort pour la nuit que les enfants aiment.") == L.FRENCH
    assert d("Der Hund ist nicht auf dem Sofa und die Katze ist mit den Kindern zu Hause.") == L.GERMAN
    assert d("El perro es de los vecinos y las flores en el jardín son para la fiesta con amigos.") == L.SPANISH
    assert d("def add(a, b):\n    return a + b\n\nclass Foo:\n    import os\n    print(add(1, 2))") == L.CODE
    assert d("The weather 今天天气很好我们去公园 is nice today for a walk") == L.MIXED


def test_domain_classifier():
    c = PiscesLxDataDomainClassifier
    assert c.classify("The patient received treatment after the diagnosis; the doctor adjusted the drug dosage.")[0] == "medical"
    assert c.classify("Solve the equation using the derivative and the integral of the polynomial.")[0] == "math"
    assert c.classify("The court heard the lawsuit; the judge read the verdict to the defendant.")[0] == "legal"
    assert c.classify("zzz qqq")[0] == "general" and c.classify(None) == ("general", 0.0)
    s = c.get_multi_domain_scores("The stock market and the bank loan interest")
    assert max(s, key=s.get) == "finance" and set(s) == set(c._DOMAIN_KEYWORDS)


def test_perplexity_model_and_fallback():
    p = PiscesLxDataPerplexityCalculator()
    rep = p.calculate("spam spam spam spam spam spam spam spam")
    var = p.calculate(EN)
    assert rep == pytest.approx(1.0) and var > 10 and p.calculate("") is None and p.calculate(None) is None
    m = PiscesLxDataPerplexityCalculator(token_logprobs=lambda t: [math.log(0.25)] * 7)
    assert m.calculate("anything") == pytest.approx(4.0)


def test_readability():
    r = PiscesLxDataReadabilityScorer
    easy = r.calculate("The cat sat on the mat. The dog ran to the park. We had fun.")
    hard = r.calculate("Notwithstanding the aforementioned considerations, institutional heterogeneity necessitates "
                       "comprehensive interdisciplinary reconceptualisation of organisational accountability.")
    assert 0.8 < easy <= 1.0 and hard < 0.2 and r.calculate("") == 0.0
    assert r._count_syllables("table") == 2 and r._count_syllables("make") == 1 and r._count_syllables("the") == 1
    good = r.calculate("今天天气很好，我们一起去公园散步吧，路上还买了一些水果和饮料。", L.CHINESE)
    assert 0.8 < good <= 1.0


def test_quality_aware_cleaner_filters_and_counts():
    cl = PiscesLxDataQualityAwareCleaner(PiscesLxDataCleaningConfig(quality_threshold=0.6, min_text_length=10, dedup_enabled=True,
                                                                   dedup_method="exact"))
    t, s, m = cl.clean_with_quality("  " + EN + "!!!!   \x00")
    assert t.endswith("arrives.!") and s >= 0.6 and m["language"] == "english" and "reason" not in m
    assert cl.clean_with_quality(EN + "!")[2]["reason"] == "duplicate"
    assert cl.clean_with_quality("short")[2]["reason"] == "too_short" and cl.clean_with_quality(None)[2]["reason"] == "empty_or_invalid"
    junk = "$$$ ### @@@ %%% ^^^ &&& *** ((( ))) " * 5
    assert cl.clean_with_quality(junk)[2]["reason"] == "low_quality"
    assert cl.clean_with_quality("buy buy buy buy buy buy buy buy buy buy buy buy buy")[2]["reason"] == "low_quality"
    st = cl.get_stats()
    assert st["total_processed"] == 1 and st["filtered_out"] == 2 and st["duplicates"] == 1
    assert cl._normalize_text("soooooooo   good") == "sooo good"
    only_en = PiscesLxDataQualityAwareCleaner(PiscesLxDataCleaningConfig(allowed_languages=("english",)))
    assert only_en.clean_with_quality("今天天气很好，我们一起去公园散步吧。")[2]["reason"] == "language"
    kept = list(only_en.clean([EN, "今天天气很好，我们一起去公园散步吧。", ""]))
    assert len(kept) == 1 and kept[0][1]["domain"] in PiscesLxDataDomainClassifier._DOMAIN_KEYWORDS | {"general": 0}.keys()


def test_incremental_cleaning_skips_unchanged_files(tmp_path):
    a, b = tmp_path / "a.jsonl", tmp_path / "b.txt"
    a.write_text(json.dumps({"text": EN, "source": "wiki"}) + "\n" + json.dumps({"text": "$$$ ### @@@ %%% ^^^ &&& ***"}) + "\n")
    b.write_text("A second document about the harvest festival that the whole village celebrates every autumn.\n\n")
    out = tmp_path / "out" / "clean.jsonl"
    ledger = tmp_path / "state" / "ledger.json"
    cl = PiscesLxDataQualityAwareCleaner(PiscesLxDataCleaningConfig(quality_threshold=0.55))
    st = PiscesLxDataIncrementalState(str(ledger))
    r1 = cl.clean_files([str(a), str(b)], str(out), st)
    assert r1 == {"files_skipped": 0, "samples_seen": 3, "samples_kept": 2}
    rows = [json.loads(l) for l in out.read_text().splitlines()]
    assert rows[0]["source"] == "wiki" and rows[0]["language"] == "english" and 0 < rows[0]["quality"] <= 1
    st2 = PiscesLxDataIncrementalState(str(ledger))                 # another run reads the ledger
    assert st2.is_processed(str(a)) and st2.processed_samples == 2
    r2 = cl.clean_files([str(a), str(b)], str(out), st2)
    assert r2["files_skipped"] == 2 and r2["samples_seen"] == 0
    b.write_text("A changed document that talks about the river and the old mill beside the wooden bridge in town.\n")
    r3 = cl.clean_files([str(a), str(b)], str(out), st2)
    assert r3["files_skipped"] == 1 and r3["samples_kept"] == 1
    assert not st2.is_processed(str(tmp_path / "missing.txt"))
