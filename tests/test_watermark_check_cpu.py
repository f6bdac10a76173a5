"""Watermark detection, model verification, content integrity, pipeline integration."""
import hashlib

import pytest
import torch
import torch.nn as nn

from pisceslx_b200.third_party.watermark_check import (InferencePipelineWatermarkOperator, InferenceWatermarkIntegrationOperator, PiscesLxContentIntegrityCheckOperator,
                                                       PiscesLxModelWatermarkVerificationOperator, PiscesLxWatermarkDetectionOperator, TrainingPipelineWatermarkOperator,
                                                       TrainingWatermarkIntegrationOperator)


def _smooth(c, h, w):
    low = torch.rand(1, c, h // 16, w // 16)
    return (torch.nn.functional.interpolate(low, size=(h, w), mode="bicubic", align_corners=False).clamp(0, 1) * 0.6 + 0.2)[0]


def test_detection_across_kinds():
    torch.manual_seed(0)
    d = PiscesLxWatermarkDetectionOperator()
    payload = {"m": "yv", "t": 1}
    marked = d.content.embed_text("some generated text", payload)
    r = d.detect_text_watermark(marked)
    assert r["detected"] and r["payload"] == payload and not r["damaged"]
    broken = marked.replace(d.content.ZW1, "", 3)
    rb = d.detect_text_watermark(broken)
    assert not rb["detected"] and rb["damaged"] and not d.detect_text_watermark("plain")["detected"]
    img = _smooth(3, 256, 256)
    out, n = d.content.embed_image(img, payload)
    ri = d.detect_image_watermark(out, num_bits=n)
    assert ri["detected"] and ri["payload"] == payload and not d.detect_image_watermark(img, num_bits=n)["detected"]
    m = nn.Linear(128, 128)
    assert not d.detect_model_watermark(m)["detected"]
    d.weights.wm.eps = 5e-3
    d.weights.embed(m)
    assert d.detect_model_watermark(m)["detected"]
    mm = d.detect_multimodal_watermark({"text": marked, "model": m, "image": img, "num_bits": n})
    assert mm["detected"] and not mm["all_detected"] and set(mm["per_modality"]) == {"text", "image", "model"}
    batch = d.batch_detect([marked, "plain", m, 3.5])
    assert [b["detected"] for b in batch] == [True, False, True, False] and "error" in batch[3]
    st = d.get_detection_statistics()
    assert st["text"]["checked"] >= 5 and 0 < st["text"]["rate"] < 1 and d.execute({"content": marked}).output["detected"]


def test_model_verification_signature_and_fingerprint():
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(64, 64), nn.Linear(64, 8))
    v = PiscesLxModelWatermarkVerificationOperator(sensitivity="high")
    sig, fp = v.signature(m), v._compute_model_fingerprint(m)
    ok = v.verify_model_integrity(m, sig, fp)
    assert ok["intact"] and ok["fingerprint_match"] and ok["similarity"] == 1.0 and ok["changed_tensors"] == [] and len(sig["0.weight"]) == 10
    with torch.no_grad():
        m[1].weight.add_(0.5)
    bad = v.verify_model_integrity(m, sig, fp)
    assert not bad["intact"] and not bad["fingerprint_match"] and bad["similarity"] < 1.0 and "1.weight" in bad["changed_tensors"]
    with torch.no_grad():
        m[0].weight[0, 0] = float("nan")
    assert "0.weight" in v.verify_model_integrity(m)["non_finite_tensors"] and not v.execute({"model": m}).output["intact"]
    assert v.transform("x") == "x"


def test_content_integrity():
    c = PiscesLxContentIntegrityCheckOperator()
    good = c.check_content_integrity("A normal sentence (with brackets) and `code`.")
    assert good["intact"] and good["kind"] == "text" and good["sha256"] == hashlib.sha256("A normal sentence (with brackets) and `code`.".encode()).hexdigest()
    bad = c.check_content_integrity("broken (text\x00 with ``` fence " + "abcd" * 20 + " �")
    assert not bad["intact"] and {"unbalanced brackets", "unclosed code fence", "degenerate repetition"} <= set(bad["issues"]) and any("control" in i for i in bad["issues"])
    assert not c.check_content_integrity("ok", expected_sha256="00")["intact"]
    rnd = torch.randint(0, 256, (8192,), dtype=torch.uint8).numpy().tobytes()
    assert any("entropy" in i for i in c.check_content_integrity(rnd)["issues"]) and any("constant" in i for i in c.check_content_integrity(b"\x00" * 100)["issues"])
    assert c.check_content_integrity(b"hello world, this is plain text " * 4)["intact"] and not c.check_content_integrity(b"")["intact"]
    t = torch.randn(4, 4)
    assert c.check_content_integrity(t)["intact"]
    t[0, 0] = float("inf")
    r = c.execute({"content": t}).output
    assert not r["intact"] and r["metrics"]["inf"] == 1 and not c.check_content_integrity(torch.ones(5))["intact"]
    with pytest.raises(TypeError):
        c.check_content_integrity(3)


def test_pipeline_integration(tmp_path):
    inf = InferenceWatermarkIntegrationOperator(jurisdiction="US", model_id="yv")
    det = PiscesLxWatermarkDetectionOperator(policy=inf.orch.policy)
    out = inf.transform({"results": ["first answer here", "second answer here"], "count": 2})
    assert out["watermarked"] and all(det.detect_text_watermark(t)["detected"] for t in out["results"]) and out["count"] == 2
    assert InferenceWatermarkIntegrationOperator(enabled=False).transform("x") == "x" and inf.execute({"data": "a b"}).output["data"] != "a b"
    cb = InferencePipelineWatermarkOperator(jurisdiction="US")
    outs = ["an answer to mark"]
    cb("postprocessing_end", processed_outputs=outs)
    assert det.detect_text_watermark(outs[0])["detected"]
    cb("batch_start", prompts=[])
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(128, 128))
    tr = TrainingWatermarkIntegrationOperator(eps=5e-3, audit_path=str(tmp_path / "a.jsonl"))
    r1 = tr.execute({"model": m}).output
    assert r1["marked"] == ["0.weight"] and not r1["already_marked"] and len(r1["fingerprint"]) == 32
    w = m[0].weight.clone()
    r2 = tr.transform(m)
    assert r2["already_marked"] and r2["marked"] == [] and torch.equal(m[0].weight, w) and len(tr.audit.records) == 2
    assert tr.verifier.verify_model_integrity(m, r1["signature"], r1["fingerprint"])["intact"]

    class T:
        model = nn.Sequential(nn.Linear(128, 128))
    tp = TrainingPipelineWatermarkOperator(eps=5e-3).bind(T())
    tp("training_start", total_epochs=1)
    assert tp.result["marked"] == ["0.weight"] and TrainingWatermarkIntegrationOperator(enabled=False).transform(m)["skipped"]
