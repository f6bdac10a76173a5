"""Watermark operators: policy / compliance, protocol framing, batched DCT mark, hash-chained audit, content, weights, orchestrator."""
import json

import pytest
import torch
import torch.nn as nn

from pisceslx_b200.third_party.watermark_ops import (
    POPSSAuditOperator, POPSSComplianceOperator, POPSSContentWatermarkOperator, POPSSDCTOperator, POPSSFrameInfo, POPSSProtocolOperator,
    POPSSWatermarkComplianceValidator, POPSSWatermarkDCTOperator, POPSSWatermarkDefaultConfigFactory, POPSSWatermarkJurisdiction, POPSSWatermarkOrchestrator,
    POPSSWatermarkPayload, POPSSWatermarkPolicy, POPSSWeightWatermarkOperator)


def _smooth(*shape):
    """A smooth picture (low-resolution noise scaled up), like a photograph: little energy in the middle frequencies."""
    lead, (h, w) = shape[:-2], shape[-2:]
    low = torch.rand(*lead, h // 16, w // 16) if len(lead) == 2 else torch.rand(1, *lead, h // 16, w // 16)
    up = torch.nn.functional.interpolate(low, size=(h, w), mode="bicubic", align_corners=False).clamp(0, 1) * 0.6 + 0.2
    return up if len(lead) == 2 else up[0]


def test_policies_and_validation():
    cn, us = POPSSWatermarkDefaultConfigFactory.create("CN"), POPSSWatermarkDefaultConfigFactory.create(POPSSWatermarkJurisdiction.US)
    assert cn.visible_label and cn.mandatory_disclosure and not us.mandatory_disclosure and us.redundancy == 2
    both = POPSSWatermarkDefaultConfigFactory.strictest(["CN", "EU"])
    assert both.visible_label and both.encrypt_payload and both.audit_retention_days == 365 and len(both.standards) == 4
    v = POPSSWatermarkComplianceValidator()
    ok = v.validate(cn)
    assert ok["compliant"] and ok["score"] == 1.0 and ok["jurisdiction"] == "CN"
    weak = POPSSWatermarkPolicy(jurisdiction="CN", mandatory_disclosure=False, audit_trail=False, redundancy=1, strength=0.01)
    bad = v.validate(weak)
    assert not bad["compliant"] and {c["name"] for c in bad["violations"]} == {"mandatory_disclosure", "audit_trail", "strength"} and bad["score"] < 0.3
    assert any("redundancy" in r for r in bad["recommendations"])
    p = POPSSWatermarkPayload(model_id="a-very-long-model-identifier")
    assert p.timestamp > 0 and len(p.nonce) == 8 and p.compact()["m"] == "a-very-long-" and set(p.compact()) == {"m", "t", "j", "r"}


def test_protocol_framing_survives_bit_errors_with_redundancy():
    pr = POPSSProtocolOperator()
    payload = {"m": "yv", "t": 1700000000, "j": "EU"}
    bits = pr.frame_payload(payload, redundancy=3)
    assert len(bits) == 3 * (16 + 16 + 8 * len(json.dumps(payload, separators=(",", ":"), sort_keys=True)) + 32)
    assert pr.extract_from_bits(bits, 3) == payload
    noisy = list(bits)
    for i in range(0, len(noisy), 3):                                                    # one error in every group of three
        noisy[i] = "1" if noisy[i] == "0" else "0"
    info = pr.decode_frame("".join(noisy), 3)
    assert isinstance(info, POPSSFrameInfo) and info.is_valid() and info.payload == payload and info.bit_errors_corrected == len(bits) // 3
    plain = pr.frame_payload(payload)
    broken = plain[:40] + ("1" if plain[40] == "0" else "0") + plain[41:]
    b = pr.decode_frame(broken)
    assert b.sync_ok and not b.crc_ok and pr.extract_from_bits(broken) is None and pr.extract_from_bits("0101") is None
    out = pr.execute({"action": "decode", "bits": "00" + plain + "11"}).output          # leading noise before the sync word
    assert out["valid"] and out["payload"] == payload
    assert pr._bits_to_bytes("0100000") is None and pr._int_to_bits(5, 4) == "0101"


def test_dct_is_orthonormal_and_batched_mark_round_trips():
    torch.manual_seed(0)
    op = POPSSWatermarkDCTOperator.create()
    C = op.dct_matrix(8)
    assert torch.allclose(C @ C.t(), torch.eye(8), atol=1e-5)
    x = torch.rand(3, 32, 40)
    X = op.block_dct2(x)
    assert X.shape == (3, 4, 5, 8, 8) and torch.allclose(op.block_idct2(X), x, atol=1e-5)
    assert torch.allclose(X[1, 2, 3], C @ x[1, 16:24, 24:32] @ C.t(), atol=1e-5)          # equals the per-block definition
    img = _smooth(2, 3, 64, 64)
    bits = "1011001110001101"
    out = op.execute({"action": "embed", "image": img, "bits": bits, "strength": 0.08}).output
    assert out["image"].shape == img.shape and out["psnr_db"] > 32 and not torch.equal(out["image"], img)
    got = op.execute({"action": "extract", "image": out["image"], "num_bits": 16}).output
    assert got["bits"] == bits and got["mean_confidence"] > 0.9
    noisy = (out["image"] + 0.005 * torch.randn_like(img)).clamp(0, 1)
    assert op.extract(noisy[1], 16)[0] == bits                                           # the second image of the batch, with noise
    assert op.extract(img, 16)[0] != bits
    gray = torch.rand(37, 45)
    assert op.embed(gray, "10").shape == gray.shape
    with pytest.raises(ValueError):
        op.embed(torch.rand(16, 16), "1" * 5)
    with pytest.raises(ValueError):
        op.embed(img, "12")
    vis = op.embed_visible(img)
    assert not torch.equal(vis[..., -4:, -4:], img[..., -4:, -4:]) and torch.equal(vis[..., :8, :8], img[..., :8, :8])
    a, b = POPSSDCTOperator.enforce_pair_relation(torch.tensor([1.0, -5.0, 0.5]), torch.tensor([2.0, 1.0, -3.0]), torch.tensor([True, True, False]), 0.5)
    assert a.tolist() == [2.5, -5.0, 0.5] and b.tolist() == [2.0, 1.0, -3.0]


def test_audit_chain_detects_tampering(tmp_path):
    path = tmp_path / "audit.jsonl"
    a = POPSSAuditOperator(path=str(path))
    for i in range(5):
        a.log_operation("embed" if i % 2 == 0 else "verify", "text", "m", "EU", success=i != 3, timestamp=1000.0 + i)
    assert a.verify_chain_integrity() == (True, []) and len(path.read_text().splitlines()) == 5
    rep = a.generate_report()
    assert rep["total"] == 5 and rep["failures"] == 1 and rep["by_operation"] == {"embed": 3, "verify": 2} and rep["chain_intact"]
    assert len(a.query({"operation": "verify"})) == 2 and len(a.query(start=1002.0, end=1003.0)) == 2 and len(a.query(limit=1)) == 1
    again = POPSSAuditOperator(path=str(path))
    assert len(again.records) == 5 and again.verify_chain_integrity()[0]
    again.records[2]["success"] = False
    ok, bad = again.verify_chain_integrity()
    assert not ok and bad == [2]
    del a.records[1]
    assert a.verify_chain_integrity()[1] == [1, 2, 3]
    fresh = POPSSAuditOperator()
    for i in range(4):
        fresh.log_operation("embed", "image", timestamp=float(i) * 86400)
    assert fresh.prune(2, now=4 * 86400.0) == 2 and len(fresh.records) == 2 and fresh.verify_chain_integrity()[0]
    assert json.loads(open(fresh.export_records(str(tmp_path / "e.json"))).read())[0]["index"] == 0
    assert fresh.export_records(str(tmp_path / "e.csv"), "csv").endswith(".csv") and fresh.execute({"action": "verify"}).output["intact"]
    with pytest.raises(ValueError):
        fresh.export_records(str(tmp_path / "e.x"), "xml")


def test_compliance_operator():
    c = POPSSComplianceOperator(POPSSWatermarkDefaultConfigFactory.create("EU"))
    assert c.validate("image")["compliant"] and any(w["name"] == "content_type" for w in c.validate("audio")["warnings"])
    md = c.generate_metadata("yv-7b", "high", "image")
    assert md["disclosure"] == "AI-generated content" and md["compact"]["r"] == "h" and "EU AI Act" in md["standards"]
    assert c.assess_risk(["realistic_media", "political_content"], "video")["risk_level"] == "high"
    low = c.assess_risk(["internal_use", "made_up"], "text")
    assert low["risk_level"] == "low" and low["unknown_factors"] == ["made_up"]
    assert c.check_requirement("redundancy", "CN")["met"] and not c.check_requirement("visible_label", "CN")["met"]
    assert not c.execute({"action": "requirement", "requirement": "nope"}).is_success()
    with pytest.raises(ValueError):
        c.generate_metadata("m", "extreme")


def test_content_text_and_image_marks():
    op = POPSSContentWatermarkOperator(POPSSWatermarkDefaultConfigFactory.create("US"))
    payload = {"m": "yv", "t": 5}
    marked = op.embed_text("Hello brave new world", payload)
    assert op.strip_text(marked) == "Hello brave new world" and marked != "Hello brave new world" and op.extract_text(marked) == payload
    assert op.extract_text("Hello") is None and op.extract_text(op.embed_text("single", payload)) == payload
    torch.manual_seed(0)
    img = _smooth(3, 128, 128)
    out = op.execute({"action": "embed", "image": img, "payload": payload}).output
    got = op.execute({"action": "extract", "image": out["image"], "num_bits": out["num_bits"]}).output
    assert got["detected"] and got["payload"] == payload
    assert not op.execute({"action": "extract", "image": img, "num_bits": out["num_bits"]}).output["detected"]


def test_weight_operator_and_orchestrator(tmp_path):
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(128, 128), nn.Linear(128, 8))
    w = POPSSWeightWatermarkOperator(key="k", eps=5e-3)
    assert not w.verify(m)["detected"]
    assert w.execute({"action": "embed", "model": m}).output["marked"] == ["0.weight"]
    assert w.verify(m)["detected"] and not POPSSWeightWatermarkOperator(key="other", eps=5e-3).verify(m)["detected"]
    o = POPSSWatermarkOrchestrator("CN", "yv-7b", audit_path=str(tmp_path / "a.jsonl"))
    r = o.mark_text("A generated answer", ["public_distribution"])
    assert r["text"].endswith("[AI-generated]") and r["risk_level"] == "medium" and r["audit_index"] == 0
    v = o.verify_text(r["text"])
    assert v["detected"] and v["payload"]["m"] == "yv-7b" and v["payload"]["j"] == "CN" and not o.verify_text("plain")["detected"]
    img = _smooth(3, 256, 256)
    ri = o.mark_image(img, ["realistic_media", "political_content"])
    assert ri["risk_level"] == "high" and o.verify_image(ri["image"], ri["num_bits"])["detected"]
    rep = o.compliance_report()
    assert rep["compliant"] and rep["audit"]["total"] == 5 and rep["audit"]["failures"] == 1 and rep["audit"]["chain_intact"]
