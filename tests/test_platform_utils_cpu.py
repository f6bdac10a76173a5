"""CPU tests of the platform utilities: device resolution, memory planning / monitor, dtype-safe linear algebra, log
bridge, console environment, modality scanner."""
from __future__ import annotations

import logging

import torch

from pisceslx_b200 import YvConfig
from pisceslx_b200.utils.platform import (PiscesLxConsoleEncoding, PiscesLxDeviceResolver, PiscesLxDtypeSafe,
                                          PiscesLxModalityScanner, PiscesLxThirdPartyLogBridge, PiscesLxVRAMMonitor,
                                          PiscesLxVRAMProfile, PiscesLxVramController)


def test_device_resolver(monkeypatch):
    assert PiscesLxDeviceResolver.resolve("cpu") == torch.device("cpu")
    t = torch.zeros(1)
    assert PiscesLxDeviceResolver.resolve(None, t) == t.device
    monkeypatch.setenv("LOCAL_RANK", "5")
    assert PiscesLxDeviceResolver.rank(None, 4) == 1 and PiscesLxDeviceResolver.rank(2, 8) == 2
    assert PiscesLxDeviceResolver.rank(None, 0) == 0
    assert PiscesLxDeviceResolver.probe(torch.device("cpu"))
    if not torch.cuda.is_available():
        assert PiscesLxDeviceResolver.default() == torch.device("cpu")


def test_vram_controller_plan_and_monitor():
    cfg = YvConfig.yv_7b_moe()
    est = PiscesLxVramController.estimate_model_vram(cfg, 2, 4096, world=1, state_bytes=2.0, recompute=True)
    assert 70 < est["weights_gb"] < 80 and est["total_gb"] > 220          # 40 B parameters
    budget = PiscesLxVRAMProfile(180.0, 178.0, "B200").safe_budget_gb()
    assert 148 < budget < 150
    plan = PiscesLxVramController.optimize_for_vram(cfg, budget + 22, micro_batch=2, seq_len=4096)
    assert plan["recompute"] and plan["state_bytes"] == 2.0 and plan["streaming_optimizer"] and plan["fits"]
    small = YvConfig.tiny_text_moe(vocab_size=512)
    p2 = PiscesLxVramController.optimize_for_vram(small, 100.0, micro_batch=8, seq_len=512)
    assert p2["fits"] and p2["steps"] == [] and not p2["recompute"]
    used = [0.5]
    mon = PiscesLxVRAMMonitor(high=0.9, low=0.7, check_interval=2, calm_checks=2, stats_fn=lambda: (used[0], 1.0))
    assert not mon.check_and_adjust() and not mon.check_and_adjust() and mon.tier == 0
    used[0] = 0.95
    mon.check_and_adjust()
    assert mon.check_and_adjust() and mon.tier == 1
    mon.check_and_adjust(); mon.check_and_adjust()
    assert mon.tier == 2
    used[0] = 0.5
    changes = [mon.check_and_adjust() for _ in range(8)]
    assert mon.tier == 0 and sum(changes) == 2


def test_dtype_safe_log_bridge_console_and_scanner():
    m = torch.randn(6, 4, dtype=torch.bfloat16)
    q = PiscesLxDtypeSafe.qr_safe(m)
    assert q.dtype == torch.bfloat16 and torch.allclose(q.float().t() @ q.float(), torch.eye(4), atol=0.05)
    u, s, vh = PiscesLxDtypeSafe.svd_safe(m)
    assert u.dtype == torch.bfloat16 and torch.allclose((u.float() * s.float()) @ vh.float(), m.float(), atol=0.1)
    assert PiscesLxDtypeSafe.finite_or_zero(torch.tensor([1.0, float("nan"), float("inf")])).tolist() == [1.0, 0.0, 0.0]
    assert PiscesLxThirdPartyLogBridge.quiet({"some.noisy.lib": "ERROR"}) == 1
    assert logging.getLogger("some.noisy.lib").level == logging.ERROR
    got = []

    class Sink(logging.Handler):
        def emit(self, record):
            got.append(record.getMessage())
    sink = Sink()
    assert PiscesLxThirdPartyLogBridge.capture("bridge.test", sink) and not PiscesLxThirdPartyLogBridge.capture("bridge.test", sink)
    logging.getLogger("bridge.test").error("hello")
    assert got == ["hello"] and PiscesLxThirdPartyLogBridge.release("bridge.test", sink)
    env = PiscesLxConsoleEncoding.child_environment({"A": "1"})
    assert env["PYTHONIOENCODING"] == "utf-8" and env["A"] == "1" and PiscesLxConsoleEncoding.ensure_utf8() in (True, False)
    sc = PiscesLxModalityScanner
    assert sc.scan_sample({"input_ids": [1], "pixel_values": torch.zeros(1)}) == {"text", "image"}
    assert sc.scan_sample({"messages": [{"content": "x", "file": "clip.MP4"}]}) == {"text", "video"}
    assert sc.scan_dataset([{"waveform": [0.1], "text": "hi"}, {"text": "b"}]) == {"audio", "text"}
    assert sc.scan_dataset([]) == {"text"}
