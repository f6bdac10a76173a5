"""CPU tests of the inference operators (operator ABI: execute -> result with status)."""
from __future__ import annotations

import torch

from pisceslx_b200 import YvConfig
from pisceslx_b200.models import build_model
from pisceslx_b200.serve.operators import (PiscesLxBeamSearchOperator, PiscesLxGPUCheckOperator, PiscesLxGPUMemoryInfo,
                                           PiscesLxMamba2Operator, PiscesLxMambaConfig, PiscesLxMambaOperator,
                                           PiscesLxNativeInferenceOperator, PiscesLxSamplingConfig,
                                           PiscesLxSamplingOperator, PiscesLxToolRegistry, PiscesLxToolType)


def tiny():
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    cfg.n_layer = 2
    return cfg


def test_sampling_and_beam_search_operators():
    logits = torch.tensor([[0.1, 5.0, 4.9, -3.0]])
    greedy = PiscesLxSamplingOperator(PiscesLxSamplingConfig(temperature=0.0)).execute({"logits": logits})
    assert greedy.is_success() and greedy.output["tokens"].tolist() == [1]
    topk = PiscesLxSamplingOperator(PiscesLxSamplingConfig(temperature=1.0, top_k=2, seed=0))
    assert {int(topk.execute({"logits": logits}).output["tokens"]) for _ in range(40)} <= {1, 2}
    bad = PiscesLxSamplingOperator().execute({"logits": torch.zeros(3)})
    assert not bad.is_success() and bad.error == "invalid inputs"
    m = build_model(tiny())
    r = PiscesLxBeamSearchOperator().execute({"model": m, "input_ids": torch.randint(0, 512, (1, 5)), "num_beams": 2,
                                              "max_new_tokens": 3})
    assert r.is_success() and r.output["sequence"].shape == (1, 8)


def test_gpu_check_operator_with_a_fake_probe():
    gpus = [PiscesLxGPUMemoryInfo(0, "NVIDIA B200", 178.4, 170.0, "10.0"), PiscesLxGPUMemoryInfo(1, "Old", 16.0, 2.0, "7.5")]
    op = PiscesLxGPUCheckOperator(probe=lambda: gpus)
    out = op.execute({"required_gb": 100.0, "require_sm100": True}).output
    assert out["ok"] and out["fits_on"] == [0] and out["sm_100_devices"] == [0] and abs(gpus[0].used_gb - 8.4) < 1e-9
    assert not op.execute({"required_gb": 175.0}).output["ok"]
    assert not PiscesLxGPUCheckOperator(probe=lambda: []).execute({}).output["ok"]
    assert PiscesLxGPUCheckOperator().execute({}).is_success()            # the real probe works with or without a GPU


def test_mamba_operators_and_native_inference():
    x = torch.randn(2, 12, 32)
    for op in (PiscesLxMambaOperator(PiscesLxMambaConfig(hidden_size=32, d_state=8), n_layers=2),
               PiscesLxMamba2Operator(PiscesLxMambaConfig(hidden_size=32, d_state=8))):
        r = op.execute({"hidden_states": x})
        assert r.is_success(), r.error
        assert r.output["hidden_states"].shape == x.shape and torch.isfinite(r.output["hidden_states"]).all()
    # causality of the stack: changing the last position leaves earlier outputs alone
    op = PiscesLxMambaOperator(PiscesLxMambaConfig(hidden_size=32, d_state=8))
    a = op.execute({"hidden_states": x}).output["hidden_states"]
    x2 = x.clone(); x2[:, -1] += 1
    b = op.execute({"hidden_states": x2}).output["hidden_states"]
    assert torch.allclose(a[:, :-1], b[:, :-1], atol=1e-5)
    m = build_model(tiny())
    nat = PiscesLxNativeInferenceOperator(model=m)
    ids = torch.randint(0, 512, (1, 6))
    r = nat.execute({"input_ids": ids, "max_new_tokens": 4, "eos_token_id": -1})
    ref, _ = m.generate(ids, max_new_tokens=4, eos_token_id=-1)
    assert r.is_success() and r.output["output_ids"] == ref[0, 6:].tolist() and r.output["stats"]["seconds"] > 0
    assert not nat.execute({}).is_success()


def test_tool_registry_statistics_search_and_agent_view():
    reg = PiscesLxToolRegistry()
    reg.register("add", lambda a, b: a + b, "adds two numbers", {"a": "number", "b": "number"}, tags=["math"])
    reg.register("fetch", lambda url: 1 / 0, "fetches a page", {"url": "string"}, PiscesLxToolType.MCP, tags=["web"])
    ok = reg.execute("add", a=2, b=3)
    assert ok.success and ok.output == 5 and ok.seconds >= 0
    err = reg.execute("fetch", url="x")
    assert not err.success and "ZeroDivisionError" in err.error and reg.infos["fetch"].failures == 1
    assert not reg.execute("nope").success
    assert [i.name for i in reg.search("numbers")] == ["add"] and [i.name for i in reg.search(tag="web")] == ["fetch"]
    agent_reg = reg.as_agent_registry()
    assert agent_reg.call("add", {"a": 1, "b": 1}) == 2 and "add(a, b)" in agent_reg.describe()
    assert reg.unregister("add") and not reg.unregister("add") and reg.infos["fetch"].calls == 1
