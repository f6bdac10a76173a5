"""Inference configuration tree: serialisation, overrides, model specifications, mappings onto the engine."""
import pytest
import torch

from pisceslx_b200.config import YvConfig
from pisceslx_b200.serve.infer_config import (MODEL_SPECS, PiscesLxAccelerationConfig, PiscesLxConfig, PiscesLxGenerationConfig, PiscesLxInferenceConfig,
                                              PiscesLxModelSpec, PiscesLxMoEConfig, PiscesLxServiceConfig)


def test_round_trip_json_yaml_and_unknown_keys(tmp_path):
    c = PiscesLxInferenceConfig()
    c.generation.temperature, c.acceleration.spec_gamma, c.moe.top_k, c.model.model_path = 0.3, 7, 6, "/m"
    d = c.to_dict()
    assert d["generation"]["temperature"] == 0.3 and d["moe"]["top_k"] == 6
    d2 = dict(d, bogus=1)
    d2["generation"] = dict(d["generation"], nope=2)
    assert PiscesLxInferenceConfig.from_dict(d2).to_dict() == d
    c.save_to_json(str(tmp_path / "a" / "c.json"))
    c.save_to_yaml(str(tmp_path / "c.yaml"))
    assert PiscesLxInferenceConfig.load_from_json(str(tmp_path / "a" / "c.json")).to_dict() == d
    assert PiscesLxInferenceConfig.load_from_yaml(str(tmp_path / "c.yaml")).to_dict() == d
    with pytest.raises(ValueError):
        PiscesLxInferenceConfig(dtype="int3")
    with pytest.raises(ValueError):
        PiscesLxGenerationConfig(top_p=0)


def test_cli_overrides():
    c = PiscesLxInferenceConfig()
    c.apply_cli_overrides({"infer_mode": "vllm", "speculative": True, "spec_gamma": "6", "min_new_tokens": "x", "quant": True, "quant_bits": 8,
                           "temperature": "0.2", "device": "cpu", "model_path": "/w", "tp": 4})
    a = c.acceleration
    assert a.use_vllm and a.use_speculative_decoding and a.spec_gamma == 6 and a.min_new_tokens == 16 and a.tensor_parallel_size == 4
    assert c.quantization.enable_quantization and c.quantization.bits == 8 and c.generation.temperature == 0.2 and c.device == "cpu" and c.model.model_path == "/w"
    c.apply_cli_overrides({"infer_mode": "standard", "no_quant": True})
    assert not a.use_vllm and not c.quantization.enable_quantization


def test_mappings_onto_engine_sampler_moe_and_quant():
    cfg = YvConfig.tiny_text_moe(vocab_size=128)
    c = PiscesLxInferenceConfig()
    c.acceleration.max_num_seqs, c.acceleration.enforce_eager, c.acceleration.use_vllm = 8, True, True
    per = c.kv_bytes_per_token(cfg)
    assert per > 0
    weights = cfg.count_parameters()["total"] * 2
    c.memory_limit = (weights + 100 * per * 64) // (1 << 20) + 1
    e = c.to_engine_config(cfg)
    assert e.max_num_seqs == 8 and not e.use_cuda_graphs and e.block_size == 64 and 8 <= e.num_blocks < 4096
    assert e.max_model_len == min(cfg.max_position_embeddings, c.acceleration.max_sequence_length)
    c.acceleration.tensor_parallel_size = 2
    assert c.kv_bytes_per_token(cfg) <= per
    s = c.to_sampling()
    assert s.strategy == "top_k_top_p" and s.temperature == 0.7 and s.top_k == 50
    c.generation.do_sample = False
    assert c.to_sampling().strategy == "greedy"
    c.sampling.contrastive_search = True
    assert c.to_sampling().strategy == "contrastive"
    c.generation.num_beams = 4
    assert c.to_sampling().strategy == "beam" and c.to_sampling().num_beams == 4
    assert c.torch_dtype() is torch.bfloat16
    m = PiscesLxMoEConfig(top_k=6, priority_routing=True, adaptive_temp_cap=1.5).to_runtime_config()
    assert m.top_k == 6 and m.routing_strategy == "priority" and m.adaptive_temp_cap == 1.5
    q = c.quantization
    q.quant_method = "gptq"
    assert q.to_pipeline_config().method.value == "gptq"
    q.quant_method = "fp8"
    assert q.to_pipeline_config().bits == 8 and q.to_pipeline_config().method.value == "rtn"


def test_model_specs_come_from_the_presets():
    assert "7B" in MODEL_SPECS and "7B" in PiscesLxConfig.list_available_models()
    s = PiscesLxConfig.get_model_spec("7B")
    assert (s.hidden_size, s.num_layers, s.num_heads, s.num_kv_heads, s.moe_experts, s.moe_active) == (4096, 32, 32, 8, 64, 6)
    assert s.max_position_embeddings == s.context_length == 131072
    d = PiscesLxModelSpec("x", 96, 2, 4, 1024)
    assert d.intermediate_size == 96 * 4 // 3 * 2 and d.num_kv_heads == 4 and d.max_position_embeddings == 1024
    with pytest.raises(ValueError):
        PiscesLxConfig.get_model_spec("9Z")


def test_service_config():
    s = PiscesLxConfig.default_service("7B", port=9000, api_key="secret")
    assert s.model_spec.hidden_size == 4096 and s.run.max_concurrency == 8 and s.opss.swarm_topology == "hierarchical"
    d = s.to_dict()
    assert d["api_key"] == "***" and s.to_dict(redact=False)["api_key"] == "secret"
    back = PiscesLxServiceConfig.from_dict(s.to_dict(redact=False))
    assert back.port == 9000 and isinstance(back.model_spec, PiscesLxModelSpec) and isinstance(back.inference.acceleration, PiscesLxAccelerationConfig)
    assert back.to_dict(redact=False) == s.to_dict(redact=False)
    with pytest.raises(ValueError):
        PiscesLxServiceConfig(port=70000)
