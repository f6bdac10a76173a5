"""Inference operator fronts: flash attention, ring attention with log-sum-exp merging, speculative / assisted decoding,
the batch engine front."""
import math

import pytest
import torch

from pisceslx_b200.config import YvConfig
from pisceslx_b200.models.model import YvModelForCausalLM
from pisceslx_b200.serve import infer_operators as IO


def _ref(q, k, v, causal):
    g = q.shape[2] // k.shape[2]
    kk, vv = k.float().repeat_interleave(g, 2), v.float().repeat_interleave(g, 2)
    s = torch.einsum("bshd,bthd->bhst", q.float(), kk) / math.sqrt(q.shape[-1])
    if causal:
        S, T = s.shape[-2:]
        s = s.masked_fill(torch.ones(S, T, dtype=torch.bool).triu(1 + T - S), float("-inf"))
    return torch.einsum("bhst,bthd->bshd", torch.softmax(s, -1), vv)


def test_flash_attention_operator_matches_the_oracle():
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 12, 4, 16), torch.randn(2, 12, 2, 16), torch.randn(2, 12, 2, 16)
    for causal in (True, False):
        op = IO.PiscesLxFlashAttention3Operator(IO.PiscesLxFlashAttention3Config(num_heads=4, num_kv_heads=2, head_dim=16, causal=causal, precision="fp32"))
        out = op.execute({"q": q, "k": k, "v": v}).output["output"]
        assert torch.allclose(out, _ref(q, k, v, causal), atol=1e-5)
    win = IO.PiscesLxFlashAttention3Operator(IO.PiscesLxFlashAttention3Config(num_heads=4, num_kv_heads=2, head_dim=16, window_size=3, precision="fp32"))
    o = win.attend(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[:, :5], v2[:, :5] = 0, 7.0                                       # outside the window of the late queries
    assert torch.allclose(o[:, 8:], win.attend(q, k2, v2)[:, 8:], atol=1e-6) and not torch.allclose(o[:, :5], win.attend(q, k2, v2)[:, :5])
    cu = torch.tensor([0, 12, 24], dtype=torch.int32)
    packed = IO.PiscesLxFlashAttention3Operator(IO.PiscesLxFlashAttention3Config(num_heads=4, num_kv_heads=2, head_dim=16, precision="fp32"))
    po = packed.attend(q.reshape(24, 64), k.reshape(24, 32), v.reshape(24, 32), cu, cu, 12, 12)
    assert torch.allclose(po.view(2, 12, 4, 16), _ref(q, k, v, True), atol=1e-5)
    for bad in ({"precision": "fp8_e4m3"}, {"dropout": 0.1}, {"num_heads": 3, "num_kv_heads": 2}):
        with pytest.raises(ValueError):
            IO.PiscesLxFlashAttention3Config(**bad)
    layer = IO.PiscesLxFlashAttention3Layer(32, IO.PiscesLxFlashAttention3Config(num_heads=4, num_kv_heads=2, head_dim=8, precision="fp32"))
    x = torch.randn(2, 6, 32, requires_grad=True)
    layer(x).sum().backward()
    assert x.grad is not None and layer.qkv.grad is not None


def test_merge_of_partial_attention_is_exact():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 3, 2, 8), torch.randn(1, 10, 2, 8), torch.randn(1, 10, 2, 8)
    blk = IO.PiscesLxRingAttentionOperator._block
    o1, l1 = blk(q, k[:, :4], v[:, :4], 8 ** -0.5, None)
    o2, l2 = blk(q, k[:, 4:], v[:, 4:], 8 ** -0.5, None)
    o, l = IO.merge_partial_attention(o1, l1, o2, l2)
    full, lf = blk(q, k, v, 8 ** -0.5, None)
    assert torch.allclose(o, full, atol=1e-6) and torch.allclose(l, lf, atol=1e-6)
    empty = torch.full_like(l1, float("-inf"))
    o3, l3 = IO.merge_partial_attention(torch.zeros_like(o1), empty, o2, l2)
    assert torch.allclose(o3, o2, atol=1e-6) and torch.allclose(l3, l2, atol=1e-6)


@pytest.mark.parametrize("causal,ring", [(True, 4), (False, 4), (True, 3), (True, 1), (True, 64)])
def test_ring_attention_equals_full_attention(causal, ring):
    torch.manual_seed(1)
    q, k, v = torch.randn(2, 22, 4, 8), torch.randn(2, 22, 2, 8), torch.randn(2, 22, 2, 8)
    op = IO.PiscesLxRingAttentionOperator(IO.PiscesLxRingAttentionConfig(ring_size=ring, num_heads=4, num_kv_heads=2, head_dim=8, causal=causal))
    r = op.execute({"q": q, "k": k, "v": v})
    assert r.is_success() and torch.allclose(r.output["output"], _ref(q, k, v, causal), atol=1e-5)
    R = min(ring, 22)
    assert r.output["blocks_visited"] == (R * (R + 1) // 2 if causal else R * R)          # future blocks are skipped


def test_ring_attention_layer_and_config():
    layer = IO.PiscesLxRingAttentionLayer(16, IO.PiscesLxRingAttentionConfig(ring_size=2, num_heads=2, head_dim=8, topology="bidirectional"))
    assert layer.config.topology is IO.PiscesLxRingTopology.BIDIRECTIONAL and layer.config.num_kv_heads == 2
    y = layer(torch.randn(1, 9, 16))
    assert tuple(y.shape) == (1, 9, 16)
    with pytest.raises(ValueError):
        IO.PiscesLxRingAttentionConfig(ring_size=0)


def _model(seed=0, layers=1):
    torch.manual_seed(seed)
    cfg = YvConfig.tiny_text_moe(vocab_size=64)
    cfg.n_layer = layers
    return YvModelForCausalLM(cfg).eval()


def test_speculative_and_assisted_decoding_operators():
    target, draft = _model(0), _model(1)
    ids = torch.randint(0, 64, (1, 6))
    op = IO.PiscesLxSpeculativeDecodingOperator(target, draft, IO.PiscesLxSpeculativeConfig(gamma=3, target_temperature=0.0, max_new_tokens=8))
    r = op.execute({"input_ids": ids})
    assert r.is_success(), r.error
    out = r.output
    assert out["output_ids"].shape[1] == 14 and torch.equal(out["output_ids"][:, :6], ids) and 0.0 <= out["acceptance_rate"] <= 1.0
    same = IO.PiscesLxSpeculativeDecodingOperator(target, target, IO.PiscesLxSpeculativeConfig(gamma=3, target_temperature=0.0, max_new_tokens=8))
    o2 = same.execute({"input_ids": ids}).output
    assert o2["acceptance_rate"] == 1.0 and not o2["fell_back"]                      # the target agrees with itself
    from pisceslx_b200.models.generation import generate
    assert torch.equal(o2["output_ids"], generate(target, ids, max_new_tokens=8, eos_token_id=-1)[0])   # and the text is the target's own
    asst = IO.PiscesLxAssistedDecodingOperator(target, {"twin": target, "other": draft}, IO.PiscesLxSpeculativeConfig(gamma=2, target_temperature=0.0, max_new_tokens=4))
    a = asst.execute({"input_ids": ids, "assistant": "other"}).output
    b = asst.execute({"input_ids": ids}).output
    assert a["assistant"] == "other" and b["assistant"] == "twin" and asst.best_assistant() == "twin"
    assert not asst.execute({"input_ids": ids, "assistant": "missing"}).is_success()
    with pytest.raises(ValueError):
        IO.PiscesLxAssistedDecodingOperator(target, {})


def test_batch_engine_front_returns_outputs_in_prompt_order():
    model = _model(0)
    op = IO.PiscesLxVLLMInferenceOperator(model, IO.PiscesLxVLLMConfig(max_num_seqs=4, num_blocks=64, block_size=16, enforce_eager=True))
    prompts = [[1, 2, 3], [4, 5], [6, 7, 8, 9]]
    outs = op.generate(prompts, IO.PiscesLxSamplingParams(max_tokens=5))
    assert [o["prompt_token_ids"] for o in outs] == prompts and all(len(o["token_ids"]) <= 5 and o["finish_reason"] for o in outs)
    from pisceslx_b200.models.generation import generate
    want = generate(model, torch.tensor([prompts[0]]), max_new_tokens=5, eos_token_id=-1)[0][0, 3:].tolist()
    assert outs[0]["token_ids"] == want[: len(outs[0]["token_ids"])]
    r = op.execute({"prompts": prompts[:1], "sampling_params": {"max_tokens": 2}})
    assert r.is_success() and len(r.output["outputs"]) == 1 and r.output["stats"]["requests"] >= 4
    assert not op.execute({"prompts": []}).is_success()
    with pytest.raises(ValueError):
        IO.PiscesLxVLLMInferenceOperator()
