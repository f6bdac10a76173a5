"""Teacher providers: local model, server and remote API through injected transports, factory."""
import math

import pytest
import torch
import torch.nn as nn

from pisceslx_b200.data.teacher_providers import (PiscesLxLocalTeacherProvider, PiscesLxRemoteTeacherProvider, PiscesLxServerTeacherProvider, PiscesLxTeacherConfig,
                                                  PiscesLxTeacherProvider, PiscesLxTeacherProviderFactory, PiscesLxTeacherProviderType)


class _Teacher(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb, self.head, self.forwards = nn.Embedding(20, 8), nn.Linear(8, 20), 0

    def forward(self, input_ids, return_logits=True, return_hidden=False):
        self.forwards += 1
        h = self.emb(input_ids)
        return {"logits": self.head(h), "hidden_states": h}


def test_local_provider_memoises_one_forward_and_selects_layers():
    t = _Teacher()
    p = PiscesLxLocalTeacherProvider(PiscesLxTeacherConfig(device="cpu", output_attentions=False, layer_indices=[0, 5]), model=t)
    ids = torch.randint(0, 20, (2, 5))
    out = p.get_all_outputs(ids)
    assert out["logits"].shape == (2, 5, 20) and len(out["hidden_states"]) == 1 and "attentions" not in out and t.forwards == 1
    assert not any(q.requires_grad for q in t.parameters()) and not out["logits"].requires_grad
    soft = p.soft_targets(ids)
    assert torch.allclose(soft.sum(-1), torch.ones(2, 5), atol=1e-5) and t.forwards == 1
    p.get_logits(torch.randint(0, 20, (2, 5)) + 0)
    assert t.forwards >= 1 and p.is_available()
    with PiscesLxLocalTeacherProvider(PiscesLxTeacherConfig(), model=t) as q:
        assert q.get_logits(ids).shape[-1] == 20
    assert q._model is None
    with pytest.raises(ValueError):
        PiscesLxLocalTeacherProvider(PiscesLxTeacherConfig()).get_logits(ids)
    with pytest.raises(ValueError):
        PiscesLxTeacherConfig(alpha=1.5)


def test_server_provider_with_retries():
    calls, fail = [], [2]

    def transport(url, payload, headers, timeout):
        calls.append((url, headers.get("Authorization")))
        if url.endswith("/health"):
            return {"ok": True}
        if fail[0] > 0:
            fail[0] -= 1
            raise ConnectionError("down")
        B, T = len(payload["input_ids"]), len(payload["input_ids"][0])
        out = {"logits": torch.zeros(B, T, 4).tolist()}
        if payload.get("output_hidden_states"):
            out["hidden_states"] = [torch.ones(B, T, 2).tolist(), torch.zeros(B, T, 2).tolist()]
        return out

    slept = []
    p = PiscesLxServerTeacherProvider(PiscesLxTeacherConfig(provider_type="server", server_url="http://h:1/", api_key="k", layer_indices=[1]), transport, slept.append)
    ids = torch.zeros(2, 3, dtype=torch.long)
    assert p.get_logits(ids).shape == (2, 3, 4) and p.retries == 2 and slept == [0.5, 1.0]
    assert calls[0] == ("http://h:1/v1/distill/forward", "Bearer k")
    hs = p.get_hidden_states(ids)
    assert len(hs) == 1 and float(hs[0].sum()) == 0.0 and p.get_attentions(ids) is None and p.is_available()
    fail[0] = 99
    with pytest.raises(RuntimeError):
        p.get_logits(ids)
    assert not PiscesLxServerTeacherProvider(PiscesLxTeacherConfig(provider_type="server"), transport).is_available()


class _Tok:
    def encode(self, s):
        return [int(s[1:])] if s.startswith("t") else [0]

    def decode(self, ids):
        return " ".join(f"t{i}" for i in ids)

    def __len__(self):
        return 10


def test_remote_provider_sparse_and_dense_targets():
    def transport(url, payload, headers, timeout):
        assert url == "https://api.x/v1/completions"
        if payload.get("max_tokens", 0) > 0:
            return {"choices": [{"text": "answer to " + payload["prompt"]}]}
        n = len(payload["prompt"].split())
        return {"choices": [{"logprobs": {"top_logprobs": [None] + [{"t3": math.log(0.6), "5": math.log(0.3)} for _ in range(n - 1)]}}]}

    cfg = PiscesLxTeacherConfig(provider_type="remote", base_url="api.x", model_name="m", top_logprobs=3)
    p = PiscesLxRemoteTeacherProvider(cfg, _Tok(), transport)
    ids = torch.tensor([[1, 2, 3]])
    si, sl = p.get_sparse_targets(ids)
    assert si.shape == (1, 3, 3) and si[0, 0].tolist() == [-1, -1, -1] and si[0, 1].tolist() == [3, 5, -1] and abs(float(sl[0, 1, 0].exp()) - 0.6) < 1e-6
    dense = p.get_logits(ids)
    probs = torch.softmax(dense, -1)
    assert dense.shape == (1, 3, 10) and abs(float(probs[0, 1, 3]) - 0.6) < 1e-5 and abs(float(probs[0, 1, 5]) - 0.3) < 1e-5
    assert abs(float(probs[0, 1, 0]) - 0.1 / 8) < 1e-5 and torch.allclose(probs[0, 0], torch.full((10,), 0.1), atol=1e-6)
    assert p.generate_for_distillation(["q1", "q2"]) == [{"prompt": "q1", "response": "answer to q1"}, {"prompt": "q2", "response": "answer to q2"}]
    assert p._normalize_base_url("http://a/v1/") == "http://a/v1" and p.is_available()
    with pytest.raises(ValueError):
        PiscesLxRemoteTeacherProvider(PiscesLxTeacherConfig(provider_type="remote", base_url="x"), None, transport).get_logits(ids)


def test_factory():
    F = PiscesLxTeacherProviderFactory
    assert isinstance(F.create(PiscesLxTeacherConfig(provider_type=PiscesLxTeacherProviderType.LOCAL), model=_Teacher()), PiscesLxLocalTeacherProvider)
    assert isinstance(F.create(PiscesLxTeacherConfig(provider_type="SERVER", server_url="u"), transport=lambda *a: {}), PiscesLxServerTeacherProvider)
    with pytest.raises(ValueError):
        F.create(PiscesLxTeacherConfig(provider_type="carrier_pigeon"))

    class Const(PiscesLxTeacherProvider):
        closed = False

        def get_logits(self, input_ids):
            return torch.zeros(*input_ids.shape, 2)

        def close(self):
            Const.closed = True
    F.register("const", Const)
    with F.create_with_cleanup(PiscesLxTeacherConfig(provider_type="const")) as p:
        assert p.get_all_outputs(torch.zeros(1, 2, dtype=torch.long))["hidden_states"] is None
    assert Const.closed
    with pytest.raises(TypeError):
        F.register("bad", dict)
    F._registry.pop("const")
