"""CPU tests of the parallel draft verifier, the adaptive speculative decoder, and the reasoning verifiers /
test-time trainer / self-adaptation loops."""
from __future__ import annotations

import torch
import torch.nn as nn

from pisceslx_b200 import YvConfig
from pisceslx_b200.models import build_model


def tiny():
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    cfg.n_layer = 2
    return cfg


def test_parallel_verifier_and_adaptive_decoder():
    from pisceslx_b200.models.speculative import YvAdaptiveSpeculativeDecoder, YvParallelVerifier, YvSpeculativeConfig
    torch.manual_seed(0)
    m = build_model(tiny())
    m.eval()
    ids = torch.randint(0, 512, (1, 6))
    greedy, _ = m.generate(ids, max_new_tokens=5, eos_token_id=-1)
    g = greedy[0, 6:]
    good = g[:4]
    bad = good.clone(); bad[2] = (bad[2] + 1) % 512
    ver = YvParallelVerifier(m)
    r = ver.verify(ids, torch.stack([good, bad]))
    assert r["accepted"].tolist() == [4, 2]
    assert int(r["next_token"][0]) == int(g[4]) and int(r["next_token"][1]) == int(g[2])
    toks, k = ver.best(ids, torch.stack([bad, good]))
    assert k == 4 and toks == g[:5].tolist()
    ad = YvAdaptiveSpeculativeDecoder(m, YvSpeculativeConfig(draft_length=3), draft_cost=0.05, draft_model=m)
    assert ad.best_length(0.95) > ad.best_length(0.5) > ad.best_length(0.05) == 1
    out, st = ad.speculative_generate(ids, 8, eos_token_id=-1)
    full, _ = m.generate(ids, max_new_tokens=8, eos_token_id=-1)
    assert torch.equal(out, full) and st["acceptance_rate"] == 1.0
    assert st["next_draft_length"] > 3 and ad.cfg.draft_length == st["next_draft_length"]


def test_reasoning_verifiers():
    from pisceslx_b200.models.reasoning_verify import YvARES, YvCRV, YvCRVIntegration, YvOTV
    torch.manual_seed(1)
    steps = torch.randn(5, 16)
    crv = YvCRV(16, threshold=0.5)
    r = crv(steps)
    assert r["scores"].shape == (4,) and (r["consistent"] == (r["first_bad_step"] is None))
    crv.threshold = -1.0
    assert crv(steps)["first_bad_step"] == 1
    assert crv(steps[:1])["consistent"]
    integ = YvCRVIntegration(16, keep=3)
    for _ in range(5):
        integ.record(torch.randn(2, 7, 16))
    assert len(integ.checkpoints) == 3
    assert "scores" in integ.verify() and not integ.checkpoints
    otv = YvOTV(16)
    q = otv(steps)
    assert q.shape == (5,) and ((q >= 0) & (q <= 1)).all() and otv.filter_steps(steps, 0.0).all()
    ares = YvARES(16)
    a = ares(steps)
    assert a["step_entailment"].shape == (4,) and 0 <= float(a["chain_soundness"]) <= 1
    assert torch.isclose(a["chain_soundness"], a["step_entailment"].prod())


def test_test_time_trainer_adapts_and_restores():
    from pisceslx_b200.models.reasoning_verify import YvTestTimeTrainer
    torch.manual_seed(2)
    m = build_model(tiny())
    m.eval()
    ids = torch.randint(0, 512, (1, 40))
    before = [p.detach().clone() for p in m.parameters()]
    ttt = YvTestTimeTrainer(m, update_layers=1, lr=1e-2, max_steps=3, min_tokens=8)
    with ttt.adapted(ids) as st:
        assert st["steps"] == 3 and st["losses"][-1] < st["losses"][0]
        changed = [not torch.equal(a, b) for a, b in zip(before, m.parameters())]
        assert any(changed)
        first_layer = [not torch.equal(a, b) for a, b in zip([p.detach() for p in m.model.layers[0].parameters()],
                                                              [q for q in before[1:1 + len(list(m.model.layers[0].parameters()))]])]
    assert all(torch.equal(a, b) for a, b in zip(before, m.parameters()))
    assert not m.training and all(p.requires_grad for p in m.parameters())
    assert ttt.adapt(ids[:, :4])["steps"] == 0


def test_seal_and_solar():
    from pisceslx_b200.models.reasoning_verify import YvSEAL, YvSOLAR
    confs = iter([0.95, 0.5, 0.99, 0.97])
    trained = []
    seal = YvSEAL(lambda p: (torch.cat([p, p]), next(confs)), lambda batch: trained.append(len(batch)) or 0.25,
                  confidence_threshold=0.9, verifier=lambda ids: ids.numel() > 2)
    kept = seal.collect([torch.tensor([1, 2]), torch.tensor([3, 4]), torch.tensor([5, 6]), torch.tensor([7])])
    assert kept == 2 and seal.self_edit() == 0.25 and trained == [2] and seal.self_edit() is None
    torch.manual_seed(3)
    w = nn.Parameter(torch.tensor([5.0, -3.0]))
    sol = YvSOLAR([w], meta_lr=0.2, lr=0.01)
    for _ in range(10):
        w.grad = 2 * w.detach()
        sol.step()
    assert sol.scale[0] > 2.0                       # gradients kept their sign: the step size grew
    plain = torch.tensor([5.0, -3.0]) * (1 - 0.02) ** 10
    assert w.detach().abs().sum() < plain.abs().sum()


def test_graph_decode_runner_falls_back_on_cpu():
    from pisceslx_b200.serve.engine import YvEngineConfig, YvInferenceEngine
    m = build_model(tiny())
    m.eval()
    eng = YvInferenceEngine(m, cfg=YvEngineConfig(max_num_seqs=2, num_blocks=16, block_size=16, eos_token_id=-1))
    free0 = eng.cache.alloc.available()
    r = eng.add_request([5, 6, 7], max_new_tokens=4)
    eng.run_until_done()
    ref, _ = m.generate(torch.tensor([[5, 6, 7]]), max_new_tokens=4, eos_token_id=-1)
    st = eng.get_stats()["decode_graphs"]
    assert r.output_ids == ref[0, 3:].tolist()
    assert st["disabled_reason"] == "no CUDA device" and st["eager_steps"] == 3 and st["graph_replays"] == 0
    assert eng.cache.alloc.available() == free0          # nothing reserved for padding when graphs are off
