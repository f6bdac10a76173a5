"""Draft model with cache, neural n-gram head, batched-candidate DSpark decoder, one-forward-per-round Medusa decoder."""
import pytest
import torch

from pisceslx_b200.config import YvConfig
from pisceslx_b200.models.model import YvModelForCausalLM
from pisceslx_b200.models.speculative_extras import (YvDraftModel, YvDSparkSpeculativeDecoder, YvMedusaDecoder, YvNeuralDSparkHead,
                                                     YvVerificationResult, YvVerificationStrategy, verify_candidates)


@pytest.fixture(scope="module")
def target():
    torch.manual_seed(0)
    m = YvModelForCausalLM(YvConfig.tiny_text_moe(vocab_size=96)).eval()
    return m


def _greedy(model, ids, n):
    with torch.no_grad():
        for _ in range(n):
            ids = torch.cat([ids, model(input_ids=ids).logits[:, -1].argmax(-1, keepdim=True)], 1)
    return ids


def test_draft_model_is_causal_and_cache_matches_full_forward():
    torch.manual_seed(0)
    d = YvDraftModel(50, 32, 2, 4, max_position_embeddings=64).eval()
    ids = torch.randint(0, 50, (2, 9))
    full = d(ids)
    changed = ids.clone()
    changed[:, -1] = (changed[:, -1] + 1) % 50
    assert torch.allclose(d(changed)[:, :-1], full[:, :-1], atol=1e-5)                  # the future does not leak back
    perm = ids[:, [1, 0] + list(range(2, 9))]
    assert not torch.allclose(d(perm)[:, 2], full[:, 2], atol=1e-4)                     # order matters
    toks, probs = d.draft(ids, 5)
    ref = ids
    for _ in range(5):
        ref = torch.cat([ref, d(ref)[:, -1].argmax(-1, keepdim=True)], 1)
    assert torch.equal(toks, ref[:, 9:]) and probs.shape == (2, 5) and (probs > 0).all()
    # chunked continuation through the cache
    lg1, c = d._run(ids[:, :5])
    lg2, _ = d._run(ids[:, 5:], c, 5)
    assert torch.allclose(torch.cat([lg1, lg2], 1), full, atol=1e-5)
    with pytest.raises(ValueError):
        YvDraftModel(10, 30, 1, 4)


def test_draft_model_distills_towards_target(target):
    torch.manual_seed(0)
    d = YvDraftModel(96, 32, 1, 4)
    opt = torch.optim.Adam(d.parameters(), lr=3e-3)
    ids = torch.randint(4, 90, (4, 12))
    with torch.no_grad():
        tl = target(input_ids=ids).logits
    losses = [float(d.distill_step(tl, ids, opt)) for _ in range(30)]
    assert losses[-1] < losses[0]


def test_neural_dspark_head_learns_a_cycle():
    torch.manual_seed(0)
    h = YvNeuralDSparkHead(12, markov_order=2, embed_dim=16, hidden=32)
    opt = torch.optim.Adam(h.parameters(), lr=1e-2)
    seq = torch.arange(40).remainder(7).view(1, -1)
    for _ in range(150):
        loss = h.fit_step(seq, opt)
    assert float(loss) < 0.1 and int(h(torch.tensor([[3, 4]])).argmax()) == 5 and int(h(torch.tensor([[5, 6]])).argmax()) == 0
    assert float(h.fit_step(seq[:, :2], opt)) == 0.0


def test_verify_candidates_picks_the_longest_agreement(target):
    ids = torch.randint(4, 90, (1, 6))
    g = _greedy(target, ids, 4)[:, 6:]
    bad = (g + 1) % 96
    half = torch.cat([g[:, :2], bad[:, 2:]], 1)
    r = verify_candidates(target, ids, torch.cat([bad, half, g], 0))
    assert isinstance(r, YvVerificationResult) and r.num_accepted == 4 and r.candidate == 2 and r.rejection_position == -1
    assert int(r.next_token) == int(_greedy(target, ids, 5)[0, -1])
    r2 = verify_candidates(target, ids, torch.cat([bad, half], 0))
    assert r2.num_accepted == 2 and r2.rejection_position == 2 and int(r2.next_token) == int(g[0, 2])
    assert YvVerificationStrategy("medusa") is YvVerificationStrategy.MEDUSA


def test_dspark_decoder_equals_greedy_and_benefits_from_a_trained_head(target):
    torch.manual_seed(0)
    ids = torch.randint(4, 90, (1, 6))
    ref = _greedy(target, ids, 20)
    cfg = {"dspark_confidence_threshold": 0.0, "dspark_parallel_candidates": 4, "dspark_draft_len": 3, "dspark_ngram_embed_dim": 16}
    seen = []
    dec = YvDSparkSpeculativeDecoder(cfg, target, on_stats=seen.append)
    out, st = dec.speculative_generate(ids, 20, generator=torch.Generator().manual_seed(0))
    assert torch.equal(out, ref) and st["generated_tokens"] == 20 and seen and st["rounds"] <= 20
    # a head fitted to what the target writes gets drafts accepted: fewer target forwards
    opt = torch.optim.Adam(dec.markov_head.parameters(), lr=1e-2)
    text = _greedy(target, ids, 40)
    for _ in range(200):
        dec.markov_head.fit_step(text, opt)
    dec.current_draft_len = 3
    out2, st2 = dec.speculative_generate(ids, 20, generator=torch.Generator().manual_seed(0))
    assert torch.equal(out2, ref) and st2["rounds"] < st["rounds"] and st2["acceptance_rate"] > st["acceptance_rate"]
    assert st2["tokens_per_target_forward"] > 1.2
    with pytest.raises(ValueError):
        dec.speculative_generate(torch.cat([ids, ids]), 4)
    dec._ema = None
    for _ in range(6):
        dec._confidence_schedule(0, 4)
    assert dec.current_draft_len == 1
    for _ in range(30):
        dec._confidence_schedule(4, 4)
    assert dec.current_draft_len == dec.max_draft_len


def test_dspark_stops_at_eos(target):
    ids = torch.randint(4, 90, (1, 6))
    ref = _greedy(target, ids, 10)
    eos = int(ref[0, 9])
    first = int((ref[0, 6:] == eos).nonzero()[0])
    dec = YvDSparkSpeculativeDecoder({"dspark_confidence_threshold": 0.0, "dspark_ngram_embed_dim": 8}, target)
    out, _ = dec.speculative_generate(ids, 10, eos_token_id=eos)
    assert torch.equal(out, ref[:, : 6 + first + 1])


def test_medusa_decoder_equals_greedy_and_trained_heads_cut_forwards(target):
    torch.manual_seed(0)
    ids = torch.randint(4, 90, (1, 6))
    ref = _greedy(target, ids, 16)
    dec = YvMedusaDecoder(target, num_heads=3)
    out, st = dec.generate(ids, max_new_tokens=16)
    assert torch.equal(out, ref) and st["generated_tokens"] == 16 and st["total_predicted"] > 0
    text = _greedy(target, ids, 40)
    opt = torch.optim.Adam(dec.medusa.parameters(), lr=3e-3)
    losses = [float(dec.train_step(text, opt)) for _ in range(150)]
    assert losses[-1] < 0.5 * losses[0]
    assert all(p.grad is None for p in target.parameters())                              # the target stays frozen
    out2, st2 = dec.generate(ids, max_new_tokens=16)
    assert torch.equal(out2, ref) and st2["target_forwards"] < st["target_forwards"] and st2["speedup"] > 1.2
    out3, _ = dec.generate(ids, max_length=10)
    assert torch.equal(out3, ref[:, :10])
