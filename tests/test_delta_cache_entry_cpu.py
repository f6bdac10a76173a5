"""Delta-coded cache entry: packing, decoding with and without kept predictions, moves and copies."""
import pytest
import torch

from pisceslx_b200.models.cache_extras import YvDeltaCacheEntry, YvPredictiveDeltaCoder


def test_entry_round_trip_packed_and_unpacked():
    torch.manual_seed(0)
    ck, cv = YvPredictiveDeltaCoder(16, 8, bits=4, warmup=True), YvPredictiveDeltaCoder(16, 8, bits=4, warmup=True)
    h = torch.randn(2, 5, 16)
    prev_k, prev_v = torch.randn(2, 5, 8), torch.randn(2, 5, 8)
    k, v = prev_k + 0.1 * torch.randn(2, 5, 8), prev_v + 0.1 * torch.randn(2, 5, 8)
    e = YvDeltaCacheEntry.encode(ck, cv, k, v, h, prev_k, prev_v)
    assert e._packed and e._rk.dtype == torch.uint8 and e._rk.shape[-1] == 4 and e.residual_k.shape == k.shape and e.num_tokens == 5
    qk, sk = ck.encode(k, h, prev_k)
    assert torch.equal(e.residual_k, qk)
    k2, v2 = e.decode(ck, cv, h, prev_k, prev_v)
    assert (k2 - k).abs().max() < 0.05 and (v2 - v).abs().max() < 0.05
    with pytest.raises(ValueError):
        e.decode()
    kept = YvDeltaCacheEntry.encode(ck, cv, k, v, h, prev_k, prev_v, keep_predictions=True)
    k3, _ = kept.decode()
    assert torch.allclose(k3, k2) and kept.nbytes > e.nbytes
    c8 = YvPredictiveDeltaCoder(16, 8, bits=8, warmup=True)
    e8 = YvDeltaCacheEntry.encode(c8, c8, k, v, h, prev_k, prev_v)
    assert not e8._packed and e8.nbytes > e.nbytes
    assert (e8.decode(c8, c8, h, prev_k, prev_v)[0] - k).abs().max() < (k2 - k).abs().max()


def test_entry_copies_are_independent():
    e = YvDeltaCacheEntry(torch.ones(1, 3, 4, dtype=torch.int8), torch.ones(1, 3, 4, dtype=torch.int8), torch.ones(1, 3, 1), torch.ones(1, 3, 1),
                          torch.zeros(1, 3, 4), torch.zeros(1, 3, 4))
    c = e.clone()
    c.scale_k.mul_(2)
    assert float(e.scale_k.sum()) == 3 and float(c.scale_k.sum()) == 6
    d = e.to("cpu").detach()
    assert torch.equal(d.residual_v, e.residual_v) and d.decode()[0].shape == (1, 3, 4)
    odd = YvDeltaCacheEntry(torch.ones(2, 3, dtype=torch.int8), torch.ones(2, 3, dtype=torch.int8), torch.ones(2, 1), torch.ones(2, 1), pack=True)
    assert not odd._packed and odd.num_tokens == 2
