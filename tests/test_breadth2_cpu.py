"""CPU tests of the long-context helpers, the multimodal output heads, the lattice / ternary / salient-token
quantisers, the Kronecker-factored preconditioner and the layout planner."""
from __future__ import annotations

import math

import pytest
import torch
import torch.nn as nn


def test_oomb_windows_and_blending():
    from pisceslx_b200.models.long_context import YvOOMBContext
    ctx = YvOOMBContext(chunk=64, overlap=16)
    wins = ctx.windows(200)
    assert wins[0] == (0, 64) and wins[-1][1] == 200
    assert all(b - a <= 64 for a, b in wins) and all(wins[i + 1][0] < wins[i][1] for i in range(len(wins) - 1))
    x = torch.randn(2, 200, 8)
    # a position-wise function is reproduced exactly whatever the blending weights
    y = ctx.run(x, lambda t: t * 2 + 1)
    assert torch.allclose(y, x * 2 + 1, atol=1e-5)
    assert ctx.run(x[:, :50], lambda t: t + 1).shape == (2, 50, 8)


def test_reform_memory_hyperconnection_and_route_adapter():
    from pisceslx_b200.models.long_context import YvLayerRouteAdapter, YvMHCLiteHyperConnection, YvREFORM
    torch.manual_seed(0)
    r = YvREFORM(32, n_slots=4, n_head=4)
    a = r(torch.randn(2, 10, 32))
    assert r.memory.shape == (2, 4, 32)
    b = r(torch.randn(2, 10, 32))
    assert r.memory.shape == (2, 8, 32) and b.shape == (2, 10, 32)
    r.reset()
    assert r.memory is None
    hc = YvMHCLiteHyperConnection(2)
    s = torch.randn(2, 1, 5, 8)
    out = hc(s, lambda t: t * 0 + 1)
    assert torch.allclose(out, s + 1)            # identity mix + unit write = plain residual on every stream
    ad = YvLayerRouteAdapter(16, n_routes=3, rank=2)
    x = torch.randn(4, 16)
    assert torch.allclose(ad(x), x)              # up-projection starts at zero
    ad.up.data.normal_()
    assert not torch.allclose(ad(x), x)


def test_trace_addresser_and_block_pool():
    from pisceslx_b200.models.long_context import YvResidentBlockPool, YvResonantTraceAddresser
    ad = YvResonantTraceAddresser(min_dwell=2, margin=0.1)
    assert ad.step(torch.tensor([0.1, 0.9, 0.2])) == 1
    assert ad.step(torch.tensor([0.95, 0.9, 0.2])) == 1     # dwell not reached
    assert ad.step(torch.tensor([0.95, 0.9, 0.2])) == 1     # margin not reached
    ad.step(torch.tensor([0.95, 0.9, 0.2]))
    assert ad.step(torch.tensor([2.0, 0.9, 0.2])) == 0
    pool = YvResidentBlockPool(2, lambda i: torch.full((2,), float(i)))
    pool.get(0); pool.get(1); pool.get(0); pool.get(2)
    assert list(pool.resident) == [0, 2] and pool.loads == 3


def test_lfq_tokenizer_and_vision_heads():
    from pisceslx_b200.models.multimodal.heads import YvDetectionHead, YvLFQTokenizer, YvSegmentationHead, YvVQAHead
    torch.manual_seed(0)
    tok = YvLFQTokenizer(32, bits=6)
    x = torch.randn(2, 9, 32, requires_grad=True)
    out, ids, aux = tok(x)
    assert out.shape == x.shape and ids.shape == (2, 9) and int(ids.max()) < 64
    (out.sum() + aux["commit"] + aux["entropy"]).backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
    assert torch.allclose(tok.decode(ids), out.detach(), atol=1e-5)
    feats = torch.randn(2, 16, 32)
    det = YvDetectionHead(32, n_classes=5, n_queries=7)(feats)
    assert det["logits"].shape == (2, 7, 6) and det["boxes"].min() >= 0 and det["boxes"].max() <= 1
    seg = YvSegmentationHead(32, 3, patch=4)(feats, (4, 4))
    assert seg.shape == (2, 3, 16, 16)
    assert YvVQAHead(32, 24, 11)(feats, torch.randn(2, 24)).shape == (2, 11)


def test_talker_vocoder_and_cross_modal_injection():
    from pisceslx_b200.models.multimodal.heads import (YvDeepCrossLayerInjector, YvNeuralVocoder,
                                                      YvRecursiveCrossModalFusion, YvTalker)
    torch.manual_seed(0)
    talker = YvTalker(48, codebook_size=32, n_codebooks=3, dim=24)
    h = torch.randn(2, 5, 48)
    codes = torch.randint(0, 32, (2, 5, 3))
    tr = talker(h, codes)
    assert tr["logits"].shape == (2, 5, 3, 32) and torch.isfinite(tr["loss"])
    tr["loss"].backward()
    gen = talker(h)
    assert gen["codes"].shape == (2, 5, 3)
    voc = YvNeuralVocoder(32, 3, dim=16, rates=(4, 2))
    wav = voc(gen["codes"])
    assert wav.shape == (2, 5 * voc.hop) and wav.abs().max() <= 1
    inj = YvDeepCrossLayerInjector(32, 16, n_head=4)
    x, m = torch.randn(2, 6, 32), torch.randn(2, 3, 16)
    assert torch.allclose(inj(x, m), x)          # zero gate: untouched
    inj.gate.data.fill_(1.0)
    assert not torch.allclose(inj(x, m), x)
    t2, m2 = YvRecursiveCrossModalFusion(32, 16, rounds=2, n_head=4)(x, m)
    assert t2.shape == x.shape and m2.shape == m.shape


def test_e8_lattice_and_hyperquant():
    from pisceslx_b200.quant.extras import PiscesLxHyperQuant, hadamard, nearest_e8
    torch.manual_seed(0)
    H = hadamard(16)
    assert torch.allclose(H @ H.t(), torch.eye(16), atol=1e-6)
    x = torch.randn(500, 8) * 2
    p = nearest_e8(x)
    # lattice membership: all-integer or all-half-integer coordinates, with an even sum
    frac = (p * 2).round() % 2
    assert ((frac == 0).all(-1) | (frac == 1).all(-1)).all()
    assert (p.sum(-1).round() % 2 == 0).all()
    # and it is at least as close as plain rounding to the even-sum integer lattice
    assert ((x - p).pow(2).sum(-1) <= (x - torch.round(x)).pow(2).sum(-1) + 1.0).all()
    w = torch.randn(24, 40)
    errs = []
    for bits in (3.0, 5.0):
        hq = PiscesLxHyperQuant(bits)
        q = hq.quantize(w)
        errs.append(float((hq.dequantize(q) - w).norm() / w.norm()))
    assert errs[1] < errs[0] < 0.5 and errs[1] < 0.08


def test_twla_and_star_kv():
    from pisceslx_b200.quant.extras import PiscesLxSTARKVQuantizer, PiscesLxTWLAQuantizer
    torch.manual_seed(0)
    w = torch.randn(32, 48)
    e0 = None
    for rank in (0, 8, 32):
        q = PiscesLxTWLAQuantizer(rank=rank).quantize(w)
        assert set(q["ternary"].unique().tolist()) <= {-1, 0, 1}
        e = float((PiscesLxTWLAQuantizer.dequantize(q) - w).norm() / w.norm())
        assert e0 is None or e < e0
        e0 = e
    assert e0 < 1e-4                              # full-rank correction restores the matrix
    kv = torch.randn(64, 2, 16)
    kv[5] *= 20
    mass = torch.zeros(64); mass[5] = 1.0; mass[9] = 0.5
    sq = PiscesLxSTARKVQuantizer(bits=4, keep=2)
    c = sq.quantize(kv, mass)
    assert c["salient_idx"].tolist() == [5, 9]
    d = sq.dequantize(c)
    assert torch.equal(d[5], kv[5]) and torch.equal(d[9], kv[9])
    assert float((d - kv).abs().max()) < float((kv[torch.arange(64) != 5].abs().max())) / 7


def test_yv_quantizer_types_and_model_swap():
    from pisceslx_b200.quant.extras import YvQuantizationConfig, YvQuantizer
    torch.manual_seed(0)
    w = torch.randn(16, 64)
    err = {}
    for t in ("int4", "int8", "fp8", "bf16", "fp16"):
        q = YvQuantizer(YvQuantizationConfig(t))
        r = q.quantize_tensor(w)
        err[t] = float((q.dequantize_tensor(r) - w).norm() / w.norm())
    assert err["int4"] > err["int8"] > err["fp16"] and err["fp8"] < 0.05 and err["int8"] < 0.01
    asym = YvQuantizer(YvQuantizationConfig("int8", symmetric=False))
    shifted = w + 3.0
    ea = float((asym.dequantize_tensor(asym.quantize_tensor(shifted)) - shifted).norm() / shifted.norm())
    sym = YvQuantizer(YvQuantizationConfig("int8"))
    es = float((sym.dequantize_tensor(sym.quantize_tensor(shifted)) - shifted).norm() / shifted.norm())
    assert ea < es                                  # a zero point pays off on shifted data
    net = nn.Sequential()
    net.add_module("proj", nn.Linear(64, 32))
    net.add_module("lm_head", nn.Linear(32, 10))
    x = torch.randn(4, 64)
    ref = net(x)
    qz = YvQuantizer(YvQuantizationConfig("int8"))
    assert qz.quantize_model(net) == 1 and isinstance(net.lm_head, nn.Linear)
    assert float((net(x) - ref).abs().max()) < 0.05 and "proj.q" in qz.get_state_dict()
    with pytest.raises(ValueError):
        YvQuantizationConfig("int3")


def test_kfac_preconditioner_whitens_gradient():
    from pisceslx_b200.optim.kfac import PiscesLxKFACPreconditioner
    torch.manual_seed(0)
    lin = nn.Linear(6, 4, bias=False)
    pre = PiscesLxKFACPreconditioner([lin], damping=1e-3, ema=0.0, update_every=1)
    # strongly anisotropic inputs: the raw gradient is dominated by the loud input direction
    scale = torch.tensor([10.0, 1, 1, 1, 1, 1])
    x = torch.randn(512, 6) * scale
    lin.train()
    y = lin(x)
    (y - torch.randn_like(y)).pow(2).mean().backward()
    raw = lin.weight.grad.clone()
    pre.precondition()
    new = lin.weight.grad
    assert torch.isclose(new.norm(), raw.norm(), rtol=1e-4)
    ratio_raw = raw[:, 0].norm() / raw[:, 1:].norm()
    ratio_new = new[:, 0].norm() / new[:, 1:].norm()
    assert ratio_new < ratio_raw * 0.5
    pre.close()


def test_layout_planner_memory_and_buckets():
    from pisceslx_b200 import YvConfig
    from pisceslx_b200.parallel.planner import (PiscesLxCommComputeOverlapOptimizer, PiscesLxFSDPOperator,
                                                PiscesLxParallel3DConfig, PiscesLxParallel3DOperator, YvModelFootprint)
    cfg = YvConfig.yv_7b_moe()
    fp = YvModelFootprint.from_config(cfg)
    total = fp.dense_params + fp.expert_params + fp.embed_params
    assert abs(total - cfg.count_parameters()["total"]) < 0.01 * total      # about 40 B (35 B of them routed experts)
    op = PiscesLxParallel3DOperator()
    c8, est8 = op.plan(cfg, 8, tokens_per_microbatch=8192)
    assert est8["fits"] and c8.pp_size == 1 and c8.world_size == 8 and c8.dp_size % c8.ep_size == 0
    c1, est1 = op.plan(cfg, 1, tokens_per_microbatch=8192, state_bytes_per_param=4.0)
    assert (c1.tp_size, c1.ep_size, c1.pp_size) == (1, 1, 1)
    assert est1["total_gb"] > est8["total_gb"] * 3
    # more sharding never raises the estimate
    e_a = op.memory_estimate(fp, PiscesLxParallel3DConfig(8, 1, 1, 1), 8192)
    e_b = op.memory_estimate(fp, PiscesLxParallel3DConfig(8, 1, 8, 1), 8192)
    e_c = op.memory_estimate(fp, PiscesLxParallel3DConfig(8, 2, 4, 1), 8192)
    assert e_b["total_gb"] < e_a["total_gb"] and e_c["weights_gb"] < e_a["weights_gb"]
    # coordinates invert
    c = PiscesLxParallel3DConfig(16, 2, 4, 2)
    for r in range(16):
        k = c.coords(r)
        assert c.rank_of(k["tp"], k["dp"], k["pp"]) == r and k["ep"] == k["dp"] % 4
    ov = PiscesLxCommComputeOverlapOptimizer(latency_us=35, bus_gbs=725)
    b = ov.bucket_bytes(8)
    assert 64 * 2 ** 20 < b < 256 * 2 ** 20
    params = [nn.Parameter(torch.zeros(1024, 1024)) for _ in range(10)]
    small = PiscesLxCommComputeOverlapOptimizer(min_mb=1, max_mb=8, latency_us=1, bus_gbs=10)
    buckets = small.build_buckets(params, 8)
    assert sorted(i for bk in buckets for i in bk) == list(range(10)) and buckets[0][0] == 9
    sim = ov.exposed_time([b] * 8, backward_s=0.05, world=8)
    assert sim["exposed_s"] < sim["comm_total_s"]
    assert PiscesLxFSDPOperator("full_shard").zero_stage == 3
    with pytest.raises(ValueError):
        PiscesLxFSDPOperator("nope")
