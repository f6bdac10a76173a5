"""CPU tests of the cross-modal fusion extras."""
from __future__ import annotations

import torch

from pisceslx_b200.models.multimodal.fusion_extras import (YvContrastiveCrossModalAligner, YvEnhancedModalFusion,
                                                           YvHighResolutionTileProcessor, YvModalFusionConfig,
                                                           YvOnlineQualityAdaptation, YvRCACrossCorrelationAttention,
                                                           YvRecurrentModalRefiner, YvTaskAwareModalityImportance,
                                                           YvUnifiedMultimodalTokenizer, YvVisionPrefixTuning)


def test_contrastive_aligner_learns_pairs_and_hard_negatives():
    torch.manual_seed(0)
    base = torch.randn(16, 12)
    a, b = base @ torch.randn(12, 20), base @ torch.randn(12, 24)          # two views of the same 16 items
    al = YvContrastiveCrossModalAligner(20, 24, embed=16, hard_k=4)
    opt = torch.optim.Adam(al.parameters(), lr=0.02)
    first = None
    for _ in range(80):
        out = al(a, b)
        first = first if first is not None else float(out["loss"])
        opt.zero_grad(); out["loss"].backward(); opt.step()
    assert float(out["loss"]) < 0.5 * first and float(out["accuracy"]) > 0.9
    full = YvContrastiveCrossModalAligner(20, 24, embed=16)
    l0 = float(full(a, b)["loss"].detach())
    assert l0 > 1.0 and l0 == l0                                            # untrained: no better than chance


def test_importance_online_adaptation_and_tokenizer():
    torch.manual_seed(1)
    imp = YvTaskAwareModalityImportance(16, 3, n_tasks=2)
    pooled = torch.randn(2, 3, 16)
    present = torch.tensor([[True, True, False], [True, True, True]])
    w = imp(pooled, torch.tensor([0, 1]), present)
    assert torch.allclose(w.sum(-1), torch.ones(2)) and float(w[0, 2]) == 0.0
    oq = YvOnlineQualityAdaptation(3, lr=0.5)
    for _ in range(30):
        oq.update(torch.tensor([1.0, 0.0, 0.0]), 1.0)                      # answers that leaned on modality 0 were rewarded
        oq.update(torch.tensor([0.0, 1.0, 0.0]), 0.0)
    wt = oq.weights()
    assert wt[0] > wt[1] and wt[0] > wt[2] and abs(float(wt.sum()) - 1) < 1e-6
    tok = YvUnifiedMultimodalTokenizer(16, {"image": 10, "audio": 6})
    out, spans = tok({"audio": torch.randn(2, 3, 6), "image": torch.randn(2, 4, 10)})
    assert out.shape == (2, 4 + 2 + 3 + 2, 16) and spans == [("image", 0, 6), ("audio", 6, 11)]
    only, sp = tok({"audio": torch.randn(2, 3, 6)})
    assert only.shape == (2, 5, 16) and sp == [("audio", 0, 5)]


def test_rca_attention_refiner_and_enhanced_fusion():
    torch.manual_seed(2)
    a, b = torch.randn(2, 5, 32), torch.randn(2, 7, 32)
    rca = YvRCACrossCorrelationAttention(32, 4)
    na, nb = rca(a, b)
    assert torch.equal(na, a) and torch.equal(nb, b)                       # zero-initialised output projections
    rca.oa.data.normal_(std=0.05); rca.ob.data.normal_(std=0.05)
    na, nb = rca(a, b)
    assert na.shape == a.shape and nb.shape == b.shape and not torch.equal(na, a)
    ref = YvRecurrentModalRefiner(32, rounds=2, n_head=4)
    ra, rb = ref(a, b)
    assert ra.shape == a.shape and rb.shape == b.shape and torch.isfinite(ra).all()
    fus = YvEnhancedModalFusion(YvModalFusionConfig(hidden_size=32, modalities=("text", "image", "audio"), n_head=4,
                                                    n_output_tokens=6, n_tasks=2))
    out = fus({"image": torch.randn(2, 9, 32), "audio": torch.randn(2, 4, 32)}, task_id=torch.tensor([0, 1]))
    assert out["tokens"].shape == (2, 6, 32)
    assert torch.allclose(out["modality_weights"].sum(-1), torch.ones(2)) and float(out["modality_weights"][:, 0].sum()) == 0
    out["tokens"].sum().backward()
    assert fus.importance.score.grad is not None


def test_high_resolution_tiles_roundtrip_and_prefix_tuning():
    torch.manual_seed(3)
    proc = YvHighResolutionTileProcessor(tile=16, overlap=4)
    img = torch.rand(3, 40, 52)
    s = proc.split(img)
    assert s["tiles"].shape[1:] == (3, 16, 16) and s["global"].shape == (3, 16, 16)
    ys = sorted({y for y, _ in s["origins"]}); xs = sorted({x for _, x in s["origins"]})
    assert ys[0] == 0 and ys[-1] == 40 - 16 and xs[-1] == 52 - 16          # the tiles cover the whole image
    merged = proc.merge(s["tiles"], s["origins"], s["size"])
    assert torch.allclose(merged, img, atol=1e-5)                          # identity maps blend back to the image
    pt = YvVisionPrefixTuning(32, n_prefix=4, n_head=4)
    x = torch.randn(2, 9, 32)
    assert torch.equal(pt(x), x)
    pt.o.data.normal_(std=0.05)
    y = pt(x)
    assert y.shape == x.shape and not torch.equal(y, x)
    y.sum().backward()
    assert pt.prefix.grad is not None and pt.prefix.grad.abs().sum() > 0
