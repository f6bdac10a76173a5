"""Selective state-space branch: scan semantics, incremental decoding, hybrid block, and the CUDA scan kernels against
the fp32 PyTorch recurrence."""
import pytest
import torch

from pisceslx_b200 import YvConfig
from pisceslx_b200.models.ssm import (YvHybridBlock, YvMamba3Block, YvSelectiveSSM, selective_scan,
                                      selective_scan_reference)


def _inputs(b, l, d, n, device="cpu", seed=0):
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(b, l, d, generator=g)
    delta = torch.nn.functional.softplus(torch.randn(b, l, d, generator=g) - 2.0)
    A = -torch.exp(torch.randn(d, n, generator=g) * 0.3)
    B, C, D = torch.randn(b, l, n, generator=g), torch.randn(b, l, n, generator=g), torch.randn(d, generator=g)
    return [t.to(device) for t in (u, delta, A, B, C, D)]


def test_scan_reference_matches_closed_form_and_step_decoding():
    u, delta, A, B, C, D = _inputs(2, 6, 8, 4)
    y, h = selective_scan_reference(u, delta, A, B, C, D)
    # closed form for the last step: h_L = sum_s exp(A * sum_{r>s} delta_r) delta_s B_s u_s
    acc = torch.zeros(2, 8, 4)
    for s in range(6):
        tail = delta[:, s + 1:].sum(1)
        acc += torch.exp(tail[..., None] * A) * delta[:, s, :, None] * B[:, s, None, :] * u[:, s, :, None]
    assert torch.allclose(h, acc, atol=1e-5)
    assert torch.allclose(y[:, -1], (acc * C[:, -1, None, :]).sum(-1) + u[:, -1] * D, atol=1e-5)


def test_ssm_module_step_matches_full_forward_and_trains():
    torch.manual_seed(0)
    m = YvSelectiveSSM(32, state_dim=16, expansion_factor=2)
    x = torch.randn(2, 7, 32)
    full = m(x)
    st = m.init_state(2, x.device)
    steps = torch.cat([m.step(x[:, t:t + 1], st) for t in range(7)], 1)
    assert torch.allclose(full, steps, atol=1e-5)
    full.pow(2).mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters())


def test_hybrid_and_mamba_blocks_shapes_and_gate_objective():
    cfg = YvConfig.tiny_text_moe(vocab_size=128)
    x = torch.randn(2, 5, cfg.hidden_size)
    assert YvMamba3Block(cfg)(x).shape == x.shape
    attn = torch.nn.Linear(cfg.hidden_size, cfg.hidden_size)
    mlp = torch.nn.Linear(cfg.hidden_size, cfg.hidden_size)
    blk = YvHybridBlock(cfg, 0, attn, mlp)
    y, aux = blk(x)
    assert y.shape == x.shape and float(blk.sparsity_objective()) > 0
    (y.mean() + blk.sparsity_objective()).backward()
    assert blk.sparse_gate_ssm.grad is not None and blk.residual_scale_ssm.grad is not None


@pytest.mark.gpu
@pytest.mark.parametrize("b,l,d", [(2, 33, 64), (1, 257, 256)])
def test_cuda_selective_scan_fwd_bwd_matches_reference(b, l, d):
    ins = _inputs(b, l, d, 16, "cuda", seed=3)
    ref_in = [t.clone().requires_grad_(True) for t in ins]
    got_in = [t.clone().requires_grad_(True) for t in ins]
    yr, _ = selective_scan_reference(*ref_in)
    yg = selective_scan(*got_in)
    assert torch.allclose(yg, yr, atol=2e-4, rtol=2e-4)
    go = torch.randn_like(yr)
    yr.backward(go)
    yg.backward(go)
    for name, a, r in zip("u delta A B C D".split(), got_in, ref_in):
        err = float((a.grad - r.grad).norm() / r.grad.norm().clamp_min(1e-12))
        assert err < 2e-3, (name, err)


@pytest.mark.gpu
def test_cuda_scan_step_carries_state():
    from pisceslx_b200.models.ssm import selective_scan_step
    u, delta, A, B, C, D = _inputs(2, 9, 64, 16, "cuda", seed=5)
    full, h = selective_scan_reference(u, delta, A, B, C, D)
    st = torch.zeros(2, 64, 16, device="cuda")
    ys = [selective_scan_step(u[:, t:t + 1].contiguous(), delta[:, t:t + 1].contiguous(), A, B[:, t:t + 1].contiguous(),
                              C[:, t:t + 1].contiguous(), D, st) for t in range(9)]
    assert torch.allclose(torch.cat(ys, 1), full, atol=2e-4) and torch.allclose(st, h, atol=2e-4)


def test_model_with_hybrid_backbone_trains_on_cpu():
    from pisceslx_b200.models import build_model
    cfg = YvConfig.tiny_text_moe(vocab_size=256)
    cfg.n_layer = 2
    cfg.use_mamba3, cfg.backbone_allow_legacy_blocks = True, False
    m = build_model(cfg)
    assert m.model.layers[0].ssm is not None
    ids = torch.randint(0, 256, (2, 16))
    out = m(input_ids=ids, labels=ids)
    out["loss"].backward()
    assert m.model.layers[0].ssm.A_log.grad is not None and torch.isfinite(out["loss"])


@pytest.mark.gpu
def test_hybrid_backbone_trains_on_gpu_with_recompute():
    from pisceslx_b200.engine.trainer import YvTrainer, YvTrainerConfig
    from pisceslx_b200.models import build_model
    cfg = YvConfig.tiny_text_moe(vocab_size=512)
    cfg.n_layer = 2
    cfg.use_mamba3, cfg.backbone_allow_legacy_blocks, cfg.use_gradient_checkpointing = True, False, True
    m = build_model(cfg, "cuda", torch.bfloat16, seed=1)
    tr = YvTrainer(m, YvTrainerConfig(micro_batch_size=2, optimizer="adamw", lr=2e-3, max_steps=50, clip_grad_norm=1.0))
    ids = torch.randint(0, 512, (2, 128), generator=torch.Generator().manual_seed(0))
    losses = [tr.train_step({"input_ids": ids, "labels": ids})["loss"] for _ in range(6)]
    assert all(l == l for l in losses) and losses[-1] < losses[0]
