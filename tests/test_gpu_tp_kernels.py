"""The fused tensor-parallel GEMM kernels on one GPU: the "peers" are other buffers of the same device, which is
all the kernels need (they read or write peer memory and wait only on counters that their own CTAs advance)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 2)])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("rows,K,N", [(256, 512, 384), (1024, 1024, 1536)])
def test_allgather_gemm_single_kernel(world, rank, b_mn, rows, K, N):
    from pisceslx_b200.ops import check_status, kernels, status_word
    torch.manual_seed(world * 10 + rank)
    Kn = kernels()
    shards = [torch.randn(rows, K, device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    wb = w.t().contiguous() if b_mn else w
    xg = torch.zeros(world * rows, K, device=DEV, dtype=torch.bfloat16)
    xg[rank * rows:(rank + 1) * rows] = shards[rank]
    y = torch.empty(world * rows, N, device=DEV, dtype=torch.bfloat16)
    ptrs = torch.tensor([s.data_ptr() for s in shards], dtype=torch.int64)
    flags = torch.full((world * rows // 128 + 3,), 7, dtype=torch.int32, device=DEV)     # stale values are reset
    st = status_word(torch.device(DEV, 0))
    Kn.gemm_tp(xg, wb, y, 1, ptrs, flags, rank, rows, b_mn, 0, st)
    torch.cuda.synchronize()
    check_status()
    full = torch.cat(shards)
    assert torch.equal(xg, full)
    assert _rel(y, full.float() @ w.float().t()) < 5e-3
    assert int(flags[: world * rows // 128].min()) >= 0


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 3)])
@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_reduce_scatter_push_single_kernel(world, rank, b_mn):
    from pisceslx_b200.ops import check_status, kernels, status_word
    torch.manual_seed(world * 10 + rank + 100)
    Kn = kernels()
    rows, K, N = 256, 768, 448
    x = torch.randn(world * rows, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    wb = w.t().contiguous() if b_mn else w
    inboxes = [torch.zeros(world, rows, N, device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    ptrs = torch.tensor([t.data_ptr() for t in inboxes], dtype=torch.int64)
    full = torch.full((world * rows, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    st = status_word(torch.device(DEV, 0))
    Kn.gemm_tp(x, wb, full, 2, ptrs, None, rank, rows, b_mn, 0, st)
    torch.cuda.synchronize()
    check_status()
    ref = x.float() @ w.float().t()
    own = slice(rank * rows, (rank + 1) * rows)
    assert _rel(full[own], ref[own]) < 5e-3
    for owner in range(world):
        blk = ref[owner * rows:(owner + 1) * rows]
        if owner == rank:
            assert float(inboxes[owner].abs().max()) == 0.0            # nothing is pushed to oneself
            continue
        assert _rel(inboxes[owner][rank], blk) < 5e-3
        others = [s for s in range(world) if s != rank]
        assert all(float(inboxes[owner][s].abs().max()) == 0.0 for s in others)
        assert torch.isnan(full[owner * rows:(owner + 1) * rows].float()).all()   # remote rows are not stored locally


@pytest.mark.parametrize("M,N,K", [(1, 6144, 4096), (64, 4096, 5632), (100, 1408, 4096), (128, 4096, 4096)])
def test_split_k_skinny_linear_matches_reference_and_is_batch_invariant(M, N, K):
    from pisceslx_b200.ops import check_status, functional as F_
    torch.manual_seed(M + N)
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.02
    assert F_._splitk_plan(M, N, K) > 1
    y = F_.linear(x, w)
    torch.cuda.synchronize()
    check_status()
    assert _rel(y, x.float() @ w.float().t()) < 4e-3
    assert torch.equal(y, F_.linear(x, w))                      # fixed summation order
    assert torch.equal(F_.linear(x[:1], w), y[:1])              # a row does not depend on its neighbours
    assert F_._splitk_plan(4096, N, K) == 0 and F_._splitk_plan(64, 154856, 4096) == 0


@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (1000, 1408, 4096), (4096, 4096, 4096)])
def test_fp8_gemm_matches_dequantised_reference(M, N, K):
    from pisceslx_b200.ops import check_status, kernels, status_word
    torch.manual_seed(M)
    Kn = kernels()
    x = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    sx = (448.0 / x.abs().max().float()).reshape(1)
    sw = (448.0 / w.abs().max().float()).reshape(1)
    xq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=DEV)
    wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device=DEV)
    ax, aw = torch.zeros(1, device=DEV), torch.zeros(1, device=DEV)
    Kn.fp8_quantize(x, sx, xq, ax)
    Kn.fp8_quantize(w, sw, wq, aw)
    assert abs(float(ax) - float(x.abs().max())) < 1e-6 and abs(float(aw) - float(w.abs().max())) < 1e-6
    assert torch.equal(xq.float(), (x.float() * sx).to(torch.float8_e4m3fn).float())      # same rounding as torch
    y = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    Kn.gemm_fp8(xq, wq, y, 1.0 / (sx * sw), 0, status_word(torch.device(DEV, 0)))
    torch.cuda.synchronize()
    check_status()
    ref = (xq.float() @ wq.float().t()) / (sx * sw)
    assert _rel(y, ref) < 4e-3                                   # exact products, fp32 accumulation, bf16 output
    assert _rel(y, x.float() @ w.float().t()) < 6e-2            # quantisation error of per-tensor e4m3


def test_fp8_linear_module_delayed_scaling_trains():
    from pisceslx_b200.quant.fp8 import YvFP8GemmLinear
    torch.manual_seed(0)
    lin = YvFP8GemmLinear(512, 256, scaling="delayed")
    x = torch.randn(64, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    for _ in range(3):
        y = lin(x)
    ref = x.float() @ lin.weight.float().t()
    assert _rel(y, ref) < 6e-2 and lin.meta_x.steps >= 3
    y.float().pow(2).mean().backward()
    assert x.grad is not None and lin.weight.grad is not None and torch.isfinite(lin.weight.grad.float()).all()


def test_mx_quantize_kernel_matches_reference_bytes_and_layout():
    from pisceslx_b200.quant import fp8 as q8
    torch.manual_seed(3)
    x = (torch.randn(300, 512, device=DEV) * torch.logspace(-3, 2, 512, device=DEV)).to(torch.bfloat16)
    x[5, :32] = 0                                               # an all-zero block keeps scale 1
    x[6, 0] = 448.0                                             # a block whose maximum needs no scaling at all
    x[6, 1:32] = 0.25
    q, sf = q8.quantize_mx(x)
    q_ref, e_ref = q8.quantize_mx_reference(x)
    e_k = q8.mx_chunks_to_scales(sf, 300)
    bad = (e_k != e_ref).nonzero()
    assert bad.numel() == 0, (bad[:4].tolist(), e_k[e_k != e_ref][:4].tolist(), e_ref[e_k != e_ref][:4].tolist(),
                              x.float().view(300, 16, 32).abs().amax(-1)[e_k != e_ref][:4].tolist())
    assert torch.equal(sf, q8.mx_scales_to_chunks(e_ref))       # pad rows of the last tile hold 127
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    d = q8.dequantize_mx(q, e_ref)
    assert _rel(d, x.float()) < 4e-2 and float(d[6, 0]) == 448.0 and int(e_ref[5, 0]) == 127


@pytest.mark.parametrize("M,N,K,bn", [(256, 384, 512, 128), (256, 384, 512, 256), (1000, 1408 + 128, 4096, 0),
                                      (4096, 4096, 1408 - 128, 256), (4096, 4096, 4096, 128)])
def test_mxfp8_gemm_matches_dequantised_reference(M, N, K, bn):
    """Block-scaled tensor-core product against the fp32 product of the dequantised operands: the scales are powers
    of two and the products exact, so only fp32 accumulation order and the bf16 output round."""
    from pisceslx_b200.ops import check_status
    from pisceslx_b200.quant import fp8 as q8
    torch.manual_seed(M + N)
    # per-column magnitudes spread over five decades: a per-tensor scale would flush most of them to zero
    x = (torch.randn(M, K, device=DEV) * torch.logspace(-3, 2, K, device=DEV)).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05 * torch.logspace(1, -2, K, device=DEV)).to(torch.bfloat16)
    xq, xs = q8.quantize_mx(x)
    wq, ws = q8.quantize_mx(w)
    y = q8.gemm_mx(xq, xs, wq, ws, bn=bn)
    torch.cuda.synchronize()
    check_status()
    ref = q8.dequantize_mx(xq, q8.mx_chunks_to_scales(xs, M)) @ q8.dequantize_mx(wq, q8.mx_chunks_to_scales(ws, N)).t()
    assert _rel(y, ref) < 4e-3
    assert _rel(y, x.float() @ w.float().t()) < 5e-2            # quantisation error of e4m3 with block scales


def test_mxfp8_grouped_gemm_and_expert_forward():
    from pisceslx_b200.ops import check_status, moe as moe_ops
    from pisceslx_b200.quant import fp8 as q8
    torch.manual_seed(11)
    E, H, F, T, k = 8, 512, 384, 1500, 2
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    w13 = (torch.randn(E, 2 * F, H, device=DEV) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, F, device=DEV) * 0.05).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(T)]).int()
    wts = torch.softmax(torch.randn(T, k, device=DEV), -1)
    # grouped product alone
    counts = torch.bincount(idx.flatten().long(), minlength=E).int()
    xp, plan = moe_ops.permute_tokens(x, idx, counts, E, False, zero_pad=True)
    xq, xs = q8.quantize_mx(xp)
    wq, ws = q8.quantize_mx(w13.view(E * 2 * F, H))
    y = q8.gemm_mx(xq, xs, wq.view(E, 2 * F, H), ws, plan.tile_expert, plan.num_m_tiles)
    torch.cuda.synchronize()
    check_status()
    n_t = int(plan.num_m_tiles)
    xd = q8.dequantize_mx(xq, q8.mx_chunks_to_scales(xs, xp.shape[0]))
    wd = q8.dequantize_mx(wq, q8.mx_chunks_to_scales(ws, E * 2 * F)).view(E, 2 * F, H)
    te = plan.tile_expert[:n_t].long()
    ref = torch.einsum("trh,tnh->trn", xd[:n_t * 128].view(n_t, 128, H), wd[te]).reshape(n_t * 128, 2 * F)
    assert _rel(y[:n_t * 128], ref) < 4e-3
    # whole expert layer: fp8 forward close to the bf16 one, backward runs
    xg = x.clone().requires_grad_(True)
    w13g, w2g = w13.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    out8 = moe_ops.moe_experts(xg, w13g, w2g, wts, idx, fp8="mx")
    out16 = moe_ops.moe_experts(x, w13, w2, wts, idx)
    check_status()
    assert _rel(out8, out16.float()) < 1e-1                      # two chained e4m3 products
    out8.float().pow(2).mean().backward()
    assert torch.isfinite(w13g.grad.float()).all() and torch.isfinite(xg.grad.float()).all()


def test_fp8_linear_module_mx_forward_backward():
    from pisceslx_b200.quant.fp8 import YvFP8GemmLinear
    torch.manual_seed(0)
    lin = YvFP8GemmLinear(512, 256)
    assert lin.scaling == "mx"
    x = torch.randn(3, 70, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = lin(x)
    assert y.shape == (3, 70, 256) and _rel(y, x.float() @ lin.weight.float().t()) < 5e-2
    y.float().pow(2).mean().backward()
    assert torch.isfinite(lin.weight.grad.float()).all() and torch.isfinite(x.grad.float()).all()


@pytest.mark.parametrize("G,n", [(3, 256), (2, 1408)])
def test_batched_gemm_affine_epilogue_forms_newton_schulz_polynomial(G, n):
    from pisceslx_b200.ops import check_status, kernels, status_word
    torch.manual_seed(n)
    Kn = kernels()
    x = torch.randn(G, n, 2 * n, device=DEV) / (2 * n) ** 0.5
    A = (x @ x.transpose(1, 2)).to(torch.bfloat16)                     # symmetric
    out = torch.empty_like(A)
    a, b, c = 3.4445, -4.7750, 2.0315
    Kn.gemm_batched_affine(A, A, A, out, a, b, c, status_word(torch.device(DEV, 0)))
    torch.cuda.synchronize()
    check_status()
    Af = A.float()
    ref = a * torch.eye(n, device=DEV) + b * Af + c * (Af @ Af.transpose(1, 2))
    assert _rel(out, ref) < 4e-3


def test_newton_schulz_with_fused_polynomial_matches_reference():
    from pisceslx_b200.ops.reference import newton_schulz
    from pisceslx_b200.optim.muon import newton_schulz_batched
    torch.manual_seed(0)
    for shape in [(2, 256, 512), (2, 512, 256)]:
        g = torch.randn(*shape, device=DEV, dtype=torch.bfloat16)
        o = newton_schulz_batched(g).float()
        r = newton_schulz(g.float())
        assert _rel(o, r) < 5e-2
        s = torch.linalg.svdvals(o)
        assert float(s.max()) < 1.3 and float(s.min()) > 0.5
