"""Numerics of every sm_100a kernel against a plain PyTorch fp32 statement of the same op (B200 only)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def Y():
    from pisceslx_b200.ops import kernels
    return kernels()


@pytest.fixture()
def status():
    from pisceslx_b200.ops import status_word
    st = status_word(torch.device("cuda", torch.cuda.current_device()))
    st.zero_()
    yield st
    torch.cuda.synchronize()
    assert st.tolist() == [0, 0, 0, 0], f"kernel status word set: {st.tolist()}"


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


# ---------------------------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (1000, 520, 328), (300, 1408, 4096), (2048, 64, 512)])
@pytest.mark.parametrize("layout", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_layouts(Y, status, shape, layout, bn):
    M, N, K = shape
    a_mn, b_mn = layout
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("leading dimension must be a multiple of 8 elements for TMA")
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=torch.bfloat16)
    c = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    Y.gemm(a, b, c, a_mn, b_mn, False, bn, status)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    assert rel(c, ref) < 4e-3


def test_gemm_fp32_out_and_accumulate(Y, status):
    torch.manual_seed(1)
    a = torch.randn(512, 384, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(768, 384, device=DEV, dtype=torch.bfloat16)
    c = torch.randn(512, 768, device=DEV, dtype=torch.float32)
    c0 = c.clone()
    Y.gemm(a, b, c, False, False, True, 0, status)
    assert rel(c, c0 + a.float() @ b.float().t()) < 1e-5
    cb = torch.randn(512, 768, device=DEV, dtype=torch.bfloat16)
    cb0 = cb.clone()
    Y.gemm(a, b, cb, False, False, True, 0, status)
    assert rel(cb, cb0.float() + a.float() @ b.float().t()) < 6e-3


def _plan(Y, counts):
    E = counts.numel()
    max_tiles = (int(counts.sum()) + E * 127) // 128 + 1
    seg = torch.zeros(E + 1, dtype=torch.int32, device=DEV)
    te = torch.zeros(max_tiles, dtype=torch.int32, device=DEV)
    nt = torch.zeros(1, dtype=torch.int32, device=DEV)
    cur = torch.zeros(E, dtype=torch.int32, device=DEV)
    Y.moe_plan(counts, seg, te, nt, cur)
    return seg, te, nt, cur, max_tiles


def test_gemm_grouped_modes(Y, status):
    torch.manual_seed(2)
    E, K, N = 8, 512, 768
    counts = torch.tensor([100, 0, 128, 300, 1, 255, 129, 64], dtype=torch.int32, device=DEV)
    seg, te, nt, _, max_tiles = _plan(Y, counts)
    segl = seg.tolist()
    assert segl == [0, 128, 128, 256, 640, 768, 1024, 1280, 1408] and nt.item() == 11
    rows = max_tiles * 128
    a = torch.randn(rows, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(E, N, K, device=DEV, dtype=torch.bfloat16)
    c = torch.zeros(rows, N, device=DEV, dtype=torch.bfloat16)
    Y.gemm_grouped_m(a, w, c, te, nt, False, 0, status)
    for e in range(E):
        r0, r1 = segl[e], segl[e + 1]
        if r1 > r0:
            assert rel(c[r0:r1], a[r0:r1].float() @ w[e].float().t()) < 4e-3
    c2 = torch.zeros_like(c)
    Y.gemm_grouped_m(a, w.transpose(1, 2).contiguous(), c2, te, nt, True, 0, status)
    assert torch.equal(c2[: segl[-1]], c[: segl[-1]])
    M2, N2 = 256, 384
    dy = torch.randn(rows, M2, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(rows, N2, device=DEV, dtype=torch.bfloat16)
    dw = torch.full((E, M2, N2), 7.0, device=DEV, dtype=torch.bfloat16)
    Y.gemm_grouped_k(dy, x, dw, seg, False, 0, status)
    for e in range(E):
        r0, r1 = segl[e], segl[e + 1]
        ref = dy[r0:r1].float().t() @ x[r0:r1].float()
        assert (dw[e].float() - ref).abs().max().item() <= 0.01 * (ref.abs().max().item() + 1.0)


@pytest.mark.parametrize("shape", [(3, 256, 512), (2, 512, 256), (5, 128, 128)])
def test_gemm_batched_and_newton_schulz(Y, status, shape):
    from pisceslx_b200.ops import reference as ref
    from pisceslx_b200.optim.muon import newton_schulz_batched
    torch.manual_seed(3)
    G, n, m = shape
    x = torch.randn(G, n, m, device=DEV, dtype=torch.bfloat16)
    a = torch.empty(G, n, n, device=DEV, dtype=torch.bfloat16)
    Y.gemm_batched(x, x, a, False, False, False, 0, status)
    assert rel(a, x.float() @ x.float().transpose(1, 2)) < 4e-3
    o = newton_schulz_batched(x)
    r = ref.newton_schulz(x.float())
    assert rel(o, r) < 0.08
    s = torch.linalg.svdvals(o.float())
    assert s.max() < 1.35 and s.min() > 0.3


@pytest.mark.parametrize("n,k,bn", [(1408, 512, 256), (1408, 512, 128), (640, 192, 256), (128, 64, 128), (1024, 256, 0)])
def test_gemm_batched_symmetric_matches_full_product(Y, status, n, k, bn):
    """Symmetric mode computes the tiles on or above the diagonal and mirrors them: the result must equal the full
    product bit for bit wherever both wrote, be exactly symmetric in the mirrored region, and leave nothing unwritten."""
    torch.manual_seed(33)
    G = 3
    x = torch.randn(G, n, k, device=DEV, dtype=torch.bfloat16)
    full = torch.empty(G, n, n, device=DEV, dtype=torch.bfloat16)
    Y.gemm_batched(x, x, full, False, False, False, bn, status, False)
    sym = torch.full((G, n, n), float("nan"), device=DEV, dtype=torch.bfloat16)
    Y.gemm_batched(x, x, sym, False, False, False, bn, status, True)
    assert not torch.isnan(sym.float()).any()
    assert torch.equal(sym, full)                           # x x^T is bitwise symmetric: products commute, same K order
    # the polynomial epilogue: aI + bA + cA^2 of a symmetric A
    a2_full, a2_sym = torch.empty_like(full), torch.full_like(full, float("nan"))
    A = (full.float() / n).bfloat16()
    Y.gemm_batched_affine(A, A, A, a2_full, 3.4445, -4.775, 2.0315, status, False)
    Y.gemm_batched_affine(A, A, A, a2_sym, 3.4445, -4.775, 2.0315, status, True)
    assert not torch.isnan(a2_sym.float()).any()
    assert rel(a2_sym, a2_full) < 1e-3                      # A A differs from its transpose only in accumulation order
    assert torch.equal(a2_sym.triu(), a2_full.triu())
    # transposed operands (the n > m branch of Newton-Schulz: A = X^T X)
    xt = torch.randn(G, k, n, device=DEV, dtype=torch.bfloat16)
    f2, s2 = torch.empty_like(full), torch.full_like(full, float("nan"))
    Y.gemm_batched(xt, xt, f2, True, True, False, bn, status, False)
    Y.gemm_batched(xt, xt, s2, True, True, False, bn, status, True)
    assert torch.equal(s2, f2)


# ---------------------------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("rows,cols", [(1, 256), (37, 1024), (1000, 4096), (65, 8192)])
def test_rmsnorm_fwd_bwd(Y, rows, cols):
    torch.manual_seed(4)
    x = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    r = torch.randn_like(x)
    w = torch.randn(cols, device=DEV, dtype=torch.bfloat16)
    y, ro, rstd = torch.empty_like(x), torch.empty_like(x), torch.empty(rows, device=DEV)
    Y.rmsnorm_fwd(x, r, w, None, None, 1, y, ro, rstd, 1e-6)
    s = (x.float() + r.float()).bfloat16().float()
    assert torch.equal(ro.float(), s)
    ref = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert rel(y, ref) < 4e-3
    dy, dx = torch.randn_like(x), torch.empty_like(x)
    dwp = torch.empty(min(rows, 592), cols, device=DEV)
    dw = torch.zeros(cols, device=DEV)
    Y.rmsnorm_bwd(dy, ro, w, rstd, None, dx, dwp, dw, False)
    sx = s.clone().requires_grad_(True)
    wf = w.float().clone().requires_grad_(True)
    (sx * torch.rsqrt(sx.pow(2).mean(-1, keepdim=True) + 1e-6) * wf).backward(dy.float())
    assert rel(dx, sx.grad) < 5e-3 and rel(dw, wf.grad) < 1e-4


def test_rmsnorm_film_epilogue(Y):
    torch.manual_seed(5)
    B, S, H = 3, 16, 512
    x = torch.randn(B * S, H, device=DEV, dtype=torch.bfloat16)
    w = torch.ones(H, device=DEV, dtype=torch.bfloat16)
    fs = torch.randn(B, H, device=DEV, dtype=torch.bfloat16) * 0.1
    fb = torch.randn(B, H, device=DEV, dtype=torch.bfloat16) * 0.1
    y, rstd = torch.empty_like(x), torch.empty(B * S, device=DEV)
    Y.rmsnorm_fwd(x, None, w, fs, fb, S, y, None, rstd, 1e-6)
    n = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    ref = n.view(B, S, H) * (1 + fs.float().unsqueeze(1)) + fb.float().unsqueeze(1)
    assert rel(y, ref.view(B * S, H)) < 4e-3


def test_rope_and_inverse(Y):
    from pisceslx_b200.ops import reference as ref
    torch.manual_seed(6)
    T, hq, hk, d = 333, 8, 2, 128
    cos, sin = ref.rope_tables(512, 64, 1e4, device=DEV)
    qkv = torch.randn(T, (hq + 2 * hk) * d, device=DEV, dtype=torch.bfloat16)
    orig = qkv.clone()
    pos = torch.randint(0, 512, (T,), device=DEV, dtype=torch.int32)
    q, k = qkv[:, : hq * d], qkv[:, hq * d:(hq + hk) * d]
    Y.rope(q, k, cos, sin, pos, hq, hk, d, 64, False)
    rq = ref.apply_rope(orig[:, : hq * d].reshape(T, hq, d).float(), cos, sin, pos, 64).reshape(T, hq * d)
    rk = ref.apply_rope(orig[:, hq * d:(hq + hk) * d].reshape(T, hk, d).float(), cos, sin, pos, 64).reshape(T, hk * d)
    assert rel(q, rq) < 4e-3 and rel(k, rk) < 4e-3
    assert torch.equal(qkv[:, (hq + hk) * d:], orig[:, (hq + hk) * d:])
    Y.rope(q, k, cos, sin, pos, hq, hk, d, 64, True)
    assert rel(qkv, orig) < 6e-3


def test_rope3d(Y):
    from pisceslx_b200.models.norms import YvSpatioTemporalRoPE3D
    from pisceslx_b200.ops import reference as ref
    torch.manual_seed(7)
    rope = YvSpatioTemporalRoPE3D(64)
    pos = YvSpatioTemporalRoPE3D.grid_positions(3, 5, 7, DEV)
    q = torch.randn(pos.shape[0], 4, 64, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(pos.shape[0], 2, 64, device=DEV, dtype=torch.bfloat16)
    q2, k2 = rope(q, k, pos)
    assert rel(q2, ref.apply_rope3d(q.float(), pos, rope.sections)) < 4e-3
    assert rel(k2, ref.apply_rope3d(k.float(), pos, rope.sections)) < 4e-3


def test_swiglu(Y):
    torch.manual_seed(8)
    T, F = 777, 1408
    g = torch.randn(T, 2 * F, device=DEV, dtype=torch.bfloat16)
    o = torch.empty(T, F, device=DEV, dtype=torch.bfloat16)
    Y.swiglu_fwd(g, o)
    gf = g.float().requires_grad_(True)
    ro = torch.nn.functional.silu(gf[:, :F]) * gf[:, F:]
    assert rel(o, ro) < 4e-3
    do, dg = torch.randn_like(o), torch.empty_like(g)
    Y.swiglu_bwd(g, do, dg)
    ro.backward(do.float())
    assert rel(dg, gf.grad) < 4e-3


# ---------------------------------------------------------------------------------------------- MoE
@pytest.mark.parametrize("E,k,mode", [(64, 6, 0), (8, 2, 0), (64, 6, 1), (128, 8, 0)])
def test_gate_topk(Y, E, k, mode):
    from pisceslx_b200.ops import reference as ref
    torch.manual_seed(9)
    T = 3001
    lg = torch.randn(T, E, device=DEV)
    bias = torch.randn(E, device=DEV) * 0.1
    w = torch.empty(T, k, device=DEV)
    idx = torch.empty(T, k, dtype=torch.int32, device=DEV)
    probs = torch.empty(T, E, device=DEV)
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    Y.gate_topk(lg, bias, w, idx, probs, counts, True, mode)
    rw, ri, rp, rc = ref.gate_topk(lg, bias, k, True, mode)
    assert torch.equal(idx.long(), ri)
    assert rel(w, rw) < 1e-5 and rel(probs, rp) < 1e-5
    assert torch.equal(counts.long(), rc)
    dwt = torch.randn(T, k, device=DEV)
    dl = torch.empty(T, E, device=DEV)
    Y.gate_topk_bwd(dwt, probs, idx, w, dl, mode)
    lgr = lg.clone().requires_grad_(True)
    rw2, _, _, _ = ref.gate_topk(lgr, bias, k, True, mode)
    rw2.backward(dwt)
    assert rel(dl, lgr.grad) < 1e-4


@pytest.mark.parametrize("deterministic", [False, True])
def test_moe_experts_matches_dense_loop(deterministic):
    from pisceslx_b200.ops import moe as moe_ops, reference as ref
    torch.manual_seed(10)
    T, H, E, F, k = 700, 256, 8, 128, 2
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16().requires_grad_(True)
    w13 = (torch.randn(E, 2 * F, H, device=DEV) * 0.05).bfloat16().requires_grad_(True)
    w2 = (torch.randn(E, H, F, device=DEV) * 0.05).bfloat16().requires_grad_(True)
    logits = torch.randn(T, E, device=DEV)
    logits[:, 3] = -50.0                                    # an expert that receives no token
    wts, idx, counts, _ = moe_ops.gate_topk(logits, None, k)
    wts = wts.detach().clone()
    wts[::7, 0] = 0.0                                       # assignments dropped by a capacity rule keep their row
    wts = wts.requires_grad_(True)
    out = moe_ops.moe_experts(x, w13, w2, wts, idx, counts, deterministic)
    do = torch.randn_like(out)
    out.backward(do)
    xr = x.detach().float().requires_grad_(True)
    w13r = w13.detach().float().requires_grad_(True)
    w2r = w2.detach().float().requires_grad_(True)
    wr = wts.detach().clone().requires_grad_(True)
    ro = ref.moe_experts(xr, w13r, w2r, wr, idx.long())
    ro.backward(do.float())
    assert rel(out, ro) < 1e-2
    assert rel(x.grad, xr.grad) < 2e-2
    assert rel(w13.grad, w13r.grad) < 2e-2 and rel(w2.grad, w2r.grad) < 2e-2
    assert rel(wts.grad, wr.grad) < 2e-2
    assert w13.grad[3].abs().max().item() == 0.0            # empty expert: exact zero gradient


def test_gate_bias_update(Y):
    bias = torch.zeros(8, device=DEV)
    counts = torch.tensor([10, 0, 0, 0, 0, 0, 0, 6], dtype=torch.int32, device=DEV)
    Y.gate_bias_update(bias, counts, 0.05, 2.0)
    ref = 0.05 * (1 / 8 - counts.float() / 16)
    assert rel(bias, ref) < 1e-6


# ---------------------------------------------------------------------------------------------- attention
def _attn_case(lens, hq, hk, d, causal):
    from pisceslx_b200.ops import functional as F_, reference as ref
    T = sum(lens)
    qkv = torch.randn(T, (hq + 2 * hk) * d, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    o = F_.rope_attention(qkv.clone(), None, None, None, cu, max(lens), hq, hk, d, d, causal)
    do = torch.randn_like(o)
    # autograd through the clone
    qkv2 = qkv.detach().clone().requires_grad_(True)
    o2 = F_.rope_attention(qkv2 * 1.0, None, None, None, cu, max(lens), hq, hk, d, d, causal)
    o2.backward(do)
    qf = qkv.detach().float().requires_grad_(True)
    q = qf[:, : hq * d].reshape(T, hq, d)
    k = qf[:, hq * d:(hq + hk) * d].reshape(T, hk, d)
    v = qf[:, (hq + hk) * d:].reshape(T, hk, d)
    ro = ref.attention_varlen(q, k, v, cu.cpu(), None, causal, 1 / math.sqrt(d)).reshape(T, hq * d)
    ro.backward(do.float())
    return rel(o, ro), rel(o2, ro), rel(qkv2.grad, qf.grad)


@pytest.mark.parametrize("lens,hq,hk,d,causal", [
    ([128], 1, 1, 128, False), ([128], 1, 1, 128, True), ([256], 2, 1, 128, True),
    ([300, 77, 513], 4, 2, 128, True), ([300, 77, 513], 4, 2, 64, False), ([1024], 8, 2, 128, True), ([1], 2, 2, 64, True)])
def test_flash_attention_fwd_bwd(status, lens, hq, hk, d, causal):
    torch.manual_seed(11)
    e1, e2, eg = _attn_case(lens, hq, hk, d, causal)
    assert e1 < 6e-3 and e2 < 6e-3 and eg < 1.2e-2


def test_cross_attention_unequal_lengths(status):
    from pisceslx_b200.ops import functional as F_, reference as ref
    torch.manual_seed(12)
    hq, hk, d = 4, 4, 64
    lq, lk = [5, 130], [200, 64]
    q = torch.randn(sum(lq), hq * d, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(sum(lk), hk * d, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(sum(lk), hk * d, device=DEV, dtype=torch.bfloat16)
    cq = torch.tensor([0, 5, 135], dtype=torch.int32, device=DEV)
    ck = torch.tensor([0, 200, 264], dtype=torch.int32, device=DEV)
    o = F_.attention(q, k, v, cq, ck, 130, 200, hq, hk, d, False)
    ro = ref.attention_varlen(q.view(-1, hq, d), k.view(-1, hk, d), v.view(-1, hk, d), cq.cpu(), ck.cpu(), False,
                              1 / math.sqrt(d)).reshape(-1, hq * d)
    assert rel(o, ro) < 6e-3


@pytest.mark.parametrize("splits", [1, 4])
@pytest.mark.parametrize("hq,hk,d", [(32, 8, 128), (4, 4, 64), (8, 1, 128)])
@pytest.mark.parametrize("blk", [64, 24, 128])        # 64 / 128: TMA-fed ring; 24: direct-load kernel
def test_paged_decode(status, splits, hq, hk, d, blk):
    from pisceslx_b200.ops import functional as F_, reference as ref
    torch.manual_seed(13)
    lens = [1, 63, 64, 200, 1000]
    B, maxb = len(lens), (1000 + blk - 1) // blk + 1
    nblocks = B * maxb + 5
    kc = torch.randn(nblocks, blk, hk, d, device=DEV, dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    bt = torch.randperm(nblocks)[: B * maxb].view(B, maxb).to(torch.int32).to(DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    q = torch.randn(B, hq, d, device=DEV, dtype=torch.bfloat16)
    o = F_.paged_decode(q, kc, vc, bt, sl, splits=splits)
    assert rel(o, ref.paged_decode(q, kc, vc, bt, sl, 1 / math.sqrt(d))) < 4e-3


def test_kv_cache_write_and_bounds(Y):
    from pisceslx_b200.ops import status_word
    st = status_word(torch.device("cuda", torch.cuda.current_device()))
    st.zero_()
    T, row, slots = 10, 256, 64
    k = torch.randn(T, row, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(T, row, device=DEV, dtype=torch.bfloat16)
    kc = torch.zeros(slots, row, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    sm = torch.tensor([5, 6, 7, -1, 9, 10, 63, 0, 1, 2], dtype=torch.int32, device=DEV)
    Y.kv_cache_write(k, v, kc, vc, sm, st)
    keep = sm >= 0
    assert torch.equal(kc[sm[keep].long()], k[keep]) and torch.equal(vc[sm[keep].long()], v[keep])
    assert st[0].item() == 0
    # an out-of-range slot is skipped and reported through the status word; nothing is written
    bad = torch.tensor([64] + [-1] * 9, dtype=torch.int32, device=DEV)
    before = kc.clone()
    Y.kv_cache_write(k, v, kc, vc, bad, st)
    torch.cuda.synchronize()
    assert st[0].item() == 8 and torch.equal(kc, before)
    st.zero_()


# ---------------------------------------------------------------------------------------------- loss / optim
def test_linear_cross_entropy():
    from pisceslx_b200.ops.loss import linear_cross_entropy
    torch.manual_seed(14)
    T, H, V = 600, 256, 5000
    h = (torch.randn(T, H, device=DEV) * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(V, H, device=DEV) * 0.05).bfloat16().requires_grad_(True)
    lab = torch.randint(0, V, (T,), device=DEV)
    lab[::7] = -100
    loss = linear_cross_entropy(h, w, lab, -100, None, chunk=256)
    (loss * 2.0).backward()
    hr = h.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    rl = torch.nn.functional.cross_entropy(hr @ wr.t(), lab, ignore_index=-100)
    (rl * 2.0).backward()
    assert abs(loss.item() - rl.item()) < 2e-3 * abs(rl.item())
    assert rel(h.grad, hr.grad) < 1.5e-2 and rel(w.grad, wr.grad) < 1.5e-2


@pytest.mark.parametrize("pdt,sdt", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32), (torch.bfloat16, torch.float32)])
def test_adamw_kernel(Y, pdt, sdt):
    from pisceslx_b200.ops import reference as ref
    torch.manual_seed(15)
    n = 10007
    p = torch.randn(n, device=DEV).to(pdt)
    g = torch.randn(n, device=DEV).to(pdt)
    m = torch.zeros(n, device=DEV, dtype=sdt)
    v = torch.zeros(n, device=DEV, dtype=sdt)
    pr, mr, vr = p.float().clone(), m.float().clone(), v.float().clone()
    for step in (1, 2, 3):
        Y.adamw(p, g, m, v, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 1.0)
        ref.adamw_step(pr, g.float(), mr, vr, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
    tol = 2e-2 if pdt == torch.bfloat16 else 1e-5
    assert rel(p, pr) < tol


@pytest.mark.parametrize("n,offset", [(8 * 4096, 0), (10007, 0), (10007, 3), (5, 0)])
@pytest.mark.parametrize("nesterov,first", [(True, True), (False, False), (True, False)])
def test_muon_streaming_kernels_vector_and_tail(Y, n, offset, nesterov, first):
    # 16-byte vector path, its scalar tail (n not a multiple of 8) and the scalar fallback (unaligned views)
    torch.manual_seed(21)
    base_m = torch.randn(n + 8, device=DEV).bfloat16()
    base_g = torch.randn(n + 8, device=DEV).bfloat16()
    base_o = torch.zeros(n + 8, device=DEV, dtype=torch.bfloat16)
    m, g, out = base_m[offset:offset + n], base_g[offset:offset + n], base_o[offset:offset + n]
    mu, gs = 0.95, 0.5
    gv = g.float() * gs
    mr = (m.float() * mu if first else m.float()) + gv
    outr = gv + mu * mr if nesterov else mr
    Y.momentum_fold(m, g, out, mu, gs, nesterov, first)
    close = lambda a, b: torch.allclose(a.float(), b, rtol=2 ** -7, atol=1e-3)      # one bf16 ulp (FMA contraction)
    assert close(m, mr) and close(out, outr)
    assert float(base_o[offset + n:].abs().sum()) == 0 and float(base_o[:offset].abs().sum()) == 0
    p = base_m[offset:offset + n].clone() if offset == 0 else base_m[offset:offset + n]
    p0 = p.float().clone()
    Y.muon_apply(p, g, 1e-2, 0.1, 0.7)
    assert close(p, p0 * (1 - 1e-2 * 0.1) - 1e-2 * 0.7 * g.float())


@pytest.mark.parametrize("first", [True, False])
def test_momentum_q8_fold_within_one_step_and_unbiased(Y, first):
    """Block-quantised momentum fold against the exact fp32 fold: each element lands within one quantisation step
    of its block (stochastic rounding), the block scale is max|m| / 127, and the rounding is unbiased."""
    torch.manual_seed(31)
    n = 128 * 4099                                           # odd block count: the grid's ragged last pass
    m0 = torch.randn(n, device=DEV) * torch.rand(n // 128, device=DEV).repeat_interleave(128)
    sc = (m0.view(-1, 128).abs().amax(1) / 127).clamp_min(1e-30)
    q = torch.round(m0.view(-1, 128) / sc.view(-1, 1)).clamp(-127, 127).to(torch.int8).view(-1)
    m_start = q.view(-1, 128).float() * sc.view(-1, 1)
    g = (torch.randn(n, device=DEV) * 0.05).bfloat16()
    mu, gs = 0.95, 0.25
    exact = (m_start * mu if first else m_start) + g.float().view(-1, 128) * gs
    q1, sc1 = q.clone(), sc.clone()
    Y.momentum_fold_q8(q1, sc1, g, mu, gs, first, 12345)
    new_scale = exact.abs().amax(1) / 127
    assert torch.allclose(sc1, new_scale, rtol=1e-5, atol=1e-30)
    got = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    Y.dequant_q8(q1, sc1, got)
    err = (q1.view(-1, 128).float() * sc1.view(-1, 1) - exact).abs() / sc1.view(-1, 1)
    assert float(err.max()) <= 1.0 + 1e-3
    assert torch.allclose(got.float().view(-1, 128), q1.view(-1, 128).float() * sc1.view(-1, 1), rtol=2 ** -7, atol=0)
    # unbiased: the mean signed error over 500 k elements is far below half a step; another seed rounds differently
    assert abs(float(((q1.view(-1, 128).float() * sc1.view(-1, 1) - exact) / sc1.view(-1, 1)).mean())) < 5e-3
    q2, sc2 = q.clone(), sc.clone()
    Y.momentum_fold_q8(q2, sc2, g, mu, gs, first, 999)
    assert not torch.equal(q1, q2)
    q3, sc3 = q.clone(), sc.clone()
    Y.momentum_fold_q8(q3, sc3, g, mu, gs, first, 12345)
    assert torch.equal(q1, q3)                               # same seed, same rounding


def test_muon_int8_momentum_tracks_bf16_momentum():
    """Thirty-two folds per step for three steps (the streaming trainer's pattern): the de-quantised int8 momentum
    follows the fp32 accumulation.  The gradients here are pure noise (the worst case: nothing accumulates coherently),
    and every fold adds a rounding error of variance 1/12 step, so after 96 folds the expected relative Frobenius
    error is about 6 %; it must stay below 9 % and the error must be unbiased."""
    torch.manual_seed(32)
    from pisceslx_b200.optim.muon import YvMuon, dequantize_q8
    p = torch.nn.Parameter(torch.randn(256, 512, device=DEV).bfloat16())
    opt = YvMuon([("w", p)], state_dtype=torch.int8)
    group = opt.param_groups[0]
    exact = torch.zeros(256, 512, device=DEV)
    for step in range(3):
        opt._step_count = step
        for i in range(32):
            g = (torch.randn(256, 512, device=DEV) * 0.1).bfloat16()
            opt._grad_scale = 1.0 / 32
            opt._fold(p, g, group, i == 0, False)
            exact = (exact * 0.95 if i == 0 else exact) + g.float() / 32
    st = opt.state[p]
    assert st["momentum_q"].dtype == torch.int8 and "momentum_buffer" not in st
    m = dequantize_q8(st["momentum_q"], st["momentum_scale"])
    assert rel(m, exact) < 9e-2
    assert abs(float((m.float() - exact).mean())) < 2e-2 * float(exact.abs().mean())


def test_frob_normalize_vector_and_scalar(Y):
    torch.manual_seed(22)
    for shape in ((5, 64, 96), (5, 7, 143)):
        x = torch.randn(*shape, device=DEV).bfloat16()
        ref = x.float() / x.float().flatten(1).norm(dim=1).view(-1, 1, 1)
        sq = x.float().pow(2).sum((1, 2))
        norms = torch.empty(5, device=DEV)
        Y.frob_normalize(x, norms, 1e-7)
        assert rel(x, ref) < 5e-3 and rel(norms, sq) < 1e-4


def test_pq_gather_and_argmax(Y):
    from pisceslx_b200.ops import reference as ref
    torch.manual_seed(16)
    C, N, D, T = 16, 1024, 128, 500
    table = (torch.randn(C, N, D, device=DEV) * 0.02).bfloat16()
    logits = torch.randn(T, C * 64, device=DEV)
    idx = torch.empty(T, C, dtype=torch.int32, device=DEV)
    Y.argmax_rows(logits, idx, C)
    assert torch.equal(idx.long(), logits.view(T, C, 64).argmax(-1))
    out = torch.empty(T, D, device=DEV, dtype=torch.bfloat16)
    Y.pq_gather_sum(table, idx, out, None)
    assert rel(out, ref.pq_gather_sum(table.float(), idx)) < 4e-3


@pytest.mark.parametrize("T,H,C,world", [(300, 256, 16, 1), (1000, 512, 7, 4)])
def test_pq_film_fused_kernel_matches_fp32_reference(Y, T, H, C, world):
    """Gather + sum + projection + modulation in one kernel against the same arithmetic in fp32.  The "ranks" of the
    sharded table are separate buffers of this device (the kernel only reads them)."""
    from pisceslx_b200.ops import check_status, status_word
    torch.manual_seed(T)
    rows = 96
    shards = [(torch.randn(C, rows, 128, device=DEV) * 0.5).bfloat16() for _ in range(world)]
    ptrs = torch.tensor([s.data_ptr() for s in shards], dtype=torch.int64)
    idx = torch.randint(0, rows * world, (T, C), device=DEV, dtype=torch.int32)
    w = (torch.randn(2 * H, 128, device=DEV) * 0.05).bfloat16()
    h = torch.randn(T, H, device=DEV).bfloat16()
    out = torch.empty_like(h)
    e = torch.empty(T, 128, device=DEV, dtype=torch.bfloat16)
    Y.pq_film(ptrs, idx, w, h, out, e, C, rows, status_word(torch.device(DEV, 0)))
    torch.cuda.synchronize()
    check_status()
    full = torch.cat([s.float() for s in shards], 1)                       # [C, rows * world, 128]
    e_ref = full[torch.arange(C, device=DEV).view(1, C), idx.long()].sum(1)
    assert rel(e, e_ref) < 4e-3
    f = e.float() @ w.float().t()                                          # the kernel projects the bf16-rounded sum
    ref_out = h.float() * (1 + f[:, :H]) + f[:, H:]
    assert rel(out, ref_out) < 4e-3
    out2 = h.clone()                                                       # in place, without the side output
    Y.pq_film(ptrs, idx, w, out2, out2, None, C, rows, None)
    assert torch.equal(out2, out)


def test_pq_field_fused_path_matches_unfused_forward_and_backward():
    from pisceslx_b200.config import YvConfig
    from pisceslx_b200.models.subconscious import YvPQKnowledgeField
    from pisceslx_b200.models.norms import YvFiLMModulation
    torch.manual_seed(5)
    cfg = YvConfig(hidden_size=256, n_layer=4, n_head=4, n_kv_head=2, vocab_size=512, use_pq_field=True,
                   pq_codebook_size=2048, pq_nav_hidden=128)
    field = YvPQKnowledgeField(cfg).to(device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        field.film_proj.normal_(std=0.05)
    assert field.fused_ok
    h = torch.randn(2 * 150, 256, device=DEV).bfloat16()
    g = torch.randn_like(h)
    outs, grads = [], []
    for fused in (True, False):
        field.zero_grad()
        hh = h.clone().requires_grad_(True)
        field.begin(hh, 2)
        if fused:
            y = field.apply_fused(hh)
        else:
            film = field.film_params(0, hh)
            y = YvFiLMModulation.apply(hh.view(2, -1, 256), film).view(hh.shape)
        (y.float() * g.float()).sum().backward()
        outs.append(y.detach())
        grads.append((hh.grad.clone(), field.film_proj.grad.clone(), field.codebook.grad.clone()))
    assert rel(outs[0], outs[1].float()) < 1e-2
    for a, b in zip(grads[0], grads[1]):
        assert rel(a, b.float()) < 2e-2


def test_patchify(Y):
    from pisceslx_b200.ops import reference as ref
    torch.manual_seed(17)
    img = torch.randn(2, 3, 56, 70, device=DEV)
    mean = torch.tensor([0.48, 0.45, 0.40], device=DEV)
    std = torch.tensor([0.26, 0.26, 0.27], device=DEV)
    out = torch.empty(2 * 4 * 5, 640, device=DEV, dtype=torch.bfloat16)
    Y.patchify(img, out, 14, mean, std)
    assert rel(out, ref.patchify(img, 14, mean, std, 640)) < 4e-3


def test_moe_rank_kernel_gives_stable_sort_order(Y):
    torch.manual_seed(31)
    T, k, E = 3001, 6, 64
    idx = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(T)]).int()
    counts = torch.bincount(idx.flatten().long(), minlength=E).int()
    seg = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    te = torch.empty((T * k + E * 127 + 127) // 128, dtype=torch.int32, device=DEV)
    nt, cur = torch.empty(1, dtype=torch.int32, device=DEV), torch.empty(E, dtype=torch.int32, device=DEV)
    Y.moe_plan(counts, seg, te, nt, cur)
    row_map = torch.empty(T, k, dtype=torch.int32, device=DEV)
    Y.moe_rank(idx, seg, row_map)
    flat = idx.flatten().long()
    order = torch.sort(flat, stable=True).indices
    rank = torch.empty_like(order)
    rank[order] = torch.arange(order.numel(), device=DEV)
    starts = torch.cumsum(counts.long(), 0) - counts.long()
    ref_rows = seg[:-1].long()[flat] + (rank - starts[flat])
    assert torch.equal(row_map.flatten().long(), ref_rows)


@pytest.mark.parametrize("capacity", [1, 40, 300, 100000])
def test_moe_capacity_mask_kernel_matches_sorted_reference(capacity):
    from pisceslx_b200.models.moe import capacity_mask
    torch.manual_seed(capacity)
    T, k, E = 2000, 4, 16
    probs = torch.softmax(torch.randn(T, E, device=DEV) * 2, -1)
    probs[::7] = probs[0]                                        # many exact ties: token order must decide
    idx = probs.topk(k, -1).indices.int()
    w = probs.gather(-1, idx.long())
    w = (w / w.sum(-1, keepdim=True)).requires_grad_(True)
    got = capacity_mask(w, idx, probs, capacity)
    ref_w = capacity_mask(w.detach().cpu(), idx.cpu(), probs.cpu(), capacity)          # eager sort-based form
    assert torch.allclose(got.detach().cpu(), ref_w, atol=1e-6)
    kept_per_expert = torch.bincount(idx.flatten().long()[(got.detach() > 0).flatten()], minlength=E)
    assert int(kept_per_expert.max()) <= capacity
    got.sum().backward()
    assert w.grad is not None and torch.isfinite(w.grad).all()


def test_attn_merge_kernel_matches_logaddexp_merge(Y):
    from pisceslx_b200.parallel.cp import merge_partials
    torch.manual_seed(41)
    L, h, d = 300, 6, 128
    o1, o2 = torch.randn(L, h, d, device=DEV), torch.randn(L, h, d, device=DEV)
    l1, l2 = torch.randn(L, h, device=DEV) * 3, torch.randn(L, h, device=DEV) * 3
    l2[5] = float("-inf")                                       # a row whose second block had no visible keys
    l1[7], l2[7] = float("-inf"), float("-inf")                 # and one with none at all
    ref_o, ref_l = merge_partials(o1, l1, o2, l2)
    a, la = o1.clone(), l1.clone()
    Y.attn_merge(a, la, o2, l2)
    assert torch.allclose(a[torch.isfinite(ref_l)], ref_o[torch.isfinite(ref_l)], atol=2e-5)
    assert torch.allclose(la[torch.isfinite(ref_l)], ref_l[torch.isfinite(ref_l)], atol=2e-5)
    assert torch.equal(a[5], o1[5]) and float(a[7].abs().max()) == 0.0 and la[7, 0] == float("-inf")
