"""Kernel micro-benchmarks and the small cases used for ``ncu`` captures.

    python -m pisceslx_b200.ops.bench_kernels --kernel gemm --m 8192 --n 8192 --k 8192 --iters 10
    python -m pisceslx_b200.ops.bench_kernels --kernel attn_fwd --batch 4 --seq 4096
    python -m pisceslx_b200.ops.bench_kernels --all --json out.json

Timing: CUDA events on the launching stream, 3 warm-up launches, a write of a 256 MB buffer between timed
launches (larger than L2) unless the operands themselves exceed L2.  Fractions are taken against the measured
peaks in ``MEASURED_PEAKS.json`` at the repository root when present (copy bandwidth and cuBLAS bf16 burst
throughput), else against 6.65 TB/s and 1.59 PFLOP/s.
"""
from __future__ import annotations

import argparse
import json
import math
import os
from typing import Any, Callable, Dict, List

import torch

from . import kernels, status_word

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks() -> Dict[str, Any]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


def timeit(fn: Callable[[], None], iters: int, flush: bool = True) -> float:
    K = kernels()
    buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if buf is not None:
            K.l2_flush(buf)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def bench_gemm(a: argparse.Namespace) -> Dict[str, Any]:
    K, st = kernels(), status_word(torch.device("cuda"))
    M, N, Kd = a.m, a.n, a.k
    A = torch.randn(M, Kd, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, Kd, device="cuda", dtype=torch.bfloat16)
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: K.gemm(A, B, C, False, False, False, a.bn, st), a.iters)
    tf = 2.0 * M * N * Kd / ms / 1e9
    return {"kernel": "gemm_sm100", "shape": [M, N, Kd], "ms": ms, "tflops": tf, "frac_of_peak": tf / peaks()["bf16_tflops"]}


def bench_attn(a: argparse.Namespace, bwd: bool) -> Dict[str, Any]:
    K, st = kernels(), status_word(torch.device("cuda"))
    B, S, hq, hk, d = a.batch, a.seq, a.hq, a.hk, a.d
    T = B * S
    qkv = torch.randn(T, (hq + 2 * hk) * d, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, : hq * d], qkv[:, hq * d:(hq + hk) * d], qkv[:, (hq + hk) * d:]
    o = torch.empty(T, hq * d, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(hq, T, device="cuda")
    cu = torch.arange(0, T + 1, S, dtype=torch.int32, device="cuda")
    sc = 1.0 / math.sqrt(d)
    flops = 4.0 * B * hq * S * S * d / 2
    K.attn_fwd(q, k, v, o, lse, cu, None, S, S, hq, hk, d, True, sc, st)
    if not bwd:
        ms = timeit(lambda: K.attn_fwd(q, k, v, o, lse, cu, None, S, S, hq, hk, d, True, sc, st), a.iters)
        tf = flops / ms / 1e9
        return {"kernel": "attn_fwd", "shape": [B, S, hq, hk, d], "ms": ms, "tflops": tf,
                "frac_of_peak": tf / peaks()["bf16_tflops"]}
    do = torch.randn_like(o)
    dqkv = torch.empty_like(qkv)
    dq, dk, dv = dqkv[:, : hq * d], dqkv[:, hq * d:(hq + hk) * d], dqkv[:, (hq + hk) * d:]
    delta = torch.empty(hq, T, device="cuda")
    ms = timeit(lambda: K.attn_bwd(do, q, k, v, o, lse, dq, dk, dv, delta, cu, None, S, S, hq, hk, d, True, sc, st), a.iters)
    tf = 2.5 * flops / ms / 1e9
    return {"kernel": "attn_bwd", "shape": [B, S, hq, hk, d], "ms": ms, "tflops_5gemm": tf,
            "frac_of_peak": tf / peaks()["bf16_tflops"]}


def bench_rmsnorm(a: argparse.Namespace) -> Dict[str, Any]:
    K = kernels()
    T, H = a.m, a.n
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    r = torch.randn_like(x)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    y, ro, rstd = torch.empty_like(x), torch.empty_like(x), torch.empty(T, device="cuda")
    ms = timeit(lambda: K.rmsnorm_fwd(x, r, w, None, None, 1, y, ro, rstd, 1e-6), a.iters)
    gbs = 4.0 * T * H * 2 / ms / 1e6
    return {"kernel": "rmsnorm_fwd(+residual)", "shape": [T, H], "ms": ms, "gbs": gbs, "frac_of_peak": gbs / peaks()["hbm_gbs"]}


def bench_muon_fold(a: argparse.Namespace) -> Dict[str, Any]:
    """The streaming kernels of the Muon step on one stack of expert matrices [batch, m, n]: gradient fold into the
    momentum (read g, read-modify-write m), Frobenius normalisation (two passes) and the parameter update."""
    K = kernels()
    G, m_, n_ = a.batch, a.m, a.n
    mom = torch.randn(G, m_, n_, device="cuda", dtype=torch.bfloat16)
    g = torch.randn_like(mom)
    p = torch.randn_like(mom)
    norms = torch.empty(G, device="cuda")
    nbytes = mom.numel() * 2
    t_fold = timeit(lambda: K.momentum_fold(mom, g, None, 0.95, 1.0, True, False), a.iters)
    t_frob = timeit(lambda: K.frob_normalize(g, norms, 1e-7), a.iters)
    t_apply = timeit(lambda: K.muon_apply(p, g, 1e-3, 0.0, 1.0), a.iters)
    gbs = {"fold": 3.0 * nbytes / t_fold / 1e6, "frob_normalize": 3.0 * nbytes / t_frob / 1e6,
           "apply": 3.0 * nbytes / t_apply / 1e6}
    return {"kernel": "muon_streaming", "shape": [G, m_, n_], "ms": {"fold": t_fold, "frob_normalize": t_frob, "apply": t_apply},
            "gbs": gbs, "frac_of_peak": {k: v / peaks()["hbm_gbs"] for k, v in gbs.items()}}


def bench_decode(a: argparse.Namespace) -> Dict[str, Any]:
    from . import functional as F_
    B, hq, hk, d, blk, ctx = a.batch, a.hq, a.hk, a.d, 64, a.seq
    nb = B * (ctx // blk)
    kc = torch.randn(nb, blk, hk, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    bt = torch.arange(nb, dtype=torch.int32, device="cuda").view(B, ctx // blk)
    sl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    q = torch.randn(B, hq, d, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: F_.paged_decode(q, kc, vc, bt, sl), a.iters, flush=False)
    gbs = 2.0 * kc.numel() * 2 / ms / 1e6
    return {"kernel": "paged_decode", "shape": [B, ctx, hq, hk, d], "ms": ms, "gbs": gbs,
            "frac_of_peak": gbs / peaks()["hbm_gbs"]}


def bench_gemm_fp8(a: argparse.Namespace) -> Dict[str, Any]:
    """e4m3 x e4m3 GEMM (tcgen05 kind::f8f6f4) with per-tensor scales; the fraction is of the bf16 peak."""
    K, st = kernels(), status_word(torch.device("cuda"))
    M, N, Kd = a.m, a.n, a.k
    A = torch.randn(M, Kd, device="cuda").to(torch.float8_e4m3fn)
    B = torch.randn(N, Kd, device="cuda").to(torch.float8_e4m3fn)
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    sc = torch.ones(1, device="cuda")
    ms = timeit(lambda: K.gemm_fp8(A, B, C, sc, a.bn, st), a.iters)
    tf = 2.0 * M * N * Kd / ms / 1e9
    return {"kernel": "gemm_sm100_fp8", "shape": [M, N, Kd], "ms": ms, "tflops": tf,
            "frac_of_bf16_peak": tf / peaks()["bf16_tflops"]}


def bench_gemm_mx(a: argparse.Namespace) -> Dict[str, Any]:
    """Block-scaled e4m3 GEMM (tcgen05 kind::mxf8f6f4.block_scale, one e8m0 scale per 32 elements of K, applied by the
    tensor cores); also times the quantise kernel that produces the operands.  The fraction is of the bf16 peak."""
    from ..quant import fp8 as q8
    K, st = kernels(), status_word(torch.device("cuda"))
    M, N, Kd = a.m, a.n, a.k
    X = torch.randn(M, Kd, device="cuda", dtype=torch.bfloat16)
    W = torch.randn(N, Kd, device="cuda", dtype=torch.bfloat16)
    xq, xs = q8.quantize_mx(X)
    wq, ws = q8.quantize_mx(W)
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: K.gemm_mxfp8(xq, xs, wq, ws, C, None, None, a.bn, st), a.iters)
    ms_q = timeit(lambda: K.mx_quantize(X, xq, xs), a.iters)
    tf = 2.0 * M * N * Kd / ms / 1e9
    return {"kernel": "gemm_sm100_mxfp8", "shape": [M, N, Kd], "bn": a.bn, "ms": ms, "tflops": tf,
            "frac_of_bf16_peak": tf / peaks()["bf16_tflops"], "quantize_ms": ms_q,
            "quantize_gbs": X.numel() * 3.03 / ms_q / 1e6, "status": int(st[0].item())}


def bench_ssm(a: argparse.Namespace) -> Dict[str, Any]:
    """Selective scan forward (batch x seq x d_inner = --batch x --seq x --n, 16 states), bytes = u, delta, y."""
    K = kernels()
    B, L, D = a.batch, a.seq, a.n
    u = torch.randn(B, L, D, device="cuda")
    dl = torch.rand(B, L, D, device="cuda") * 0.1
    A = -torch.rand(D, 16, device="cuda")
    Bm, Cm, Dp = torch.randn(B, L, 16, device="cuda"), torch.randn(B, L, 16, device="cuda"), torch.ones(D, device="cuda")
    y = torch.empty_like(u)
    ms = timeit(lambda: K.ssm_scan_fwd(u, dl, A, Bm, Cm, Dp, y, None, None), a.iters)
    return {"kernel": "ssm_scan_fwd", "shape": [B, L, D, 16], "ms": ms, "gbs": 3.0 * u.numel() * 4 / ms / 1e6,
            "state_updates_per_s": B * L * D * 16 / ms * 1e3}


def bench_gemm_tp(a: argparse.Namespace, mode: int) -> Dict[str, Any]:
    """The fused tensor-parallel GEMM kernels on ONE GPU: the "peers" are other buffers of this device (the kernels
    only read or write peer memory and wait on counters their own CTAs advance), world = --batch ranks.  Shows the
    kernel's own cost (copier warps / inbox stores beside the MMA pipeline) without NVLink in the way; the two-GPU
    numbers come from ``parallel/bench_tp.py``."""
    K, st = kernels(), status_word(torch.device("cuda"))
    world, rank = max(2, a.batch), 0
    M, N, Kd = a.m, a.n, a.k
    rows = M // world
    w = torch.randn(N, Kd, device="cuda", dtype=torch.bfloat16) * 0.02
    y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    if mode == 1:
        shards = [torch.randn(rows, Kd, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
        xg = torch.empty(M, Kd, device="cuda", dtype=torch.bfloat16)
        xg[:rows] = shards[0]
        ptrs = torch.tensor([s.data_ptr() for s in shards], dtype=torch.int64)
        flags = torch.zeros(M // 128 + 8, dtype=torch.int32, device="cuda")
        fn = lambda: K.gemm_tp(xg, w, y, 1, ptrs, flags, rank, rows, False, 0, st)
        name = "gemm_tp_allgather"
    else:
        x = torch.randn(M, Kd, device="cuda", dtype=torch.bfloat16)
        inboxes = [torch.empty(world, rows, N, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
        ptrs = torch.tensor([t.data_ptr() for t in inboxes], dtype=torch.int64)
        fn = lambda: K.gemm_tp(x, w, y, 2, ptrs, None, rank, rows, False, 0, st)
        name = "gemm_tp_reduce_scatter_push"
    ms = timeit(fn, a.iters)
    tf = 2.0 * M * N * Kd / ms / 1e9
    return {"kernel": name, "shape": [M, N, Kd], "world": world, "ms": ms, "tflops": tf,
            "frac_of_peak": tf / peaks()["bf16_tflops"]}


def bench_newton_schulz(a: argparse.Namespace) -> Dict[str, Any]:
    """Batched Newton-Schulz on [batch, m, n] (the Muon orthogonalisation of a stack of expert matrices), plus the
    three batched GEMMs of one iteration timed separately."""
    from ..optim.muon import NS_COEFFS, newton_schulz_batched
    K, st = kernels(), status_word(torch.device("cuda"))
    G, n, m = a.batch, a.m, a.n
    x = torch.randn(G, n, m, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: newton_schulz_batched(x), max(1, a.iters // 3))
    s, l = min(n, m), max(n, m)
    flops = len(NS_COEFFS) * G * (4.0 * s * s * l + 2.0 * s ** 3)
    A = torch.empty(G, s, s, device="cuda", dtype=torch.bfloat16)
    A2, Y = torch.empty_like(A), torch.empty_like(x)
    if n <= m:
        t_gram = timeit(lambda: K.gemm_batched(x, x, A, False, False, False, 0, st), a.iters)
        t_sq = timeit(lambda: K.gemm_batched(A, A, A2, False, False, False, 0, st), a.iters)
        t_apply = timeit(lambda: K.gemm_batched(A2, x, Y, False, True, False, 0, st), a.iters)
    else:
        t_gram = timeit(lambda: K.gemm_batched(x, x, A, True, True, False, 0, st), a.iters)
        t_sq = timeit(lambda: K.gemm_batched(A, A, A2, False, False, False, 0, st), a.iters)
        t_apply = timeit(lambda: K.gemm_batched(x, A2, Y, False, False, False, 0, st), a.iters)
    tf = flops / ms / 1e9
    return {"kernel": "newton_schulz_batched", "shape": [G, n, m], "ms": ms, "tflops": tf,
            "frac_of_peak": tf / peaks()["bf16_tflops"],
            "gemm_tflops": {"gram": 2.0 * G * s * s * l / t_gram / 1e9, "square": 2.0 * G * s ** 3 / t_sq / 1e9,
                            "apply": 2.0 * G * s * s * l / t_apply / 1e9}}


def _bw(name: str, shape, ms: float, nbytes: float) -> Dict[str, Any]:
    gbs = nbytes / ms / 1e6
    return {"kernel": name, "shape": list(shape), "ms": ms, "gbs": gbs, "frac_of_peak": gbs / peaks()["hbm_gbs"]}


def bench_moe(a: argparse.Namespace) -> List[Dict[str, Any]]:
    """The routed-expert path at the benchmark's layer shape for one micro-batch: gate, plan, permute, grouped GEMMs
    (up: [rows, H] x [E, 2F, H]; down: [rows, F] x [E, H, F]; weight gradient over expert segments), SwiGLU forward and
    the row-wise backward, combine and its backward, un-permute."""
    from . import moe as moe_ops
    K, st = kernels(), status_word(torch.device("cuda"))
    T, H, E, F, k = a.m, a.n, 64, 1408, 6
    dev = "cuda"
    x = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
    logits = torch.randn(T, E, device=dev)
    w = torch.empty(T, k, device=dev)
    idx = torch.empty(T, k, dtype=torch.int32, device=dev)
    probs = torch.empty(T, E, device=dev)
    counts = torch.zeros(E, dtype=torch.int32, device=dev)

    def gate():
        counts.zero_()
        K.gate_topk(logits, None, w, idx, probs, counts, True, 0)
    out = [_bw("gate_topk", (T, E), timeit(gate, a.iters), T * E * 8 + T * k * 8)]
    xp, plan = moe_ops.permute_tokens(x, idx, counts, E, False, True)
    rows = plan.max_rows
    cursor = torch.empty(E, dtype=torch.int32, device=dev)

    def permute():
        K.moe_plan(counts, plan.seg_offsets, plan.tile_expert, plan.num_m_tiles, cursor)
        K.moe_permute(x, idx, cursor, plan.row_map, xp)
    out.append(_bw("moe_plan + moe_permute", (T, H, k), timeit(permute, a.iters), (T + T * k) * H * 2))
    w13 = (torch.randn(E, 2 * F, H, device=dev) * 0.02).bfloat16()
    w2 = (torch.randn(E, H, F, device=dev) * 0.02).bfloat16()
    y1 = torch.empty(rows, 2 * F, dtype=torch.bfloat16, device=dev)
    act = torch.empty(rows, F, dtype=torch.bfloat16, device=dev)
    y2 = torch.empty(rows, H, dtype=torch.bfloat16, device=dev)
    real = T * k
    for name, fn, fl in (
            ("gemm_grouped_m up [rows,H]x[E,2F,H]", lambda: K.gemm_grouped_m(xp, w13, y1, plan.tile_expert, plan.num_m_tiles, False, 0, st), 2.0 * real * H * 2 * F),
            ("gemm_grouped_m down [rows,F]x[E,H,F]", lambda: K.gemm_grouped_m(act, w2, y2, plan.tile_expert, plan.num_m_tiles, False, 0, st), 2.0 * real * H * F),
            ("gemm_grouped_m dX [rows,H]x[E,H,F]^T", lambda: K.gemm_grouped_m(y2, w2, act, plan.tile_expert, plan.num_m_tiles, True, 0, st), 2.0 * real * H * F)):
        ms = timeit(fn, a.iters)
        out.append({"kernel": name, "shape": [rows, H, F], "ms": ms, "tflops": fl / ms / 1e9,
                    "frac_of_peak": fl / ms / 1e9 / peaks()["bf16_tflops"]})
    dw13 = torch.empty_like(w13)
    ms = timeit(lambda: K.gemm_grouped_k(y1, xp, dw13, plan.seg_offsets, False, 0, st), a.iters)
    fl = 2.0 * real * H * 2 * F
    out.append({"kernel": "gemm_grouped_k dW [2F,rows_e]x[rows_e,H]", "shape": [E, 2 * F, H], "ms": ms,
                "tflops": fl / ms / 1e9, "frac_of_peak": fl / ms / 1e9 / peaks()["bf16_tflops"]})
    out.append(_bw("swiglu_fwd", (rows, F), timeit(lambda: K.swiglu_fwd(y1, act), a.iters), rows * F * 6))
    row_w = torch.rand(rows, device=dev)
    dy1, actw, rowdot = torch.empty_like(y1), torch.empty_like(act), torch.empty(rows, device=dev)
    out.append(_bw("swiglu_bwd_rows", (rows, F), timeit(lambda: K.swiglu_bwd_rows(y1, act, row_w, dy1, actw, rowdot), a.iters),
                   rows * F * 2 * (2 + 1 + 2 + 1)))
    o = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    out.append(_bw("moe_combine", (T, H, k), timeit(lambda: K.moe_combine(y2, plan.row_map, w, None, o), a.iters),
                   (T * k + T) * H * 2))
    dx = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    out.append(_bw("moe_unpermute_sum", (T, H, k), timeit(lambda: K.moe_unpermute_sum(y2, plan.row_map, dx, k), a.iters),
                   (T * k + T) * H * 2))
    return out


def bench_streaming(a: argparse.Namespace) -> List[Dict[str, Any]]:
    """Bandwidth-bound kernels at model shapes: quantised momentum fold, AdamW, cross-entropy over a logits chunk, RoPE,
    RMSNorm backward, patch extraction."""
    K = kernels()
    dev = "cuda"
    out = []
    n = 64 * 2816 * 4096                                                      # one layer's expert up-projections
    q = torch.zeros(n, dtype=torch.int8, device=dev)
    sc = torch.ones(n // 128, device=dev)
    g = (torch.randn(n, device=dev) * 0.01).bfloat16()
    out.append(_bw("momentum_q8 (fold into int8 momentum)", (64, 2816, 4096),
                   timeit(lambda: K.momentum_fold_q8(q, sc, g, 0.95, 1.0 / 32, False, 7), a.iters), n * 4.0 + n / 32))
    mt = torch.empty(n, dtype=torch.bfloat16, device=dev)
    out.append(_bw("dequant_q8", (64, 2816, 4096), timeit(lambda: K.dequant_q8(q, sc, mt), a.iters), n * 3.0))
    na = 154856 * 4096
    p, ga = torch.randn(na, device=dev).bfloat16(), torch.randn(na, device=dev).bfloat16()
    m1, v1 = torch.zeros_like(p), torch.zeros_like(p)
    out.append(_bw("adamw (bf16 p, g, m, v)", (154856, 4096),
                   timeit(lambda: K.adamw(p, ga, m1, v1, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3, 1.0), a.iters), na * 2.0 * 7))
    Tc, V = 2048, 154856
    logits = torch.randn(Tc, V, device=dev)
    labels = torch.randint(0, V, (Tc,), device=dev)
    loss = torch.zeros(1, device=dev)
    dl = torch.empty(Tc, V, dtype=torch.bfloat16, device=dev)
    out.append(_bw("ce_fwd_bwd (fp32 logits chunk -> loss + bf16 dlogits)", (Tc, V),
                   timeit(lambda: K.ce_fwd_bwd(logits, labels, loss, dl, -100, 1.0), a.iters), Tc * V * 6.0))
    T, hq, hk, d = 8192, 32, 8, 128
    qk = torch.randn(T, (hq + 2 * hk) * d, device=dev).bfloat16()
    from . import reference as ref
    cos, sin = ref.rope_tables(4096, d, 1e4, 1.0, device=dev)
    pos = (torch.arange(T, device=dev) % 4096).int()
    qv, kv = qk[:, : hq * d], qk[:, hq * d:(hq + hk) * d]
    out.append(_bw("rope (q and k in place)", (T, hq + hk, d),
                   timeit(lambda: K.rope(qv, kv, cos, sin, pos, hq, hk, d, d, False), a.iters), T * (hq + hk) * d * 4.0))
    x = torch.randn(32768, 4096, device=dev).bfloat16()
    dy, dx = torch.randn_like(x), torch.empty_like(x)
    w = torch.ones(4096, device=dev).bfloat16()
    y, rstd = torch.empty_like(x), torch.empty(32768, device=dev)
    K.rmsnorm_fwd(x, None, w, None, None, 1, y, None, rstd, 1e-6)
    from .functional import _NORM_BWD_BLOCKS
    dwp = torch.empty(_NORM_BWD_BLOCKS, 4096, device=dev)
    dwo = torch.empty(4096, device=dev)
    try:
        out.append(_bw("rmsnorm_bwd", (32768, 4096),
                       timeit(lambda: K.rmsnorm_bwd(dy, x, w, rstd, None, dx, dwp, dwo, False), a.iters), 32768 * 4096 * 6.0))
    except Exception as e:                                                    # workspace shape differs between builds
        out.append({"kernel": "rmsnorm_bwd", "skipped": str(e)[:120]})
    img = torch.randn(4, 3, 1022, 1022, device=dev).bfloat16()
    patches = torch.empty(4 * 73 * 73, 640, dtype=torch.bfloat16, device=dev)       # 588 padded to a multiple of 64
    try:
        out.append(_bw("patchify 14x14", (4, 3, 1022, 1022), timeit(lambda: K.patchify(img, patches, 14, None, None), a.iters),
                       img.numel() * 4.0))
    except Exception as e:
        out.append({"kernel": "patchify", "skipped": str(e)[:120]})
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="gemm", choices=["gemm", "gemm_fp8", "gemm_mx", "attn_fwd", "attn_bwd", "rmsnorm", "decode", "ns", "ssm", "gemm_tp_ag", "gemm_tp_rs", "muon_fold", "moe", "streaming"])
    ap.add_argument("--all", action="store_true")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hk", type=int, default=8)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    res = []
    if a.all:
        for shape in [(8192, 8192, 8192), (16384, 6144, 4096), (16384, 4096, 4096), (8192, 5632, 4096)]:
            a.m, a.n, a.k = shape
            res.append(bench_gemm(a))
        res.append(bench_attn(a, False))
        res.append(bench_attn(a, True))
        a.m, a.n = 32768, 4096
        res.append(bench_rmsnorm(a))
        a.batch, a.seq = 64, 4096
        res.append(bench_decode(a))
        a.m, a.n, a.k = 8192, 8192, 8192
        res.append(bench_gemm_fp8(a))
        a.batch, a.seq, a.n = 2, 4096, 8192
        res.append(bench_ssm(a))
        a.batch, a.m, a.n = 128, 1408, 4096
        res.append(bench_newton_schulz(a))
    else:
        fn = {"gemm": bench_gemm, "attn_fwd": lambda x: bench_attn(x, False), "attn_bwd": lambda x: bench_attn(x, True),
              "rmsnorm": bench_rmsnorm, "decode": bench_decode, "ns": bench_newton_schulz, "gemm_fp8": bench_gemm_fp8,
              "gemm_mx": bench_gemm_mx, "ssm": bench_ssm, "gemm_tp_ag": lambda x: bench_gemm_tp(x, 1),
              "gemm_tp_rs": lambda x: bench_gemm_tp(x, 2), "muon_fold": bench_muon_fold, "moe": bench_moe,
              "streaming": bench_streaming}[a.kernel]
        r = fn(a)
        res.extend(r if isinstance(r, list) else [r])
    out = {"peaks": peaks(), "results": res}
    print(json.dumps(out, indent=1))
    if a.json:
        json.dump(out, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
