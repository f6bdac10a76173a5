"""Micro-benchmark of the tensor-parallel GEMM + collective pairs: NCCL + GEMM (the baseline) against the fused
single-kernel path, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29531 \
        -m pisceslx_b200.parallel.bench_tp --tokens 16384 --hidden 4096 --out 6144

Times are CUDA-event times on the launching stream after warm-up, maximum over ranks; the L2 is flushed between
iterations.  The roofline of a pair is the slower of FLOPs / measured bf16 peak and the bytes that must cross
NVLink / the peer-copy bandwidth per direction, which this program measures first on the same GPUs
(``parallel.bench_nvlink.measure``; ``--nvlink-gbs`` overrides it)."""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--out", type=int, default=6144, help="output features of the column-parallel layer (all ranks)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--nvlink-gbs", type=float, default=0.0, help="link bandwidth for the roofline (0 = measure it now)")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from pisceslx_b200.ops import check_status, functional as F_, kernels
    from pisceslx_b200.ops.bench_kernels import peaks
    from pisceslx_b200.parallel import fused_tp as ft
    from pisceslx_b200.parallel import tp as tpm
    K = kernels()
    group = dist.group.WORLD
    probe = {}
    if a.nvlink_gbs <= 0:
        from pisceslx_b200.parallel.bench_nvlink import measure
        probe = measure(group, 256, 5)
    NVLINK_GBS = a.nvlink_gbs if a.nvlink_gbs > 0 else probe["peer_copy_gbs"]
    T, H, N = a.tokens, a.hidden, a.out
    rows, n_loc, k_loc = T // world, N // world, H // world
    torch.manual_seed(rank)
    x_shard = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
    w_col = torch.randn(n_loc, H, device=dev, dtype=torch.bfloat16) * 0.02           # column-parallel weight
    x_full = torch.randn(T, k_loc, device=dev, dtype=torch.bfloat16)
    w_row = torch.randn(H, k_loc, device=dev, dtype=torch.bfloat16) * 0.02           # row-parallel weight
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        tot = 0.0
        for _ in range(a.iters):
            K.l2_flush(flush)
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            tot += s.elapsed_time(e)
        t = torch.tensor([tot / a.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def ag_nccl():
        return F_.gemm(tpm.all_gather_rows(x_shard, group), w_col)

    def ag_fused():
        return ft.allgather_gemm(x_shard, w_col, group)[1]

    def rs_nccl():
        return tpm.reduce_scatter_rows(F_.gemm(x_full, w_row), group)

    def rs_fused():
        return ft.gemm_reduce_scatter(x_full, w_row, group)

    # numerics of the fused paths against the NCCL ones
    err_ag = float((ag_fused().float() - ag_nccl().float()).abs().max())
    err_rs = float((rs_fused().float() - rs_nccl().float()).abs().max() / rs_nccl().float().abs().max())
    res = {"ag_nccl_ms": timed(ag_nccl), "ag_fused_ms": timed(ag_fused), "rs_nccl_ms": timed(rs_nccl),
           "rs_fused_ms": timed(rs_fused)}
    check_status()
    pk = peaks()
    ag_flops, rs_flops = 2.0 * T * n_loc * H, 2.0 * T * H * k_loc
    ag_bytes = (world - 1) * rows * H * 2                      # received per rank
    rs_bytes = (world - 1) * rows * H * 2                      # sent per rank
    ag_roof = max(ag_flops / (pk["bf16_tflops"] * 1e9), ag_bytes / (NVLINK_GBS * 1e6))
    rs_roof = max(rs_flops / (pk["bf16_tflops"] * 1e9), rs_bytes / (NVLINK_GBS * 1e6))
    if rank == 0:
        print(json.dumps({"world": world, "tokens": T, "hidden": H, "out": N, **res,
                          "ag_roofline_ms": ag_roof, "rs_roofline_ms": rs_roof,
                          "ag_fused_frac_of_roofline": ag_roof / res["ag_fused_ms"],
                          "rs_fused_frac_of_roofline": rs_roof / res["rs_fused_ms"],
                          "ag_speedup_vs_nccl": res["ag_nccl_ms"] / res["ag_fused_ms"],
                          "rs_speedup_vs_nccl": res["rs_nccl_ms"] / res["rs_fused_ms"],
                          "max_abs_err_ag": err_ag, "rel_err_rs": err_rs, "peaks": pk["kind"],
                          "nvlink_gbs_used": NVLINK_GBS, "nvlink_probe": probe}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
