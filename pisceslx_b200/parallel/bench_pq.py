"""Benchmark of the Subconscious knowledge field's hot operation: 16 codebooks x 131 072 entries x 128 dims, sharded by
rows over the ranks; every token gathers one entry per codebook, the entries are summed, projected to FiLM scale and
shift and applied to the residual stream.  Three implementations of the same arithmetic, one process per GPU:

  * ``nccl``   the baseline: all-gather the ids, every rank sums the entries IT owns for all tokens of the group,
               reduce-scatter the partial sums (NCCL), then projection GEMM + modulation kernel;
  * ``peer``   gather kernel with peer loads, then projection GEMM + modulation kernel (three kernels, ``e`` and the
               scale / shift matrices round-trip through device memory);
  * ``fused``  the one-kernel path (``ops/csrc/pq_film.cu``).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29551 \
        -m pisceslx_b200.parallel.bench_pq --tokens 16384

Also runs on one GPU (``python -m pisceslx_b200.parallel.bench_pq``): the table is then local.  CUDA-event times after
warm-up, maximum over ranks, L2 flushed between iterations.  The roofline is the slower of the bytes that must cross
NVLink / the measured peer-copy bandwidth and the device-memory bytes (h in, h out, the gathered entries) / the measured
copy bandwidth."""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384, help="tokens per rank")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--codebooks", type=int, default=16)
    ap.add_argument("--entries", type=int, default=131072)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--nvlink-gbs", type=float, default=0.0)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from pisceslx_b200.ops import check_status, functional as F_, kernels, status_word
    from pisceslx_b200.ops.bench_kernels import peaks
    K = kernels()
    st = status_word(dev)
    T, H, C, N, D = a.tokens, a.hidden, a.codebooks, a.entries, 128
    rows = N // world
    torch.manual_seed(1234 + rank)
    nvlink = a.nvlink_gbs
    probe = {}
    if world > 1:
        from pisceslx_b200.parallel import fused as fz
        heap = fz.heap_for(dist.group.WORLD)
        buf = heap.get("bench_pq_table", C * rows * D * 2)
        table = buf.tensor(torch.bfloat16, C * rows * D).view(C, rows, D)
        table.normal_(std=0.02)
        heap.barrier()
        ptrs = buf.ptrs
        if nvlink <= 0:
            from pisceslx_b200.parallel.bench_nvlink import measure
            probe = measure(dist.group.WORLD, 256, 5)
            nvlink = probe["peer_copy_gbs"]
    else:
        table = torch.empty(C, rows, D, device=dev, dtype=torch.bfloat16).normal_(std=0.02)
        ptrs = torch.tensor([table.data_ptr()], dtype=torch.int64)
    idx = torch.randint(0, N, (T, C), device=dev, dtype=torch.int32)
    w = (torch.randn(2 * H, D, device=dev) * 0.05).to(torch.bfloat16)
    h = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(h)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        tot = 0.0
        for _ in range(a.iters):
            K.l2_flush(flush)
            if world > 1:
                dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            tot += s.elapsed_time(e)
        t = torch.tensor([tot / a.iters], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def project_and_modulate(e):
        f = F_.gemm(e, w)                                                  # [T, 2H]
        return F_.film(h.view(1, T, H), f[:, :H].reshape(1, T, H), f[:, H:].reshape(1, T, H)).view(T, H)

    def fused():
        K.pq_film(ptrs, idx, w, h, out, None, C, rows, st)
        return out

    def peer():
        e = torch.empty(T, D, device=dev, dtype=torch.bfloat16)
        if world > 1:
            K.pq_gather_sum_peer(ptrs, idx, e, C, rows, st)
        else:
            K.pq_gather_sum(table, idx, e, st)
        return project_and_modulate(e)

    def nccl():
        if world == 1:
            return peer()
        all_idx = torch.empty(world * T, C, device=dev, dtype=torch.int32)
        dist.all_gather_into_tensor(all_idx, idx)
        local = all_idx - rank * rows
        mine = (local >= 0) & (local < rows)
        local = torch.where(mine, local, torch.full_like(local, -1))      # ids of other shards contribute nothing
        part = torch.empty(world * T, D, device=dev, dtype=torch.bfloat16)
        K.pq_gather_sum(table, local.contiguous(), part, None)
        e = torch.empty(T, D, device=dev, dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(e, part)
        return project_and_modulate(e)

    ref = peer().float()
    err_fused = float((fused().float() - ref).norm() / ref.norm())
    err_nccl = float((nccl().float() - ref).norm() / ref.norm()) if world > 1 else 0.0
    res = {"fused_ms": timed(fused), "peer_ms": timed(peer), "nccl_ms": timed(nccl) if world > 1 else None}
    check_status()
    pk = peaks()
    hbm_bytes = 2.0 * T * H * 2 + T * C * D * 2
    link_bytes = T * C * D * 2 * (world - 1) / world
    roof = max(hbm_bytes / (pk["hbm_gbs"] * 1e6), link_bytes / (nvlink * 1e6) if world > 1 else 0.0)
    if rank == 0:
        print(json.dumps({"world": world, "tokens_per_rank": T, "hidden": H, "field": [C, N, D], **res,
                          "roofline_ms": roof, "fused_frac_of_roofline": roof / res["fused_ms"],
                          "fused_speedup_vs_nccl": (res["nccl_ms"] / res["fused_ms"]) if res["nccl_ms"] else None,
                          "fused_speedup_vs_three_kernels": res["peer_ms"] / res["fused_ms"],
                          "rel_err_fused_vs_three_kernels": err_fused, "rel_err_nccl": err_nccl,
                          "hbm_bytes": hbm_bytes, "nvlink_bytes_per_rank": link_bytes, "nvlink_gbs_used": nvlink,
                          "peaks": pk["kind"], "nvlink_probe": probe}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
