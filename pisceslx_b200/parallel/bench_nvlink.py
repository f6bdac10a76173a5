"""Measured NVLink bandwidth of this node: the denominators of every communication roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29541 \\
        -m pisceslx_b200.parallel.bench_nvlink [--mib 256] [--out profiles/nvlink_probe.json]

Two figures, device-timed (CUDA events, maximum over ranks, after warm-up):
  * ``peer_copy_gbs``: one direction, rank r pulling ``--mib`` MiB from rank r+1's symmetric buffer with the
    16-byte-per-lane peer copy kernel that the fused kernels' transfers are built from (all ranks pull at once, so
    the figure is per GPU under full load);
  * ``allgather_busbw_gbs`` / ``allreduce_busbw_gbs``: NCCL bus bandwidth at the same size.
``measure()`` is importable: the tensor-parallel benchmark calls it first and uses ``peer_copy_gbs`` instead of a
constant."""
from __future__ import annotations

import argparse
import json
import os
from typing import Any, Dict

import torch
import torch.distributed as dist


def _time(fn, iters: int, dev: torch.device) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize(dev)
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def measure(group: Any = None, mib: int = 256, iters: int = 10) -> Dict[str, float]:
    """Must be called by every rank of ``group`` (default: all ranks)."""
    from ..ops import kernels
    from .fused import heap_for
    group = group or dist.group.WORLD
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    dev = torch.device("cuda", torch.cuda.current_device())
    nbytes = mib << 20
    K = kernels()
    heap = heap_for(group)
    buf = heap.get("nvlink_probe", nbytes)
    dst = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    buf.tensor(torch.uint8, nbytes).fill_(rank + 1)
    heap.barrier()
    peer = (rank + 1) % world
    res: Dict[str, float] = {"world": world, "mib": mib}
    if world > 1:
        ms = _time(lambda: K.peer_copy(dst.data_ptr(), buf.peer_ptrs[peer], nbytes), iters, dev)
        assert int(dst[0]) == peer + 1 and int(dst[-1]) == peer + 1, "peer copy returned the wrong data"
        res["peer_copy_gbs"] = nbytes / (ms * 1e-3) / 1e9
        res["peer_copy_ms"] = ms
    x = torch.empty(nbytes // 2, dtype=torch.bfloat16, device=dev).normal_()
    out = torch.empty(world * x.numel(), dtype=torch.bfloat16, device=dev)
    ms = _time(lambda: dist.all_gather_into_tensor(out, x, group=group), iters, dev)
    res["allgather_busbw_gbs"] = (world - 1) * nbytes / (ms * 1e-3) / 1e9
    ms = _time(lambda: dist.all_reduce(x, group=group), iters, dev)
    res["allreduce_busbw_gbs"] = 2 * (world - 1) / world * nbytes / (ms * 1e-3) / 1e9
    heap.barrier()
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    rank = int(os.environ["RANK"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    res = measure(None, a.mib, a.iters)
    if rank == 0:
        print(json.dumps(res))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(res, f, indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
