"""Process-group mesh: one process per GPU, ranks laid out as  pp x dp x tp  with expert parallelism carved
out of the data-parallel dimension (experts are sharded over ``ep`` ranks of a dp row and replicated over
the remaining ``dp / ep`` "expert data parallel" ranks).

rank = ((pp_rank * dp_size) + dp_rank) * tp_size + tp_rank           (tp fastest: neighbours share NVLink hops)

The reference initialises a single world group and forces TP = PP = 1 (opss/train/parallel_3d.py:237-268);
its expert parallel operator is never called (utils/opsc/distributed.py:1018-1158).  Here every dimension
is a real group, on NCCL for GPUs and Gloo for CPU tests.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import Any, List, Optional

import torch
import torch.distributed as dist


@dataclass
class YvParallelState:
    world_size: int = 1
    rank: int = 0
    local_rank: int = 0
    tp_size: int = 1
    ep_size: int = 1
    pp_size: int = 1
    dp_size: int = 1
    cp_size: int = 1
    tp_rank: int = 0
    ep_rank: int = 0
    pp_rank: int = 0
    dp_rank: int = 0
    edp_size: int = 1            # expert-data-parallel size = dp / ep
    edp_rank: int = 0
    tp_group: Any = None
    ep_group: Any = None
    dp_group: Any = None         # gradient reduction of dense (non-expert) parameters
    edp_group: Any = None        # gradient reduction of expert parameters
    pp_group: Any = None
    model_parallel_group: Any = None   # tp x pp (norm reductions for clipping)
    expert_grad_group: Any = None      # tp x edp: ranks that hold replicas of the same routed experts
    stage_group: Any = None            # tp x dp: all ranks of one pipeline stage
    cp_group: Any = None               # context parallel: cp consecutive data-parallel ranks share their sequences
    cp_rank: int = 0
    world_group: Any = None
    backend: str = "none"
    device: torch.device = field(default_factory=lambda: torch.device("cpu"))
    pp_prev: Optional[int] = None
    pp_next: Optional[int] = None

    @property
    def is_distributed(self) -> bool:
        return self.world_size > 1

    @property
    def data_rank(self) -> int:
        """Index of the distinct data shard this rank reads: context-parallel peers read the same sequences."""
        return self.dp_rank // max(self.cp_size, 1)

    @property
    def data_size(self) -> int:
        return self.dp_size // max(self.cp_size, 1)


_STATE: Optional[YvParallelState] = None


def get_state() -> YvParallelState:
    global _STATE
    if _STATE is None:
        _STATE = YvParallelState()
    return _STATE


def default_nccl_env() -> None:
    """Single-node NVSwitch defaults.  (The reference pins NCCL_ALGO=Ring / NCCL_PROTO=Simple /
    NCCL_MIN_NCHANNELS=1, tools/train/orchestrator.py:1085-1088, which leaves NVLS and tree off; nothing is
    pinned here so NCCL may use NVLS.)"""
    os.environ.setdefault("TORCH_NCCL_AVOID_RECORD_STREAMS", "1")
    os.environ.setdefault("NCCL_SOCKET_IFNAME", "lo")
    os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")


def init_parallel(tp: int = 1, ep: int = 1, pp: int = 1, backend: Optional[str] = None,
                  timeout_s: float = 600.0, device: Optional[torch.device] = None, cp: int = 1,
                  ep_over_tp: bool = False) -> YvParallelState:
    """Create (or reuse) the default process group from the torchrun environment and build the mesh.

    ``ep_over_tp`` is the serving layout "tensor-parallel attention with expert-parallel experts on the same GPUs"
    (TP 8 x EP 8 on one node): the expert-parallel group IS the tensor-parallel group - attention shards heads over it,
    the sequence-parallel token shards between attention and the MoE layer are what the experts' all-to-all
    dispatches, and every GPU holds 1 / tp of the routed experts instead of a replica of all of them."""
    global _STATE
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if device is None:
        device = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if backend is None:
        backend = "nccl" if device.type == "cuda" else "gloo"
    st = YvParallelState(world_size=world, rank=rank, local_rank=local_rank, backend=backend, device=device)
    if world == 1:
        st.tp_size = st.ep_size = st.pp_size = st.dp_size = 1
        _STATE = st
        return st
    default_nccl_env()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = device
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    assert world % (tp * pp) == 0, f"world {world} not divisible by tp*pp = {tp * pp}"
    dp = world // (tp * pp)
    if ep_over_tp:
        ep = 1                                             # the mesh below is built without a separate ep dimension
    assert dp % ep == 0, f"dp {dp} not divisible by ep {ep}"
    st.tp_size, st.pp_size, st.dp_size, st.ep_size, st.edp_size = tp, pp, dp, ep, dp // ep
    st.tp_rank = rank % tp
    st.dp_rank = (rank // tp) % dp
    st.pp_rank = rank // (tp * dp)
    st.ep_rank = st.dp_rank % ep
    st.edp_rank = st.dp_rank // ep
    st.world_group = dist.group.WORLD

    def make(groups: List[List[int]]):
        mine = None
        for ranks in groups:
            g = dist.new_group(ranks=ranks, backend=backend) if len(ranks) > 1 else None
            if rank in ranks:
                mine = g
        return mine

    r = lambda p, d, t: (p * dp + d) * tp + t
    st.tp_group = make([[r(p, d, t) for t in range(tp)] for p in range(pp) for d in range(dp)])
    st.dp_group = make([[r(p, d, t) for d in range(dp)] for p in range(pp) for t in range(tp)])
    st.ep_group = make([[r(p, e0 * ep + e, t) for e in range(ep)] for p in range(pp) for t in range(tp)
                        for e0 in range(dp // ep)])
    st.edp_group = make([[r(p, e0 * ep + e, t) for e0 in range(dp // ep)] for p in range(pp) for t in range(tp)
                         for e in range(ep)])
    st.pp_group = make([[r(p, d, t) for p in range(pp)] for d in range(dp) for t in range(tp)])
    st.model_parallel_group = make([[r(p, d, t) for p in range(pp) for t in range(tp)] for d in range(dp)])
    st.expert_grad_group = make([[r(p, e0 * ep + e, t) for e0 in range(dp // ep) for t in range(tp)]
                                 for p in range(pp) for e in range(ep)])
    st.stage_group = make([[r(p, d, t) for d in range(dp) for t in range(tp)] for p in range(pp)])
    if ep_over_tp and tp > 1:
        st.ep_size, st.ep_rank, st.ep_group = tp, st.tp_rank, st.tp_group
        st.edp_size, st.edp_rank = dp, st.dp_rank
    # Context parallelism is carved out of the data-parallel dimension: cp consecutive dp ranks hold consecutive
    # chunks of the SAME sequences.  Gradients are still reduced over the whole dp group (different tokens).
    assert dp % cp == 0, f"dp {dp} not divisible by cp {cp}"
    st.cp_size, st.cp_rank = cp, st.dp_rank % cp
    if cp > 1:
        st.cp_group = make([[r(p, c0 * cp + c, t) for c in range(cp)] for p in range(pp) for t in range(tp)
                            for c0 in range(dp // cp)])
    if pp > 1:
        st.pp_prev = r(st.pp_rank - 1, st.dp_rank, st.tp_rank) if st.pp_rank > 0 else None
        st.pp_next = r(st.pp_rank + 1, st.dp_rank, st.tp_rank) if st.pp_rank < pp - 1 else None
    _STATE = st
    return st


def destroy_parallel() -> None:
    global _STATE
    if dist.is_initialized():
        dist.destroy_process_group()
    _STATE = None


def barrier() -> None:
    if dist.is_initialized():
        dist.barrier()
