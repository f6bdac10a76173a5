"""Layout planning for the parallel runtime: which tp x ep x pp x dp mesh fits a model into 180 GB parts, how much
memory each rank then holds, and how gradient buckets are sized so that their reduction hides under backward.

Reference counterparts: ``PiscesLxParallel3DOperator`` (opss/train/parallel_3d.py:136-730: config with dp/tp/pp sizes
and a ZeRO stage, rank <-> coordinate mapping, ``get_memory_estimate`` :696), ``PiscesLxCommComputeOverlapOptimizer``
(:731-900: gradient buckets of a fixed 25 MB reduced asynchronously), ``PiscesLxFSDPTrainingOperator``
(opss/train/fsdp.py:170: sharding strategy chosen by name).  Here the mesh itself is built by
``parallel.state.init_parallel``; this module decides its shape.  On an NVSwitch node every pair of GPUs has the same
bandwidth, so the choice is driven by memory and by launch latency, not by link topology."""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch


@dataclass
class PiscesLxParallel3DConfig:
    world_size: int = 1
    tp_size: int = 1
    ep_size: int = 1
    pp_size: int = 1
    zero_stage: int = 1
    sequence_parallel: bool = True
    pipeline_schedule: str = "1f1b"
    num_micro_batches: int = 1
    param_bytes: int = 2                  # bf16 working weights
    master_bytes: int = 4                 # fp32 master copy held by the optimizer shard
    state_bytes_per_param: float = 8.0    # AdamW: two fp32 moments; Muon: one -> 4.0

    @property
    def dp_size(self) -> int:
        return self.world_size // (self.tp_size * self.pp_size)

    def validate(self) -> None:
        assert self.world_size % (self.tp_size * self.pp_size) == 0, "world not divisible by tp*pp"
        assert self.dp_size % self.ep_size == 0, "dp not divisible by ep"

    # rank <-> coordinates, matching the mesh of parallel.state.init_parallel (tp fastest, then dp, then pp)
    def coords(self, rank: int) -> Dict[str, int]:
        tp, dp = self.tp_size, self.dp_size
        d = (rank // tp) % dp
        return {"tp": rank % tp, "dp": d, "pp": rank // (tp * dp), "ep": d % self.ep_size, "edp": d // self.ep_size}

    def rank_of(self, tp: int, dp: int, pp: int) -> int:
        return (pp * self.dp_size + dp) * self.tp_size + tp


@dataclass
class YvModelFootprint:
    """Parameter counts split by how they shard."""
    dense_params: int                     # attention, norms, shared experts, router: replicated over ep, split by tp/pp
    expert_params: int                    # routed experts: split by ep (and tp), replicated over edp
    embed_params: int                     # embedding + output head: vocab-parallel over tp
    n_layer: int
    hidden: int
    act_bytes_per_token_layer: float      # stored activations of one layer for one token without recomputation

    @staticmethod
    def from_config(cfg: Any) -> "YvModelFootprint":
        h, L = cfg.hidden_size, cfg.n_layer
        hd = getattr(cfg, "head_dim", h // cfg.n_head)
        nkv = getattr(cfg, "n_kv_head", cfg.n_head)
        attn = h * (cfg.n_head * hd) * 2 + h * (nkv * hd) * 2
        n_exp = getattr(cfg, "moe_num_experts", 0)
        ffe = getattr(cfg, "moe_expert_intermediate_size", None) or getattr(cfg, "intermediate_size", 4 * h)
        n_sh = getattr(cfg, "moe_shared_experts", 0) if n_exp else 0
        ffs = getattr(cfg, "moe_shared_intermediate_size", None) or 2 * ffe
        if n_exp:
            expert = L * n_exp * 3 * h * ffe
            dense = L * (attn + n_sh * 3 * h * ffs + n_exp * h + 2 * h)
            topk = getattr(cfg, "moe_top_k", 2)
            act_ff = topk * ffe + n_sh * ffs
        else:
            ff = getattr(cfg, "intermediate_size", 4 * h)
            expert, dense, act_ff = 0, L * (attn + 3 * h * ff + 2 * h), ff
        embed = cfg.vocab_size * h * (1 if getattr(cfg, "tie_word_embeddings", False) else 2)
        # bf16 bytes kept per token per layer: residual in, normed x, q/k/v, attention out, FFN gate/up/act, residuals
        act = 2.0 * (6 * h + 2 * nkv * hd + 3 * act_ff)
        return YvModelFootprint(dense, expert, embed, L, h, act)


class PiscesLxParallel3DOperator:
    """Plans and (optionally) initialises the mesh.  ``plan`` returns the cheapest layout that fits: it prefers no
    tensor parallelism (no per-layer collectives), then expert parallelism (moves tokens, not weights), then tensor
    parallelism, and pipeline stages last."""

    def __init__(self, hbm_gb: float = 180.0, usable_fraction: float = 0.86, reserve_gb: float = 6.0):
        self.hbm = hbm_gb * 2 ** 30
        self.usable = usable_fraction * self.hbm - reserve_gb * 2 ** 30

    def memory_estimate(self, fp: YvModelFootprint, c: PiscesLxParallel3DConfig, tokens_per_microbatch: int = 0,
                        stored_layers: int = 0) -> Dict[str, float]:
        c.validate()
        tp, pp, ep, dp = c.tp_size, c.pp_size, c.ep_size, c.dp_size
        dense = (fp.dense_params / pp + fp.embed_params / max(1, min(pp, 2))) / tp
        expert = fp.expert_params / (pp * tp * ep)
        weights = (dense + expert) * c.param_bytes
        grads = (dense + expert) * c.param_bytes
        opt_per_param = c.master_bytes + c.state_bytes_per_param
        if c.zero_stage >= 1:
            opt = dense * opt_per_param / dp + expert * opt_per_param / max(1, dp // ep)
        else:
            opt = (dense + expert) * opt_per_param
        if c.zero_stage >= 2:
            grads = dense * c.param_bytes / dp + expert * c.param_bytes / max(1, dp // ep)
        if c.zero_stage >= 3:
            weights = dense * c.param_bytes / dp + expert * c.param_bytes / max(1, dp // ep)
        layers_here = fp.n_layer / pp
        sp = tp if c.sequence_parallel else 1
        boundary = tokens_per_microbatch * fp.hidden * 2 / sp * layers_here          # checkpoints of recomputed layers
        stored = tokens_per_microbatch * fp.act_bytes_per_token_layer / tp * min(stored_layers, layers_here)
        total = weights + grads + opt + boundary + stored
        g = 2 ** 30
        return {"weights_gb": weights / g, "grads_gb": grads / g, "optimizer_gb": opt / g,
                "activations_gb": (boundary + stored) / g, "total_gb": total / g, "fits": total <= self.usable,
                "headroom_gb": (self.usable - total) / g}

    def candidates(self, world: int, n_experts: int, n_kv_head: int) -> List[Tuple[int, int, int]]:
        out = []
        for pp in (1, 2, 4, 8):
            for tp in (1, 2, 4, 8):
                if world % (tp * pp) or (n_kv_head and n_kv_head % tp):
                    continue
                dp = world // (tp * pp)
                for ep in (1, 2, 4, 8, 16, 32, 64):
                    if dp % ep or (n_experts and n_experts % ep) or (not n_experts and ep > 1):
                        continue
                    out.append((tp, ep, pp))
        # cost order: pipeline stages, then tensor parallel degree, then prefer the largest ep (most memory freed)
        return sorted(out, key=lambda t: (t[2], t[0], -t[1]))

    def plan(self, cfg: Any, world: int, tokens_per_microbatch: int, zero_stage: int = 1,
             state_bytes_per_param: float = 8.0) -> Tuple[PiscesLxParallel3DConfig, Dict[str, float]]:
        fp = YvModelFootprint.from_config(cfg)
        n_exp = getattr(cfg, "moe_num_experts", 0)
        best = None
        for tp, ep, pp in self.candidates(world, n_exp, getattr(cfg, "n_kv_head", 0)):
            c = PiscesLxParallel3DConfig(world, tp, ep, pp, zero_stage, state_bytes_per_param=state_bytes_per_param)
            est = self.memory_estimate(fp, c, tokens_per_microbatch)
            if est["fits"]:
                return c, est
            if best is None or est["total_gb"] < best[1]["total_gb"]:
                best = (c, est)
        assert best is not None, "no valid layout for this world size"
        return best

    def initialize(self, c: PiscesLxParallel3DConfig, **kw):
        from .state import init_parallel
        c.validate()
        return init_parallel(tp=c.tp_size, ep=c.ep_size, pp=c.pp_size, **kw)


class PiscesLxCommComputeOverlapOptimizer:
    """Sizes gradient-reduction buckets from two measured constants of the node: the fixed cost of one collective
    (launch + synchronisation, ``latency_us``) and its bus bandwidth.  A bucket of ``b`` bytes costs
    ``latency + b / bandwidth``; buckets are made large enough that latency is at most ``latency_share`` of that, and
    no larger, so that the first reduction starts early in backward and the last (exposed) one is short."""

    def __init__(self, latency_us: float = 35.0, bus_gbs: float = 725.0, latency_share: float = 0.1,
                 min_mb: float = 8.0, max_mb: float = 512.0):
        self.latency_s, self.bw = latency_us * 1e-6, bus_gbs * 1e9
        self.share, self.min_b, self.max_b = latency_share, min_mb * 2 ** 20, max_mb * 2 ** 20

    def bucket_bytes(self, world: int) -> int:
        # ring / NVLS all-reduce moves 2 (w-1)/w of the payload per rank
        eff = self.bw / (2 * (world - 1) / world) if world > 1 else self.bw
        b = self.latency_s * eff * (1 - self.share) / self.share
        return int(min(self.max_b, max(self.min_b, b)))

    def build_buckets(self, params: Sequence[torch.nn.Parameter], world: int) -> List[List[int]]:
        """Indices of ``params`` grouped in reverse registration order (the order backward produces gradients)."""
        cap, out, cur, size = self.bucket_bytes(world), [], [], 0
        for i in reversed(range(len(params))):
            p = params[i]
            if not p.requires_grad:
                continue
            n = p.numel() * p.element_size()
            if cur and size + n > cap:
                out.append(cur)
                cur, size = [], 0
            cur.append(i)
            size += n
        if cur:
            out.append(cur)
        return out

    def exposed_time(self, bucket_sizes: Sequence[int], backward_s: float, world: int) -> Dict[str, float]:
        """Simulates backward producing buckets at a uniform rate while one communication stream drains them."""
        total = float(sum(bucket_sizes)) or 1.0
        eff = self.bw / (2 * (world - 1) / world) if world > 1 else float("inf")
        t_ready, t_comm = 0.0, 0.0
        for b in bucket_sizes:
            t_ready += backward_s * b / total
            t_comm = max(t_comm, t_ready) + self.latency_s + b / eff
        return {"comm_total_s": sum(self.latency_s + b / eff for b in bucket_sizes), "exposed_s": max(0.0, t_comm - backward_s),
                "finish_s": t_comm}


class PiscesLxFSDPOperator:
    """Name-compatible selector of the sharding strategy: maps the reference's FSDP strategy names to the ZeRO stage
    of this runtime's sharded optimizer (parallel.zero)."""

    STRATEGIES = {"no_shard": 0, "shard_grad_op": 2, "full_shard": 3, "hybrid_shard": 3, "zero1": 1, "zero2": 2, "zero3": 3}

    def __init__(self, strategy: str = "zero1"):
        if strategy.lower() not in self.STRATEGIES:
            raise ValueError(f"unknown sharding strategy {strategy!r}; one of {sorted(self.STRATEGIES)}")
        self.strategy = strategy.lower()

    @property
    def zero_stage(self) -> int:
        return self.STRATEGIES[self.strategy]

    def apply(self, trainer_cfg: Any) -> Any:
        setattr(trainer_cfg, "zero_stage", self.zero_stage)
        return trainer_cfg
