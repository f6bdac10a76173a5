"""Gradient-clustering initialisation of experts (reference model/moe/expert_init.py:115-1000): gradient statistics
per parameter, k-means (k-means++ seeding, elbow choice of k) over them, experts initialised from the clusters.

Memory: the reference keeps a clone of EVERY collected gradient of every parameter in a list and recomputes the
statistics from the whole list at each call (expert_init.py:320-380) - its footprint grows by one model-sized copy per
step.  Here the statistics are streamed (Welford: a count, a running mean and a running sum of squared deviations per
parameter), so the footprint is two parameter-sized buffers whatever the number of steps, and a call is two fused
updates per parameter.

Features: the reference concatenates the four full-size statistics of each parameter, which only stacks when all
parameters have one shape.  Here every parameter is reduced to a fixed-length sketch - a signed count sketch of its
gradient direction and of its relative deviation (the hash depends only on the flat index, so equal shapes are sketched
alike and inner products between directions are preserved in expectation) plus three scale features - so parameters of
any shapes can be clustered together and the feature matrix is [parameters, 2 x sketch + 3].

Initialisation: the reference overwrites an expert's weight with ``mean gradient + std x noise`` (expert_init.py:
890-905), i.e. with numbers of gradient size that carry no trained function.  Here an expert keeps its weight (a dense
layer being up-cycled, or its fresh initialisation) and is DISPLACED against the mean gradient direction of its cluster's
matching member, by ``init_scale`` x the weight's root mean square, with noise shaped by the gradient's deviation: the
experts of different clusters start apart along directions the data distinguishes, and none of them starts broken."""
from __future__ import annotations

import math
import re
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn


@dataclass
class YvGradientStatistics:
    mean: torch.Tensor            # flat, the parameter's number of elements
    std: torch.Tensor
    norm: torch.Tensor            # scalar: running mean of the gradient's L2 norm
    direction: torch.Tensor       # mean / |mean|
    count: int
    param_shape: Tuple[int, ...]
    param_name: str


@dataclass
class YvClusterInfo:
    cluster_id: int
    centroid: torch.Tensor
    member_indices: List[int]
    member_names: List[str]
    intra_cluster_variance: float
    size: int


class YvGradientClusterInitializer:
    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, min_clusters: int = 4, max_clusters: int = 16,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None, sketch_dim: int = 128):
        self.hidden_size, self.intermediate_size, self.num_experts = hidden_size, intermediate_size, num_experts
        self.min_clusters, self.max_clusters = min_clusters, max_clusters
        self.device, self.dtype, self.sketch_dim = device or torch.device("cpu"), dtype or torch.float32, sketch_dim
        self.gradient_features: Dict[str, YvGradientStatistics] = {}
        self.clusters: List[YvClusterInfo] = []
        self._acc: Dict[str, Dict[str, Any]] = {}
        self._collection_count = 0
        self._hash_cache: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}

    # -- statistics ---------------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def collect_gradients(self, model: nn.Module, param_filter: Optional[str] = None) -> Dict[str, YvGradientStatistics]:
        """After ``backward()`` and before the optimizer step; every call adds one sample per parameter."""
        self._collection_count += 1
        pat = re.compile(param_filter) if param_filter else None
        for name, p in model.named_parameters():
            if p.grad is None or (pat is not None and not pat.search(name)):
                continue
            g = p.grad.detach().to(device=self.device, dtype=self.dtype).reshape(-1)
            a = self._acc.get(name)
            if a is None:
                a = self._acc[name] = {"n": 0, "mean": torch.zeros_like(g), "m2": torch.zeros_like(g),
                                       "norm": torch.zeros((), device=self.device, dtype=self.dtype), "shape": tuple(p.shape)}
            a["n"] += 1
            delta = g - a["mean"]
            a["mean"].add_(delta, alpha=1.0 / a["n"])
            a["m2"].addcmul_(delta, g - a["mean"])
            a["norm"].add_((g.norm() - a["norm"]) / a["n"])
        self.gradient_features = self._compute_gradient_statistics()
        return self.gradient_features

    def _compute_gradient_statistics(self) -> Dict[str, YvGradientStatistics]:
        out = {}
        for name, a in self._acc.items():
            std = (a["m2"] / max(a["n"] - 1, 1)).sqrt() if a["n"] > 1 else torch.zeros_like(a["mean"])
            out[name] = YvGradientStatistics(a["mean"], std, a["norm"], a["mean"] / a["mean"].norm().clamp_min(1e-12), a["n"], a["shape"], name)
        return out

    def reset_statistics(self) -> None:
        self._acc.clear()
        self.gradient_features, self.clusters, self._collection_count = {}, [], 0

    # -- features -----------------------------------------------------------------------------------------------------------------
    def _hash(self, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
        h = self._hash_cache.get(n)
        if h is None:
            i = torch.arange(n, device=self.device, dtype=torch.int64)
            x = (i * 2654435761 + 40503) & 0xFFFFFFFF                                  # multiplicative hashes of the flat index
            bucket = ((x >> 7) % self.sketch_dim)
            sign = (((x * 2246822519) >> 15) & 1).to(self.dtype) * 2 - 1
            h = self._hash_cache[n] = (bucket, sign)
        return h

    def _sketch(self, v: torch.Tensor) -> torch.Tensor:
        bucket, sign = self._hash(v.numel())
        return torch.zeros(self.sketch_dim, device=self.device, dtype=self.dtype).index_add_(0, bucket, v * sign)

    def _extract_clustering_features(self, gradient_stats: Dict[str, YvGradientStatistics]) -> Tuple[torch.Tensor, List[str]]:
        feats, names = [], []
        for name, s in gradient_stats.items():
            d = self._sketch(s.direction)
            rel = s.std / s.mean.abs().mean().clamp_min(1e-12)
            r = self._sketch(rel / rel.norm().clamp_min(1e-12))
            scal = torch.stack([torch.log10(s.norm.clamp_min(1e-20)), torch.log10(s.mean.abs().mean().clamp_min(1e-20)),
                                torch.log10(s.std.mean().clamp_min(1e-20))]) * 0.1
            feats.append(torch.cat([d, 0.5 * r, scal]))
            names.append(name)
        return torch.stack(feats), names

    # -- k-means ------------------------------------------------------------------------------------------------------------------
    def _kmeans_plusplus_init(self, features: torch.Tensor, k: int, generator: torch.Generator) -> torch.Tensor:
        n = features.shape[0]
        first = int(torch.randint(n, (1,), generator=generator))
        cent = [features[first]]
        d2 = (features - cent[0]).pow(2).sum(1)
        for _ in range(1, k):
            p = (d2 / d2.sum().clamp_min(1e-30)).cpu()
            nxt = int(torch.multinomial(p, 1, generator=generator)) if float(p.sum()) > 0 else int(torch.randint(n, (1,), generator=generator))
            cent.append(features[nxt])
            d2 = torch.minimum(d2, (features - cent[-1]).pow(2).sum(1))
        return torch.stack(cent)

    def _kmeans_clustering(self, features: torch.Tensor, num_clusters: int, max_iterations: int = 100, tolerance: float = 1e-4,
                           seed: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        k = max(1, min(num_clusters, features.shape[0]))
        g = torch.Generator().manual_seed(0 if seed is None else seed)
        cent = self._kmeans_plusplus_init(features, k, g)
        labels = torch.zeros(features.shape[0], dtype=torch.long, device=features.device)
        for it in range(max_iterations):
            labels = torch.cdist(features, cent).argmin(1)
            onehot = torch.nn.functional.one_hot(labels, k).to(features.dtype)          # [n, k]
            counts = onehot.sum(0)
            new = (onehot.t() @ features) / counts.clamp_min(1).unsqueeze(1)
            new = torch.where(counts.unsqueeze(1) > 0, new, cent)                        # an empty cluster keeps its centre
            shift = (new - cent).norm()
            cent = new
            if it % 5 == 4 and float(shift) < tolerance:                                 # looked at every fifth round
                break
        return cent, torch.cdist(features, cent).argmin(1)

    def auto_detect_clusters(self, features: torch.Tensor, min_k: int = 4, max_k: int = 16) -> int:
        """The elbow of the within-cluster sum of squares over k (largest second difference)."""
        n = features.shape[0]
        if n < min_k:
            return max(1, n)
        max_k = min(max_k, n)
        ks = list(range(min_k, max_k + 1))
        if len(ks) < 3:
            return min_k
        wcss = []
        for k in ks:
            cent, lab = self._kmeans_clustering(features, k, 50, 1e-3, 42)
            wcss.append((features - cent[lab]).pow(2).sum())
        w = torch.stack(wcss)
        second = (w[2:] - w[1:-1]) - (w[1:-1] - w[:-2])
        return ks[min(int(second.abs().argmax()) + 1, len(ks) - 1)]

    def _build_cluster_info(self, centroids: torch.Tensor, labels: torch.Tensor, param_names: List[str], features: torch.Tensor) -> List[YvClusterInfo]:
        out = []
        lab = labels.tolist()
        for c in range(centroids.shape[0]):
            idx = [i for i, l in enumerate(lab) if l == c]
            if not idx:
                continue
            var = float((features[idx] - centroids[c]).pow(2).sum(1).mean())
            out.append(YvClusterInfo(len(out), centroids[c], idx, [param_names[i] for i in idx], var, len(idx)))
        return out

    def discover_expert_specializations(self, gradient_stats: Optional[Dict[str, YvGradientStatistics]] = None, auto_detect_k: bool = True,
                                        num_clusters: Optional[int] = None, max_iterations: int = 100, tolerance: float = 1e-4,
                                        seed: Optional[int] = None) -> List[YvClusterInfo]:
        stats = self.gradient_features if gradient_stats is None else gradient_stats
        if not stats:
            raise ValueError("No gradient statistics available for clustering: call collect_gradients() first")
        features, names = self._extract_clustering_features(stats)
        if auto_detect_k:
            num_clusters = self.auto_detect_clusters(features, self.min_clusters, min(self.max_clusters, features.shape[0]))
        elif num_clusters is None:
            raise ValueError("num_clusters must be specified when auto_detect_k is False")
        cent, lab = self._kmeans_clustering(features, num_clusters, max_iterations, tolerance, seed)
        self.clusters = self._build_cluster_info(cent, lab, names, features)
        return self.clusters

    # -- initialisation -----------------------------------------------------------------------------------------------------------
    @staticmethod
    def _assign_clusters_to_experts(num_experts: int, num_clusters: int, clusters: List[YvClusterInfo]) -> List[int]:
        """Experts per cluster in proportion to cluster size, at least one each while experts last (largest remainders)."""
        if num_clusters >= num_experts:
            order = sorted(range(num_clusters), key=lambda i: -clusters[i].size)[:num_experts]
            return sorted(order)
        total = sum(c.size for c in clusters)
        per = [1] * num_clusters
        for _ in range(num_experts - num_clusters):
            i = max(range(num_clusters), key=lambda j: clusters[j].size / total / per[j])
            per[i] += 1
        out: List[int] = []
        for i, n in enumerate(per):
            out += [i] * n
        return out

    @staticmethod
    def _reshape_stats(source: torch.Tensor, target_shape: Tuple[int, ...]) -> torch.Tensor:
        n = math.prod(target_shape)
        if source.numel() < n:
            source = source.repeat((n + source.numel() - 1) // source.numel())
        return source[:n].view(target_shape)

    @staticmethod
    def _default_expert_init(experts: Sequence[nn.Module], init_scale: float = 0.02) -> None:
        for e in experts:
            for p in e.parameters():
                if p.requires_grad:
                    nn.init.kaiming_uniform_(p, a=math.sqrt(5)) if p.dim() >= 2 else nn.init.zeros_(p)

    @torch.no_grad()
    def _initialize_single_expert(self, expert: nn.Module, cluster: YvClusterInfo, gradient_stats: Dict[str, YvGradientStatistics], init_scale: float,
                                  preserve_structure: bool, generator: Optional[torch.Generator] = None) -> int:
        touched = 0
        for _, p in expert.named_parameters():
            if not p.requires_grad or p.dim() < 2:
                continue
            same = [gradient_stats[n] for n in cluster.member_names if n in gradient_stats and gradient_stats[n].param_shape == tuple(p.shape)]
            src = same[0] if same else next((gradient_stats[n] for n in cluster.member_names if n in gradient_stats), None)
            if src is None:
                continue
            if not same and preserve_structure:
                continue                                                                # no member of this shape: leave the weight alone
            d = self._reshape_stats(src.direction, tuple(p.shape)).to(p.device, torch.float32)
            s = self._reshape_stats(src.std, tuple(p.shape)).to(p.device, torch.float32)
            rms = p.float().pow(2).mean().sqrt().clamp_min(1e-8)
            d = d / d.pow(2).mean().sqrt().clamp_min(1e-12)                              # unit root mean square
            noise = torch.randn(p.shape, generator=generator).to(p.device) * (s / s.mean().clamp_min(1e-12)).clamp(max=4.0)
            p.add_((-init_scale * rms * d + 0.1 * init_scale * rms * noise).to(p.dtype))
            touched += 1
        return touched

    def initialize_experts_from_clusters(self, experts: Sequence[nn.Module], clusters: Optional[List[YvClusterInfo]] = None,
                                         gradient_stats: Optional[Dict[str, YvGradientStatistics]] = None, init_scale: float = 0.02,
                                         preserve_structure: bool = True, seed: int = 0) -> List[int]:
        """Returns the cluster of every expert (an empty list after the default initialisation when there are no clusters)."""
        clusters = self.clusters if clusters is None else clusters
        stats = self.gradient_features if gradient_stats is None else gradient_stats
        if not clusters:
            self._default_expert_init(experts, init_scale)
            return []
        assign = self._assign_clusters_to_experts(len(experts), len(clusters), clusters)
        g = torch.Generator().manual_seed(seed)
        for e, c in zip(experts, assign):
            self._initialize_single_expert(e, clusters[c], stats, init_scale, preserve_structure, g)
        return assign

    def get_cluster_summary(self) -> Dict[str, Any]:
        return {"num_clusters": len(self.clusters), "collection_count": self._collection_count, "num_parameters": len(self.gradient_features),
                "clusters": [{"cluster_id": c.cluster_id, "size": c.size, "intra_cluster_variance": c.intra_cluster_variance,
                              "members": c.member_names[:8]} for c in self.clusters]}
