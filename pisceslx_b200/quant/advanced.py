"""The rest of the quantisation layer: Hessian collection for GPTQ, low-rank KV compression, the advanced (sensitivity-
driven mixed-precision) quantiser, the quantisation benchmark operator and the engine / pipeline configurations (reference
opss/quantize/methods.py:60-124,1385-1545, advanced.py:54-760, benchmark.py:59-650, engine.py:66-86, pipeline.py:63-110).

* ``PiscesLxGPTQHessianComputer``: the reference runs the calibration batches through the model and returns an EMPTY
  dictionary - no hook ever records anything (methods.py:77-121).  Here a forward pre-hook on every linear layer accumulates
  H += x^T x as one GEMM per batch (fp32 accumulation on the device, no activation is kept), and the damped Hessian is what
  ``quant.ptq.PiscesLxGPTQQuantizer`` consumes.
* ``PiscesLxSTARKVCompression``: the reference's ``decompress`` returns the compressed coefficients unchanged and its
  ``compress`` divides them by the singular values but keeps no basis to undo it (methods.py:1516-1535), so nothing can be
  reconstructed.  Here each head keeps (coefficients [T, r], basis [D, r]); the rank per head is the smallest that keeps
  ``energy`` of the spectrum (capped by the compression target), found for all heads at once from one batched SVD of the
  small D x D Gram matrices - the long T axis only ever appears in GEMMs."""
from __future__ import annotations

import json
import statistics
import time
from dataclasses import asdict, dataclass, field
from enum import Enum
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..utils.opsc import PiscesLxOperatorInterface
from .extras import PiscesLxHyperQuant
from .pipeline import (PiscesLxAdaptiveBitAllocationOperator, PiscesLxQuantizationConfig, PiscesLxQuantizationEngine, PiscesLxQuantizationMethod,
                       PiscesLxSensitivityAnalysisOperator)


class YvQuantizationType(str, Enum):
    NONE = "none"
    INT8 = "int8"
    INT4 = "int4"
    FP8 = "fp8"
    FP4 = "fp4"
    NF4 = "nf4"
    MX = "mx"


PiscesLxHyperQuantizer = PiscesLxHyperQuant


@dataclass
class PiscesLxQuantizationEngineConfig:
    name: str = "quantize.engine.config"
    method: str = "gptq"
    bits: int = 4
    group_size: int = 128
    damp_percent: float = 0.01
    desc_act: bool = False
    symmetric: bool = True
    num_calibration_samples: int = 128
    calibration_dataset: Optional[str] = None
    enable_kv_cache_quant: bool = False
    kv_cache_bits: int = 8
    mixed_precision: bool = False
    sensitive_layers: List[str] = field(default_factory=list)
    preserve_accuracy_layers: List[str] = field(default_factory=list)
    device: str = "cuda"
    export_format: str = "safetensors"

    def to_quantization_config(self) -> PiscesLxQuantizationConfig:
        skip = tuple(dict.fromkeys(("lm_head", "embed", "router", "gate", *self.preserve_accuracy_layers)))
        return PiscesLxQuantizationConfig(method=PiscesLxQuantizationMethod(self.method), bits=self.bits, group_size=self.group_size, skip=skip,
                                          per_layer_bits={n: 8 for n in self.sensitive_layers} if self.mixed_precision else {})


@dataclass
class PiscesLxQuantizationPipelineConfig:
    name: str = "quantize.pipeline.config"
    method: str = "auto"
    bits: int = 8
    group_size: int = 128
    enable_sensitivity_analysis: bool = True
    enable_adaptive_allocation: bool = True
    target_compression_ratio: float = 0.5
    calibration_dataset: str = "wikitext"
    calibration_samples: int = 128
    sequence_length: int = 512
    preserve_layers: Optional[List[str]] = None
    exclude_layers: Optional[List[str]] = None
    validate_after_quantization: bool = True
    validation_metric: str = "perplexity"

    def resolved_method(self, has_calibration: bool) -> str:
        """``auto``: GPTQ when there is calibration data and the target is 4 bits or fewer, AWQ for 5-7, round-to-nearest at 8."""
        if self.method != "auto":
            return self.method
        if not has_calibration or self.bits >= 8:
            return "rtn"
        return "gptq" if self.bits <= 4 else "awq"


# ---- Hessians --------------------------------------------------------------------------------------------------------------------
class PiscesLxGPTQHessianComputer:
    def __init__(self, device: Optional[torch.device] = None, dtype: torch.dtype = torch.float32, damp_percent: float = 0.01, skip: Sequence[str] = ("lm_head",)):
        self.device, self.dtype, self.damp_percent, self.skip = device, dtype, damp_percent, tuple(skip)
        self.samples: Dict[str, int] = {}

    def compute_hessian(self, model: nn.Module, dataloader: Iterable[Any], num_samples: int = 128, layers: Optional[Sequence[str]] = None) -> Dict[str, torch.Tensor]:
        """{layer name: H [in, in]} with H = 2 / N sum x^T x over the calibration tokens (undamped; see ``damped``)."""
        hs: Dict[str, torch.Tensor] = {}
        self.samples = {}
        handles = []

        def hook(name: str):
            def fn(mod: nn.Module, args: Tuple[Any, ...]) -> None:
                x = args[0].detach().reshape(-1, args[0].shape[-1]).to(self.dtype)
                h = hs.get(name)
                if h is None:
                    h = hs[name] = torch.zeros(x.shape[1], x.shape[1], device=x.device, dtype=self.dtype)
                h.addmm_(x.t(), x)
                self.samples[name] = self.samples.get(name, 0) + x.shape[0]
            return fn
        for name, m in model.named_modules():
            if isinstance(m, nn.Linear) and not any(s in name for s in self.skip) and (layers is None or name in layers):
                handles.append(m.register_forward_pre_hook(hook(name)))
        was = model.training
        model.eval()
        dev = self.device or next(model.parameters()).device
        try:
            with torch.no_grad():
                for i, batch in enumerate(dataloader):
                    if i >= num_samples:
                        break
                    if isinstance(batch, dict):
                        model(**{k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in batch.items()})
                    elif isinstance(batch, (tuple, list)):
                        model(*[b.to(dev) if torch.is_tensor(b) else b for b in batch])
                    else:
                        model(batch.to(dev))
        finally:
            for h in handles:
                h.remove()
            model.train(was)
        for name, h in hs.items():
            h.mul_(2.0 / max(self.samples[name], 1))
        return hs

    def damped(self, hessian: torch.Tensor) -> torch.Tensor:
        """H + damp_percent x mean(diag H) x I, and 1 on the diagonal of dead inputs (columns never active)."""
        h = hessian.clone()
        d = h.diagonal()
        dead = d == 0
        d[dead] = 1.0
        d.add_(self.damp_percent * d[~dead].mean() if (~dead).any() else self.damp_percent)
        return h

    def inverse_cholesky(self, hessian: torch.Tensor) -> torch.Tensor:
        """The upper Cholesky factor of H^-1 that the GPTQ column sweep reads its update coefficients from."""
        h = self.damped(hessian).double()
        inv = torch.cholesky_inverse(torch.linalg.cholesky(h))
        return torch.linalg.cholesky(inv, upper=True).to(hessian.dtype)


# ---- low-rank KV compression -------------------------------------------------------------------------------------------------
class PiscesLxSTARKVCompression(nn.Module):
    """``compress(key, value)`` [B, H, T, D] -> a dictionary per tensor with coefficients [B, H, T, r_max], bases [B, H, D, r_max]
    and the rank kept per head (columns beyond a head's rank are zero); ``decompress`` rebuilds [B, H, T, D].
    ``attend(query, packed_k, packed_v)`` computes attention WITHOUT rebuilding the keys: q^T k = (q^T basis) coefficients^T."""

    def __init__(self, kv_dim: int, max_rank: Optional[int] = None, compression_target: float = 0.75, energy: float = 0.99, threshold_eps: float = 1e-6):
        super().__init__()
        self.kv_dim, self.target, self.energy, self.eps = kv_dim, compression_target, energy, threshold_eps
        self.max_rank = max_rank or max(1, int(round(kv_dim * (1.0 - compression_target))))

    @property
    def compression(self) -> float:
        return self.target

    @torch.no_grad()
    def _pack(self, x: torch.Tensor) -> Dict[str, torch.Tensor]:
        B, H, T, D = x.shape
        xf = x.float()
        gram = xf.transpose(-1, -2) @ xf                                               # [B, H, D, D]: the only place T is reduced
        evals, evecs = torch.linalg.eigh(gram)
        evals, evecs = evals.flip(-1).clamp_min(0), evecs.flip(-1)                      # descending
        r_max = min(self.max_rank, D)
        share = evals.cumsum(-1) / evals.sum(-1, keepdim=True).clamp_min(self.eps)
        rank = ((share < self.energy).sum(-1) + 1).clamp(max=r_max)                     # [B, H]
        keep = (torch.arange(r_max, device=x.device) < rank.unsqueeze(-1)).to(xf.dtype)  # [B, H, r_max]
        basis = evecs[..., :r_max] * keep.unsqueeze(-2)
        return {"coeff": (xf @ basis).to(x.dtype), "basis": basis.to(x.dtype), "rank": rank}

    def compress(self, key: torch.Tensor, value: torch.Tensor) -> Tuple[Dict[str, torch.Tensor], Dict[str, torch.Tensor], torch.Tensor]:
        k, v = self._pack(key), self._pack(value)
        return k, v, torch.maximum(k["rank"], v["rank"])

    @staticmethod
    def _unpack(p: Dict[str, torch.Tensor]) -> torch.Tensor:
        return p["coeff"] @ p["basis"].transpose(-1, -2)

    def decompress(self, k_compressed: Dict[str, torch.Tensor], v_compressed: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        return self._unpack(k_compressed), self._unpack(v_compressed)

    def attend(self, query: torch.Tensor, k_compressed: Dict[str, torch.Tensor], v_compressed: Dict[str, torch.Tensor], causal: bool = False) -> torch.Tensor:
        """query [B, H, Tq, D] -> [B, H, Tq, D], with scores and the value product both taken in the r-dimensional space."""
        D = query.shape[-1]
        s = (query.float() @ k_compressed["basis"].float()) @ k_compressed["coeff"].float().transpose(-1, -2) / D ** 0.5
        if causal:
            Tq, Tk = s.shape[-2:]
            s = s.masked_fill(~torch.ones(Tq, Tk, dtype=torch.bool, device=s.device).tril(Tk - Tq), float("-inf"))
        out = (torch.softmax(s, -1) @ v_compressed["coeff"].float()) @ v_compressed["basis"].float().transpose(-1, -2)
        return out.to(query.dtype)

    @staticmethod
    def bytes_ratio(p: Dict[str, torch.Tensor], T: int, D: int) -> float:
        """Stored elements over original elements for the ranks actually kept."""
        r = p["rank"].float().mean().item()
        return (T * r + D * r) / (T * D)


# ---- advanced quantiser ----------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxAdvancedQuantizationConfig:
    name: str = "quantize.advanced.config"
    sensitivity_analysis: bool = True
    adaptive_bit_allocation: bool = True
    preserve_layers: Optional[List[str]] = None
    target_compression_ratio: float = 0.5
    calibration_samples: int = 128
    sensitivity_metric: str = "mse"
    candidate_bits: Tuple[int, ...] = (2, 3, 4, 8)
    method: str = "rtn"
    group_size: int = 128


class PiscesLxAdvancedQuantizer:
    """Sensitivity per layer (the error a layer's output takes when only that layer is quantised to few bits, on calibration
    inputs), then bits per layer under a size budget (the most sensitive layers get the most bits), then quantisation."""

    def __init__(self, config: Optional[PiscesLxAdvancedQuantizationConfig] = None):
        self.config = config or PiscesLxAdvancedQuantizationConfig()
        self.sensitivity: Dict[str, float] = {}
        self.allocation: Dict[str, int] = {}

    @staticmethod
    def _fake_quant(w: torch.Tensor, bits: int, group: int) -> torch.Tensor:
        g = group if (group > 0 and w.shape[1] % group == 0) else w.shape[1]
        x = w.float().view(w.shape[0], -1, g)
        qmax = 2 ** (bits - 1) - 1
        s = x.abs().amax(-1, keepdim=True).clamp_min(1e-12) / max(qmax, 1)
        return ((x / s).round().clamp(-qmax - 1, qmax) * s).view_as(w).to(w.dtype)

    def _layers(self, model: nn.Module) -> Dict[str, nn.Linear]:
        keep = tuple(self.config.preserve_layers or ("lm_head", "embed"))
        return {n: m for n, m in model.named_modules() if isinstance(m, nn.Linear) and not any(k in n for k in keep)}

    @torch.no_grad()
    def analyze_sensitivity(self, model: nn.Module, calibration: Sequence[Any], probe_bits: int = 3) -> Dict[str, float]:
        layers = self._layers(model)
        acts: Dict[str, List[torch.Tensor]] = {n: [] for n in layers}
        hs = [m.register_forward_pre_hook(lambda mod, a, n=n: acts[n].append(a[0].detach().reshape(-1, a[0].shape[-1])[:256])) for n, m in layers.items()]
        was = model.training
        model.eval()
        try:
            for b in list(calibration)[: self.config.calibration_samples]:
                model(**b) if isinstance(b, dict) else model(b)
        finally:
            for h in hs:
                h.remove()
            model.train(was)
        out = {}
        for n, m in layers.items():
            if not acts[n]:
                out[n] = 0.0
                continue
            x = torch.cat(acts[n])[:2048].to(m.weight.dtype)
            ref = x @ m.weight.t()
            err = (x @ self._fake_quant(m.weight, probe_bits, self.config.group_size).t() - ref).float().pow(2).mean() / ref.float().pow(2).mean().clamp_min(1e-12)
            out[n] = float(err)
        self.sensitivity = out
        return out

    def allocate_bits(self, model: nn.Module, sensitivity: Optional[Dict[str, float]] = None) -> Dict[str, int]:
        """Start every layer at the smallest candidate; while the size budget (``target_compression_ratio`` x 16-bit size) has room,
        raise the layer with the largest sensitivity per added byte to its next candidate."""
        sens = sensitivity if sensitivity is not None else self.sensitivity
        layers = self._layers(model)
        cands = sorted(self.config.candidate_bits)
        size = {n: m.weight.numel() for n, m in layers.items()}
        budget = self.config.target_compression_ratio * 16.0 * sum(size.values())
        alloc = {n: cands[0] for n in layers}
        used = sum(alloc[n] * size[n] for n in layers)
        while True:
            best, gain = None, 0.0
            for n in layers:
                i = cands.index(alloc[n])
                if i + 1 >= len(cands):
                    continue
                extra = (cands[i + 1] - alloc[n]) * size[n]
                if used + extra > budget:
                    continue
                g = (sens.get(n, 0.0) / 4.0 ** (alloc[n] - cands[0]) + 1e-12) / extra       # the error falls about 4x per added bit
                if g > gain:
                    best, gain = n, g
            if best is None:
                break
            nxt = cands[cands.index(alloc[best]) + 1]
            used += (nxt - alloc[best]) * size[best]
            alloc[best] = nxt
        self.allocation = alloc
        return alloc

    @torch.no_grad()
    def quantize(self, model: nn.Module, calibration: Optional[Sequence[Any]] = None) -> Dict[str, Any]:
        c = self.config
        layers = self._layers(model)
        if c.sensitivity_analysis and calibration:
            self.analyze_sensitivity(model, calibration)
        else:
            self.sensitivity = {n: 1.0 for n in layers}
        alloc = self.allocate_bits(model) if c.adaptive_bit_allocation else {n: 4 for n in layers}
        err = {}
        for n, m in layers.items():
            q = self._fake_quant(m.weight, alloc[n], c.group_size)
            err[n] = float((q.float() - m.weight.float()).pow(2).mean() / m.weight.float().pow(2).mean().clamp_min(1e-12))
            m.weight.copy_(q)
        total = sum(m.weight.numel() for m in layers.values())
        mean_bits = sum(alloc[n] * layers[n].weight.numel() for n in layers) / max(total, 1)
        return {"allocation": alloc, "sensitivity": dict(self.sensitivity), "mean_bits": mean_bits, "compression_ratio": mean_bits / 16.0, "weight_error": err,
                "layers": len(layers)}

    @staticmethod
    def advanced_quantize(model: nn.Module, calibration: Optional[Sequence[Any]] = None, config: Optional[PiscesLxAdvancedQuantizationConfig] = None) -> Dict[str, Any]:
        return PiscesLxAdvancedQuantizer(config).quantize(model, calibration)


# ---- benchmark operator ----------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxBenchmarkConfig:
    batch_size: int = 1
    sequence_length: int = 512
    num_warmup_iterations: int = 10
    num_benchmark_iterations: int = 100
    warmup_tokens: int = 100
    benchmark_tokens: int = 1000
    enable_memory_profiling: bool = True
    enable_throughput_test: bool = True
    enable_latency_test: bool = True
    enable_accuracy_test: bool = False
    test_dataset: Optional[str] = None
    metrics: List[str] = field(default_factory=lambda: ["throughput", "latency", "memory", "accuracy"])
    vocab_size: int = 32000
    quality_threshold: float = 0.05            # the largest relative loss increase that still passes


class PiscesLxQuantizationBenchmarkOperator(PiscesLxOperatorInterface):
    """Latency, throughput, memory and (given held-out batches) loss of a model, against a baseline when one is set.  Timed with CUDA
    events after warm-up on a GPU, ``perf_counter`` on the host."""

    name = "quantization_benchmark"

    def __init__(self, config: Optional[PiscesLxBenchmarkConfig] = None):
        self.config = config or PiscesLxBenchmarkConfig()
        self.baseline: Optional[Dict[str, Any]] = None
        self.history: List[Dict[str, Any]] = []

    def set_baseline(self, results: Dict[str, Any]) -> None:
        self.baseline = results

    def generate_test_inputs(self, model: nn.Module) -> torch.Tensor:
        c = self.config
        v = int(getattr(getattr(model, "cfg", None), "vocab_size", 0) or c.vocab_size)
        g = torch.Generator().manual_seed(0)
        return torch.randint(0, v, (c.batch_size, c.sequence_length), generator=g).to(next(model.parameters()).device)

    @torch.no_grad()
    def _times(self, model: nn.Module, ids: torch.Tensor) -> List[float]:
        c, dev = self.config, ids.device
        call = (lambda: model(input_ids=ids)) if "input_ids" in getattr(model.forward, "__code__", type("", (), {"co_varnames": ()})).co_varnames else (lambda: model(ids))
        for _ in range(c.num_warmup_iterations):
            call()
        if dev.type == "cuda":
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(c.num_benchmark_iterations)]
            torch.cuda.synchronize(dev)
            for a, b in evs:
                a.record()
                call()
                b.record()
            torch.cuda.synchronize(dev)
            return [a.elapsed_time(b) for a, b in evs]
        out = []
        for _ in range(c.num_benchmark_iterations):
            t0 = time.perf_counter()
            call()
            out.append((time.perf_counter() - t0) * 1e3)
        return out

    @staticmethod
    def benchmark_memory(model: nn.Module) -> Dict[str, float]:
        pb = sum(p.numel() * p.element_size() for p in model.parameters()) + sum(b.numel() * b.element_size() for b in model.buffers())
        out = {"model_mb": pb / 2 ** 20}
        dev = next(model.parameters()).device
        if dev.type == "cuda":
            out["allocated_mb"], out["peak_mb"] = torch.cuda.memory_allocated(dev) / 2 ** 20, torch.cuda.max_memory_allocated(dev) / 2 ** 20
        return out

    @torch.no_grad()
    def benchmark_accuracy(self, model: nn.Module, heldout: Sequence[Any]) -> Dict[str, float]:
        tot, n = 0.0, 0
        for b in heldout:
            out = model(**b) if isinstance(b, dict) else model(b)
            loss = out["loss"] if isinstance(out, dict) else getattr(out, "loss", None)
            if loss is not None:
                tot, n = tot + float(loss), n + 1
        return {"loss": tot / n, "perplexity": float(torch.exp(torch.tensor(min(tot / n, 30.0))))} if n else {}

    def compare_with_baseline(self, result: Dict[str, Any]) -> Dict[str, float]:
        b = self.baseline
        if not b:
            return {}
        out = {}
        if result.get("latency") and b.get("latency"):
            out["speedup"] = b["latency"]["mean_ms"] / max(result["latency"]["mean_ms"], 1e-12)
        if result.get("memory") and b.get("memory"):
            out["memory_ratio"] = result["memory"]["model_mb"] / max(b["memory"]["model_mb"], 1e-12)
        if result.get("accuracy") and b.get("accuracy"):
            out["loss_increase"] = (result["accuracy"]["loss"] - b["accuracy"]["loss"]) / max(abs(b["accuracy"]["loss"]), 1e-12)
        return out

    def run_full_benchmark(self, model: nn.Module, model_name: str = "model", quantization_method: str = "none", bits: int = 16,
                           heldout: Optional[Sequence[Any]] = None) -> Dict[str, Any]:
        c, t0 = self.config, time.perf_counter()
        was = model.training
        model.eval()
        res: Dict[str, Any] = {"model_name": model_name, "quantization_method": quantization_method, "bits": bits}
        ids = self.generate_test_inputs(model)
        if c.enable_latency_test or c.enable_throughput_test:
            ms = sorted(self._times(model, ids))
            mean = statistics.fmean(ms)
            res["latency"] = {"mean_ms": mean, "p50_ms": ms[len(ms) // 2], "p95_ms": ms[min(int(0.95 * len(ms)), len(ms) - 1)], "p99_ms": ms[min(int(0.99 * len(ms)), len(ms) - 1)]}
            res["throughput"] = {"tokens_per_second": ids.numel() / (mean / 1e3), "samples_per_second": ids.shape[0] / (mean / 1e3)}
            res["timing"] = "cuda_events" if ids.device.type == "cuda" else "host"
        if c.enable_memory_profiling:
            res["memory"] = self.benchmark_memory(model)
        if (c.enable_accuracy_test or heldout) and heldout:
            res["accuracy"] = self.benchmark_accuracy(model, heldout)
        res["comparison_with_baseline"] = self.compare_with_baseline(res)
        inc = res["comparison_with_baseline"].get("loss_increase")
        res["passes_quality_threshold"] = inc is None or inc <= c.quality_threshold
        res["benchmark_time_seconds"] = time.perf_counter() - t0
        model.train(was)
        self.history.append(res)
        return res

    def export_results(self, path: str) -> str:
        p = Path(path)
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_text(json.dumps({"baseline": self.baseline, "results": self.history}, indent=1))
        return str(p)

    def get_stats(self) -> Dict[str, Any]:
        return {"runs": len(self.history), "has_baseline": self.baseline is not None}

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return isinstance(inputs.get("model"), nn.Module)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        r = self.run_full_benchmark(inputs["model"], inputs.get("model_name", "model"), inputs.get("quantization_method", "none"), int(inputs.get("bits", 16)), inputs.get("heldout"))
        if inputs.get("as_baseline"):
            self.set_baseline(r)
        return r
