"""Quantisation engine and pipeline (reference opss/quantize: engine.py ``PiscesLxQuantizationEngine``, pipeline.py
``PiscesLxQuantizationPipelineOperator``, calibration.py activation collector / calibration loader, methods.py operator
wrappers, benchmark.py evaluator / benchmark / memory profiler, plus sensitivity analysis and adaptive bit
allocation).  Works on any module tree with ``nn.Linear`` layers; the package's own fused-weight modules are
quantised with ``quant.ptq.quantize_model_weights``."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from ..utils.opsc import PiscesLxOperatorInterface
from .ptq import (PiscesLxAWQQuantizer, PiscesLxBlockWiseINT4Quantizer, PiscesLxGPTQQuantizer, PiscesLxSmoothQuantizer)


class PiscesLxQuantizationMethod(str, Enum):
    RTN = "rtn"                  # round to nearest, group-wise
    GPTQ = "gptq"
    AWQ = "awq"
    SMOOTHQUANT = "smoothquant"


class PiscesLxScaleMethod(str, Enum):
    ABSMAX = "absmax"
    PERCENTILE = "percentile"


class PiscesLxFP8Format(str, Enum):
    E4M3 = "e4m3"
    E5M2 = "e5m2"


@dataclass
class PiscesLxCalibrationConfig:
    n_batches: int = 8
    max_rows_per_layer: int = 4096


@dataclass
class PiscesLxQuantizationConfig:
    method: PiscesLxQuantizationMethod = PiscesLxQuantizationMethod.RTN
    bits: int = 4
    group_size: int = 128
    skip: Tuple[str, ...] = ("lm_head", "embed", "router", "gate")
    per_layer_bits: Dict[str, int] = field(default_factory=dict)      # overrides from the bit allocator


@dataclass
class PiscesLxQuantizationResult:
    layers: int
    method: str
    mean_bits: float
    weight_error: Dict[str, float]
    seconds: float


# ------------------------------------------------------------------------------------------------ calibration
class PiscesLxActivationCollectorOperator(PiscesLxOperatorInterface):
    """inputs {"model", "batches": iterable of model inputs (tensor or kwargs dict)} -> {layer name: [rows, in]}
    activations seen by every ``nn.Linear`` (forward pre-hooks, at most ``max_rows_per_layer`` rows kept)."""
    name = "activation_collector"

    def __init__(self, config: Optional[PiscesLxCalibrationConfig] = None):
        self.config = config or PiscesLxCalibrationConfig()

    def run(self, inputs: Dict[str, Any]) -> Dict[str, torch.Tensor]:
        model, cap = inputs["model"], self.config.max_rows_per_layer
        store: Dict[str, List[torch.Tensor]] = {}
        handles = []
        for name, m in model.named_modules():
            if isinstance(m, nn.Linear):
                def hook(mod, args, name=name):
                    x = args[0].detach().reshape(-1, args[0].shape[-1]).float().cpu()
                    have = sum(t.shape[0] for t in store.get(name, []))
                    if have < cap:
                        store.setdefault(name, []).append(x[: cap - have])
                handles.append(m.register_forward_pre_hook(hook))
        was = model.training
        model.eval()
        with torch.no_grad():
            for i, b in enumerate(inputs["batches"]):
                if i >= self.config.n_batches:
                    break
                model(**b) if isinstance(b, dict) else model(b)
        model.train(was)
        for h in handles:
            h.remove()
        return {k: torch.cat(v) for k, v in store.items()}


class PiscesLxCalibrationDataLoaderOperator(PiscesLxOperatorInterface):
    """inputs {"texts" | "token_ids", "tokenizer", "seq_len", "batch"} -> list of [batch, seq_len] id tensors."""
    name = "calibration_loader"

    def run(self, inputs: Dict[str, Any]) -> List[torch.Tensor]:
        S, B = int(inputs.get("seq_len", 128)), int(inputs.get("batch", 4))
        if "token_ids" in inputs:
            flat = torch.as_tensor(inputs["token_ids"]).flatten()
        else:
            tok = inputs["tokenizer"]
            flat = torch.tensor([t for s in inputs["texts"] for t in tok.encode(s)])
        n = flat.numel() // (S * B)
        return list(flat[: n * S * B].view(n, B, S))


# ------------------------------------------------------------------------------------------------ analysis
class PiscesLxSensitivityAnalysisOperator(PiscesLxOperatorInterface):
    """inputs {"model", "activations"} -> per-layer output error when that layer alone is quantised to ``bits``
    (relative to the layer's fp output on its calibration activations)."""
    name = "sensitivity"

    def __init__(self, bits: int = 4, group_size: int = 128):
        self.q = PiscesLxBlockWiseINT4Quantizer(group_size, bits)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, float]:
        acts, out = inputs["activations"], {}
        for name, m in inputs["model"].named_modules():
            if isinstance(m, nn.Linear) and name in acts:
                x, w = acts[name], m.weight.detach().float().cpu()
                ref = x @ w.t()
                out[name] = float(((x @ self.q.fake_quant(w).t()) - ref).norm() / ref.norm().clamp_min(1e-12))
        return out


class PiscesLxAdaptiveBitAllocationOperator(PiscesLxOperatorInterface):
    """inputs {"sensitivity": {layer: error}, "sizes": {layer: parameters}, "target_bits": mean bits per weight} ->
    {layer: bits in ``choices``}: starts every layer at the lowest choice and gives extra bits to the layers with the
    highest sensitivity per parameter until the size-weighted mean reaches the target."""
    name = "bit_allocation"

    def __init__(self, choices: Sequence[int] = (2, 3, 4, 8)):
        self.choices = sorted(choices)

    def run(self, inputs: Dict[str, Any]) -> Dict[str, int]:
        sens, sizes, target = inputs["sensitivity"], inputs["sizes"], float(inputs["target_bits"])
        bits = {k: self.choices[0] for k in sens}
        total = sum(sizes[k] for k in sens)
        mean = lambda: sum(bits[k] * sizes[k] for k in sens) / max(total, 1)
        b0 = self.choices[0]
        # greedy: the layer whose estimated remaining error (it halves with every extra bit) is largest gets the next
        # upgrade that still fits the budget
        while True:
            best = None
            for k in sens:
                i = self.choices.index(bits[k])
                if i + 1 == len(self.choices):
                    continue
                step = (self.choices[i + 1] - bits[k]) * sizes[k] / total
                if mean() + step > target + 1e-9:
                    continue
                err = sens[k] * 2.0 ** (-(bits[k] - b0))
                if best is None or err > best[0]:
                    best = (err, k, self.choices[i + 1])
            if best is None:
                break
            bits[best[1]] = best[2]
        return bits


# ------------------------------------------------------------------------------------------------ method operators
class _LinearQuantOperator(PiscesLxOperatorInterface):
    def quantize_weight(self, w: torch.Tensor, x: Optional[torch.Tensor], bits: int, group: int) -> torch.Tensor:
        raise NotImplementedError

    def run(self, inputs: Dict[str, Any]) -> Dict[str, torch.Tensor]:
        w = inputs["weight"]
        return {"weight": self.quantize_weight(w, inputs.get("activations"), int(inputs.get("bits", 4)),
                                               int(inputs.get("group_size", 128))).to(w.dtype)}


class PiscesLxRTNOperator(_LinearQuantOperator):
    name = "rtn"

    def quantize_weight(self, w, x, bits, group):
        return PiscesLxBlockWiseINT4Quantizer(group, bits).fake_quant(w.float())


class PiscesLxGPTQOperator(_LinearQuantOperator):
    name = "gptq"

    def quantize_weight(self, w, x, bits, group):
        assert x is not None, "GPTQ needs calibration activations"
        return PiscesLxGPTQQuantizer(bits, group).quantize(w, x)


class PiscesLxAWQOperator(_LinearQuantOperator):
    name = "awq"

    def quantize_weight(self, w, x, bits, group):
        assert x is not None, "AWQ needs calibration activations"
        return PiscesLxAWQQuantizer(bits, group).quantize(w, x)[0]


class PiscesLxSmoothQuantOperator(_LinearQuantOperator):
    """Migrates activation outliers into the weights (per-channel scale), then rounds the smoothed weight; returns
    the weight mapped back to the original input scale so that it can replace the layer's weight directly."""
    name = "smoothquant"

    def quantize_weight(self, w, x, bits, group):
        assert x is not None, "SmoothQuant needs calibration activations"
        sq = PiscesLxSmoothQuantizer()
        s = sq.scales(w, x)
        return PiscesLxBlockWiseINT4Quantizer(group, bits).fake_quant(w.float() * s) / s


class PiscesLxQuantizationOperatorFactory:
    TABLE = {PiscesLxQuantizationMethod.RTN: PiscesLxRTNOperator, PiscesLxQuantizationMethod.GPTQ: PiscesLxGPTQOperator,
             PiscesLxQuantizationMethod.AWQ: PiscesLxAWQOperator, PiscesLxQuantizationMethod.SMOOTHQUANT: PiscesLxSmoothQuantOperator}

    @classmethod
    def create(cls, method: Any) -> _LinearQuantOperator:
        return cls.TABLE[PiscesLxQuantizationMethod(method)]()


# ------------------------------------------------------------------------------------------------ engine / evaluation
class PiscesLxQuantizationEngine:
    """Quantises (fake-quant: values on the integer grid, stored in the layer's dtype) every eligible ``nn.Linear``
    of a model with the configured method, layer by layer."""

    def __init__(self, config: Optional[PiscesLxQuantizationConfig] = None):
        self.config = config or PiscesLxQuantizationConfig()

    def quantize(self, model: nn.Module, activations: Optional[Dict[str, torch.Tensor]] = None) -> PiscesLxQuantizationResult:
        c, t0 = self.config, time.perf_counter()
        op = PiscesLxQuantizationOperatorFactory.create(c.method)
        errs, bits_w, n_w, layers = {}, 0.0, 0, 0
        for name, m in model.named_modules():
            if not isinstance(m, nn.Linear) or any(s in name for s in c.skip):
                continue
            bits = c.per_layer_bits.get(name, c.bits)
            group = min(c.group_size, m.in_features)
            while m.in_features % group:
                group //= 2
            x = activations.get(name) if activations else None
            w0 = m.weight.detach().clone()
            wq = op.run({"weight": w0.cpu(), "activations": x, "bits": bits, "group_size": max(group, 1)})["weight"]
            with torch.no_grad():
                m.weight.copy_(wq.to(m.weight.device, m.weight.dtype))
            errs[name] = float((wq.float() - w0.float().cpu()).norm() / w0.float().norm().clamp_min(1e-12))
            bits_w += bits * w0.numel()
            n_w += w0.numel()
            layers += 1
        # weight matrices held as bare parameters (fused QKV / gate-up matrices, stacked expert weights [E, out, in])
        linear_weights = {id(m.weight) for m in model.modules() if isinstance(m, nn.Linear)}
        for name, p in model.named_parameters():
            if p.dim() < 2 or id(p) in linear_weights or any(s in name for s in c.skip) or "norm" in name:
                continue
            bits = c.per_layer_bits.get(name, c.bits)
            w0 = p.detach().clone()
            mats = w0.reshape(-1, w0.shape[-1]).cpu()                     # rows = output channels of every stacked matrix
            group = min(c.group_size, mats.shape[1])
            while mats.shape[1] % group:
                group //= 2
            wq = op.run({"weight": mats, "activations": None, "bits": bits, "group_size": max(group, 1)})["weight"]
            with torch.no_grad():
                p.copy_(wq.reshape(w0.shape).to(p.device, p.dtype))
            errs[name] = float((wq.float() - mats.float()).norm() / mats.float().norm().clamp_min(1e-12))
            bits_w += bits * w0.numel()
            n_w += w0.numel()
            layers += 1
        return PiscesLxQuantizationResult(layers, PiscesLxQuantizationMethod(c.method).value, bits_w / max(n_w, 1), errs,
                                          time.perf_counter() - t0)


class PiscesLxQuantizationEvaluator:
    """Output agreement of a quantised model with its fp original on held-out inputs: relative logit error and
    top-1 agreement."""

    @staticmethod
    @torch.no_grad()
    def compare(fp_model: nn.Module, q_model: nn.Module, batches: Iterable[Any]) -> Dict[str, float]:
        err = agree = n = 0.0
        for b in batches:
            a = fp_model(**b) if isinstance(b, dict) else fp_model(b)
            q = q_model(**b) if isinstance(b, dict) else q_model(b)
            a = a["logits"] if isinstance(a, dict) else getattr(a, "logits", a)
            q = q["logits"] if isinstance(q, dict) else getattr(q, "logits", q)
            err += float((q.float() - a.float()).norm() / a.float().norm().clamp_min(1e-12))
            agree += float((q.argmax(-1) == a.argmax(-1)).float().mean())
            n += 1
        return {"relative_error": err / max(n, 1), "top1_agreement": agree / max(n, 1), "batches": int(n)}


class PiscesLxMemoryProfiler:
    @staticmethod
    def weight_bytes(model: nn.Module, bits_per_layer: Optional[Dict[str, int]] = None, default_bits: int = 16,
                     group_size: int = 128) -> Dict[str, float]:
        """Storage of the linear weights at the given bit widths, scales included (one fp16 scale per group)."""
        total = 0.0
        for name, m in model.named_modules():
            if isinstance(m, nn.Linear):
                bits = (bits_per_layer or {}).get(name, default_bits)
                n = m.weight.numel()
                total += n * bits / 8 + (n / group_size * 2 if bits < 16 else 0)
        return {"bytes": total, "mb": total / 2 ** 20}


@dataclass
class PiscesLxBenchmarkResult:
    method: str
    mean_bits: float
    relative_error: float
    top1_agreement: float
    weight_mb: float
    seconds: float


class PiscesLxQuantizationBenchmark:
    """Runs several (method, bits) settings on copies of a model and tabulates error, agreement and size."""

    def __init__(self, make_model: Callable[[], nn.Module], calib: Sequence[Any], heldout: Sequence[Any]):
        self.make_model, self.calib, self.heldout = make_model, list(calib), list(heldout)

    def run(self, settings: Sequence[Tuple[str, int]]) -> List[PiscesLxBenchmarkResult]:
        fp = self.make_model().eval()
        acts = PiscesLxActivationCollectorOperator().run({"model": fp, "batches": self.calib})
        out = []
        for method, bits in settings:
            q = self.make_model().eval()
            q.load_state_dict(fp.state_dict())
            res = PiscesLxQuantizationEngine(PiscesLxQuantizationConfig(PiscesLxQuantizationMethod(method), bits)).quantize(q, acts)
            ev = PiscesLxQuantizationEvaluator.compare(fp, q, self.heldout)
            mb = PiscesLxMemoryProfiler.weight_bytes(q, {k: bits for k in res.weight_error})["mb"]
            out.append(PiscesLxBenchmarkResult(method, res.mean_bits, ev["relative_error"], ev["top1_agreement"], mb, res.seconds))
        return out


class PiscesLxQuantizationPipelineOperator(PiscesLxOperatorInterface):
    """inputs {"model", "calibration": batches, "config": PiscesLxQuantizationConfig, "target_bits" (optional: turns
    on sensitivity analysis + adaptive bit allocation)} -> quantises the model in place and returns the report."""
    name = "quantization_pipeline"

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return "model" in inputs and "calibration" in inputs

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        model = inputs["model"]
        cfg: PiscesLxQuantizationConfig = inputs.get("config") or PiscesLxQuantizationConfig()
        acts = PiscesLxActivationCollectorOperator().run({"model": model, "batches": inputs["calibration"]})
        report: Dict[str, Any] = {"calibrated_layers": len(acts)}
        if "target_bits" in inputs:
            sens = PiscesLxSensitivityAnalysisOperator(min(cfg.bits, 4), cfg.group_size).run({"model": model, "activations": acts})
            sens = {k: v for k, v in sens.items() if not any(s in k for s in cfg.skip)}
            sizes = {n: m.weight.numel() for n, m in model.named_modules() if isinstance(m, nn.Linear) and n in sens}
            cfg.per_layer_bits = PiscesLxAdaptiveBitAllocationOperator().run(
                {"sensitivity": sens, "sizes": sizes, "target_bits": inputs["target_bits"]})
            report["sensitivity"], report["bits"] = sens, dict(cfg.per_layer_bits)
        res = PiscesLxQuantizationEngine(cfg).quantize(model, acts)
        report.update({"layers": res.layers, "mean_bits": res.mean_bits, "weight_error": res.weight_error, "method": res.method})
        return report


PiscesLxQuantizationEngineOperator = PiscesLxQuantizationPipelineOperator
PiscesLxPipeline = PiscesLxQuantizationPipelineOperator
