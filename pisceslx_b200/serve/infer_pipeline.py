"""The inference pipeline layer: pipeline / prompt-engineering / result-processing operators (reference
tools/infer/pipeline.py:54-600) and the monitoring operators shared by serving and training - request / step monitor,
resource monitor, visualiser, phase profiler (tools/infer/monitoring.py:53-500, tools/train/monitoring.py:120-540).

Notes on the monitoring side:
* histories are bounded rings (the reference's lists grow for the life of the server);
* phase times of the profiler come from CUDA events recorded on the launching stream when the device is a GPU and are
  read together when the request ends - ``time.time()`` between asynchronous launches, as the reference takes it
  (monitoring.py:367-400), measures launch latency, not execution;
* plots are written as SVG text, so no plotting library is needed on a serving host."""
from __future__ import annotations

import json
import re
import statistics
import threading
import time
from collections import deque
from pathlib import Path
from typing import Any, Callable, Deque, Dict, Iterator, List, Optional, Sequence, Union

from ..utils.opsc import PiscesLxOperatorInterface
from .infer_config import PiscesLxInferenceConfig


class _Callbacks:
    def __init__(self) -> None:
        self.callbacks: List[Callable] = []
        self.callback_errors: List[str] = []

    def add_callback(self, callback: Callable) -> None:
        if callback not in self.callbacks:
            self.callbacks.append(callback)

    def remove_callback(self, callback: Callable) -> None:
        if callback in self.callbacks:
            self.callbacks.remove(callback)

    def execute_callbacks(self, stage: str, **kwargs: Any) -> None:
        for cb in list(self.callbacks):
            try:
                cb(stage, **kwargs)
            except Exception as e:
                self.callback_errors.append(f"{stage}: {type(e).__name__}: {e}")


class PiscesLxInferencePipelineOperator(_Callbacks, PiscesLxOperatorInterface):
    """Around an ``inferencer`` with ``generate(prompt, **kw) -> str`` and optionally ``batch_generate(prompts, **kw)`` and
    ``_stream_generate(prompt, **kw)`` (``serve.infer_operators.PiscesLxVLLMInferenceOperator`` and the engine front have
    them): cleaning of inputs and outputs, batches, streams, a background run, callbacks at every stage."""

    name = "inference_pipeline_operator"

    def __init__(self, config: Any = None, inferencer: Any = None):
        _Callbacks.__init__(self)
        self.infer_config = self._normalize_infer_config(config)
        self.inferencer = inferencer

    @staticmethod
    def _normalize_infer_config(config: Any) -> PiscesLxInferenceConfig:
        if config is None:
            return PiscesLxInferenceConfig()
        if isinstance(config, PiscesLxInferenceConfig):
            return config
        if isinstance(config, dict):
            return PiscesLxInferenceConfig.from_dict(config)
        if isinstance(config, (str, Path)):
            p = str(config)
            return PiscesLxInferenceConfig.load_from_json(p) if p.endswith(".json") else PiscesLxInferenceConfig.load_from_yaml(p)
        params = getattr(config, "parameters", None)
        if isinstance(params, dict):
            return PiscesLxInferenceConfig.from_dict(params)
        raise TypeError(f"cannot make an inference configuration from {type(config).__name__}")

    def transform(self, data: Any) -> Any:
        if isinstance(data, (str, list)):
            return self.run({"prompts": data})["results"]
        return data

    def preprocess_inputs(self, inputs: Union[str, List[str]]) -> List[str]:
        inputs = [inputs] if isinstance(inputs, str) else list(inputs)
        self.execute_callbacks("preprocessing_start", inputs=inputs)
        out = [re.sub(r"[ \t]+\n", "\n", i).strip() for i in inputs]
        out = [i for i in out if i]
        self.execute_callbacks("preprocessing_end", processed_inputs=out)
        return out

    def postprocess_outputs(self, outputs: List[str], original_inputs: List[str]) -> Union[str, List[str]]:
        self.execute_callbacks("postprocessing_start", outputs=outputs)
        out = [(o or "").strip() for o in outputs]
        self.execute_callbacks("postprocessing_end", processed_outputs=out)
        return out[0] if (len(original_inputs) == 1 and len(out) == 1) else out

    def generate_stream(self, prompt: str, chunk_chars: int = 10, **kwargs: Any) -> Iterator[str]:
        self.execute_callbacks("stream_start", prompt=prompt)
        try:
            if hasattr(self.inferencer, "_stream_generate"):
                it = self.inferencer._stream_generate(prompt, **kwargs)
            else:
                full = self.inferencer.generate(prompt, **kwargs)
                it = (full[i:i + chunk_chars] for i in range(0, len(full), chunk_chars))
            for chunk in it:
                self.execute_callbacks("stream_chunk", chunk=chunk)
                yield chunk
        except Exception as e:
            self.execute_callbacks("stream_error", error=str(e))
            raise
        finally:
            self.execute_callbacks("stream_end")

    def batch_inference(self, prompts: List[str], batch_size: Optional[int] = None, **kwargs: Any) -> List[str]:
        """A failed batch yields empty strings for its prompts (and a ``batch_failed`` callback), the others still run."""
        bs = max(int(batch_size or self.infer_config.batch_size), 1)
        self.execute_callbacks("batch_start", prompts=prompts, batch_size=bs)
        results: List[str] = []
        for n, i in enumerate(range(0, len(prompts), bs), 1):
            part = prompts[i:i + bs]
            self.execute_callbacks("batch_processing", batch_index=n, batch_prompts=part)
            try:
                if hasattr(self.inferencer, "batch_generate"):
                    r = list(self.inferencer.batch_generate(part, **kwargs))
                else:
                    r = [self.inferencer.generate(p, **kwargs) for p in part]
                if len(r) != len(part):
                    raise RuntimeError(f"{len(r)} results for {len(part)} prompts")
                results += r
                self.execute_callbacks("batch_completed", batch_index=n, batch_results=r)
            except Exception as e:
                results += [""] * len(part)
                self.execute_callbacks("batch_failed", batch_index=n, error=str(e))
        self.execute_callbacks("batch_end", results=results)
        return results

    def async_inference(self, prompts: List[str], callback: Optional[Callable] = None, **kwargs: Any) -> threading.Thread:
        """Runs ``batch_inference`` on a thread; ``callback(results)`` or ``callback(None, error=...)`` when it ends."""
        def worker() -> None:
            try:
                r = self.batch_inference(prompts, **kwargs)
                if callback:
                    callback(r)
            except Exception as e:
                if callback:
                    callback(None, error=str(e))
        t = threading.Thread(target=worker, daemon=True)
        t.start()
        return t

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return self.inferencer is not None and "prompts" in inputs

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        raw = inputs["prompts"]
        prompts = self.preprocess_inputs(raw)
        g = self.infer_config.generation
        kw = {"max_new_tokens": g.max_new_tokens, "temperature": g.temperature, "top_p": g.top_p, "top_k": g.top_k}
        kw.update(inputs.get("generation") or {})
        outs = self.batch_inference(prompts, inputs.get("batch_size"), **kw)
        return {"results": self.postprocess_outputs(outs, prompts), "count": len(prompts)}


class PiscesLxPromptEngineeringOperator(PiscesLxOperatorInterface):
    """Named templates with ``{placeholders}``, prompt shortening / flattening and a rough quality report."""

    name = "prompt_engineering_operator"
    QUESTION_WORDS = ("what", "how", "why", "when", "where", "who", "which")

    def __init__(self, config: Any = None):
        self.templates: Dict[str, Dict[str, Any]] = {}
        self.add_template("qa", "Question: {question}\nAnswer:", "question answering")
        self.add_template("instruct", "### Instruction:\n{instruction}\n\n### Response:\n", "instruction following")
        self.add_template("summarize", "Summarize the following text in {n} sentences.\n\n{text}\n\nSummary:", "summarisation", {"n": 3})
        self.add_template("chat", "{system}\n\nUser: {user}\nAssistant:", "one chat turn", {"system": "You are a helpful assistant."})

    def transform(self, data: Any) -> Any:
        if isinstance(data, dict) and "template" in data:
            return self.render_template(data["template"], **{k: v for k, v in data.items() if k != "template"})
        return data

    def add_template(self, name: str, template: str, description: str = "", defaults: Optional[Dict[str, Any]] = None) -> None:
        self.templates[name] = {"template": template, "description": description, "defaults": dict(defaults or {}),
                                "variables": sorted(set(re.findall(r"{(\w+)}", template)))}

    def render_template(self, template_name: str, **kwargs: Any) -> str:
        if template_name not in self.templates:
            raise KeyError(f"unknown template {template_name}; known: {sorted(self.templates)}")
        t = self.templates[template_name]
        vals = {**t["defaults"], **kwargs}
        missing = [v for v in t["variables"] if v not in vals]
        if missing:
            raise ValueError(f"template {template_name} needs {missing}")
        return t["template"].format(**vals)

    @staticmethod
    def _sentences(prompt: str) -> List[str]:
        return [s.strip() for s in re.split(r"(?<=[.!?。！？])\s+", prompt.strip()) if s.strip()]

    def optimize_prompt(self, prompt: str, strategy: str = "length", max_sentences: int = 3) -> str:
        if strategy == "length":
            s = self._sentences(prompt)
            if len(s) > max_sentences:
                return " ".join(s[:max_sentences - 1] + s[-1:])
            return prompt.strip()
        if strategy == "clarity":
            return re.sub(r"\s+", " ", prompt).strip()
        if strategy == "dedupe":
            seen, out = set(), []
            for s in self._sentences(prompt):
                k = s.lower()
                if k not in seen:
                    seen.add(k)
                    out.append(s)
            return " ".join(out)
        return prompt

    def _calculate_complexity(self, prompt: str) -> float:
        words = prompt.split()
        if not words:
            return 0.0
        s = self._sentences(prompt)
        avg = sum(len(x.split()) for x in s) / max(len(s), 1)
        return min(len(set(w.lower() for w in words)) / len(words) * 0.5 + min(avg / 40.0, 0.5), 1.0)

    def _calculate_clarity(self, prompt: str) -> float:
        if not prompt.strip():
            return 0.0
        c = 0.5 + (0.3 if any(p in prompt for p in ".!?;:。？！") else 0.0)
        low = prompt.lower()
        return min(c + min(sum(1 for w in self.QUESTION_WORDS if re.search(rf"\b{w}\b", low)) * 0.1, 0.2), 1.0)

    def analyze_prompt_quality(self, prompt: str) -> Dict[str, Any]:
        a = {"length": len(prompt), "word_count": len(prompt.split()), "sentence_count": len(self._sentences(prompt)),
             "complexity_score": self._calculate_complexity(prompt), "clarity_score": self._calculate_clarity(prompt), "recommendations": []}
        if a["length"] > 500:
            a["recommendations"].append("Prompt is quite long, consider shortening")
        if a["complexity_score"] > 0.8:
            a["recommendations"].append("High complexity detected, consider simplifying")
        if a["clarity_score"] < 0.5:
            a["recommendations"].append("Low clarity detected, consider rephrasing")
        return a

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return "template" in inputs or "prompt" in inputs

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        if "template" in inputs:
            return {"prompt": self.render_template(inputs["template"], **(inputs.get("variables") or {}))}
        p = self.optimize_prompt(inputs["prompt"], inputs.get("strategy", "length"))
        return {"prompt": p, "analysis": self.analyze_prompt_quality(p)}


class PiscesLxResultProcessorOperator(PiscesLxOperatorInterface):
    """A chain of ``str -> str`` processors, then filters (length bounds, banned words, duplicates) and a format."""

    name = "result_processor_operator"

    def __init__(self, config: Any = None):
        self.processors: List[Callable[[str], str]] = []

    def transform(self, data: Any) -> Any:
        return self.process_results(data) if isinstance(data, (str, list)) else data

    def add_processor(self, processor: Callable[[str], str]) -> None:
        self.processors.append(processor)

    def process_results(self, results: Union[str, List[str]]) -> Union[str, List[str]]:
        single = isinstance(results, str)
        out = []
        for r in ([results] if single else results):
            for p in self.processors:
                try:
                    r = p(r)
                except Exception:
                    continue                                                            # a failing processor is skipped for this result
            out.append(r)
        return out[0] if single else out

    @staticmethod
    def filter_results(results: List[str], min_length: int = 0, max_length: Optional[int] = None, banned_words: Optional[Sequence[str]] = None,
                       unique: bool = False) -> List[str]:
        out, seen = [], set()
        for r in results:
            if len(r) < min_length or (max_length is not None and len(r) > max_length):
                continue
            if banned_words and any(w.lower() in r.lower() for w in banned_words):
                continue
            if unique:
                if r in seen:
                    continue
                seen.add(r)
            out.append(r)
        return out

    @staticmethod
    def format_results(results: List[str], format_type: str = "list") -> Union[str, List[str], Dict[str, Any]]:
        if format_type == "list":
            return list(results)
        if format_type == "json":
            return json.dumps({"results": list(results), "count": len(results)}, ensure_ascii=False)
        if format_type == "numbered":
            return "\n".join(f"{i}. {r}" for i, r in enumerate(results, 1))
        if format_type == "text":
            return "\n\n".join(results)
        if format_type == "dict":
            return {"results": list(results), "count": len(results)}
        raise ValueError(f"unknown format {format_type}")

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return "results" in inputs

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        r = self.process_results(inputs["results"])
        r = [r] if isinstance(r, str) else r
        r = self.filter_results(r, **(inputs.get("filter") or {}))
        return {"results": self.format_results(r, inputs.get("format", "list")), "count": len(r)}


# ---- monitoring -------------------------------------------------------------------------------------------------------------------
def percentile(values: Sequence[float], p: float) -> float:
    """Linear interpolation between order statistics, p in [0, 100]."""
    if not values:
        return 0.0
    v = sorted(values)
    k = (len(v) - 1) * p / 100.0
    lo, hi = int(k), min(int(k) + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (k - lo)


class PiscesLxSystemResourceMonitor:
    """Host CPU / memory through psutil, devices through NVML - both read only; either may be absent."""

    def __init__(self, nvml: Any = None):
        self._nvml, self._nvml_ok = nvml, nvml is not None
        if nvml is None:
            try:
                import pynvml
                pynvml.nvmlInit()
                self._nvml, self._nvml_ok = pynvml, True
            except Exception:
                self._nvml_ok = False

    def get_system_metrics(self) -> Dict[str, float]:
        out: Dict[str, float] = {}
        try:
            import psutil
            vm = psutil.virtual_memory()
            out.update(cpu_percent=float(psutil.cpu_percent(interval=None)), memory_percent=float(vm.percent), memory_used_gb=vm.used / 2 ** 30)
        except Exception:
            pass
        if self._nvml_ok:
            try:
                n = self._nvml.nvmlDeviceGetCount()
                used = total = util = 0.0
                for i in range(n):
                    h = self._nvml.nvmlDeviceGetHandleByIndex(i)
                    m = self._nvml.nvmlDeviceGetMemoryInfo(h)
                    used, total = used + m.used, total + m.total
                    util += self._nvml.nvmlDeviceGetUtilizationRates(h).gpu
                out.update(gpu_count=float(n), gpu_memory_percent=100.0 * used / max(total, 1.0), gpu_memory_used_gb=used / 2 ** 30,
                           gpu_utilization=util / max(n, 1))
            except Exception:
                pass
        return out


class _MonitorBase(PiscesLxOperatorInterface):
    SERIES: Sequence[str] = ()

    def __init__(self, log_dir: str, save_interval: int, history: int, resources: Optional[PiscesLxSystemResourceMonitor], log_name: str):
        self.log_dir = Path(log_dir)
        self.log_dir.mkdir(parents=True, exist_ok=True)
        self.save_interval, self.log_name = save_interval, log_name
        self.metrics_history: Dict[str, Deque[float]] = {k: deque(maxlen=history) for k in (*self.SERIES, "timestamps")}
        self.count = 0
        self.resources = resources
        self.start_time = time.time()
        self.anomalies: Deque[Dict[str, Any]] = deque(maxlen=256)

    _percentile = staticmethod(percentile)

    def transform(self, data: Any) -> Any:
        return data

    def _save_metrics_log(self) -> None:
        p = self.log_dir / self.log_name
        tmp = p.with_suffix(".tmp")
        tmp.write_text(json.dumps({"summary": self._generate_summary(), "history": {k: list(v)[-1000:] for k, v in self.metrics_history.items()}}))
        tmp.replace(p)

    def get_realtime_metrics(self) -> Dict[str, Any]:
        return self._generate_summary()

    def _generate_summary(self) -> Dict[str, Any]:
        raise NotImplementedError


class PiscesLxInferenceMonitorOperator(_MonitorBase):
    """``record_inference_request({"latency": s, "tokens_generated": n, "success": bool, ...})``; summaries with latency
    percentiles, throughput and error rate; anomalies: latency spike (3 x the recent mean), error rate over 5 % after 100
    requests, host or device memory over 90 %."""

    name = "inference_monitor_operator"
    SERIES = ("latency", "tokens_generated", "throughput", "memory_usage", "gpu_memory_usage")

    def __init__(self, config: Any = None, log_dir: str = "./inference_logs", save_interval: int = 100, history: int = 10000,
                 resources: Optional[PiscesLxSystemResourceMonitor] = None):
        super().__init__(log_dir, save_interval, history, resources, "inference_metrics.json")
        self.error_count = 0

    def record_inference_request(self, request_metrics: Dict[str, Any]) -> List[Dict[str, Any]]:
        h = self.metrics_history
        lat, toks = float(request_metrics.get("latency", 0.0)), float(request_metrics.get("tokens_generated", 0))
        h["timestamps"].append(float(request_metrics.get("timestamp", time.time())))
        h["latency"].append(lat)
        h["tokens_generated"].append(toks)
        h["throughput"].append(toks / lat if lat > 0 else 0.0)
        sysm = self.resources.get_system_metrics() if self.resources is not None else {}
        h["memory_usage"].append(float(request_metrics.get("memory_usage", sysm.get("memory_percent", 0.0))))
        h["gpu_memory_usage"].append(float(request_metrics.get("gpu_memory_usage", sysm.get("gpu_memory_percent", 0.0))))
        self.count += 1
        if not request_metrics.get("success", True):
            self.error_count += 1
        found = self.detect_anomalies()
        self.anomalies.extend(found)
        if self.save_interval and self.count % self.save_interval == 0:
            self._save_metrics_log()
        return found

    @property
    def request_count(self) -> int:
        return self.count

    def _generate_summary(self) -> Dict[str, Any]:
        lat = list(self.metrics_history["latency"])
        up = time.time() - self.start_time
        return {"request_count": self.count, "error_count": self.error_count, "error_rate": self.error_count / max(self.count, 1),
                "uptime_seconds": up, "qps": self.count / max(up, 1e-9), "latency_mean": statistics.fmean(lat) if lat else 0.0,
                "latency_p50": percentile(lat, 50), "latency_p95": percentile(lat, 95), "latency_p99": percentile(lat, 99),
                "tokens_total": sum(self.metrics_history["tokens_generated"]),
                "throughput_mean": statistics.fmean(self.metrics_history["throughput"]) if lat else 0.0}

    def detect_anomalies(self) -> List[Dict[str, Any]]:
        h, out = self.metrics_history, []
        lat = list(h["latency"])[-10:]
        ts = h["timestamps"][-1] if h["timestamps"] else time.time()
        if len(lat) >= 10:
            mean = statistics.fmean(lat[:-1])
            if mean > 0 and lat[-1] > 3.0 * mean:
                out.append({"type": "latency_spike", "severity": "high", "timestamp": ts, "message": f"Latency spike detected: {lat[-1]:.4f}s vs average {mean:.4f}s"})
        if self.count >= 100 and self.error_count / self.count > 0.05:
            out.append({"type": "high_error_rate", "severity": "critical", "timestamp": ts, "message": f"High error rate detected: {self.error_count / self.count:.2%}"})
        for key, label in (("memory_usage", "memory"), ("gpu_memory_usage", "device memory")):
            recent = list(h[key])[-5:]
            if recent and max(recent) > 90.0:
                out.append({"type": f"high_{key}", "severity": "warning", "timestamp": ts, "message": f"High {label} usage: {max(recent):.1f}%"})
        return out

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return True

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        if "request" in inputs:
            return {"anomalies": self.record_inference_request(inputs["request"]), "summary": self._generate_summary()}
        return {"summary": self._generate_summary(), "anomalies": list(self.anomalies)}


class PiscesLxTrainingMonitorOperator(_MonitorBase):
    """``record_training_step({"loss", "learning_rate", "grad_norm", "throughput", "step_time", ...})``; anomalies: a loss
    that is not finite, a loss spike (over 2 x the recent mean), a gradient norm over 10 x its recent median, a throughput
    drop under half of the recent mean, memory over 90 %."""

    name = "training_monitor_operator"
    SERIES = ("loss", "learning_rate", "grad_norm", "throughput", "step_time", "memory_usage", "gpu_memory_usage")

    def __init__(self, config: Any = None, log_dir: str = "./logs", save_interval: int = 100, history: int = 100000,
                 resources: Optional[PiscesLxSystemResourceMonitor] = None):
        super().__init__(log_dir, save_interval, history, resources, "training_metrics.json")

    def record_training_step(self, step_metrics: Dict[str, Any]) -> List[Dict[str, Any]]:
        h = self.metrics_history
        h["timestamps"].append(float(step_metrics.get("timestamp", time.time())))
        sysm = self.resources.get_system_metrics() if self.resources is not None else {}
        for k in self.SERIES:
            d = sysm.get("memory_percent", 0.0) if k == "memory_usage" else sysm.get("gpu_memory_percent", 0.0) if k == "gpu_memory_usage" else 0.0
            v = step_metrics.get(k, d)
            h[k].append(float(v if v is not None else 0.0))
        self.count += 1
        found = self.detect_anomalies()
        self.anomalies.extend(found)
        if self.save_interval and self.count % self.save_interval == 0:
            self._save_metrics_log()
        return found

    def _generate_summary(self) -> Dict[str, Any]:
        h = self.metrics_history
        loss, st = list(h["loss"]), list(h["step_time"])
        return {"steps": self.count, "loss_last": loss[-1] if loss else None, "loss_mean_100": statistics.fmean(loss[-100:]) if loss else None,
                "loss_min": min(loss) if loss else None, "step_time_p50": percentile(st, 50), "step_time_p95": percentile(st, 95),
                "throughput_mean": statistics.fmean(h["throughput"]) if h["throughput"] else 0.0, "elapsed_seconds": time.time() - self.start_time,
                "anomaly_count": len(self.anomalies)}

    def detect_anomalies(self) -> List[Dict[str, Any]]:
        import math
        h, out = self.metrics_history, []
        ts = h["timestamps"][-1] if h["timestamps"] else time.time()
        loss = list(h["loss"])[-11:]
        if loss and not math.isfinite(loss[-1]):
            out.append({"type": "non_finite_loss", "severity": "critical", "timestamp": ts, "message": f"Loss is {loss[-1]}"})
        elif len(loss) >= 11:
            prev = [x for x in loss[:-1] if math.isfinite(x)]
            mean = statistics.fmean(prev) if prev else 0.0
            if mean > 0 and loss[-1] > 2.0 * mean:
                out.append({"type": "loss_spike", "severity": "high", "timestamp": ts, "message": f"Loss spike: {loss[-1]:.4f} vs recent mean {mean:.4f}"})
        gn = list(h["grad_norm"])[-21:]
        if len(gn) >= 11:
            med = statistics.median(gn[:-1])
            if med > 0 and gn[-1] > 10.0 * med:
                out.append({"type": "gradient_explosion", "severity": "high", "timestamp": ts, "message": f"Gradient norm {gn[-1]:.3g} vs recent median {med:.3g}"})
        tp = list(h["throughput"])[-11:]
        if len(tp) >= 11:
            mean = statistics.fmean(tp[:-1])
            if mean > 0 and 0 < tp[-1] < 0.5 * mean:
                out.append({"type": "throughput_drop", "severity": "warning", "timestamp": ts, "message": f"Throughput {tp[-1]:.1f} vs recent mean {mean:.1f}"})
        for key, label in (("memory_usage", "memory"), ("gpu_memory_usage", "device memory")):
            recent = list(h[key])[-5:]
            if recent and max(recent) > 90.0:
                out.append({"type": f"high_{key}", "severity": "warning", "timestamp": ts, "message": f"High {label} usage: {max(recent):.1f}%"})
        return out

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return True

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        if "step" in inputs:
            return {"anomalies": self.record_training_step(inputs["step"]), "summary": self._generate_summary()}
        return {"summary": self._generate_summary(), "anomalies": list(self.anomalies)}


class PiscesLxInferenceVisualizer:
    """One SVG line chart per series of a metrics history (``generate_plots`` returns the files written)."""

    def __init__(self, log_dir: Union[str, Path], width: int = 640, height: int = 240):
        self.log_dir, self.width, self.height = Path(log_dir), width, height
        self.log_dir.mkdir(parents=True, exist_ok=True)

    def _svg(self, title: str, ys: Sequence[float]) -> str:
        W, H, pad = self.width, self.height, 36
        finite = [y for y in ys if y == y and abs(y) != float("inf")]
        lo, hi = (min(finite), max(finite)) if finite else (0.0, 1.0)
        if hi == lo:
            hi = lo + 1.0
        n = max(len(ys) - 1, 1)
        pts = " ".join(f"{pad + (W - 2 * pad) * i / n:.1f},{H - pad - (H - 2 * pad) * (y - lo) / (hi - lo):.1f}" for i, y in enumerate(ys)
                       if y == y and abs(y) != float("inf"))
        return (f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" viewBox="0 0 {W} {H}">'
                f'<rect width="{W}" height="{H}" fill="white"/><text x="{pad}" y="20" font-family="monospace" font-size="13">{title}</text>'
                f'<text x="2" y="{pad + 4}" font-family="monospace" font-size="10">{hi:.4g}</text>'
                f'<text x="2" y="{H - pad}" font-family="monospace" font-size="10">{lo:.4g}</text>'
                f'<line x1="{pad}" y1="{H - pad}" x2="{W - pad}" y2="{H - pad}" stroke="#888"/><line x1="{pad}" y1="{pad}" x2="{pad}" y2="{H - pad}" stroke="#888"/>'
                f'<polyline fill="none" stroke="#1f77b4" stroke-width="1.5" points="{pts}"/></svg>')

    def generate_plots(self, metrics_history: Dict[str, Sequence[float]], max_points: int = 2000) -> List[str]:
        out = []
        for name, series in metrics_history.items():
            ys = list(series)
            if name == "timestamps" or len(ys) < 2:
                continue
            if len(ys) > max_points:
                step = len(ys) / max_points
                ys = [ys[int(i * step)] for i in range(max_points)]
            p = self.log_dir / f"{name}.svg"
            p.write_text(self._svg(name, ys))
            out.append(str(p))
        return out


PiscesLxTrainingVisualizer = PiscesLxInferenceVisualizer


class PiscesLxPerformanceProfilerOperator(PiscesLxOperatorInterface):
    """Phase times of a request (tokenisation, forward, decoding) or of a training step (forward, backward, optimizer):
    ``start_*_profile()``, ``mark(phase)`` after each phase, ``end_*_profile()``.  On a GPU the marks are CUDA events on
    the current stream, resolved when the profile ends; on the host they are ``perf_counter`` readings."""

    name = "performance_profiler_operator"

    def __init__(self, config: Any = None, profile_interval: int = 50, history: int = 5000, use_cuda_events: Optional[bool] = None):
        self.profile_interval = max(profile_interval, 1)
        self.phase_history: Dict[str, Deque[float]] = {}
        self.total_history: Deque[float] = deque(maxlen=history)
        self.tokens_history: Deque[float] = deque(maxlen=history)
        self._history_len, self._marks, self._count = history, [], 0
        self.last_report: Dict[str, Any] = {}
        if use_cuda_events is None:
            try:
                import torch
                use_cuda_events = torch.cuda.is_available()
            except Exception:
                use_cuda_events = False
        self.use_cuda_events = bool(use_cuda_events)

    def transform(self, data: Any) -> Any:
        return data

    _percentile = staticmethod(percentile)

    def _now(self) -> Any:
        if self.use_cuda_events:
            import torch
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e
        return time.perf_counter()

    def start_request_profile(self) -> None:
        self._marks = [("start", self._now())]

    start_step_profile = start_request_profile

    def mark(self, phase: str) -> None:
        if self._marks:
            self._marks.append((phase, self._now()))

    def record_tokenization_time(self) -> None:
        self.mark("tokenization")

    def record_forward_start(self) -> None:
        self.mark("pre_forward")

    def record_forward_end(self) -> None:
        self.mark("forward")

    def record_forward_time(self) -> None:
        self.mark("forward")

    def record_backward_time(self) -> None:
        self.mark("backward")

    def record_optimizer_time(self) -> None:
        self.mark("optimizer")

    def record_decoding_time(self) -> None:
        self.mark("decoding")

    def end_request_profile(self, tokens_generated: int = 0) -> Dict[str, float]:
        if not self._marks:
            return {}
        self._marks.append(("end", self._now()))
        if self.use_cuda_events:
            self._marks[-1][1].synchronize()
            dur = lambda a, b: a.elapsed_time(b) / 1e3
        else:
            dur = lambda a, b: b - a
        phases: Dict[str, float] = {}
        for (_, t0), (name, t1) in zip(self._marks, self._marks[1:]):
            if name != "end":
                phases[name] = phases.get(name, 0.0) + dur(t0, t1)
        total = dur(self._marks[0][1], self._marks[-1][1])
        for k, v in phases.items():
            self.phase_history.setdefault(k, deque(maxlen=self._history_len)).append(v)
        self.total_history.append(total)
        self.tokens_history.append(float(tokens_generated))
        self._marks = []
        self._count += 1
        if self._count % self.profile_interval == 0:
            self._generate_performance_report()
        return {**phases, "total": total}

    def end_step_profile(self) -> Dict[str, float]:
        return self.end_request_profile(0)

    def _generate_performance_report(self) -> Dict[str, Any]:
        tot = list(self.total_history)
        rep: Dict[str, Any] = {"count": self._count, "total": {"mean": statistics.fmean(tot) if tot else 0.0, "p50": percentile(tot, 50),
                                                                 "p95": percentile(tot, 95), "p99": percentile(tot, 99)}, "phases": {}}
        s = sum(tot) or 1.0
        for k, v in self.phase_history.items():
            vals = list(v)
            rep["phases"][k] = {"mean": statistics.fmean(vals), "p95": percentile(vals, 95), "share": sum(vals) / s}
        toks = sum(self.tokens_history)
        if toks:
            rep["tokens_per_second"] = toks / s
        if rep["phases"]:
            rep["bottleneck"] = max(rep["phases"], key=lambda k: rep["phases"][k]["share"])
        self.last_report = rep
        return rep

    def get_performance_report(self) -> Dict[str, Any]:
        return self._generate_performance_report()

    def validate_inputs(self, inputs: Dict[str, Any]) -> bool:
        return True

    def run(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        return self.get_performance_report()
