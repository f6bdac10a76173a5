"""The benchmark framework around the suites: configuration, datasets, evaluator, suite runner, model comparison, result and
comparison managers, performance / long-context / agent / multimodal runners, charts and reports (reference
tools/benchmark/{benchmark,config,runner,result,comparison,builders,performance,long_context,agent,multimodal,visualization,
orchestrator,cli}.py).

``tools/benchmark_suites.py`` holds the scoring of each suite and ``tools/benchmark.py`` the measurement primitives; this module
is the layer that turns a configuration into runs, files and reports.

Performance numbers are taken on the device: every timed region is bracketed by CUDA events on the launching stream after
warm-up (``time.perf_counter`` on a host-only run) and peak memory comes from the allocator's counters; every result says
which clock it was taken with.  Reference scores of other models are NOT shipped: ``PiscesLxToolsFlagshipComparator`` compares against a table the user supplies."""
from __future__ import annotations

import html
import json
import math
import statistics
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch
from torch.utils.data import Dataset

from . import benchmark_suites as S

GenerateFn = Callable[[str, int], str]


# ---- configuration ---------------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxToolsBenchmarkConfig:
    model_path: str = ""
    model_name: Optional[str] = None
    datasets: Optional[List[str]] = None
    metrics: Optional[List[str]] = None
    batch_size: int = 8
    max_length: int = 2048
    temperature: float = 0.7
    top_p: float = 0.9
    device: str = "auto"
    output_dir: str = ".pisceslx/benchmark"
    use_cache: bool = True
    save_predictions: bool = True
    debug: bool = False
    modality: str = "text"
    eval_type: str = "LOCAL"
    api_url: Optional[str] = None
    generation_config: Optional[Dict[str, Any]] = None
    eval_batch_size: Optional[int] = None
    timeout: Optional[int] = None
    data_paths: Dict[str, str] = field(default_factory=dict)          # suite name -> jsonl file; suites without one use their smoke rows
    max_samples: Optional[int] = None

    def __post_init__(self) -> None:
        self.datasets = list(self.datasets) if self.datasets else ["mmlu", "gsm8k"]
        self.metrics = list(self.metrics) if self.metrics else ["accuracy"]
        self.model_name = self.model_name or (Path(self.model_path).name if self.model_path else "model")
        if self.modality not in ("text", "image", "audio", "video", "doc"):
            raise ValueError(f"unknown modality {self.modality}")
        if self.eval_type not in ("LOCAL", "SERVICE"):
            raise ValueError("eval_type is LOCAL or SERVICE")

    @classmethod
    def load(cls, config: Union[str, Dict[str, Any], "PiscesLxToolsBenchmarkConfig"]) -> "PiscesLxToolsBenchmarkConfig":
        if isinstance(config, cls):
            return config
        if isinstance(config, (str, Path)):
            p = Path(config)
            if p.suffix in (".yaml", ".yml"):
                import yaml
                config = yaml.safe_load(p.read_text()) or {}
            else:
                config = json.loads(p.read_text())
        names = set(cls.__dataclass_fields__)
        return cls(**{k: v for k, v in dict(config).items() if k in names})


class PiscesLxToolsBenchmarkConfigFactory:
    @staticmethod
    def create(config: Union[str, Dict[str, Any]]) -> PiscesLxToolsBenchmarkConfig:
        return PiscesLxToolsBenchmarkConfig.load(config)


@dataclass
class PiscesLxBenchmarkSuiteConfig:
    suites: List[str] = field(default_factory=lambda: ["mmlu", "gsm8k", "humaneval", "needle"])
    data_paths: Dict[str, str] = field(default_factory=dict)
    max_samples: Optional[int] = None
    output_dir: str = ".pisceslx/benchmark"
    fail_fast: bool = False


# ---- builders: a benchmark configuration as model / dataset / metric / task descriptions -------------------------------------
class PiscesLxToolsModelConfigBuilder:
    @staticmethod
    def build(config: PiscesLxToolsBenchmarkConfig) -> Dict[str, Any]:
        gen = {"max_new_tokens": min(config.max_length, 512), "temperature": config.temperature, "top_p": config.top_p, **(config.generation_config or {})}
        return {"model_id": config.model_name, "model_path": config.model_path, "device": config.device, "eval_type": config.eval_type, "api_url": config.api_url,
                "generation_config": gen, "batch_size": config.eval_batch_size or config.batch_size}


class PiscesLxToolsDatasetConfigBuilder:
    @staticmethod
    def build(config: PiscesLxToolsBenchmarkConfig) -> List[Dict[str, Any]]:
        return [{"name": d, "path": config.data_paths.get(d), "limit": config.max_samples, "modality": config.modality} for d in config.datasets]


class PiscesLxToolsMetricConfigBuilder:
    KNOWN = {"accuracy", "pass@1", "pass@k", "exact_match", "f1", "latency", "throughput"}

    @classmethod
    def build(cls, config: PiscesLxToolsBenchmarkConfig) -> List[Dict[str, Any]]:
        return [{"name": m, "known": m in cls.KNOWN} for m in config.metrics]


class PiscesLxToolsTaskConfigBuilder:
    @staticmethod
    def build(config: PiscesLxToolsBenchmarkConfig) -> Dict[str, Any]:
        return {"model": PiscesLxToolsModelConfigBuilder.build(config), "datasets": PiscesLxToolsDatasetConfigBuilder.build(config),
                "metrics": PiscesLxToolsMetricConfigBuilder.build(config), "work_dir": config.output_dir, "use_cache": config.use_cache, "debug": config.debug,
                "timeout_ms": config.timeout}


# ---- datasets ----------------------------------------------------------------------------------------------------------------------
class PiscesLxBenchmarkDataset(Dataset):
    """Rows of a suite (a jsonl file or a list); subclasses normalise field names."""

    name = "generic"

    def __init__(self, data: Union[str, Sequence[Dict[str, Any]], None] = None, max_samples: Optional[int] = None):
        rows = S.load_suite_rows(data) if isinstance(data, str) else list(data if data is not None else S._SELFTEST_ROWS.get(self.name, []))
        self.rows = [self.normalize(r) for r in rows][: max_samples or None]

    def normalize(self, row: Dict[str, Any]) -> Dict[str, Any]:
        return dict(row)

    def __len__(self) -> int:
        return len(self.rows)

    def __getitem__(self, i: int) -> Dict[str, Any]:
        return self.rows[i]


class PiscesLxMMLUDataset(PiscesLxBenchmarkDataset):
    name = "mmlu"

    def normalize(self, row: Dict[str, Any]) -> Dict[str, Any]:
        ch = row.get("choices") or [row[k] for k in ("A", "B", "C", "D") if k in row]
        ans = row.get("answer", row.get("label", 0))
        if isinstance(ans, str) and ans.strip().upper() in "ABCD" and len(ans.strip()) == 1:
            ans = "ABCD".index(ans.strip().upper())
        return {**row, "question": row.get("question", row.get("prompt", "")), "choices": list(ch), "answer": int(ans), "subject": row.get("subject", "general")}


class PiscesLxGSM8KDataset(PiscesLxBenchmarkDataset):
    name = "gsm8k"

    def normalize(self, row: Dict[str, Any]) -> Dict[str, Any]:
        ans = str(row.get("answer", ""))
        return {**row, "question": row.get("question", row.get("prompt", "")), "answer": ans.split("####")[-1].strip() if "####" in ans else ans.strip()}


class PiscesLxHumanEvalDataset(PiscesLxBenchmarkDataset):
    name = "humaneval"

    def normalize(self, row: Dict[str, Any]) -> Dict[str, Any]:
        return {**row, "task_id": row.get("task_id", ""), "prompt": row.get("prompt", ""), "test": row.get("test", ""), "entry_point": row.get("entry_point", "")}


# ---- evaluation ------------------------------------------------------------------------------------------------------------------
class PiscesLxBaseBenchmark:
    """A named benchmark: ``evaluate(model, tokenizer) -> {"score", "metric", "n", ...}``."""

    name, metric = "base", "accuracy"

    def __init__(self, data_path: Optional[str] = None, max_samples: Optional[int] = None):
        self.data_path, self.max_samples = data_path, max_samples

    def evaluate(self, model: Any, tokenizer: Any = None) -> Dict[str, Any]:
        out = S.run_suite(self.name, model, tokenizer, self.data_path, self.max_samples)
        res = out["result"]
        score = next((float(res[k]) for k in (self.metric, "accuracy", "pass@1", "exact_match", "mean") if isinstance(res, dict) and k in res), None)
        return {"benchmark": self.name, "metric": self.metric, "score": score, "n": out["rows"], "source": out["source"], "details": res}


class PiscesLxSWEBenchBenchmark(PiscesLxBaseBenchmark):
    """Patch generation scored by FORMAT only here (a unified diff that names existing paths and applies hunk headers that add
    up): running repository test suites needs their containers, which an offline host does not have."""

    name, metric = "swebench", "well_formed_rate"

    def __init__(self, rows: Optional[Sequence[Dict[str, Any]]] = None, generate: Optional[GenerateFn] = None, max_new_tokens: int = 512):
        super().__init__()
        self.rows, self.generate, self.max_new_tokens = list(rows or []), generate, max_new_tokens

    def evaluate(self, model: Any = None, tokenizer: Any = None) -> Dict[str, Any]:
        gen = self.generate or S._generate_fn(model, tokenizer)
        chk = S.PiscesLxSWEBenchFormatChecker()
        ok = 0
        details = []
        for r in self.rows:
            patch = gen(f"Repository issue:\n{r.get('problem_statement', r.get('issue', ''))}\n\nWrite a unified diff that fixes it.\n", self.max_new_tokens)
            res = chk.check(patch, r.get("repo_files", []))
            good = bool(res.get("is_diff")) and (not r.get("repo_files") or all(f in set(r["repo_files"]) for f in res.get("files", [])))
            ok += int(good)
            details.append({"instance_id": r.get("instance_id"), "well_formed": good})
        n = len(self.rows)
        return {"benchmark": self.name, "metric": self.metric, "score": ok / n if n else None, "n": n, "source": "given rows", "details": details}


class PiscesLxBenchmarkEvaluator:
    """Runs benchmarks against one model, keeping going when one fails (the failure is a result with ``error``)."""

    def __init__(self, model: Any, tokenizer: Any = None):
        self.model, self.tokenizer = model, tokenizer

    def evaluate(self, benchmarks: Sequence[PiscesLxBaseBenchmark], fail_fast: bool = False) -> Dict[str, Dict[str, Any]]:
        out: Dict[str, Dict[str, Any]] = {}
        for b in benchmarks:
            t0 = time.perf_counter()
            try:
                r = b.evaluate(self.model, self.tokenizer)
            except Exception as e:
                if fail_fast:
                    raise
                r = {"benchmark": b.name, "metric": b.metric, "score": None, "n": 0, "error": f"{type(e).__name__}: {e}"}
            r["seconds"] = time.perf_counter() - t0
            out[b.name] = r
        return out


class PiscesLxBenchmarkSuite:
    def __init__(self, config: Optional[PiscesLxBenchmarkSuiteConfig] = None):
        self.config = config or PiscesLxBenchmarkSuiteConfig()

    def benchmarks(self) -> List[PiscesLxBaseBenchmark]:
        out = []
        for s in self.config.suites:
            if s not in S.available_suites():
                raise ValueError(f"unknown suite {s!r}; available: {', '.join(S.available_suites())}")
            b = PiscesLxBaseBenchmark(self.config.data_paths.get(s), self.config.max_samples)
            b.name = s
            b.metric = {"humaneval": "pass@1", "needle": "accuracy"}.get(s, "accuracy")
            out.append(b)
        return out

    def run(self, model: Any, tokenizer: Any = None) -> Dict[str, Any]:
        res = PiscesLxBenchmarkEvaluator(model, tokenizer).evaluate(self.benchmarks(), self.config.fail_fast)
        scores = [r["score"] for r in res.values() if r.get("score") is not None]
        return {"results": res, "summary": {"mean_score": statistics.fmean(scores) if scores else None, "completed": len(scores), "failed": sum(1 for r in res.values() if "error" in r)}}


# ---- results --------------------------------------------------------------------------------------------------------------------
class PiscesLxToolsResultManager:
    def __init__(self, output_dir: str):
        self.output_dir = Path(output_dir)
        self.output_dir.mkdir(parents=True, exist_ok=True)

    def save_results(self, results: Dict[str, Any], summary: Dict[str, Any], config: Optional[PiscesLxToolsBenchmarkConfig] = None, tag: Optional[str] = None) -> str:
        tag = tag or time.strftime("%Y%m%d_%H%M%S")
        p = self.output_dir / f"results_{tag}.json"
        tmp = p.with_suffix(".tmp")
        tmp.write_text(json.dumps({"results": results, "summary": summary, "config": asdict(config) if config else None, "saved_at": time.time()}, indent=1, default=str))
        tmp.replace(p)
        return str(p)

    def load_results(self, path: Optional[str] = None) -> Dict[str, Any]:
        files = sorted(self.output_dir.glob("results_*.json"))
        if path is None and not files:
            raise FileNotFoundError(f"no results under {self.output_dir}")
        return json.loads(Path(path or files[-1]).read_text())

    def generate_comparison_report(self, results: Dict[str, Dict[str, Any]]) -> Dict[str, Any]:
        """``results``: model name -> {benchmark -> {"score"}}: per-benchmark winner and each model's mean."""
        benches = sorted({b for r in results.values() for b in r})
        table = {b: {m: (results[m].get(b) or {}).get("score") for m in results} for b in benches}
        winners = {b: max((m for m in row if row[m] is not None), key=lambda m: row[m], default=None) for b, row in table.items()}
        means = {m: (statistics.fmean([v for v in (table[b][m] for b in benches) if v is not None]) if any(table[b][m] is not None for b in benches) else None) for m in results}
        return {"benchmarks": benches, "table": table, "winners": winners, "mean_scores": means, "best_model": max((m for m in means if means[m] is not None), key=lambda m: means[m], default=None)}


class PiscesLxToolsComparisonManager:
    """Keeps named result sets and diffs two of them (regressions beyond ``tolerance``)."""

    def __init__(self, tolerance: float = 0.01):
        self.tolerance, self.runs = tolerance, {}

    def add(self, name: str, results: Dict[str, Dict[str, Any]]) -> None:
        self.runs[name] = {b: r.get("score") for b, r in results.items()}

    def diff(self, base: str, new: str) -> Dict[str, Any]:
        a, b = self.runs[base], self.runs[new]
        rows = {k: {"base": a.get(k), "new": b.get(k), "delta": (b[k] - a[k]) if (a.get(k) is not None and b.get(k) is not None) else None} for k in sorted(set(a) | set(b))}
        return {"rows": rows, "regressions": [k for k, r in rows.items() if r["delta"] is not None and r["delta"] < -self.tolerance],
                "improvements": [k for k, r in rows.items() if r["delta"] is not None and r["delta"] > self.tolerance]}


@dataclass
class PiscesLxToolsComparisonConfig:
    model_name: str = "pisceslx"
    output_dir: str = ".pisceslx/benchmark/comparison"
    reference_table: Optional[str] = None                             # json: {model: {benchmark: score}}
    higher_is_better: bool = True


class PiscesLxToolsFlagshipComparator:
    """Ranks this model's scores among a user-supplied table of other models' scores (no such table ships with the code)."""

    def __init__(self, config: Optional[PiscesLxToolsComparisonConfig] = None, reference: Optional[Dict[str, Dict[str, float]]] = None):
        self.config = config or PiscesLxToolsComparisonConfig()
        self.reference = dict(reference or {})
        self.last: Dict[str, Any] = {}

    def load_flagship_benchmarks(self) -> Dict[str, Dict[str, float]]:
        if not self.reference and self.config.reference_table:
            self.reference = json.loads(Path(self.config.reference_table).read_text())
        return self.reference

    def _compute_rankings(self, ours: Dict[str, float]) -> Dict[str, Dict[str, Any]]:
        ref, out = self.load_flagship_benchmarks(), {}
        for b, s in ours.items():
            field_ = sorted([(m, v[b]) for m, v in ref.items() if b in v] + [(self.config.model_name, s)], key=lambda t: -t[1] if self.config.higher_is_better else t[1])
            out[b] = {"rank": [m for m, _ in field_].index(self.config.model_name) + 1, "of": len(field_), "leader": field_[0][0], "leader_score": field_[0][1]}
        return out

    def _identify_gaps(self, ours: Dict[str, float]) -> Dict[str, Dict[str, Any]]:
        r = self._compute_rankings(ours)
        return {b: {"gap_to_leader": (r[b]["leader_score"] - s) if self.config.higher_is_better else (s - r[b]["leader_score"]), "leader": r[b]["leader"]} for b, s in ours.items()}

    def compare_with_flagship(self, ours: Dict[str, float]) -> Dict[str, Any]:
        rk, gaps = self._compute_rankings(ours), self._identify_gaps(ours)
        self.last = {"model": self.config.model_name, "scores": dict(ours), "rankings": rk, "gaps": gaps,
                     "strengths": sorted((b for b in rk if rk[b]["rank"] == 1), key=str), "weaknesses": sorted(gaps, key=lambda b: -gaps[b]["gap_to_leader"])[:3],
                     "mean_rank": statistics.fmean(v["rank"] for v in rk.values()) if rk else None}
        return self.last

    def generate_comparison_table(self) -> str:
        ref, ours = self.load_flagship_benchmarks(), self.last.get("scores", {})
        models = [self.config.model_name] + sorted(ref)
        rows = ["| benchmark | " + " | ".join(models) + " |", "|---|" + "---|" * len(models)]
        for b in sorted(ours):
            cells = [f"{ours[b]:.3g}"] + [f"{ref[m][b]:.3g}" if b in ref[m] else "-" for m in models[1:]]
            rows.append(f"| {b} | " + " | ".join(cells) + " |")
        return "\n".join(rows)

    def save_results(self) -> str:
        d = Path(self.config.output_dir)
        d.mkdir(parents=True, exist_ok=True)
        p = d / f"comparison_{self.config.model_name}.json"
        p.write_text(json.dumps(self.last, indent=1))
        return str(p)


# ---- runner ------------------------------------------------------------------------------------------------------------------------
class PiscesLxToolsBenchmarkRunner:
    """``run_benchmark(model)`` runs the configured suites and saves the results; ``model_loader(path)`` builds models for
    ``compare_models`` (``engine.loader.load_model_for_inference`` by default)."""

    def __init__(self, config: Union[str, Dict[str, Any], PiscesLxToolsBenchmarkConfig], model_loader: Optional[Callable[[str], Any]] = None):
        self.config = PiscesLxToolsBenchmarkConfig.load(config)
        self.results = PiscesLxToolsResultManager(self.config.output_dir)
        self.model_loader = model_loader

    def _load(self, path: str) -> Any:
        if self.model_loader is not None:
            return self.model_loader(path)
        from ..engine.loader import load_model_for_inference
        import os
        return load_model_for_inference(path if not os.path.exists(path) else "0.01B", path if os.path.exists(path) else None, None if self.config.device == "auto" else self.config.device)

    def run_benchmark(self, model: Any = None, tokenizer: Any = None, save: bool = True) -> Dict[str, Any]:
        model = model if model is not None else self._load(self.config.model_path)
        suite = PiscesLxBenchmarkSuite(PiscesLxBenchmarkSuiteConfig(self.config.datasets, self.config.data_paths, self.config.max_samples, self.config.output_dir))
        out = suite.run(model, tokenizer)
        out["model"] = self.config.model_name
        if save:
            out["saved_to"] = self.results.save_results(out["results"], out["summary"], self.config)
        return out

    def compare_models(self, model_configs: List[Dict[str, Any]]) -> Dict[str, Any]:
        """``[{"name", "model" | "model_path", "tokenizer"?}]``."""
        per = {}
        for mc in model_configs:
            m = mc.get("model") if mc.get("model") is not None else self._load(mc["model_path"])
            per[mc.get("name") or mc.get("model_path", "model")] = self.run_benchmark(m, mc.get("tokenizer"), save=False)["results"]
        return {"per_model": per, "comparison": self.results.generate_comparison_report(per)}


class PiscesLxToolsBenchmark:
    @staticmethod
    def create(config: Union[str, Dict[str, Any]]) -> PiscesLxToolsBenchmarkConfig:
        return PiscesLxToolsBenchmarkConfig.load(config)

    @staticmethod
    def run(config: Union[str, Dict[str, Any], PiscesLxToolsBenchmarkConfig], model: Any = None, tokenizer: Any = None) -> Dict[str, Any]:
        return PiscesLxToolsBenchmarkRunner(config).run_benchmark(model, tokenizer)

    @staticmethod
    def compare(model_configs: List[Dict[str, Any]], config: Optional[Union[str, Dict[str, Any]]] = None) -> Dict[str, Any]:
        return PiscesLxToolsBenchmarkRunner(config or {}).compare_models(model_configs)


class PiscesLxToolsBenchmarkComparer:
    compare = staticmethod(PiscesLxToolsBenchmark.compare)


# ---- performance ------------------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxToolsPerformanceConfig:
    output_dir: str = ".pisceslx/benchmark/performance"
    warmup_runs: int = 3
    benchmark_runs: int = 10
    batch_sizes: List[int] = field(default_factory=lambda: [1, 2, 4, 8, 16])
    sequence_lengths: List[int] = field(default_factory=lambda: [128, 256, 512, 1024, 2048, 4096])
    max_new_tokens: int = 128
    device: str = "cuda"
    measure_memory: bool = True
    measure_flops: bool = True
    measure_gpu_util: bool = True
    save_results: bool = True
    max_tokens_per_case: int = 1 << 20            # batch x length above this is skipped (a bound on the sweep's memory)


@dataclass
class PiscesLxToolsPerformanceMetrics:
    batch_size: int
    sequence_length: int
    latency_ms_mean: float
    latency_ms_p50: float
    latency_ms_p95: float
    tokens_per_second: float
    peak_memory_mb: Optional[float] = None
    tflops: Optional[float] = None
    timing: str = "host"


class PiscesLxToolsPerformanceEvaluator:
    """Forward latency and throughput over batch x length.  Timing: CUDA events on the current stream after ``warmup_runs``
    untimed calls; on the host, ``perf_counter``."""

    def __init__(self, model: Any, config: Optional[PiscesLxToolsPerformanceConfig] = None):
        self.model, self.config = model, config or PiscesLxToolsPerformanceConfig()
        self.device = next(model.parameters()).device
        self.vocab = int(getattr(getattr(model, "cfg", None), "vocab_size", 0) or 32000)

    def _time(self, fn: Callable[[], Any], runs: int) -> Tuple[List[float], str]:
        if self.device.type == "cuda":
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(runs)]
            torch.cuda.synchronize(self.device)
            for a, b in evs:
                a.record()
                fn()
                b.record()
            torch.cuda.synchronize(self.device)
            return [a.elapsed_time(b) for a, b in evs], "cuda_events"
        out = []
        for _ in range(runs):
            t0 = time.perf_counter()
            fn()
            out.append((time.perf_counter() - t0) * 1e3)
        return out, "host"

    @torch.no_grad()
    def measure(self, batch_size: int, sequence_length: int) -> PiscesLxToolsPerformanceMetrics:
        c = self.config
        ids = torch.randint(0, self.vocab, (batch_size, sequence_length), device=self.device)
        was = self.model.training
        self.model.eval()
        fn = lambda: self.model(input_ids=ids)
        for _ in range(c.warmup_runs):
            fn()
        if self.device.type == "cuda" and c.measure_memory:
            torch.cuda.reset_peak_memory_stats(self.device)
        ms, how = self._time(fn, c.benchmark_runs)
        self.model.train(was)
        s = sorted(ms)
        mean = statistics.fmean(ms)
        mem = torch.cuda.max_memory_allocated(self.device) / 2 ** 20 if (self.device.type == "cuda" and c.measure_memory) else None
        tf = None
        if c.measure_flops and getattr(self.model, "cfg", None) is not None:
            from .benchmark import model_flops_per_token
            try:
                tf = model_flops_per_token(self.model.cfg) * batch_size * sequence_length / (mean / 1e3) / 1e12
            except Exception:
                tf = None
        return PiscesLxToolsPerformanceMetrics(batch_size, sequence_length, mean, s[len(s) // 2], s[min(int(0.95 * len(s)), len(s) - 1)],
                                               batch_size * sequence_length / (mean / 1e3), mem, tf, how)

    def sweep(self) -> List[PiscesLxToolsPerformanceMetrics]:
        c, out = self.config, []
        limit = int(getattr(getattr(self.model, "cfg", None), "max_position_embeddings", 1 << 30) or (1 << 30))
        for b in c.batch_sizes:
            for n in c.sequence_lengths:
                if b * n > c.max_tokens_per_case or n > limit:
                    continue
                out.append(self.measure(b, n))
        return out


class PiscesLxToolsPerformanceBenchmarkRunner:
    def __init__(self, model: Any, config: Optional[PiscesLxToolsPerformanceConfig] = None):
        self.evaluator = PiscesLxToolsPerformanceEvaluator(model, config)

    def run(self) -> Dict[str, Any]:
        rows = [asdict(m) for m in self.evaluator.sweep()]
        best = max(rows, key=lambda r: r["tokens_per_second"], default=None)
        out = {"cases": rows, "best_throughput": best, "device": str(self.evaluator.device), "timing": rows[0]["timing"] if rows else None}
        c = self.evaluator.config
        if c.save_results:
            d = Path(c.output_dir)
            d.mkdir(parents=True, exist_ok=True)
            (d / "performance.json").write_text(json.dumps(out, indent=1))
            out["saved_to"] = str(d / "performance.json")
        return out


# ---- long context / agent / multimodal ---------------------------------------------------------------------------------------------
@dataclass
class PiscesLxToolsLongContextConfig:
    lengths: Tuple[int, ...] = (1024, 4096, 16384)
    depths: Tuple[float, ...] = (0.0, 0.25, 0.5, 0.75, 1.0)
    output_dir: str = ".pisceslx/benchmark/long_context"
    max_new_tokens: int = 16


@dataclass
class PiscesLxToolsLongContextMetrics:
    accuracy: float
    by_length: Dict[int, float]
    by_depth: Dict[float, float]
    grid: Dict[str, float]


class PiscesLxToolsLongContextEvaluator:
    def __init__(self, generate: GenerateFn, tokenizer: Any, config: Optional[PiscesLxToolsLongContextConfig] = None):
        self.bench, self.config = S.PiscesLxLongContextBenchmark(generate, tokenizer), config or PiscesLxToolsLongContextConfig()

    def evaluate(self) -> PiscesLxToolsLongContextMetrics:
        c = self.config
        grid: Dict[str, float] = {}
        for n in c.lengths:
            for d in c.depths:
                r = self.bench.evaluate(lengths=(n,), depths=(d,))
                grid[f"{n}@{d}"] = float(r["mean"])
        by_len = {n: statistics.fmean(grid[f"{n}@{d}"] for d in c.depths) for n in c.lengths}
        by_dep = {d: statistics.fmean(grid[f"{n}@{d}"] for n in c.lengths) for d in c.depths}
        return PiscesLxToolsLongContextMetrics(statistics.fmean(grid.values()) if grid else 0.0, by_len, by_dep, grid)


class PiscesLxToolsLongContextBenchmarkRunner:
    def __init__(self, model: Any, tokenizer: Any, config: Optional[PiscesLxToolsLongContextConfig] = None):
        self.evaluator = PiscesLxToolsLongContextEvaluator(S._generate_fn(model, tokenizer), tokenizer, config)

    def run(self) -> Dict[str, Any]:
        return asdict(self.evaluator.evaluate())


@dataclass
class PiscesLxToolsAgentConfig:
    max_steps: int = 8
    output_dir: str = ".pisceslx/benchmark/agent"


@dataclass
class PiscesLxToolsAgentMetrics:
    success_rate: float
    mean_steps: float
    tool_error_rate: float
    n: int


class PiscesLxToolsAgentEvaluator:
    """Tasks ``{"goal", "check": callable(final_text) -> bool}`` run by an agent ``agent(goal, max_steps) -> {"answer", "steps", "tool_errors"}``."""

    def __init__(self, agent: Callable[[str, int], Dict[str, Any]], config: Optional[PiscesLxToolsAgentConfig] = None):
        self.agent, self.config = agent, config or PiscesLxToolsAgentConfig()

    def evaluate(self, tasks: Sequence[Dict[str, Any]]) -> PiscesLxToolsAgentMetrics:
        ok = steps = errs = calls = 0
        for t in tasks:
            try:
                r = self.agent(t["goal"], self.config.max_steps)
            except Exception:
                r = {"answer": "", "steps": self.config.max_steps, "tool_errors": 1, "tool_calls": 1}
            ok += int(bool(t["check"](r.get("answer", ""))))
            steps += int(r.get("steps", 0))
            errs += int(r.get("tool_errors", 0))
            calls += int(r.get("tool_calls", max(r.get("steps", 0), 1)))
        n = len(tasks)
        return PiscesLxToolsAgentMetrics(ok / n if n else 0.0, steps / n if n else 0.0, errs / max(calls, 1), n)


class PiscesLxToolsAgentBenchmarkRunner:
    def __init__(self, agent: Callable[[str, int], Dict[str, Any]], config: Optional[PiscesLxToolsAgentConfig] = None):
        self.evaluator = PiscesLxToolsAgentEvaluator(agent, config)

    def run(self, tasks: Sequence[Dict[str, Any]]) -> Dict[str, Any]:
        return asdict(self.evaluator.evaluate(tasks))


@dataclass
class PiscesLxToolsMultimodalConfig:
    modalities: Tuple[str, ...] = ("vision",)
    output_dir: str = ".pisceslx/benchmark/multimodal"
    max_new_tokens: int = 32


class _ModalEvaluator:
    modality = "vision"

    def __init__(self, answer: Callable[[Dict[str, Any]], str]):
        self.answer = answer

    def evaluate(self, rows: Sequence[Dict[str, Any]]) -> Dict[str, Any]:
        """Rows ``{"question", "answers": [...], <modality payload>}``; a prediction counts when it contains one of the accepted answers."""
        hit = 0
        for r in rows:
            pred = str(self.answer(r)).strip().lower()
            hit += int(any(str(a).strip().lower() in pred for a in r.get("answers", [r.get("answer", "")]) if str(a).strip()))
        return {"modality": self.modality, "accuracy": hit / len(rows) if rows else 0.0, "n": len(rows)}


class PiscesLxToolsVisionEvaluator(_ModalEvaluator):
    modality = "vision"


class PiscesLxToolsAudioEvaluator(_ModalEvaluator):
    modality = "audio"


class PiscesLxToolsVideoEvaluator(_ModalEvaluator):
    modality = "video"


class PiscesLxToolsMultimodalBenchmarkRunner:
    EVALUATORS = {"vision": PiscesLxToolsVisionEvaluator, "audio": PiscesLxToolsAudioEvaluator, "video": PiscesLxToolsVideoEvaluator}

    def __init__(self, answer: Callable[[Dict[str, Any]], str], config: Optional[PiscesLxToolsMultimodalConfig] = None):
        self.answer, self.config = answer, config or PiscesLxToolsMultimodalConfig()

    def run(self, rows_by_modality: Dict[str, Sequence[Dict[str, Any]]]) -> Dict[str, Any]:
        out = {m: self.EVALUATORS[m](self.answer).evaluate(rows_by_modality.get(m, [])) for m in self.config.modalities}
        accs = [r["accuracy"] for r in out.values() if r["n"]]
        return {"per_modality": out, "mean_accuracy": statistics.fmean(accs) if accs else None}


# ---- charts and reports ----------------------------------------------------------------------------------------------------------
@dataclass
class PiscesLxToolsVisualizationConfig:
    output_dir: str = ".pisceslx/benchmark/figures"
    width: int = 640
    height: int = 420
    palette: Tuple[str, ...] = ("#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b")


class PiscesLxToolsBenchmarkVisualizer:
    """Charts as SVG text (no plotting library): radar, grouped bars, heat map, line trend, needle-in-a-haystack grid."""

    def __init__(self, config: Optional[PiscesLxToolsVisualizationConfig] = None):
        self.config = config or PiscesLxToolsVisualizationConfig()
        Path(self.config.output_dir).mkdir(parents=True, exist_ok=True)

    def _wrap(self, body: str, title: str) -> str:
        c = self.config
        return (f'<svg xmlns="http://www.w3.org/2000/svg" width="{c.width}" height="{c.height}" viewBox="0 0 {c.width} {c.height}"><rect width="100%" height="100%" fill="white"/>'
                f'<text x="{c.width / 2}" y="22" text-anchor="middle" font-family="sans-serif" font-size="15">{html.escape(title)}</text>{body}</svg>')

    def _save(self, name: str, svg: str) -> str:
        p = Path(self.config.output_dir) / name
        p.write_text(svg)
        return str(p)

    def plot_radar_chart(self, scores: Dict[str, Dict[str, float]], title: str = "Benchmarks", filename: str = "radar.svg") -> str:
        c = self.config
        axes = sorted({b for s in scores.values() for b in s})
        cx, cy, R = c.width / 2, c.height / 2 + 10, min(c.width, c.height) / 2 - 60
        hi = max([v for s in scores.values() for v in s.values()] + [1e-9])
        pt = lambda i, v: (cx + R * v / hi * math.sin(2 * math.pi * i / len(axes)), cy - R * v / hi * math.cos(2 * math.pi * i / len(axes)))
        body = "".join(f'<line x1="{cx}" y1="{cy}" x2="{pt(i, hi)[0]:.1f}" y2="{pt(i, hi)[1]:.1f}" stroke="#ccc"/><text x="{pt(i, hi * 1.12)[0]:.1f}" y="{pt(i, hi * 1.12)[1]:.1f}" '
                       f'text-anchor="middle" font-family="sans-serif" font-size="11">{html.escape(a)}</text>' for i, a in enumerate(axes))
        for k, (m, s) in enumerate(scores.items()):
            col = c.palette[k % len(c.palette)]
            pts = " ".join(f"{pt(i, s.get(a, 0.0))[0]:.1f},{pt(i, s.get(a, 0.0))[1]:.1f}" for i, a in enumerate(axes))
            body += f'<polygon points="{pts}" fill="{col}" fill-opacity="0.15" stroke="{col}"/><text x="12" y="{44 + 16 * k}" fill="{col}" font-family="sans-serif" font-size="12">{html.escape(m)}</text>'
        return self._save(filename, self._wrap(body, title))

    def plot_bar_comparison(self, scores: Dict[str, Dict[str, float]], title: str = "Comparison", filename: str = "bars.svg") -> str:
        c = self.config
        benches, models = sorted({b for s in scores.values() for b in s}), list(scores)
        hi = max([v for s in scores.values() for v in s.values()] + [1e-9])
        x0, y0, W, H = 50, c.height - 50, c.width - 70, c.height - 100
        gw = W / max(len(benches), 1)
        bw = gw * 0.8 / max(len(models), 1)
        body = f'<line x1="{x0}" y1="{y0}" x2="{x0 + W}" y2="{y0}" stroke="#444"/>'
        for i, b in enumerate(benches):
            body += f'<text x="{x0 + gw * (i + 0.5):.1f}" y="{y0 + 16}" text-anchor="middle" font-family="sans-serif" font-size="11">{html.escape(b)}</text>'
            for k, m in enumerate(models):
                v = scores[m].get(b)
                if v is None:
                    continue
                h = H * v / hi
                body += f'<rect x="{x0 + gw * i + gw * 0.1 + bw * k:.1f}" y="{y0 - h:.1f}" width="{bw:.1f}" height="{h:.1f}" fill="{c.palette[k % len(c.palette)]}"><title>{html.escape(m)}: {v:.4g}</title></rect>'
        body += "".join(f'<text x="{x0 + 8}" y="{44 + 15 * k}" fill="{c.palette[k % len(c.palette)]}" font-family="sans-serif" font-size="12">{html.escape(m)}</text>' for k, m in enumerate(models))
        return self._save(filename, self._wrap(body, title))

    def plot_heatmap(self, grid: Dict[Any, Dict[Any, float]], title: str = "Heat map", filename: str = "heatmap.svg", lo: float = 0.0, hi: float = 1.0) -> str:
        c = self.config
        rows = list(grid)
        cols = list(dict.fromkeys(k for r in grid.values() for k in r))
        x0, y0 = 90, 50
        cw, ch = (c.width - x0 - 20) / max(len(cols), 1), (c.height - y0 - 40) / max(len(rows), 1)
        body = ""
        for i, r in enumerate(rows):
            body += f'<text x="{x0 - 6}" y="{y0 + ch * (i + 0.6):.1f}" text-anchor="end" font-family="sans-serif" font-size="11">{html.escape(str(r))}</text>'
            for j, k in enumerate(cols):
                v = grid[r].get(k)
                if v is None:
                    continue
                t = min(max((v - lo) / max(hi - lo, 1e-12), 0.0), 1.0)
                col = f"rgb({int(215 - 170 * t)},{int(48 + 150 * t)},{int(39 + 40 * t)})"
                body += f'<rect x="{x0 + cw * j:.1f}" y="{y0 + ch * i:.1f}" width="{cw:.1f}" height="{ch:.1f}" fill="{col}"><title>{r} / {k}: {v:.3g}</title></rect>'
        body += "".join(f'<text x="{x0 + cw * (j + 0.5):.1f}" y="{c.height - 18}" text-anchor="middle" font-family="sans-serif" font-size="11">{html.escape(str(k))}</text>' for j, k in enumerate(cols))
        return self._save(filename, self._wrap(body, title))

    def plot_line_trend(self, series: Dict[str, Sequence[float]], title: str = "Trend", filename: str = "trend.svg") -> str:
        c = self.config
        vals = [v for s in series.values() for v in s]
        lo, hi = (min(vals), max(vals)) if vals else (0.0, 1.0)
        hi = hi if hi > lo else lo + 1.0
        x0, y0, W, H = 50, c.height - 40, c.width - 70, c.height - 90
        body = f'<line x1="{x0}" y1="{y0}" x2="{x0 + W}" y2="{y0}" stroke="#444"/><line x1="{x0}" y1="{y0}" x2="{x0}" y2="{y0 - H}" stroke="#444"/>'
        for k, (name, s) in enumerate(series.items()):
            n = max(len(s) - 1, 1)
            pts = " ".join(f"{x0 + W * i / n:.1f},{y0 - H * (v - lo) / (hi - lo):.1f}" for i, v in enumerate(s))
            col = c.palette[k % len(c.palette)]
            body += f'<polyline fill="none" stroke="{col}" stroke-width="1.6" points="{pts}"/><text x="{x0 + 8}" y="{44 + 15 * k}" fill="{col}" font-family="sans-serif" font-size="12">{html.escape(name)}</text>'
        return self._save(filename, self._wrap(body, title))

    def plot_needle_haystack_heatmap(self, grid: Dict[str, float], title: str = "Needle in a haystack", filename: str = "needle.svg") -> str:
        """``grid``: "length@depth" -> accuracy (the long-context evaluator's grid)."""
        g: Dict[str, Dict[str, float]] = {}
        for key, v in grid.items():
            n, d = key.split("@")
            g.setdefault(f"depth {d}", {})[n] = v
        return self.plot_heatmap(g, title, filename)

    @staticmethod
    def create_visualizer(output_dir: str = ".pisceslx/benchmark/figures", **kw: Any) -> "PiscesLxToolsBenchmarkVisualizer":
        return PiscesLxToolsBenchmarkVisualizer(PiscesLxToolsVisualizationConfig(output_dir=output_dir, **kw))


class PiscesLxToolsReportGenerator:
    def __init__(self, config: Optional[PiscesLxToolsVisualizationConfig] = None):
        self.config = config or PiscesLxToolsVisualizationConfig()
        Path(self.config.output_dir).mkdir(parents=True, exist_ok=True)

    @staticmethod
    def _rows(results: Dict[str, Dict[str, Any]]) -> List[Tuple[str, str, str, str]]:
        return [(b, str(r.get("metric", "")), "-" if r.get("score") is None else f"{r['score']:.4g}", str(r.get("n", ""))) for b, r in sorted(results.items())]

    def generate_markdown_report(self, results: Dict[str, Dict[str, Any]], title: str = "Benchmark report", model: str = "", filename: str = "report.md") -> str:
        lines = [f"# {title}", "", f"Model: `{model}`" if model else "", "", "| benchmark | metric | score | n |", "|---|---|---|---|"]
        lines += [f"| {b} | {m} | {s} | {n} |" for b, m, s, n in self._rows(results)]
        failed = [b for b, r in results.items() if "error" in r]
        if failed:
            lines += ["", "Failed: " + ", ".join(f"{b} ({results[b]['error']})" for b in failed)]
        p = Path(self.config.output_dir) / filename
        p.write_text("\n".join(lines) + "\n")
        return str(p)

    def generate_html_report(self, results: Dict[str, Dict[str, Any]], title: str = "Benchmark report", model: str = "", figures: Sequence[str] = (), filename: str = "report.html") -> str:
        e = html.escape
        rows = "".join(f"<tr><td>{e(b)}</td><td>{e(m)}</td><td>{e(s)}</td><td>{e(n)}</td></tr>" for b, m, s, n in self._rows(results))
        figs = "".join(f'<div>{Path(f).read_text()}</div>' for f in figures if Path(f).suffix == ".svg" and Path(f).exists())
        doc = (f"<!doctype html><html><head><meta charset='utf-8'><title>{e(title)}</title><style>body{{font-family:sans-serif;margin:2em}}table{{border-collapse:collapse}}"
               f"td,th{{border:1px solid #ccc;padding:4px 10px}}</style></head><body><h1>{e(title)}</h1><p>Model: <code>{e(model)}</code></p>"
               f"<table><tr><th>benchmark</th><th>metric</th><th>score</th><th>n</th></tr>{rows}</table>{figs}</body></html>")
        p = Path(self.config.output_dir) / filename
        p.write_text(doc)
        return str(p)

    def generate_latex_table(self, results: Dict[str, Dict[str, Any]], caption: str = "Benchmark results", label: str = "tab:bench", filename: str = "table.tex") -> str:
        esc = lambda s: s.replace("_", r"\_").replace("%", r"\%").replace("&", r"\&").replace("#", r"\#")
        body = "\n".join(f"{esc(b)} & {esc(m)} & {s} & {n} \\\\" for b, m, s, n in self._rows(results))
        tex = (f"\\begin{{table}}[t]\n\\centering\n\\begin{{tabular}}{{llrr}}\n\\toprule\nbenchmark & metric & score & n \\\\\n\\midrule\n{body}\n\\bottomrule\n\\end{{tabular}}\n"
               f"\\caption{{{esc(caption)}}}\n\\label{{{label}}}\n\\end{{table}}\n")
        p = Path(self.config.output_dir) / filename
        p.write_text(tex)
        return str(p)

    @staticmethod
    def create_report_generator(output_dir: str = ".pisceslx/benchmark/figures") -> "PiscesLxToolsReportGenerator":
        return PiscesLxToolsReportGenerator(PiscesLxToolsVisualizationConfig(output_dir=output_dir))


# ---- orchestration from the command line ---------------------------------------------------------------------------------------
class PiscesLxToolsBenchmarkOrchestrator:
    """Turns parsed command-line arguments into a run: ``--list``, ``--selftest``, ``--benchmark NAME[,NAME]``, ``--perf``, ``--report``."""

    def __init__(self, args: Any, model_loader: Optional[Callable[[str], Any]] = None):
        self.args, self.model_loader = args, model_loader

    def _parse_generation_config(self) -> Optional[Dict[str, Any]]:
        raw = getattr(self.args, "generation_config", None)
        if not raw:
            return None
        if isinstance(raw, dict):
            return raw
        try:
            return json.loads(raw)
        except ValueError:
            return dict(kv.split("=", 1) for kv in str(raw).split(",") if "=" in kv)

    def run(self, model: Any = None, tokenizer: Any = None) -> Dict[str, Any]:
        a = self.args
        if getattr(a, "list", False):
            return {"suites": S.available_suites()}
        if getattr(a, "selftest", False):
            return {"selftest": S.selftest()}
        names = [n.strip() for n in str(getattr(a, "benchmark", "") or "").split(",") if n.strip()] or None
        cfg = PiscesLxToolsBenchmarkConfig(model_path=getattr(a, "model_path", "") or "", datasets=names, output_dir=getattr(a, "output_dir", None) or ".pisceslx/benchmark",
                                           max_samples=getattr(a, "max_samples", None), generation_config=self._parse_generation_config(),
                                           data_paths=dict(getattr(a, "data_paths", None) or {}))
        runner = PiscesLxToolsBenchmarkRunner(cfg, self.model_loader)
        out = runner.run_benchmark(model, tokenizer)
        if getattr(a, "perf", False):
            m = model if model is not None else runner._load(cfg.model_path)
            out["performance"] = PiscesLxToolsPerformanceBenchmarkRunner(m, PiscesLxToolsPerformanceConfig(output_dir=cfg.output_dir + "/performance", batch_sizes=[1], sequence_lengths=[128],
                                                                                                         warmup_runs=3, benchmark_runs=5)).run()
        if getattr(a, "report", False):
            out["report"] = PiscesLxToolsReportGenerator(PiscesLxToolsVisualizationConfig(output_dir=cfg.output_dir)).generate_markdown_report(out["results"], model=cfg.model_name)
        return out


class PiscesLxBenchmarkCli:
    @staticmethod
    def build_parser():
        import argparse
        p = argparse.ArgumentParser(prog="benchmark", description="Run evaluation suites and performance sweeps")
        p.add_argument("--list", action="store_true")
        p.add_argument("--selftest", action="store_true")
        p.add_argument("--benchmark", default="")
        p.add_argument("--model-path", dest="model_path", default="")
        p.add_argument("--output-dir", dest="output_dir", default=".pisceslx/benchmark")
        p.add_argument("--max-samples", dest="max_samples", type=int, default=None)
        p.add_argument("--generation-config", dest="generation_config", default=None)
        p.add_argument("--perf", action="store_true")
        p.add_argument("--report", action="store_true")
        return p

    @classmethod
    def main(cls, argv: Optional[Sequence[str]] = None, model: Any = None, tokenizer: Any = None) -> Dict[str, Any]:
        return PiscesLxToolsBenchmarkOrchestrator(cls.build_parser().parse_args(list(argv) if argv is not None else None)).run(model, tokenizer)
