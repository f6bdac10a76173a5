"""Benchmark framework: configuration, datasets, suite runs, comparison, performance sweep, evaluators, charts and reports."""
import json

import pytest
import torch

from pisceslx_b200.config import YvConfig
from pisceslx_b200.models.model import YvModelForCausalLM
from pisceslx_b200.models.tokenizer import YvTokenizer
from pisceslx_b200.tools.benchmark_framework import (
    PiscesLxBenchmarkCli, PiscesLxBenchmarkSuite, PiscesLxBenchmarkSuiteConfig, PiscesLxGSM8KDataset, PiscesLxHumanEvalDataset, PiscesLxMMLUDataset,
    PiscesLxSWEBenchBenchmark, PiscesLxToolsAgentBenchmarkRunner, PiscesLxToolsBenchmark, PiscesLxToolsBenchmarkConfig, PiscesLxToolsBenchmarkRunner,
    PiscesLxToolsBenchmarkVisualizer, PiscesLxToolsComparisonConfig, PiscesLxToolsComparisonManager, PiscesLxToolsFlagshipComparator, PiscesLxToolsLongContextConfig,
    PiscesLxToolsLongContextEvaluator, PiscesLxToolsMultimodalBenchmarkRunner, PiscesLxToolsMultimodalConfig, PiscesLxToolsPerformanceBenchmarkRunner,
    PiscesLxToolsPerformanceConfig, PiscesLxToolsReportGenerator, PiscesLxToolsResultManager, PiscesLxToolsTaskConfigBuilder, PiscesLxToolsVisualizationConfig)


@pytest.fixture(scope="module")
def model():
    torch.manual_seed(0)
    return YvModelForCausalLM(YvConfig.tiny_text_moe(vocab_size=300)).eval()


@pytest.fixture(scope="module")
def tok():
    return YvTokenizer(use_files=False)


def test_config_builders_and_datasets(tmp_path):
    c = PiscesLxToolsBenchmarkConfig.load({"model_path": "/m/yv-7b", "datasets": ["mmlu"], "temperature": 0.2, "unknown": 1, "generation_config": {"top_k": 5}})
    assert c.model_name == "yv-7b" and c.metrics == ["accuracy"] and c.datasets == ["mmlu"]
    t = PiscesLxToolsTaskConfigBuilder.build(c)
    assert t["model"]["generation_config"]["top_k"] == 5 and t["model"]["generation_config"]["temperature"] == 0.2 and t["datasets"][0]["name"] == "mmlu" and t["metrics"][0]["known"]
    f = tmp_path / "c.json"
    f.write_text(json.dumps({"model_path": "x", "modality": "image"}))
    assert PiscesLxToolsBenchmark.create(str(f)).modality == "image"
    with pytest.raises(ValueError):
        PiscesLxToolsBenchmarkConfig(modality="smell")
    m = PiscesLxMMLUDataset([{"question": "q", "A": "1", "B": "2", "C": "3", "D": "4", "answer": "c"}])
    assert m[0]["choices"] == ["1", "2", "3", "4"] and m[0]["answer"] == 2 and len(m) == 1
    assert PiscesLxGSM8KDataset([{"question": "q", "answer": "work...\n#### 42"}])[0]["answer"] == "42"
    assert PiscesLxHumanEvalDataset([{"task_id": "t/1", "prompt": "def f():"}])[0]["entry_point"] == ""
    assert len(PiscesLxMMLUDataset()) >= 1                                               # the built-in smoke rows


def test_suite_runner_saves_and_compares(model, tok, tmp_path):
    cfg = PiscesLxToolsBenchmarkConfig(model_path="tiny", datasets=["mmlu", "gsm8k"], output_dir=str(tmp_path), max_samples=2)
    runner = PiscesLxToolsBenchmarkRunner(cfg, model_loader=lambda p: model)
    out = runner.run_benchmark(tokenizer=tok)
    assert set(out["results"]) == {"mmlu", "gsm8k"} and out["summary"]["completed"] == 2 and out["summary"]["failed"] == 0
    assert all(0.0 <= r["score"] <= 1.0 and r["seconds"] > 0 for r in out["results"].values())
    saved = PiscesLxToolsResultManager(str(tmp_path)).load_results()
    assert saved["config"]["model_path"] == "tiny" and set(saved["results"]) == {"mmlu", "gsm8k"}
    cmp_ = runner.compare_models([{"name": "a", "model": model, "tokenizer": tok}, {"name": "b", "model_path": "whatever", "tokenizer": tok}])
    rep = cmp_["comparison"]
    assert rep["benchmarks"] == ["gsm8k", "mmlu"] and set(rep["mean_scores"]) == {"a", "b"} and rep["best_model"] in ("a", "b")
    with pytest.raises(ValueError):
        PiscesLxBenchmarkSuite(PiscesLxBenchmarkSuiteConfig(suites=["nope"])).benchmarks()
    bad = PiscesLxBenchmarkSuite(PiscesLxBenchmarkSuiteConfig(suites=["mmlu"])).run(object(), tok)
    assert bad["summary"]["failed"] == 1 and "error" in bad["results"]["mmlu"]


def test_comparison_managers():
    cm = PiscesLxToolsComparisonManager(tolerance=0.01)
    cm.add("v1", {"mmlu": {"score": 0.50}, "gsm8k": {"score": 0.30}})
    cm.add("v2", {"mmlu": {"score": 0.55}, "gsm8k": {"score": 0.20}, "new": {"score": 0.1}})
    d = cm.diff("v1", "v2")
    assert d["regressions"] == ["gsm8k"] and d["improvements"] == ["mmlu"] and d["rows"]["new"]["delta"] is None
    fc = PiscesLxToolsFlagshipComparator(PiscesLxToolsComparisonConfig(model_name="yv"), reference={"big": {"mmlu": 0.9, "gsm8k": 0.8}, "small": {"mmlu": 0.4}})
    r = fc.compare_with_flagship({"mmlu": 0.6, "gsm8k": 0.85})
    assert r["rankings"]["mmlu"] == {"rank": 2, "of": 3, "leader": "big", "leader_score": 0.9} and r["rankings"]["gsm8k"]["rank"] == 1 and r["strengths"] == ["gsm8k"]
    assert abs(r["gaps"]["mmlu"]["gap_to_leader"] - 0.3) < 1e-9 and r["weaknesses"][0] == "mmlu" and "| mmlu | 0.6 | 0.9 | 0.4 |" in fc.generate_comparison_table()
    assert PiscesLxToolsFlagshipComparator().compare_with_flagship({"x": 1.0})["rankings"]["x"]["rank"] == 1      # no table: alone in the field


def test_performance_sweep_on_host(model, tmp_path):
    cfg = PiscesLxToolsPerformanceConfig(output_dir=str(tmp_path), warmup_runs=1, benchmark_runs=3, batch_sizes=[1, 2], sequence_lengths=[16, 32], max_tokens_per_case=48)
    out = PiscesLxToolsPerformanceBenchmarkRunner(model, cfg).run()
    assert [(c["batch_size"], c["sequence_length"]) for c in out["cases"]] == [(1, 16), (1, 32), (2, 16)] and out["timing"] == "host"
    assert all(c["tokens_per_second"] > 0 and c["latency_ms_p95"] >= c["latency_ms_p50"] for c in out["cases"]) and (tmp_path / "performance.json").exists()
    assert out["best_throughput"]["tokens_per_second"] == max(c["tokens_per_second"] for c in out["cases"])


def test_long_context_agent_multimodal_and_swe(tok):
    def oracle(prompt, max_new_tokens=16):
        import re
        m = re.search(r"(?:magic|secret|special)[^0-9]*([0-9]+)", prompt)
        return m.group(1) if m else "0"
    lc = PiscesLxToolsLongContextEvaluator(oracle, tok, PiscesLxToolsLongContextConfig(lengths=(128, 256), depths=(0.0, 1.0))).evaluate()
    assert set(lc.grid) == {"128@0.0", "128@1.0", "256@0.0", "256@1.0"} and 0.0 <= lc.accuracy <= 1.0 and set(lc.by_length) == {128, 256}
    agent = lambda goal, steps: {"answer": goal.upper(), "steps": 2, "tool_errors": 1 if "bad" in goal else 0, "tool_calls": 2}
    ar = PiscesLxToolsAgentBenchmarkRunner(agent).run([{"goal": "ok", "check": lambda a: a == "OK"}, {"goal": "bad", "check": lambda a: a == "nope"}])
    assert ar == {"success_rate": 0.5, "mean_steps": 2.0, "tool_error_rate": 0.25, "n": 2}
    mm = PiscesLxToolsMultimodalBenchmarkRunner(lambda r: "a red cat", PiscesLxToolsMultimodalConfig(modalities=("vision", "audio")))
    out = mm.run({"vision": [{"question": "?", "answers": ["cat"]}, {"question": "?", "answers": ["dog"]}]})
    assert out["per_modality"]["vision"]["accuracy"] == 0.5 and out["per_modality"]["audio"]["n"] == 0 and out["mean_accuracy"] == 0.5
    patch = "--- a/x.py\n+++ b/x.py\n@@ -1,1 +1,1 @@\n-a\n+b\n"
    swe = PiscesLxSWEBenchBenchmark([{"instance_id": "i1", "issue": "bug", "repo_files": ["x.py"]}, {"instance_id": "i2", "issue": "bug"}],
                                    generate=lambda p, n: patch if "bug" in p else "").evaluate()
    assert swe["n"] == 2 and swe["score"] in (0.5, 1.0) and swe["details"][0]["instance_id"] == "i1"


def test_charts_and_reports(tmp_path):
    v = PiscesLxToolsBenchmarkVisualizer(PiscesLxToolsVisualizationConfig(output_dir=str(tmp_path)))
    scores = {"yv": {"mmlu": 0.6, "gsm8k": 0.4, "humaneval": 0.3}, "other <b>": {"mmlu": 0.7, "gsm8k": 0.2}}
    files = [v.plot_radar_chart(scores), v.plot_bar_comparison(scores), v.plot_heatmap({"r1": {"a": 0.1, "b": 0.9}, "r2": {"a": 0.5}}),
             v.plot_line_trend({"loss": [3, 2, 1.5, 1.2], "flat": [1, 1]}), v.plot_needle_haystack_heatmap({"128@0.0": 1.0, "128@1.0": 0.0, "256@0.0": 0.5})]
    for f in files:
        s = open(f).read()
        assert s.startswith("<svg") and s.endswith("</svg>") and "<b>" not in s
    assert "polygon" in open(files[0]).read() and open(files[1]).read().count("<rect") == 6 and "&lt;b&gt;" in open(files[1]).read()
    rg = PiscesLxToolsReportGenerator.create_report_generator(str(tmp_path))
    res = {"mmlu": {"metric": "accuracy", "score": 0.61234, "n": 100}, "needle_x": {"metric": "accuracy", "score": None, "n": 0, "error": "boom"}}
    md = open(rg.generate_markdown_report(res, model="yv-7b")).read()
    assert "| mmlu | accuracy | 0.6123 | 100 |" in md and "Failed: needle_x (boom)" in md and "`yv-7b`" in md
    ht = open(rg.generate_html_report(res, model="yv", figures=files[:1])).read()
    assert "<td>mmlu</td>" in ht and "<svg" in ht
    assert r"needle\_x & accuracy & - & 0 \\" in open(rg.generate_latex_table(res)).read()


def test_cli_and_orchestrator(model, tok, tmp_path):
    assert PiscesLxBenchmarkCli.main(["--list"])["suites"] == ["mmlu", "gsm8k", "aime", "humaneval", "needle"]
    assert isinstance(PiscesLxBenchmarkCli.main(["--selftest"])["selftest"], dict)
    out = PiscesLxBenchmarkCli.main(["--benchmark", "mmlu", "--output-dir", str(tmp_path), "--max-samples", "1", "--report", "--perf", "--generation-config", "top_k=3,x=1"], model, tok)
    assert set(out["results"]) == {"mmlu"} and out["report"].endswith("report.md") and out["performance"]["cases"][0]["sequence_length"] == 128
