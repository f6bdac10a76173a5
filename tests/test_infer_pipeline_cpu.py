"""Inference pipeline / prompt / result operators; request and step monitors, visualiser, phase profiler."""
import json
import time

import pytest

from pisceslx_b200.serve.infer_pipeline import (PiscesLxInferenceMonitorOperator, PiscesLxInferencePipelineOperator, PiscesLxInferenceVisualizer,
                                                PiscesLxPerformanceProfilerOperator, PiscesLxPromptEngineeringOperator, PiscesLxResultProcessorOperator,
                                                PiscesLxSystemResourceMonitor, PiscesLxTrainingMonitorOperator, PiscesLxTrainingVisualizer, percentile)


class _Inf:
    def __init__(self, fail_on=None):
        self.fail_on, self.calls = fail_on, []

    def generate(self, prompt, **kw):
        return f"  echo:{prompt}  "

    def batch_generate(self, prompts, **kw):
        self.calls.append((list(prompts), kw))
        if self.fail_on and any(self.fail_on in p for p in prompts):
            raise RuntimeError("boom")
        return [self.generate(p) for p in prompts]


def test_pipeline_batches_failures_streams_and_async():
    inf = _Inf(fail_on="bad")
    op = PiscesLxInferencePipelineOperator({"batch_size": 2, "generation": {"max_new_tokens": 7}}, inf)
    ev = []
    op.add_callback(lambda stage, **kw: ev.append(stage))
    op.add_callback(lambda stage, **kw: 1 / 0)
    out = op.execute({"prompts": [" a ", "", "b", "bad", "c"]}).output
    assert out["count"] == 4 and out["results"] == ["echo:a", "echo:b", "", ""]           # the batch holding "bad" fails as a whole
    assert inf.calls[0][1]["max_new_tokens"] == 7 and ev.count("batch_failed") == 1 and ev.count("batch_completed") == 1
    assert ev[0] == "preprocessing_start" and ev[-1] == "postprocessing_end" and op.callback_errors
    assert op.transform("x") == "echo:x"
    assert "".join(op.generate_stream("hello", chunk_chars=4)) == "  echo:hello  " and "stream_end" in ev
    got = []
    t = op.async_inference(["q"], callback=lambda r, error=None: got.append((r, error)))
    t.join(5)
    assert got == [(["  echo:q  "], None)]
    with pytest.raises(TypeError):
        PiscesLxInferencePipelineOperator(3.0)
    assert not PiscesLxInferencePipelineOperator().execute({"prompts": ["a"]}).is_success()


def test_prompt_engineering():
    pe = PiscesLxPromptEngineeringOperator()
    assert pe.render_template("qa", question="2+2?") == "Question: 2+2?\nAnswer:"
    assert "3 sentences" in pe.render_template("summarize", text="T") and "in 1 sentences" in pe.render_template("summarize", text="T", n=1)
    with pytest.raises(ValueError):
        pe.render_template("instruct")
    with pytest.raises(KeyError):
        pe.render_template("nope")
    pe.add_template("t", "{a}-{b}", defaults={"b": 2})
    assert pe.execute({"template": "t", "variables": {"a": 1}}).output["prompt"] == "1-2" and pe.templates["t"]["variables"] == ["a", "b"]
    long = "First one. Second one. Third one. Fourth one. What is last?"
    assert pe.optimize_prompt(long) == "First one. Second one. What is last?"
    assert pe.optimize_prompt("a\n b\t c", "clarity") == "a b c" and pe.optimize_prompt("Hi there. hi there. Bye.", "dedupe") == "Hi there. Bye."
    q = pe.analyze_prompt_quality(long)
    assert q["sentence_count"] == 5 and q["clarity_score"] >= 0.9 and q["recommendations"] == []
    bad = pe.analyze_prompt_quality("word " * 200)
    assert any("long" in r for r in bad["recommendations"])
    assert pe.analyze_prompt_quality("")["clarity_score"] == 0.0


def test_result_processor():
    rp = PiscesLxResultProcessorOperator()
    rp.add_processor(str.strip)
    rp.add_processor(lambda s: s[0].upper() + s[1:])
    rp.add_processor(lambda s: s.bogus())                                                # skipped
    assert rp.process_results("  hi ") == "Hi" and rp.process_results([" a", "b "]) == ["A", "B"]
    r = rp.filter_results(["ok", "", "too long here", "spam inside", "ok"], min_length=1, max_length=11, banned_words=["SPAM"], unique=True)
    assert r == ["ok"]
    assert rp.format_results(["x", "y"], "numbered") == "1. x\n2. y" and json.loads(rp.format_results(["x"], "json")) == {"results": ["x"], "count": 1}
    out = rp.execute({"results": [" a ", " a ", " bb "], "filter": {"unique": True}, "format": "dict"}).output
    assert out["results"] == {"results": ["A", "Bb"], "count": 2}
    with pytest.raises(ValueError):
        rp.format_results([], "xml")


def test_percentile():
    assert percentile([], 50) == 0.0 and percentile([1, 2, 3, 4], 50) == 2.5 and percentile([5], 99) == 5 and percentile([1, 2, 3], 100) == 3


class _Res:
    def __init__(self, mem=10.0):
        self.mem = mem

    def get_system_metrics(self):
        return {"memory_percent": self.mem, "gpu_memory_percent": 5.0}


def test_inference_monitor_summary_anomalies_and_log(tmp_path):
    res = _Res()
    m = PiscesLxInferenceMonitorOperator(log_dir=str(tmp_path), save_interval=10, history=50, resources=res)
    for i in range(10):
        assert m.record_inference_request({"latency": 0.1, "tokens_generated": 20}) == []
    assert (tmp_path / "inference_metrics.json").exists()
    s = m.get_realtime_metrics()
    assert s["request_count"] == 10 and abs(s["latency_p50"] - 0.1) < 1e-9 and abs(s["throughput_mean"] - 200) < 1e-6 and s["tokens_total"] == 200
    spike = m.record_inference_request({"latency": 1.0, "tokens_generated": 20})
    assert [a["type"] for a in spike] == ["latency_spike"]
    res.mem = 95.0
    assert "high_memory_usage" in [a["type"] for a in m.record_inference_request({"latency": 0.1})]
    res.mem = 10.0
    for i in range(100):
        m.record_inference_request({"latency": 0.1, "success": i % 10 != 0})
    assert "high_error_rate" in [a["type"] for a in m.detect_anomalies()] and len(m.metrics_history["latency"]) == 50
    out = m.execute({}).output
    assert out["summary"]["error_count"] == 10 and len(out["anomalies"]) >= 3
    assert isinstance(PiscesLxSystemResourceMonitor().get_system_metrics(), dict)


def test_training_monitor_anomalies(tmp_path):
    m = PiscesLxTrainingMonitorOperator(log_dir=str(tmp_path), save_interval=0)
    for i in range(12):
        assert m.record_training_step({"loss": 2.0 - 0.01 * i, "grad_norm": 1.0, "throughput": 1000.0, "step_time": 0.5, "learning_rate": 1e-4}) == []
    assert [a["type"] for a in m.record_training_step({"loss": 5.0, "grad_norm": 1.0, "throughput": 1000.0})] == ["loss_spike"]
    assert [a["type"] for a in m.record_training_step({"loss": 1.8, "grad_norm": 50.0, "throughput": 1000.0})] == ["gradient_explosion"]
    assert [a["type"] for a in m.record_training_step({"loss": 1.8, "grad_norm": 1.0, "throughput": 100.0})] == ["throughput_drop"]
    assert "non_finite_loss" in [a["type"] for a in m.record_training_step({"loss": float("nan"), "grad_norm": 1.0, "throughput": 1000.0})]
    s = m.execute({}).output["summary"]
    assert s["steps"] == 16 and s["anomaly_count"] == 4 and s["step_time_p50"] >= 0


def test_visualizer_writes_svg(tmp_path):
    v = PiscesLxInferenceVisualizer(tmp_path)
    files = v.generate_plots({"latency": [0.1, 0.2, float("nan"), 0.15], "timestamps": [1, 2, 3, 4], "one": [1.0], "flat": [2.0] * 5000})
    assert sorted(f.rsplit("/", 1)[-1] for f in files) == ["flat.svg", "latency.svg"]
    svg = (tmp_path / "latency.svg").read_text()
    assert svg.startswith("<svg") and "polyline" in svg and "nan" not in svg and svg.count(",") >= 3
    assert (tmp_path / "flat.svg").read_text().count(",") <= 2001 and PiscesLxTrainingVisualizer is PiscesLxInferenceVisualizer


def test_phase_profiler_on_host():
    p = PiscesLxPerformanceProfilerOperator(profile_interval=2, use_cuda_events=False)
    for _ in range(2):
        p.start_request_profile()
        time.sleep(0.002)
        p.record_tokenization_time()
        p.record_forward_start()
        time.sleep(0.01)
        p.record_forward_end()
        time.sleep(0.002)
        p.record_decoding_time()
        r = p.end_request_profile(tokens_generated=10)
    assert set(r) == {"tokenization", "pre_forward", "forward", "decoding", "total"} and r["forward"] > r["tokenization"]
    assert abs(sum(v for k, v in r.items() if k != "total") - r["total"]) < 2e-3
    rep = p.last_report
    assert rep["count"] == 2 and rep["bottleneck"] == "forward" and rep["tokens_per_second"] > 0 and 0.3 < rep["phases"]["forward"]["share"] < 1.0
    p.start_step_profile()
    p.record_forward_time()
    p.record_backward_time()
    p.record_optimizer_time()
    assert set(p.end_step_profile()) == {"forward", "backward", "optimizer", "total"}
    assert p.end_request_profile() == {} and p.execute({}).output["count"] == 3
