"""CPU tests of the quantisation engine and pipeline."""
from __future__ import annotations

import torch
import torch.nn as nn

from pisceslx_b200.quant.pipeline import (PiscesLxActivationCollectorOperator, PiscesLxAdaptiveBitAllocationOperator,
                                          PiscesLxCalibrationDataLoaderOperator, PiscesLxMemoryProfiler,
                                          PiscesLxQuantizationBenchmark, PiscesLxQuantizationConfig,
                                          PiscesLxQuantizationEngine, PiscesLxQuantizationEvaluator,
                                          PiscesLxQuantizationMethod, PiscesLxQuantizationOperatorFactory,
                                          PiscesLxQuantizationPipelineOperator, PiscesLxSensitivityAnalysisOperator)


def make():
    torch.manual_seed(0)
    net = nn.Sequential()
    net.add_module("fc1", nn.Linear(64, 128))
    net.add_module("act", nn.GELU())
    net.add_module("fc2", nn.Linear(128, 64))
    net.add_module("lm_head", nn.Linear(64, 32))
    return net


def data(n, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, 16, 64, generator=g)
    x[..., 3] *= 12.0                                        # an outlier channel, as activations have
    return list(x)


def test_collector_loader_sensitivity_and_bit_allocation():
    net = make()
    acts = PiscesLxActivationCollectorOperator().run({"model": net, "batches": data(4, 1)})
    assert set(acts) == {"fc1", "fc2", "lm_head"} and acts["fc1"].shape == (64, 64) and acts["fc2"].shape == (64, 128)
    ld = PiscesLxCalibrationDataLoaderOperator().run({"token_ids": torch.arange(1000), "seq_len": 16, "batch": 4})
    assert len(ld) == 15 and ld[0].shape == (4, 16) and int(ld[1][0, 0]) == 64
    sens = PiscesLxSensitivityAnalysisOperator(bits=3, group_size=32).run({"model": net, "activations": acts})
    assert all(0 < v < 1 for v in sens.values())
    alloc = PiscesLxAdaptiveBitAllocationOperator((2, 4, 8)).run(
        {"sensitivity": {"a": 0.9, "b": 0.01, "c": 0.02}, "sizes": {"a": 100, "b": 100, "c": 100}, "target_bits": 4.0})
    assert alloc == {"a": 8, "b": 2, "c": 2}                 # one very sensitive layer takes the whole budget
    even = PiscesLxAdaptiveBitAllocationOperator((2, 4, 8)).run(
        {"sensitivity": {"a": 0.9, "b": 0.1, "c": 0.5}, "sizes": {"a": 100, "b": 100, "c": 100}, "target_bits": 4.0})
    assert even == {"a": 4, "b": 4, "c": 4}                  # comparable layers: spreading the bits loses least


def test_engine_methods_and_evaluator():
    held = data(3, 9)
    errs = {}
    for method in ("rtn", "gptq", "awq", "smoothquant"):
        fp, q = make(), make()
        from pisceslx_b200.quant.pipeline import PiscesLxCalibrationConfig
        acts = PiscesLxActivationCollectorOperator(PiscesLxCalibrationConfig(n_batches=48)).run({"model": fp, "batches": data(48, 2)})
        res = PiscesLxQuantizationEngine(PiscesLxQuantizationConfig(PiscesLxQuantizationMethod(method), bits=4, group_size=32)).quantize(q, acts)
        assert res.layers == 2 and res.mean_bits == 4.0 and "lm_head" not in res.weight_error
        assert torch.equal(q.lm_head.weight, fp.lm_head.weight) and not torch.equal(q.fc1.weight, fp.fc1.weight)
        ev = PiscesLxQuantizationEvaluator.compare(fp, q, held)
        errs[method] = ev["relative_error"]
        assert ev["relative_error"] < 0.2 and ev["top1_agreement"] > 0.7 and ev["batches"] == 3
    assert errs["gptq"] < errs["rtn"] and errs["awq"] <= errs["rtn"] * 1.05     # calibrated methods do not lose to rounding
    assert type(PiscesLxQuantizationOperatorFactory.create("gptq")).__name__ == "PiscesLxGPTQOperator"
    full = PiscesLxMemoryProfiler.weight_bytes(make())["bytes"]
    q4 = PiscesLxMemoryProfiler.weight_bytes(make(), {"fc1": 4, "fc2": 4})["bytes"]
    assert q4 < 0.45 * full


def test_pipeline_with_bit_allocation_and_benchmark_table():
    net = make()
    rep = PiscesLxQuantizationPipelineOperator().execute(
        {"model": net, "calibration": data(4, 3), "config": PiscesLxQuantizationConfig(bits=4, group_size=32), "target_bits": 4.0})
    assert rep.is_success(), rep.error
    out = rep.output
    assert out["layers"] == 2 and set(out["bits"]) == {"fc1", "fc2"} and 2.0 <= out["mean_bits"] <= 8.0
    assert not PiscesLxQuantizationPipelineOperator().execute({"model": net}).is_success()
    table = PiscesLxQuantizationBenchmark(make, data(4, 4), data(2, 5)).run([("rtn", 8), ("rtn", 3), ("gptq", 3)])
    assert [r.method for r in table] == ["rtn", "rtn", "gptq"]
    assert table[0].relative_error < table[1].relative_error and table[2].relative_error < table[1].relative_error
    assert table[0].weight_mb > table[1].weight_mb
