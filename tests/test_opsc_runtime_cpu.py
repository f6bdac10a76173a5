"""CPU tests of the operator runtime extras: base / transform / filter operators, pipeline core, schedulers, memory
pool, estimator, offload manager, load balancer, parallel operators."""
from __future__ import annotations

import torch
import torch.nn as nn

from pisceslx_b200.utils import opsc_runtime as R


def test_base_operators_hub_and_pipeline_core():
    hub = R.PiscesLxOperatorRegistryHub()

    @hub.registrar("data/double")
    class Double(R.PiscesLxBaseOperator):
        def run(self, inputs):
            return {**inputs, "data": [2 * x for x in inputs["data"]]}
    hub.register("data/keep_big", lambda: R.PiscesLxFilterOperator(lambda v: v > 4))
    assert hub.namespace("data") == ["data/double", "data/keep_big"] and hub.namespace("train") == []
    core = R.PiscesLxOperatorCore(hub)
    out, ctx = core.run_pipeline(["data/double", R.PiscesLxTransformOperator(lambda d: d + [100]), "data/keep_big"], {"data": [1, 2, 3]})
    assert out["data"] == [6, 100] and [t[1] for t in ctx.trace] == ["SUCCESS"] * 3

    class Flaky(R.PiscesLxBaseOperator):
        def run(self, inputs):
            if self.calls < 2:
                raise RuntimeError("not yet")
            return {"ok": True}
    fl = Flaky(R.PiscesLxOperatorConfig("flaky", retries=3))
    assert fl.execute({}).is_success() and fl.calls == 3
    bad, ctx2 = core.run_pipeline([Flaky(R.PiscesLxOperatorConfig("fails")), "data/double"], {"data": [1]})
    assert ctx2.trace == [("fails", "FAILED", ctx2.trace[0][2])] and "not yet" in ctx2.shared["error"] and bad == {"data": [1]}


def test_streams_events_scheduler_and_gpu_placement():
    a, b = R.PiscesLxCUDAEvent(), R.PiscesLxCUDAEvent()
    a.record()
    with R.PiscesLxCUDAStream() as s:
        x = torch.ones(4).sum()
    b.record(s)
    assert float(x) == 4 and a.elapsed_ms(b) >= 0
    sch = R.PiscesLxCUDAScheduler(n_streams=2)
    sch.submit(lambda: "low", R.PiscesLxAllocationPriority.LOW, "low")
    sch.submit(lambda: "high", R.PiscesLxAllocationPriority.HIGH, "high")
    sch.submit(lambda: "normal", name="normal")
    assert sch.run_all() == ["low", "high", "normal"] and sch.last_order == ["high", "normal", "low"]
    loads = [R.PiscesLxDeviceLoad(0, 0.9, 80), R.PiscesLxDeviceLoad(1, 0.2, 10), R.PiscesLxDeviceLoad(2, 0.25, 10)]
    gs = R.PiscesLxGPUScheduler(lambda: [R.PiscesLxDeviceLoad(l.index, l.memory_used_frac, l.utilization) for l in loads])
    assert gs.place("t1") == 1 and gs.place("t2") == 2 and gs.place("t3", min_free_frac=0.95) is None
    gs.release("t1")
    assert gs.place("t4") == 1


def test_memory_pool_and_resource_estimator():
    pool = R.PiscesLxMemoryPool(max_cached_bytes=1 << 20)
    t = pool.get(1000)
    assert t.shape == (1000,) and pool.misses == 1
    pool.put(t)
    u = pool.get(700)                                       # 700 and 1000 share the 1024 bucket
    assert pool.hits == 1 and u.shape == (700,) and u.data_ptr() == t.data_ptr()
    pool.put(u)
    big = pool.get(1 << 19)                                 # 2 MB: larger than the cache limit, not kept
    pool.put(big)
    assert pool.cached_bytes == 4096
    net = nn.Linear(10, 10)
    est = R.PiscesLxResourceEstimator.module_bytes(net, training=True)
    assert est["parameters"] == 440 and est["gradients"] == 440 and est["optimizer"] == 880 and est["total"] == 1760
    assert R.PiscesLxResourceEstimator.module_bytes(net, training=False)["total"] == 440
    assert R.PiscesLxResourceEstimator.tensor_bytes((2, 4096, 4096)) == 2 * 4096 * 4096 * 2
    req = R.PiscesLxResourceRequest(R.PiscesLxResourceType.GPU_MEMORY, 1e9, R.PiscesLxAllocationPriority.HIGH)
    assert R.PiscesLxResourceAllocation(req, 1e9, device=0).request.priority == 2


def test_offload_manager_load_balancer_and_heterogeneous_executor():
    torch.manual_seed(0)
    layers = [nn.Linear(8, 8) for _ in range(4)]
    ref = nn.Sequential(*layers)
    x = torch.randn(3, 8)
    want = ref(x)
    off = R.PiscesLxOffloadManager(layers, "cpu", R.PiscesLxHeterogeneousConfig(prefetch=1, pin_host=False))
    assert torch.allclose(off.run(x), want) and off.moves == 4 and off.resident == []
    lb = R.PiscesLxLoadBalancer(["gpu", "cpu"], ema=0.0)
    assert lb.split(10) == {"gpu": 5, "cpu": 5}
    lb.observe("gpu", 90, 1.0); lb.observe("cpu", 10, 1.0)
    assert lb.split(10) == {"gpu": 9, "cpu": 1} and sum(lb.split(7).values()) == 7
    calls = []
    ex = R.PiscesLxHeterogeneousExecutor(lambda chunk, target: calls.append((target, len(chunk))) or chunk * 2)
    out = ex.run(torch.arange(6.0).view(6, 1))
    assert torch.equal(out, torch.arange(6.0).view(6, 1) * 2) and sum(n for _, n in calls) == 6


def test_parallel_operators_single_process():
    net = nn.Linear(4, 4)
    net(torch.randn(2, 4)).sum().backward()
    g0 = net.weight.grad.clone()
    dp = R.PiscesLxDataParallelOperator()
    r = dp.execute({"parameters": list(net.parameters())})
    assert r.is_success() and r.output == {"reduced_tensors": 2, "world": 1} and torch.allclose(net.weight.grad, g0)
    assert dp.stats.calls == {"all_reduce": 1} and dp.stats.total_bytes() == 20 * 4
    pp = R.PiscesLxPipelineParallelOperator().execute({"stages": [lambda t: t + 1, lambda t: t * 2], "micro_batches": [torch.zeros(2), torch.ones(2)]})
    assert [o.tolist() for o in pp.output["outputs"]] == [[2.0, 2.0], [4.0, 4.0]] and abs(pp.output["bubble_fraction"] - 1 / 3) < 1e-9
    x = torch.arange(12.0).view(6, 2)
    idx = torch.tensor([2, 0, 1, 0, 2, 2])
    ep = R.PiscesLxExpertParallelOperator().execute({"tokens": x, "expert_idx": idx, "experts": [lambda t: t + 10, lambda t: t + 20, lambda t: t + 30]})
    want = x + torch.tensor([30.0, 10, 20, 10, 30, 30])[:, None]
    assert torch.equal(ep.output["output"], want) and ep.output["tokens_per_expert"] == [2, 1, 3]
    hy = R.PiscesLxHybridParallelOperator(R.PiscesLxParallelConfig(R.PiscesLxParallelismType.HYBRID)).execute({"device": torch.device("cpu")})
    assert hy.is_success() and hy.output["world"] == 1 and hy.output["dp"] == 1
