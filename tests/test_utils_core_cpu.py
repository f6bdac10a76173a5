"""Application kit: errors, configuration, filesystem, token budgets, templates, LLM client, batch processor, lifecycle,
devices and resource pool, system metrics."""
import asyncio
import json
import types

import pytest

from pisceslx_b200.utils import core as C


def test_errors_carry_code_and_context():
    e = C.PiscesLxCoreTimeoutError("too slow", C.PiscesLxCoreErrorContext("engine", "decode", request_id="r1"))
    assert isinstance(e, C.PiscesLxCoreError) and e.code is C.PiscesLxCoreErrorCode.TIMEOUT_ERROR
    assert str(e) == "[P-008] too slow" and e.to_dict()["context"]["request_id"] == "r1"
    assert C.PiscesLxCoreError().code.id == "P-001" and C.PiscesLxCoreValidationError().message == "Validation error"
    with pytest.raises(C.PiscesLxCoreError):
        raise C.PiscesLxCoreMemoryError()


def test_configuration_layers(tmp_path):
    cfg = C.PiscesLxConfiguration({"train": {"lr": 1e-3, "steps": 10}})
    f = tmp_path / "c.json"
    f.write_text(json.dumps({"train": {"steps": 20}, "name": "run"}))
    cfg.load_from_file(str(f))
    y = tmp_path / "c.yaml"
    y.write_text("serve:\n  port: 8000\n")
    cfg.load_from_file(str(y))
    n = cfg.load_from_env("PX_", {"PX_TRAIN__LR": "0.01", "PX_DEBUG": "true", "OTHER": "1", "PX_TAG": "abc"})
    assert n == 3 and cfg.get("train.lr") == 0.01 and cfg.get("train.steps") == 20 and cfg.get("serve.port") == 8000
    assert cfg.get_bool("debug") and cfg.get("tag") == "abc" and cfg.get("missing.key", 7) == 7
    cfg.set("a.b.c", "5")
    assert cfg.get_int("a.b.c") == 5 and cfg.get_float("train.lr") == 0.01 and cfg.to_dict()["a"]["b"]["c"] == "5"
    bad = tmp_path / "bad.json"
    bad.write_text("{nope")
    with pytest.raises(C.PiscesLxCoreError) as ei:
        cfg.load_from_file(str(bad))
    assert ei.value.code is C.PiscesLxCoreErrorCode.CONFIG_PARSE_ERROR


def test_filesystem_is_confined_and_atomic(tmp_path):
    fs = C.PiscesLxFilesystem(str(tmp_path))
    fs.write("a/b.txt", "hello")
    fs.write_bytes("a/c.bin", b"\x00\x01")
    assert fs.read("a/b.txt") == "hello" and fs.read_bytes("a/c.bin") == b"\x00\x01" and fs.list_dir("a") == ["b.txt", "c.bin"]
    assert fs.exists("a/b.txt") and fs.delete("a/b.txt") and not fs.exists("a/b.txt") and not fs.delete("a/b.txt")
    fs.mkdir("d/e")
    assert fs.delete("d") and not fs.exists("d")
    with pytest.raises(C.PiscesLxCoreError):
        fs.read("../outside.txt")
    with pytest.raises(C.PiscesLxCoreError):
        fs.write("/etc/x", "no")
    assert not [p for p in (tmp_path / "a").iterdir() if p.name.startswith(".tmp_")]


def test_context_ids_and_error_logging(tmp_path):
    ctx = C.PiscesLxCoreContext.create("svc", base_path=str(tmp_path))
    ctx.set_request_id("r9")
    ctx.set_correlation_id("c1")
    ec = ctx.error_context("x", "y", k=1)
    assert (ec.request_id, ec.correlation_id, ec.details) == ("r9", "c1", {"k": 1})
    assert ctx.metrics is C.PiscesLxCoreContext("other").metrics
    with pytest.raises(ValueError):
        with ctx:
            raise ValueError("boom")

    async def use():
        async with ctx as c:
            return c.get_request_id()
    assert asyncio.run(use()) == "r9"


def test_token_manager_limits_and_truncation():
    tm = C.PiscesLxTokenManager(limits={"m": 5})
    assert tm.count_tokens("abcdefgh") == 2 and tm.count_tokens("今天天气") == 4 and tm.get_limit("other") == -1
    assert tm.is_within_limit("x" * 20, "m") and not tm.is_within_limit("x" * 21, "m") and tm.is_within_limit("x" * 999, "other")
    assert tm.truncate("x" * 50, "m") == "x" * 20 and tm.truncate("short", "m") == "short"
    with pytest.raises(C.PiscesLxCoreError) as ei:
        tm.require("x" * 40, "m")
    assert ei.value.code is C.PiscesLxCoreErrorCode.TOKEN_LIMIT_EXCEEDED
    exact = C.PiscesLxTokenManager(counter=lambda t: len(t.split()))
    assert exact.count_tokens("a b c") == 3


def test_prompt_template():
    t = C.PiscesLxPromptTemplate("Hello {name}, you are {age}. {{literal}} {name}!")
    assert t.get_variables() == ["name", "age"]
    assert t.render(name="Ann", age=3) == "Hello Ann, you are 3. {literal} Ann!"
    assert t.render(name="Ann") == "Hello Ann, you are {age}. {{literal}} Ann!"
    with pytest.raises(C.PiscesLxCoreError):
        t.render(strict=True, name="Ann")
    p = t.partial(name="{x}")
    assert p.get_variables() == ["age"] and p.render(age=1) == "Hello {x}, you are 1. {literal} {x}!"


def test_llm_client_sync_async_stream_and_failures():
    tm = C.PiscesLxTokenManager(limits={"pisces": 10})

    def backend(prompt, max_tokens=None, temperature=0.7, stream=False, **kw):
        if stream:
            return iter(["a", "b", "c"])
        if "fail" in prompt:
            raise RuntimeError("down")
        return "x" * 8

    cl = C.PiscesLxLLMClient(backend=backend, token_manager=tm)
    r = asyncio.run(cl.generate("hi there", max_tokens=2))
    assert r.content == "x" * 8 and r.finish_reason == "length" and r.metadata == {"prompt_tokens": 2, "completion_tokens": 2}
    assert r.token_count == 4 and r.duration_ms >= 0

    async def agen(prompt, **kw):
        return "async ok"
    assert asyncio.run(C.PiscesLxLLMClient(backend=agen).generate("q")).content == "async ok"

    async def collect():
        return [p async for p in cl.generate_stream("hi")]
    assert asyncio.run(collect()) == ["a", "b", "c"]
    with pytest.raises(C.PiscesLxCoreError) as e1:
        asyncio.run(cl.generate("fail"))
    assert e1.value.code is C.PiscesLxCoreErrorCode.LLM_REQUEST_FAILED
    with pytest.raises(C.PiscesLxCoreError) as e2:
        asyncio.run(cl.generate("y" * 100))
    assert e2.value.code is C.PiscesLxCoreErrorCode.TOKEN_LIMIT_EXCEEDED
    with pytest.raises(C.PiscesLxCoreError) as e3:
        asyncio.run(C.PiscesLxLLMClient().generate("q"))
    assert e3.value.code is C.PiscesLxCoreErrorCode.SERVICE_UNAVAILABLE


def test_batch_processor_bounds_concurrency_and_keeps_order():
    live = {"now": 0, "max": 0}

    async def work(i):
        live["now"] += 1
        live["max"] = max(live["max"], live["now"])
        await asyncio.sleep(0.01)
        live["now"] -= 1
        if i == 3:
            raise ValueError("three")
        return i * i

    bp = C.PiscesLxBatchProcessor(max_concurrent=2, timeout=1.0)
    out = bp.run(list(range(6)), work, return_exceptions=True)
    assert out[:3] == [0, 1, 4] and isinstance(out[3], ValueError) and out[4:] == [16, 25] and live["max"] == 2

    async def slow(i):
        await asyncio.sleep(0.2)
    res = C.PiscesLxBatchProcessor(timeout=0.02).run([1], slow, return_exceptions=True)
    assert isinstance(res[0], C.PiscesLxCoreTimeoutError)


def test_application_lifecycle_order_hooks_and_failures():
    log = []

    class M(C.PiscesLxServiceModule):
        def on_init(self, ctx): log.append(("init", self.name()))
        def on_start(self, ctx): log.append(("start", self.name()))
        def on_shutdown(self, ctx): log.append(("stop", self.name()))

    class AM(C.PiscesLxAsyncServiceModule):
        async def on_start(self, ctx): log.append(("start", self.name()))

    class Broken(C.PiscesLxServiceModule):
        def on_init(self, ctx): raise RuntimeError("nope")

    app = C.PiscesLxApplication("app")
    app.add(M("api", dependencies=["engine"])).add(M("engine", priority=5)).add(AM("metrics", priority=9))
    app.add(Broken("optional", critical=False)).add(M("needs_optional", dependencies=["optional"]))
    app.hooks.on_before_init(lambda ctx: log.append(("hook", "before_init")))

    async def after_start(ctx):
        log.append(("hook", "after_start"))
    app.hooks.on_after_start(after_start)
    assert app.order() == ["metrics", "engine", "api", "optional", "needs_optional"]
    asyncio.run(app.start())
    assert log[0] == ("hook", "before_init") and log[-1] == ("hook", "after_start")
    assert [n for k, n in log if k == "init"] == ["engine", "api"]
    assert [n for k, n in log if k == "start"] == ["metrics", "engine", "api"]
    assert set(app.failed) == {"optional", "needs_optional"}
    asyncio.run(app.shutdown())
    assert [n for k, n in log if k == "stop"] == ["api", "engine"]
    cyc = C.PiscesLxApplication().add(M("a", dependencies=["b"])).add(M("b", dependencies=["a"]))
    with pytest.raises(C.PiscesLxCoreError):
        cyc.order()
    crit = C.PiscesLxApplication().add(Broken("must"))
    with pytest.raises(RuntimeError):
        asyncio.run(crit.start())


def _dev(i, mem, status=C.PiscesLxDeviceStatus.AVAILABLE, temp=40.0):
    d = C.PiscesLxDevice(f"gpu:{i}", C.PiscesLxDeviceType.GPU)
    d.set_capabilities(C.PiscesLxDeviceCapabilities(compute_units=148, memory_gb=mem))
    d.set_health_metrics(C.PiscesLxDeviceHealthMetrics(temperature_celsius=temp))
    d.set_status(status)
    return d


def test_devices_health_and_pool_allocation():
    hm = C.PiscesLxDeviceHealthMetrics(cpu_usage_percent=100, memory_usage_percent=100, temperature_celsius=100, error_count=10)
    assert hm.health_score == 100 - 10 - 10 - 9 - 30 and not hm.is_healthy
    pool = C.PiscesLxResourcePool("p")
    for d in (_dev(0, 180), _dev(1, 180, temp=95.0), _dev(2, 80), _dev(3, 180, C.PiscesLxDeviceStatus.OFFLINE)):
        pool.add_device(d)
    need = C.PiscesLxDeviceCapabilities(memory_gb=100)
    a = pool.allocate("job1", need, C.PiscesLxDeviceType.GPU)
    b = pool.allocate("job2", need)
    assert a.id == "gpu:0" and b.id == "gpu:1" and pool.allocate("job3", need) is None and pool.owner_of("gpu:0") == "job1"
    st = pool.get_status()
    assert (st.total_devices, st.available_devices, st.allocated_devices) == (4, 1, 2)
    assert st.utilization_percent == pytest.approx(75.0) and st.status_distribution["offline"] == 1 and pool.is_healthy()
    assert pool.release("gpu:0") and not pool.release("gpu:0") and pool.allocate("job3", need).id == "gpu:0"
    stats = pool.get_statistics()
    assert stats.offline_devices == 1 and stats.total_memory_gb == 620 and stats.total_compute_units == 4 * 148
    assert pool.remove_device("gpu:2") and pool.get_device("gpu:2") is None
    assert not C.PiscesLxDeviceCapabilities(custom={"nvlink": 1}).meets_requirements(C.PiscesLxDeviceCapabilities(custom={"nvlink": 2}))
    assert C.PiscesLxConnectionPoolStatistics(total_successful_ops=3, total_failed_ops=1).success_rate == 0.75


def test_pool_from_a_fake_nvml():
    mem = types.SimpleNamespace(total=180 * 2 ** 30, used=18 * 2 ** 30)
    calls = []
    nvml = types.SimpleNamespace(
        nvmlInit=lambda: calls.append("init"), nvmlShutdown=lambda: calls.append("shutdown"), nvmlDeviceGetCount=lambda: 2,
        nvmlDeviceGetHandleByIndex=lambda i: i, nvmlDeviceGetName=lambda h: b"NVIDIA B200",
        nvmlDeviceGetMemoryInfo=lambda h: mem, nvmlDeviceGetNumGpuCores=lambda h: 148 * 128,
        nvmlDeviceGetTemperature=lambda h, k: 55, nvmlDeviceGetUtilizationRates=lambda h: types.SimpleNamespace(gpu=30))
    pool = C.PiscesLxResourcePool.from_local_gpus(nvml=nvml)
    d = pool.get_device("gpu:1")
    assert len(pool.get_all_devices()) == 2 and d.name == "NVIDIA B200" and d.capabilities.compute_units == 148
    assert d.capabilities.memory_gb == 180 and d.health_metrics.memory_usage_percent == pytest.approx(10.0) and d.is_available
    assert calls == ["init", "shutdown"]
    broken = types.SimpleNamespace(nvmlInit=lambda: (_ for _ in ()).throw(RuntimeError("no driver")))
    assert C.PiscesLxResourcePool.from_local_gpus(nvml=broken).get_all_devices() == []


def test_system_metrics_sample():
    a = C.PiscesLxSystemMetrics.collect()
    b = C.PiscesLxSystemMetrics.collect(previous=a)
    assert 0 <= a.memory_usage_percent <= 100 and 0 <= a.disk_usage_percent <= 100 and a.cpu_usage_percent >= 0
    d = b.to_dict()
    assert set(d) == {"timestamp", "cpu", "memory", "disk", "network"} and d["memory"]["total_bytes"] > 0
