"""Monitor helpers: TTL cache, dotted configuration, context with hooks, utilities."""
from pisceslx_b200.tools.monitor_tool import (PiscesLxCoreConfigManager, PiscesLxCoreEnhancedCacheManager, PiscesLxMonitorCache, PiscesLxMonitorContext,
                                              PiscesLxMonitorContextManager, PiscesLxMonitorUtils)


def test_cache_ttl_and_dirs(tmp_path):
    t = [0.0]
    c = PiscesLxMonitorCache(str(tmp_path), clock=lambda: t[0])
    c.set("a", 1)
    c.set("b", 2, ttl=5)
    t[0] = 4.9
    assert c.get("b") == 2
    t[0] = 5.0
    assert c.get("b") is None and c.get("a") == 1 and c.get("x", 7) == 7 and len(c) == 1
    assert c.get_cache_dir("gpu").startswith(str(tmp_path))
    e = PiscesLxCoreEnhancedCacheManager(str(tmp_path), clock=lambda: t[0])
    e.set("k", "v")
    t[0] = 304.0
    assert e.get("k") == "v"
    t[0] = 306.0
    assert e.get("k") is None


def test_config_context_and_utils():
    cfg = PiscesLxCoreConfigManager({"alerts": {"gpu": {"temp": 85}}})
    cfg.set("alerts.gpu.mem", 0.9)
    assert cfg.get("alerts.gpu.temp") == 85 and cfg.get("alerts.gpu.mem") == 0.9 and cfg.get("alerts.cpu.x", "d") == "d"
    ctx = PiscesLxMonitorContext()
    seen = []
    ctx.add_hook(lambda ev, d: seen.append((ev, d)))
    ctx.add_hook(lambda ev, d: 1 / 0)
    ctx.set_context("run", 3)
    assert ctx.get_context("run") == 3 and ctx.emit_event("tick", {"a": 1}, b=2) == 1 and seen == [("tick", {"a": 1, "b": 2})] and len(ctx.hook_errors) == 1
    sentinel = object()
    m = PiscesLxMonitorContextManager()
    m.set_utils(device_manager=sentinel, fs_manager="fs")
    assert m.get_device_manager() is sentinel and m.get_fs_manager() == "fs" and m.PiscesLxLogger().name == "PiscesLx.Tools.Monitor"
    u = PiscesLxMonitorUtils(system_monitor=sentinel)
    assert u.get_device_manager() is sentinel and isinstance(u.get_cache_manager(), PiscesLxMonitorCache) and u.get_fs_manager() is not None
