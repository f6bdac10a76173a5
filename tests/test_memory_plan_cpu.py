"""The recompute planner's arithmetic, driven by a fake CUDA memory model (no GPU needed)."""
import types

import torch

from pisceslx_b200.engine.memory_plan import YvRecomputePlanner

GIB = 2 ** 30


class _Layer:
    def __init__(self):
        self.use_recompute, self.measure_stored, self.stored_bytes = True, False, 0


def _planner(monkeypatch, n_layers, total_gib, peak_all_recompute_gib, layer_gib, outside_gib=0.0, budget=0.95):
    layers = [_Layer() for _ in range(n_layers)]
    model = types.SimpleNamespace(model=types.SimpleNamespace(layers=layers))
    state = {"peak": 0}

    def peak_now():
        stored = sum(1 for l in layers if not l.use_recompute)
        return int((peak_all_recompute_gib + stored * layer_gib) * GIB)
    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda d: types.SimpleNamespace(total_memory=int(total_gib * GIB)))
    monkeypatch.setattr(torch.cuda, "reset_peak_memory_stats", lambda d=None: None)
    monkeypatch.setattr(torch.cuda, "max_memory_allocated", lambda d=None: peak_now())
    monkeypatch.setattr(torch.cuda, "memory_reserved", lambda d=None: peak_now())
    monkeypatch.setattr(torch.cuda, "mem_get_info",
                        lambda d=None: (int(total_gib * GIB) - peak_now() - int(outside_gib * GIB), int(total_gib * GIB)))
    p = YvRecomputePlanner(model, torch.device("cuda", 0), budget=budget)
    return p, layers


def _run_steps(p, layers, layer_gib):
    for _ in range(3):
        p.before_step()
        if layers[-1].measure_stored:
            layers[-1].stored_bytes = int(layer_gib * GIB)        # what the block reports after its measured forward
        p.after_step()


def test_planner_stores_as_many_layers_as_fit(monkeypatch):
    # 180 GiB device, 120 GiB with everything recomputed, 2 GiB per stored layer: limit 171 -> (171 - 122) // 2 - 1 = 23 more
    p, layers = _planner(monkeypatch, 32, 180, 120, 2.0)
    _run_steps(p, layers, 2.0)
    assert p.stage == 3 and p.stored_layers == 24 and p.layer_bytes == 2 * GIB
    assert [l.use_recompute for l in layers] == [True] * 8 + [False] * 24           # counted from the last layer
    assert "24/32 layers keep their activations (2.00 GiB each" in p.summary()


def test_planner_caps_at_the_layer_count_and_respects_outside_memory(monkeypatch):
    p, layers = _planner(monkeypatch, 8, 180, 40, 1.0)
    _run_steps(p, layers, 1.0)
    assert p.stored_layers == 8 and not any(l.use_recompute for l in layers)
    # 30 GiB held outside the allocator (symmetric heaps, NCCL): limit 171 - 30 = 141 -> (141 - 122) // 2 - 1 = 8 more
    p2, layers2 = _planner(monkeypatch, 32, 180, 120, 2.0, outside_gib=30)
    _run_steps(p2, layers2, 2.0)
    assert p2.stored_layers == 9


def test_planner_keeps_full_recompute_without_headroom(monkeypatch):
    p, layers = _planner(monkeypatch, 32, 180, 168, 2.0)          # 171 - 168 = 3 GiB < the 6 GiB headroom
    _run_steps(p, layers, 2.0)
    assert p.stage == 3 and p.stored_layers == 0 and all(l.use_recompute for l in layers)
    cpu = YvRecomputePlanner(types.SimpleNamespace(model=types.SimpleNamespace(layers=[_Layer()])), torch.device("cpu"))
    assert cpu.stage == 3                                          # nothing to plan without a CUDA device
