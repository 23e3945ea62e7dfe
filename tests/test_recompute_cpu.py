"""Recomputation engine, cache, memory tracker, hooks, strategies, profiler, recommender and the distributed variants."""
import json
import threading
import time

import pytest
import torch

from ml_framework_b200.checkpoint.activation import CheckpointConfig, CheckpointStrategyKind
from ml_framework_b200.checkpoint import recompute as rc
from ml_framework_b200.dist.process_group import run_fake_world


def test_dependency_graph_orders_dependencies_first_and_detects_cycles():
    g = rc.DependencyGraph()
    g.add_dependency("c", ["b"])
    g.add_dependency("b", ["a"])
    g.add_dependency("d", ["a"])
    order = g.topological_order(["c"])
    assert order == ["a", "b", "c"]
    both = g.topological_order(["d", "c"])
    assert both.index("a") < both.index("d") and both.index("b") < both.index("c") and len(both) == 4
    assert not g.has_cycle()
    g.add_dependency("a", ["c"])
    assert g.has_cycle()
    with pytest.raises(rc.RecomputationError):
        g.topological_order(["c"])
    with pytest.raises(ValueError):
        g.add_dependency("x", ["x"])


def test_cache_evicts_least_recently_used_by_bytes():
    c = rc.RecomputationCache(max_size_bytes=3 * 400)
    for k in "abc":
        assert c.add(k, torch.zeros(100))
    assert c.get("a") is not None              # a becomes most recent
    c.add("d", torch.zeros(100))               # evicts b
    assert not c.contains("b") and c.contains("a") and c.contains("c") and c.contains("d")
    assert c.get("b") is None
    assert not c.add("huge", torch.zeros(1000))
    s = c.stats()
    assert (s.entries, s.size_bytes, s.hits, s.misses, s.evictions) == (3, 1200, 1, 1, 1)
    assert s.hit_rate == 0.5
    c.clear()
    assert c.stats().entries == 0 and c.stats().size_bytes == 0


def test_engine_runs_dependencies_first_counts_and_caches():
    calls = []
    eng = rc.RecomputationEngine(cache=rc.RecomputationCache(1 << 20))
    eng.register_recompute_function("l0", lambda: calls.append("l0") or torch.ones(4))
    eng.register_recompute_function("l1", lambda: calls.append("l1") or torch.full((4,), 2.0), dependencies=["l0"])
    out = eng.recompute("l1")
    assert calls == ["l0", "l1"] and out.sum().item() == 8.0
    eng.recompute("l1")                          # both served by the cache
    assert calls == ["l0", "l1"]
    s = eng.stats()
    assert s.total_recomputations == 2 and s.registered_layers == 2 and s.cache.hits == 2
    assert eng.layer_stats("l1").call_count == 1 and eng.layer_stats("l1").average_ms >= 0
    res = eng.recompute_multiple(["l0", "l1"])
    assert set(res) == {"l0", "l1"}
    with pytest.raises(rc.RecomputationError):
        eng.recompute("nope")
    eng.register_recompute_function("bad", lambda: 1 / 0)
    with pytest.raises(rc.RecomputationError, match="bad"):
        eng.recompute("bad")
    eng.clear()
    assert not eng.has_recompute_function("l0")


def test_async_engine_runs_closures_on_worker_threads():
    eng = rc.AsyncRecomputationEngine(max_workers=4)
    names = set()

    def make(k):
        def fn():
            names.add(threading.current_thread().name)
            time.sleep(0.05)
            return torch.full((2,), float(k))
        return fn
    for k in range(4):
        eng.register_recompute_function(f"l{k}", make(k))
    t0 = time.perf_counter()
    out = eng.wait_all(eng.recompute_multiple_async([f"l{k}" for k in range(4)]), timeout=5)
    assert time.perf_counter() - t0 < 0.15         # four closures of 50 ms each, not one after the other
    assert [out[f"l{k}"][0].item() for k in range(4)] == [0.0, 1.0, 2.0, 3.0]
    assert all(n.startswith("mlf-recompute") for n in names)
    with pytest.raises(rc.RecomputationError):
        eng.recompute_async("missing")
    eng.close()
    with pytest.raises(rc.RecomputationError):
        eng.recompute_async("l0")


def test_memory_tracker_limit_fires_once_per_crossing():
    tr = rc.MemoryTracker(limit_bytes=1000)
    crossed, allocs = [], []
    tr.on_limit_exceeded.append(lambda lid, cur, lim: crossed.append((lid, cur, lim)))
    tr.on_allocated.append(lambda lid, n: allocs.append(n))
    tr.record_allocation("a", 600)
    tr.record_allocation("b", 600)
    tr.record_allocation("b", 100)
    assert crossed == [("b", 1200, 1000)] and allocs == [600, 600, 100]
    assert tr.record_deallocation("b") == 100 and tr.record_deallocation("b") == 600
    assert tr.record_deallocation("b") == 0
    tr.record_allocation("c", 500)
    assert len(crossed) == 2
    s = tr.stats()
    assert s.current_bytes == 1100 and s.peak_bytes == 1300 and s.allocation_count == 4 and s.deallocation_count == 2 and s.layers == 3
    assert tr.layer_stats("b").peak_bytes == 700 and tr.layer_stats("b").current_bytes == 0
    tr.record_tensor("t", torch.zeros(10, dtype=torch.float64))
    assert tr.layer_stats("t").current_bytes == 80
    tr.reset_stats()
    assert tr.stats().current_bytes == 0 and tr.stats().limit_bytes == 1000


def test_backward_hooks_fire_from_autograd_and_can_replace_the_gradient():
    m = rc.BackwardHookManager()
    seen = []
    h1 = m.register_hook("blk", lambda g: seen.append(g.clone()))
    h2 = m.register_hook("blk", lambda g: g * 2)
    x = torch.ones(3, requires_grad=True)
    y = x * 3
    m.attach(y, "blk")
    y.sum().backward()
    assert torch.equal(seen[0], torch.ones(3)) and torch.equal(x.grad, torch.full((3,), 6.0))
    assert m.hook_count_for_layer("blk") == 2 and m.has_hook(h1)
    assert m.remove_hook(h2) and not m.remove_hook(h2)
    assert m.remove_hooks_for_layer("blk") == 1 and not m.has_hook(h1)
    m.register_hook("e", lambda g: 1 / 0)
    ran = []
    m.register_hook("e", lambda g: ran.append(1))
    with pytest.raises(ZeroDivisionError):
        m.invoke_hooks("e", torch.zeros(1))
    assert ran == [1]
    m.clear_all_hooks()
    assert m.hook_count_for_layer("e") == 0


def test_gradient_accumulator_averages_over_steps():
    acc = rc.CheckpointedGradientAccumulator(2)
    acc.accumulate({"w": torch.tensor([2.0, 4.0]), "b": torch.tensor([1.0])})
    assert not acc.should_apply_gradients()
    acc.accumulate({"w": torch.tensor([4.0, 0.0]), "b": torch.tensor([3.0])})
    assert acc.should_apply_gradients()
    assert torch.equal(acc.get_gradient("w"), torch.tensor([3.0, 2.0]))
    assert acc.remove_gradient("b") and acc.get_gradient("b") is None
    g = acc.get_accumulated_gradients()
    assert list(g) == ["w"] and acc.current_step == 0 and acc.peek_gradients() == {}
    acc.accumulate({"w": torch.zeros(2)})
    with pytest.raises(ValueError):
        acc.accumulate({"w": torch.zeros(3)})


def test_strategies_and_factory():
    a = torch.zeros(1024)                        # 4 KB
    assert [rc.IntervalCheckpointStrategy(3).should_checkpoint("l", a, i) for i in range(4)] == [True, False, False, True]
    sel = rc.SelectiveCheckpointStrategy(["x"], ["y"])
    assert sel.should_checkpoint("x", a, 0) and not sel.should_checkpoint("y", a, 0) and not sel.should_checkpoint("z", a, 0)
    with pytest.raises(ValueError):
        rc.SelectiveCheckpointStrategy(["x"], ["x"])
    sz = rc.SizeBasedCheckpointStrategy(4096)
    assert sz.should_checkpoint("l", a, 0) and not sz.should_checkpoint("l", torch.zeros(8), 0)
    ma = rc.MemoryAwareCheckpointStrategy(0.5, 20000)            # budget 10 000 bytes
    assert [ma.should_checkpoint(f"l{i}", a, i) for i in range(4)] == [False, False, True, True]
    ma.reset()
    assert not ma.should_checkpoint("l", a, 0)
    smart = rc.SmartCheckpointStrategy(0.5, 20000)
    for k, (n, ms) in {"big_cheap": (8000, 1.0), "big_slow": (8000, 100.0), "small": (2000, 1.0)}.items():
        smart.observe(k, n, ms)
    assert smart.plan() == ["big_cheap"]                          # 18 000 -> 10 000 fits
    assert smart.should_checkpoint("big_cheap", a, 0) and not smart.should_checkpoint("big_slow", a, 1)
    assert smart.should_checkpoint("unknown", a, 0) and not smart.should_checkpoint("unknown2", a, 1)
    for kind, cls in [(CheckpointStrategyKind.INTERVAL, rc.IntervalCheckpointStrategy), (CheckpointStrategyKind.SELECTIVE, rc.SelectiveCheckpointStrategy),
                      (CheckpointStrategyKind.SIZE_BASED, rc.SizeBasedCheckpointStrategy), (CheckpointStrategyKind.MEMORY_AWARE, rc.MemoryAwareCheckpointStrategy),
                      (CheckpointStrategyKind.SMART, rc.SmartCheckpointStrategy)]:
        assert isinstance(rc.make_strategy(CheckpointConfig(strategy=kind)), cls)


def test_profiler_summary_report_monitor_and_recommendations():
    p = rc.CheckpointProfiler()
    p.record_event(rc.CheckpointEventType.CHECKPOINT, "ignored")      # not profiling yet
    p.start_profiling()
    E = rc.CheckpointEventType
    for _ in range(2):
        p.record_event(E.CHECKPOINT, "hot", 1.0, 1 << 20)
    for _ in range(6):
        p.record_event(E.RECOMPUTE, "hot", 50.0)
    for _ in range(12):
        p.record_event(E.CHECKPOINT, "cold", 0.1, 1 << 10)
        p.record_event(E.CACHE_MISS, "cold")
    p.record_event(E.CACHE_HIT, "cold")
    p.record_event(E.CHECKPOINT, "waste", 40.0, 10)
    p.record_event(E.RECOMPUTE, "waste", 1.0)
    fired = []
    mon = rc.CheckpointMonitor(p, memory_threshold_bytes=1 << 20, recompute_threshold_ms=100.0, interval_s=30.0)
    mon.on_memory_threshold.append(lambda cur, thr: fired.append("mem"))
    mon.on_recompute_threshold.append(lambda cur, thr: fired.append("time"))
    mon.check_now()
    mon.close()
    assert fired == ["mem", "time"]
    p.stop_profiling()
    s = p.summary()
    assert s.total_events == 2 + 6 + 25 + 2 and s.total_recompute_ms == 301.0 and len(s.layer_profiles) == 3
    assert p.layer_profile("hot").average_recompute_ms == 50.0 and abs(p.layer_profile("cold").cache_hit_rate - 1 / 13) < 1e-9
    assert "hot: 2 checkpoints, 6 recomputes" in p.generate_report()
    assert json.loads(p.export_json())["total_memory_saved"] == s.total_memory_saved
    recs = rc.OptimizationRecommender().generate(s)
    kinds = [(r.type, r.affected_layer_id) for r in recs]
    T = rc.RecommendationType
    assert (T.REDUCE_RECOMPUTATION, "hot") in kinds and (T.IMPROVE_CACHE_HIT_RATE, "cold") in kinds and (T.IMPROVE_EFFICIENCY, "waste") in kinds
    assert any(r.type == T.ENABLE_ASYNC_RECOMPUTATION for r in recs)
    assert [r.priority.value for r in recs] == sorted(r.priority.value for r in recs)
    assert "could save 300ms" in next(r for r in recs if r.affected_layer_id == "hot").expected_impact


def test_distributed_manager_fetches_from_owner_and_aggregates_memory():
    def worker(pg):
        m = rc.DistributedCheckpointManager(pg)
        if pg.rank == 1:
            m.register_checkpoint("act", torch.arange(6, dtype=torch.float32).view(2, 3))
        else:
            m.register_checkpoint("other", torch.zeros(2))
        m.synchronize_checkpoints()
        got = m.retrieve_or_fetch("act", source_rank=1)
        m.register_checkpoint_broadcast("shared", torch.full((4,), float(pg.rank + 5)), source_rank=0)
        stats = m.aggregated_memory_stats()
        local_missing = False
        try:
            m.retrieve_or_fetch("nowhere")
        except KeyError:
            local_missing = True
        shared = m.retrieve_or_fetch("shared")
        m.clear_checkpoints_distributed()
        return got.tolist(), shared.tolist(), stats.per_rank_bytes, stats.imbalance, local_missing, m.tracker.stats().current_bytes

    res = run_fake_world(2, worker)
    for got, shared, per_rank, imb, missing, left in res:
        assert got == [[0.0, 1.0, 2.0], [3.0, 4.0, 5.0]] and shared == [5.0] * 4 and missing and left == 0
        assert per_rank == [8 + 16, 24 + 16] and abs(imb - (40 / 32 - 1)) < 1e-9


def test_model_and_pipeline_parallel_variants():
    s = rc.ModelParallelCheckpointStrategy(rank=3, tensor_parallel_size=2)
    assert not s.should_checkpoint("l", None, is_tensor_parallel=True) and s.should_checkpoint("l", None)
    assert rc.ModelParallelCheckpointStrategy(4, 2).should_checkpoint("l", None, is_tensor_parallel=True)
    s.register_layer_rank("pinned", 3)
    assert s.should_checkpoint("pinned", None, True) and s.checkpoint_rank("pinned") == 3 and s.checkpoint_rank("l") == 0
    pp = rc.PipelineParallelCheckpointManager(stage=1, num_stages=3)
    a, b = torch.zeros(1), torch.ones(1)
    pp.register_stage_checkpoint(1, "inner", a)
    pp.register_stage_checkpoint(1, "out", b, is_boundary=True)
    assert len(pp.stage_checkpoints(1)) == 2 and pp.next_stage_boundaries() == [b]
    last = rc.PipelineParallelCheckpointManager(2, 3)
    last.register_stage_checkpoint(2, "out", b, True)
    assert last.next_stage_boundaries() == []
    pp.clear_stage_checkpoints()
    assert pp.stage_checkpoints(1) == []
    with pytest.raises(ValueError):
        pp.register_stage_checkpoint(5, "x", a)


def test_checkpoint_scopes_sequential_and_selective_wrapping():
    import torch.nn as nn
    from ml_framework_b200.checkpoint import activation as act
    calls = {"n": 0}

    def f(t):
        calls["n"] += 1
        return torch.tanh(t) * 2
    x = torch.randn(4, requires_grad=True)
    act.maybe_checkpoint(f, x).sum().backward()
    assert calls["n"] == 1 and not act.in_checkpoint_scope()
    g_plain = x.grad.clone()
    x.grad = None
    with act.checkpoint_scope():
        assert act.in_checkpoint_scope()
        with act.checkpoint_scope(False):
            assert not act.in_checkpoint_scope()
        y = act.maybe_checkpoint(f, x)
    y.sum().backward()
    assert calls["n"] == 3 and torch.allclose(x.grad, g_plain)                  # forward once more during backward
    layers = [nn.Linear(4, 4) for _ in range(5)]
    x2 = torch.randn(2, 4, requires_grad=True)
    ref = x2
    for l in layers:
        ref = l(ref)
    out = act.checkpoint_sequential(layers, 2, x2)
    assert torch.allclose(out, ref)
    out.sum().backward()
    assert all(l.weight.grad is not None for l in layers)
    with pytest.raises(ValueError):
        act.checkpoint_sequential(layers, 0, x2)
    model = nn.Sequential(nn.Sequential(nn.Linear(4, 4), nn.ReLU()), nn.Linear(4, 2))
    assert act.selective_checkpointing(model, lambda path, m: isinstance(m, nn.Sequential)) == ["0"]
    assert isinstance(model[0], act.CheckpointedModuleWrapper) and act.selective_checkpointing(model, lambda p, m: True) == ["1"]
    model(torch.randn(3, 4, requires_grad=True)).sum().backward()
    a = torch.zeros(10)
    assert act.tensor_checkpoint_bytes(a, a, torch.zeros(3, dtype=torch.float64)) == 40 + 24
