"""Hardware abstraction layer on CPU: device ids, streams and events of the CPU backend, the operation table of both
backends against PyTorch, the registry, dynamic-shape memory (bounds, adaptive padding, predictive allocation,
pressure handling)."""
import pytest
import torch

from ml_framework_b200.hal import core as H


def test_device_ids_streams_events_and_properties_on_cpu():
    did = H.DeviceId(H.DeviceType.CUDA, 3)
    assert str(did) == "cuda:3" and did.torch() == torch.device("cuda", 3) and str(H.DeviceId(H.DeviceType.CPU)) == "cpu:0"
    be = H.BackendRegistry.get("cpu")
    d = be.device(0)
    assert not d.is_cuda and d.properties()["name"] == "cpu" and d.properties()["cores"] >= 1
    d.synchronize()
    s = d.create_stream(priority=-1)
    order = []
    s.enqueue(lambda: order.append("a"))
    s.enqueue(lambda: order.append("b"))
    assert order == ["a", "b"] and s.handle == 0
    ev = d.create_event()
    assert not ev.query()
    ev.record(s)
    assert ev.query() and ev.elapsed_ms(s.record_event()) == 0.0
    ev.synchronize()
    s.wait_event(ev)
    s.synchronize()
    b = d.allocate(100)
    assert b.ptr == b.tensor.data_ptr() and b.size >= 100
    b.free()
    assert b.freed
    d.allocator.empty_cache()
    with pytest.raises(ValueError):
        d.allocate(0)
    with pytest.raises(NotImplementedError):
        H.MemoryAllocator(d).allocate(8)


def test_operation_table_matches_torch_on_both_backends():
    torch.manual_seed(0)
    a, b = torch.randn(4, 6), torch.randn(4, 6)
    O = H.Operation
    for name in ("cpu", "b200"):                                   # the B200 backend falls back to PyTorch for CPU tensors
        be = H.BackendRegistry.get(name)
        assert all(be.supports(op) for op in O)
        assert torch.equal(be.execute(O.ADD, [a, b]), a + b) and torch.equal(be.execute(O.SUBTRACT, [a, b]), a - b)
        assert torch.equal(be.execute(O.MULTIPLY, [a, b]), a * b) and torch.equal(be.execute(O.DIVIDE, [a, b]), a / b)
        assert torch.equal(be.execute(O.MATMUL, [a, b.t()]), a @ b.t()) and torch.equal(be.execute(O.TRANSPOSE, [a]), a.t())
        assert torch.equal(be.execute(O.SUM, [a], dim=1), a.sum(1)) and torch.equal(be.execute(O.SUM, [a]), a.sum())
        assert torch.equal(be.execute(O.MEAN, [a], dim=0), a.mean(0)) and torch.equal(be.execute(O.MAX, [a]), a.max())
        assert torch.equal(be.execute(O.MIN, [a], dim=1), a.amin(1)) and torch.equal(be.execute(O.MAX, [a], dim=0), a.amax(0))
        c = be.execute(O.COPY, [a])
        assert torch.equal(c, a) and c.data_ptr() != a.data_ptr()
        assert torch.equal(be.execute(O.FILL, [a], value=2.5), torch.full_like(a, 2.5))
        assert torch.equal(be.execute(O.RELU, [a]), torch.relu(a)) and torch.equal(be.execute(O.SIGMOID, [a]), torch.sigmoid(a))
        assert torch.equal(be.execute(O.TANH, [a]), torch.tanh(a))
        x, w, bias = torch.randn(1, 2, 8, 8), torch.randn(3, 2, 3, 3), torch.randn(3)
        assert torch.allclose(be.execute(O.CONV2D, [x, w, bias], padding=1), torch.nn.functional.conv2d(x, w, bias, padding=1))
        assert torch.equal(be.execute(O.MAXPOOL2D, [x]), torch.nn.functional.max_pool2d(x, 2))
        assert be.execute(O.CAST, [a], dtype=torch.float64).dtype == torch.float64
        assert be.execute(O.RESHAPE, [a], shape=(6, 4)).shape == (6, 4)
    assert "cpu" in H.BackendRegistry.available() and H.BackendRegistry.best().name in ("cpu", "b200")
    assert H.BackendRegistry.get("b200").is_available() == torch.cuda.is_available()
    assert H.BackendRegistry.get("b200").device_count() == torch.cuda.device_count() and H.Backend().device_count() == 1
    with pytest.raises(KeyError):
        H.BackendRegistry.get("tpu")

    class Custom(H.Backend):
        name = "custom"
    H.BackendRegistry.register(Custom())
    assert H.BackendRegistry.get("custom").is_available() and "custom" in H.BackendRegistry.available()


def test_shape_bounds_adaptive_padding_and_predictive_allocation():
    bnd = H.ShapeBounds((1, 8), (64, 8), expected_shape=(16, 8))
    assert bnd.contains((32, 8)) and not bnd.contains((65, 8)) and not bnd.contains((4,)) and bnd.max_elements() == 512
    with pytest.raises(ValueError):
        H.ShapeBounds((2, 2), (1, 2))
    with pytest.raises(ValueError):
        H.ShapeBounds((1,), (1, 2))
    pad = H.AdaptivePaddingStrategy(initial=1.2, lo=1.0, hi=1.5)
    assert pad.padded(100) == 120
    for _ in range(16):
        pad.observe(True)                                           # re-allocating all the time: pad more
    grown = pad.factor
    assert grown > 1.2
    for _ in range(64):
        pad.observe(True)
    assert pad.factor == 1.5                                        # capped
    for _ in range(16 * 60):
        pad.observe(False)                                          # padding never needed: shrink to the floor
    assert pad.factor == 1.0
    d = H.BackendRegistry.get("cpu").device(0)
    pa = H.PredictiveAllocator(H.SimpleAllocator(d), padding=H.AdaptivePaddingStrategy(1.5))
    t = pa.get("kv", (10, 4), torch.float32)
    t.fill_(3.0)
    assert t.shape == (10, 4) and pa.reallocations == 0
    t2 = pa.get("kv", (14, 4), torch.float32)                       # fits the padded capacity (15 rows): same storage
    assert t2.data_ptr() == t.data_ptr() and pa.reallocations == 0 and float(t2[0, 0]) == 3.0
    t3 = pa.get("kv", (40, 4), torch.float32)
    assert pa.reallocations == 1 and t3.shape == (40, 4) and pa.predict_elements("kv") == 160
    t4 = pa.get("kv", (8, 4), torch.bfloat16)                       # another dtype needs its own buffer
    assert t4.dtype == torch.bfloat16 and pa.reallocations == 2
    capped = pa.get("bounded", (60, 8), torch.float32, H.ShapeBounds((1, 8), (64, 8)))
    assert capped.shape == (60, 8) and pa._handles["bounded"].capacity_elements == 512      # never beyond the bound
    with pytest.raises(ValueError):
        pa._handles["bounded"].view((65, 8))
    pa.release("kv")
    pa.release("kv")                                                # releasing twice is harmless
    assert "kv" not in pa._handles and pa.predict_elements("nothing") == 0


def test_memory_pressure_handler_releases_low_priority_first_until_below_the_low_mark():
    used = [95]
    log = []

    def rel(name, amount):
        def f():
            log.append(name)
            used[0] -= amount
            return amount
        return f
    h = H.MemoryPressureHandler(100, high=0.9, low=0.75, usage_fn=lambda: used[0])
    h.register(rel("important", 50), priority=10)
    h.register(rel("cache", 10), priority=0)
    h.register(rel("scratch", 15), priority=5)
    assert h.pressure() == 0.95 and h.check() == 25 and log == ["cache", "scratch"] and used[0] == 70 and h.events == 1
    assert h.check() == 0 and h.events == 1                         # below the high mark: nothing to do
    used[0] = 99
    assert h.check() == 25 and used[0] == 74 and h.events == 2      # stops as soon as usage is under the low mark
    used[0] = 140
    assert h.check() == 75 and log[-1] == "important" and used[0] == 65


def test_graph_fallback_handler_proxy_allocator_and_static_facade():
    import torch
    import torch.nn as nn
    from ml_framework_b200.hal import cuda_graphs as cg
    seen = []
    fb = cg.CUDAGraphFallbackHandler(max_failures=2, on_fallback=seen.append)
    assert fb.execute_with_fallback(lambda: "graph", lambda: "eager") == "graph"

    def boom():
        raise RuntimeError("capture failed")
    assert fb.execute_with_fallback(boom, lambda: "eager") == "eager" and fb.graph_path_enabled
    assert fb.execute_with_fallback(boom, lambda: "eager") == "eager" and not fb.graph_path_enabled
    calls = []
    assert fb.execute_with_fallback(lambda: calls.append(1), lambda: "eager") == "eager" and calls == []      # graph path is off
    st = fb.stats()
    assert st["successes"] == 1 and st["fallbacks"] == 3 and st["by_type"] == {"RuntimeError": 2} and len(seen) == 2
    fb.reset()
    assert fb.graph_path_enabled and fb.last_error is None

    lin = nn.Linear(3, 2)
    px = cg.CUDAGraphProxy(lin, name="lin")
    x = torch.randn(4, 3)
    for _ in range(5):
        assert torch.equal(px(x), lin(x))                    # CPU tensors: warm-up, then the eager fall-back
    assert px.calls == 5 and not px.is_captured and px.manager.fallbacks == 2
    assert px.update_weights({"weight": torch.zeros(2, 3), "other": torch.zeros(1)}) == 1 and float(lin.weight.detach().abs().sum()) == 0.0
    with __import__("pytest").raises(ValueError):
        px.update_weights({"weight": torch.zeros(3, 3)})
    with __import__("pytest").raises(TypeError):
        cg.CUDAGraphProxy(lambda t: t).update_weights({})
    px.invalidate()
    px.enabled = False
    px(x)
    assert px.manager._calls == {}

    al = cg.GraphCompatibleMemoryAllocator(cg.GraphMemoryPool(4096, torch.device("cpu")))
    a = al.allocate((8,), torch.float32)
    with al.capture_scope():
        b = al.allocate((100,), torch.float32)
        c = al.allocate((10,), torch.bfloat16)
        assert al.in_capture and c.data_ptr() - b.data_ptr() == 512
        with __import__("pytest").raises(RuntimeError):
            al.reset_pool()
        with __import__("pytest").raises(MemoryError):
            al.allocate((2000,), torch.float32)
    s = al.stats()
    assert (s.pool_allocations, s.fallback_allocations, s.fallback_bytes, s.pool_used, s.pool_blocks) == (2, 1, 32, 768, 2) and abs(s.pool_utilization - 768 / 4096) < 1e-9
    assert al.free(c) and not al.free(a) and al.stats().pool_used == 512
    al.reset_pool()
    assert al.stats().pool_used == 0 and al.stats().pool_peak == 768

    cg.CUDAGraphStatic.reset()
    f = lambda t: t * 2      # noqa: E731
    assert torch.equal(cg.CUDAGraphStatic.run("dbl", f, x), x * 2) and cg.CUDAGraphStatic.stats()["graphs"] == 0
    p2 = cg.CUDAGraphStatic.proxy(f, "dbl2")
    assert p2.manager is cg.CUDAGraphStatic.manager() and torch.equal(p2(x), x * 2)
    cg.CUDAGraphStatic.enabled = False
    assert torch.equal(cg.CUDAGraphStatic.run("dbl", f, x), x * 2)
    cg.CUDAGraphStatic.configure(cg.CaptureOptions())
    cg.CUDAGraphStatic.reset()


def test_graph_validation_rules_context_result_and_fallback_strategies():
    from ml_framework_b200.hal import cuda_graphs as cg
    ctx = cg.CUDAGraphValidationContext()
    for name, kind in (("gemm", "kernel"), ("gemm", "kernel"), ("print", "io"), ("if x.item()", "branch"), ("cudaDeviceSynchronize", "sync"),
                       ("callback", "host"), ("", "kernel")):
        ctx.record_operation(name, kind)
    ctx.record_memory_allocation(0x7000)
    ctx.record_memory_allocation(0)
    assert ctx.get_operation_count("gemm") == 2 and ctx.has_operation("print") and not ctx.has_operation("nope")
    assert ctx.allocated_memory == frozenset({0x7000}) and len(ctx.captured_operations) == 6 and ctx.operation_counts["gemm"] == 2
    v = cg.GraphValidator()
    res = v.validation_result(ctx.ops())
    assert not res.is_valid and res.operation_count == 7 and len(res.errors) == 4 and len(res.warnings) == 1
    assert {e.split("]")[0][1:] for e in res.errors} == {"IOOperation", "ControlFlow", "Synchronization", "DynamicMemory"}
    assert v.validation_result([]).errors == ["[EmptyGraph] capture recorded no operations"]
    assert [r.rule_name for r in v.rules][:5] == ["EmptyGraph", "DynamicMemory", "ControlFlow", "IOOperation", "Synchronization"]
    assert all(r.description for r in v.rules)

    class TooManyKernels(cg.ValidationRule):
        rule_name, description = "KernelBudget", "a capture should stay small"

        def validate(self, ops):
            n = sum(o.kind == "kernel" for o in ops)
            return [cg.ValidationIssue(self.rule_name, f"{n} kernels", cg.ValidationSeverity.WARNING)] if n > 1 else []
    v.add_rule(TooManyKernels())
    with pytest.raises(ValueError):
        v.add_rule(TooManyKernels())
    assert any("KernelBudget" in w for w in v.validation_result(ctx.ops()).warnings)
    assert v.remove_rule("IOOperation") and not v.remove_rule("IOOperation") and len(v.validation_result(ctx.ops()).errors) == 3
    only = cg.GraphValidator([cg.EmptyGraphRule()])
    assert only.is_valid(ctx.ops())
    ctx.clear()
    assert ctx.ops() == [] and cg.CUDAGraphValidationResult.success(3).is_valid and not cg.CUDAGraphValidationResult.failure(["x"]).is_valid
    assert cg.GraphPhase.FULL_TRAINING_STEP.value == "full_training_step" and cg.CUDAGraphState.INVALIDATED.value == "invalidated"

    S = cg.CUDAGraphFallbackStrategy

    def boom():
        raise RuntimeError("capture failed")
    never = cg.CUDAGraphFallbackHandler(strategy=S.NEVER_CAPTURE)
    assert never.execute_with_fallback(boom, lambda: "eager") == "eager" and never.by_type == {}
    always = cg.CUDAGraphFallbackHandler(max_failures=1, strategy=S.CAPTURE_OR_FALLBACK)
    for _ in range(3):
        assert always.execute_with_fallback(boom, lambda: "eager") == "eager"
    assert always.by_type == {"RuntimeError": 3} and always.graph_path_enabled          # keeps trying
    strict = cg.CUDAGraphFallbackHandler(strategy=S.CAPTURE_ONLY)
    with pytest.raises(cg.CUDAGraphCaptureException, match="capture failed"):
        strict.execute_with_fallback(boom, lambda: "eager")
    once = cg.CUDAGraphFallbackHandler(max_failures=5, strategy=S.TRY_ONCE_THEN_FALLBACK)
    assert once.execute_with_fallback(lambda: "graph", lambda: "eager") == "graph"
    assert once.execute_with_fallback(boom, lambda: "eager") == "eager" and not once.graph_path_enabled
    assert once.execute_with_fallback(lambda: "graph", lambda: "eager") == "eager"
    retry = cg.CUDAGraphFallbackHandler(max_failures=2)
    retry.execute_with_fallback(boom, lambda: 0); assert retry.graph_path_enabled
    retry.execute_with_fallback(boom, lambda: 0); assert not retry.graph_path_enabled


def test_allocation_stats_and_model_memory_pressure():
    from ml_framework_b200.hal import core as H
    alloc = H.PredictiveAllocator(H.SimpleAllocator(H.BackendRegistry.get("cpu").device(0)))
    for n in (100, 110, 300, 120):
        alloc.get("act", (n,), torch.float32)
    st = alloc.stats()
    assert st.total_allocations >= 2 and st.total_resizes >= 1 and st.total_bytes_allocated >= 300 * 4 and st.total_bytes_wasted > 0
    assert 0 < st.average_utilization <= 1 and "resizes" in st.to_report()

    now = [0.0]
    unloaded, busy = [], {("m", "2")}
    h = H.ModelMemoryPressureHandler(1000, lambda n, v: unloaded.append((n, v)), lambda n, v: (n, v) not in busy, clock=lambda: now[0])
    for i, v in enumerate(("1", "2", "3", "4")):
        now[0] = float(i)
        h.track_model_load("m", v, 300)
    assert h.get_total_memory_usage() == 1200 and len(h.get_loaded_models_info()) == 4
    now[0] = 10.0
    h.track_model_access("m", "1")                         # the oldest load becomes the most recently used
    h.pin_model("m", "3")
    r = h.evict_if_needed()
    assert r.evicted_versions == ["m:4"] and r.bytes_freed == 300 and r.sufficient and unloaded == [("m", "4")]   # 2 is busy, 3 pinned
    assert "freed 300 bytes" in str(r) and h.evict_if_needed().evicted_versions == []
    r = h.evict_if_needed(required_bytes=400)               # 900 used, 600 allowed: only version 1 can go
    assert r.evicted_versions == ["m:1"] and r.sufficient
    r = h.evict_if_needed(required_bytes=900)               # nothing evictable is left
    assert r.evicted_versions == [] and not r.sufficient and "NOT enough" in str(r)
    busy.clear()
    h.unpin_model("m", "3")
    assert h.evict_if_needed(required_bytes=900).evicted_versions == ["m:2", "m:3"] and h.get_total_memory_usage() == 0 and h.evictions == 4
    assert not h.untrack_model("m", "9")
    with pytest.raises(KeyError):
        h.pin_model("m", "9")
    with pytest.raises(ValueError):
        h.set_memory_threshold(0)
    info = H.ModelMemoryInfo("a", "1", 10, clock=lambda: 5.0)
    w0 = info.weight
    info.record_access()
    assert info.weight == w0 + 86400.0 and info.access_count == 1
