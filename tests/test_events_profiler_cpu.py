"""Event system, collectors, scalar series and the host-side profilers on CPU (NVML is replaced by a fake)."""
import gc
import time

import pytest
import torch

from ml_framework_b200.obs import events as E
from ml_framework_b200.obs import profiler as P


def test_event_factory_json_round_trip_subscriptions_and_storage(tmp_path):
    evs = [E.EventFactory.scalar("loss", 0.5, 3, run="a"), E.EventFactory.histogram("w", [1, 2, 3]), E.EventFactory.profiling_start("fwd"),
           E.EventFactory.profiling_end("fwd", duration_ns=1200), E.EventFactory.memory("act", 1 << 20), E.EventFactory.tensor_op("matmul", [(2, 3), (3, 4)])]
    back = [E.Event.from_json(e.to_json()) for e in evs]
    assert [b.type for b in back] == [e.type for e in evs] and back[0].metadata == {"run": "a"} and back[1].value == [1.0, 2.0, 3.0]
    assert back[3].value == 1200 and back[4].value == 1 << 20 and back[5].value == [[2, 3], [3, 4]]
    bus = E.EventSystem()
    all_seen, scalars = [], []
    bus.subscribe(all_seen.append)
    un = bus.subscribe(scalars.append, E.EventType.SCALAR)
    for e in evs:
        bus.publish(e)
    un()
    un()                                                                       # unsubscribing twice is harmless
    bus.publish(evs[0])
    assert len(all_seen) == 7 and len(scalars) == 1 and bus.published == 7
    assert isinstance(E.storage_backend("memory"), E.MemoryStorageBackend)
    fb = E.storage_backend("file", log_dir=str(tmp_path))
    fb.write(evs)
    fb.flush()
    assert [e.name for e in E.FileStorageBackend.read(fb.path)] == [e.name for e in evs]
    fb.close()
    with pytest.raises(KeyError):
        E.storage_backend("s3")
    with pytest.raises(NotImplementedError):
        E.StorageBackend().write([])


def test_collectors_backpressure_and_background_flush():
    mem = E.MemoryStorageBackend()
    col = E.EventCollector(mem, E.EventCollectorConfig(buffer_capacity=3, flush_batch=100, backpressure=E.BackpressureStrategy.DROP_OLDEST))
    for i in range(5):
        col.collect(E.EventFactory.scalar("x", i))
    col.close()
    assert col.dropped == 2 and [e.value for e in mem.events] == [2.0, 3.0, 4.0]          # the oldest two were displaced
    mem2 = E.MemoryStorageBackend()
    acol = E.AsyncEventCollector(mem2, E.EventCollectorConfig(buffer_capacity=2, flush_interval_s=0.01))
    for i in range(6):
        acol.collect(E.EventFactory.scalar("y", i))
        time.sleep(0.02)                                                       # slower than the flusher: nothing is dropped
    acol.close()
    assert [e.value for e in mem2.events] == [float(i) for i in range(6)] and acol.dropped == 0
    mem3 = E.MemoryStorageBackend()
    burst = E.AsyncEventCollector(mem3, E.EventCollectorConfig(buffer_capacity=2, flush_interval_s=5.0, backpressure=E.BackpressureStrategy.DROP_NEWEST))
    for i in range(5):
        burst.collect(E.EventFactory.scalar("z", i))
    burst.close()
    assert burst.dropped == 3 and [e.value for e in mem3.events] == [0.0, 1.0]


def test_scalar_series_smoothing_resampling_and_stats():
    s = E.ScalarSeries("loss")
    for i, v in enumerate([4.0, 2.0, 2.0, 0.0, 2.0, 2.0, 2.0, 2.0, 2.0, 2.0]):
        s.add(i * 10, v)
    assert s.moving_average(2)[:4] == [4.0, 3.0, 2.0, 1.0] and s.moving_average(100)[-1] == pytest.approx(2.0)
    ema = s.ema(0.5)
    assert ema[0] == pytest.approx(4.0) and ema[1] == pytest.approx((0.5 * 2 + 0.25 * 4) / 0.75)          # debiased
    steps, vals = s.resample(4)
    assert steps == [0, 30, 60, 90] and vals == [4.0, 0.0, 2.0, 2.0] and s.resample(50) == (s.steps, s.values)
    assert s.stats() == {"count": 10, "min": 0.0, "max": 4.0, "mean": 2.0, "last": 2.0} and E.ScalarSeries("e").stats() == {"count": 0}
    log = E.ScalarLogger()
    log.log("a", 1.0, 0)
    assert log.get("a").values == [1.0]
    with pytest.raises(KeyError):
        log.get("b")


def test_scope_profiler_report_reset_and_disabled_mode():
    prof = P.Profiler()
    for _ in range(3):
        with prof.scope("step"):
            with prof.scope("fwd"):
                time.sleep(0.001)
    r = prof.result("fwd")
    assert r.count == 3 and r.parent == "step" and r.mean_ns == r.total_ns / 3 and r.min_ns <= r.p50_ns <= r.max_ns
    rep = prof.report()
    assert rep.splitlines()[0].startswith("step") and "(in step)" in rep.splitlines()[1]                # sorted by total time
    prof.record_instant("mark")
    prof.reset()
    assert prof.results() == {} and prof.instants == []
    off = P.Profiler(enabled=False)
    with off.scope("x"):
        pass
    assert off.results() == {}


def test_memory_gc_and_utilisation_trackers_with_a_fake_nvml():
    mp = P.MemoryProfiler()
    assert mp.delta() == 0.0
    a = mp.snapshot("start")
    keep = [[i] for i in range(20000)]                                       # container objects are what the collector tracks
    b = mp.snapshot("end")
    assert a["tag"] == "start" and b["py_objects"] > a["py_objects"] and mp.delta("py_objects") >= 20000
    del keep
    mon = P.GCMonitor()
    mon.start()
    gc.collect()
    gc.collect()
    mon.stop()
    mon.stop()
    n = mon.collections
    gc.collect()
    assert n >= 2 and mon.collections == n and mon.pause_ns > 0                                          # stopped: no further counting

    class U:
        gpu, memory = 70, 40

    class M:
        used, total = 10 << 30, 180 << 30

    class FakeNvml:
        NVML_CLOCK_SM = 1
        calls = 0

        def nvmlDeviceGetUtilizationRates(self, h):
            self.calls += 1
            return U()

        def nvmlDeviceGetMemoryInfo(self, h): return M()
        def nvmlDeviceGetClockInfo(self, h, k): return 1600
        def nvmlDeviceGetMaxClockInfo(self, h, k): return 1965
        def nvmlDeviceGetPowerUsage(self, h): return 950_000
        def nvmlDeviceGetCurrentClocksEventReasons(self, h): return 4
    tr = P.GpuUtilizationTracker(0, interval_s=0.005)
    fake = FakeNvml()
    tr._nv, tr._h = fake, object()
    one = tr.sample()
    assert one["gpu_util"] == 70 and one["sm_mhz"] == 1600 and one["power_w"] == 950.0 and one["throttle_reasons"] == 4
    tr.start()
    time.sleep(0.05)
    mean = tr.stop()
    assert fake.calls >= 3 and mean["gpu_util"] == 70 and mean["sm_max_mhz"] == 1965 and "time" not in mean and "throttle_reasons" not in mean
    none = P.GpuUtilizationTracker(0)
    none._nv = None
    assert none.sample() == {} and none.stop() == {}


def test_percentile_calculator_duration_tracker_and_shape_profile_optimizer():
    import pytest as _p
    from ml_framework_b200.compiler.cache import GlobalShapeProfiler, ShapeProfileOptimizer
    from ml_framework_b200.obs.profiler import DurationTracker, PercentileCalculator
    pc = PercentileCalculator([5, 1, 3])
    pc.add(2); pc.add(4)
    assert len(pc) == 5 and pc.percentile(50) == 3.0 and pc.percentile(0) == 1.0 and pc.percentile(100) == 5.0 and pc.percentiles([25, 75]) == {25: 2.0, 75: 4.0}
    assert pc.summary()["mean"] == 3.0 and PercentileCalculator().summary() == {"count": 0}
    with _p.raises(ValueError):
        pc.percentile(101)
    dt = DurationTracker(max_samples_per_name=3)
    for v in (10, 20, 30, 40):
        dt.record("step", v)
    with dt.track("blk"):
        pass
    st = dt.statistics("step")
    assert st["count"] == 4 and st["total_ns"] == 100 and st["mean_ns"] == 25 and st["min_ns"] == 20 and st["p50_ns"] == 30 and dt.names() == ["blk", "step"]
    assert dt.statistics("blk")["count"] == 1 and dt.statistics("none") == {"count": 0}
    with _p.raises(ValueError):
        dt.record("x", -1)
    dt.reset("step")
    assert dt.names() == ["blk"]
    dt.reset()
    assert dt.names() == []
    prof = GlobalShapeProfiler()
    for _ in range(60):
        prof.record("linear", (8, 4096))
    for _ in range(30):
        prof.record("linear", (64, 4096))
    for b in (3, 5, 7, 100, 200):
        for _ in range(2):
            prof.record("linear", (b, 4096))
    opt = ShapeProfileOptimizer(prof, coverage=0.9, max_variants=4)
    st = opt.statistics("linear")
    assert st.calls == 100 and st.distinct_shapes == 7 and st.most_common == (8, 4096) and st.most_common_share == 0.6 and st.dynamic_dims == (0,)
    assert st.min_dims == (3, 4096) and st.max_dims == (200, 4096)
    plan = opt.plan("linear")
    assert plan.specialize[:2] == [(8, 4096), (64, 4096)] and plan.expected_hit_rate >= 0.9 and plan.bucket_dims == {0: [4, 8, 16, 32, 64, 128, 200]}
    built = []
    assert opt.apply(None, "linear", built.append) == len(plan.specialize) and built == plan.specialize
    prof.record("rare", (1,))
    assert opt.plan("rare") is None and set(opt.plan_all()) == {"linear"} and opt.statistics("none") is None
