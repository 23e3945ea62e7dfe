"""Queues, prefetch, worker pool with supervision, object / array / tensor pools, extra datasets, async loader, loading metrics."""
import asyncio
import threading
import time

import numpy as np
import pytest
import torch

from ml_framework_b200.data import workers as W
from ml_framework_b200.data.loader import (AdvancedDataLoader, ArrayDataset, DataLoaderConfig, InMemoryDataset, TensorDataset, dict_collate,
                                           stack_collate)
from ml_framework_b200.obs.metrics import DataLoadingMetrics, MetricsCollector, PerformanceCounter, ProfilingScope


def test_shared_queue_blocks_times_out_batches_and_completes():
    q = W.SharedQueue(2)
    q.enqueue(1)
    q.enqueue(2)
    assert not q.try_enqueue(3, timeout_ms=20) and len(q) == 2 and q.try_peek() == (True, 1)
    got = []
    t = threading.Thread(target=lambda: got.extend(q.dequeue() for _ in range(3)))
    t.start()
    q.enqueue(3)                                  # room appears once the consumer starts taking
    t.join(timeout=5)
    assert got == [1, 2, 3] and q.try_dequeue(10) == (False, None)
    q.enqueue_batch([4, 5])
    assert q.dequeue_batch(5, timeout_ms=30) == [4, 5]
    q.enqueue(6)
    q.complete_adding()
    with pytest.raises(W.QueueClosed):
        q.enqueue(7)
    assert not q.is_completed and list(q) == [6] and q.is_completed and q.wait_for_completion(0.5)
    with pytest.raises(W.QueueClosed):
        q.dequeue()
    s = q.statistics()
    assert (s.enqueued, s.dequeued, s.max_size, s.capacity) == (6, 6, 2, 2) and s.average_consumer_wait_ms >= 0
    q2 = W.SharedQueue(4, enable_statistics=False)
    q2.enqueue("x")
    q2.shutdown()
    assert len(q2) == 0 and q2.statistics().enqueued == 0 and "complete=True" in repr(q2)
    with pytest.raises(ValueError):
        W.SharedQueue(0)


def test_prefetch_buffer_and_strategy():
    b = W.PrefetchBuffer(2)
    b.add(1)
    b.add(2)
    with pytest.raises(OverflowError):
        b.add(3)
    assert b.peek() == 1 and b.get_next() == 1 and b.try_get() == (True, 2) and b.try_get() == (False, None)
    with pytest.raises(IndexError):
        b.get_next()
    q = W.SharedQueue(16)
    q.enqueue_batch(range(6))
    p = W.SimplePrefetchStrategy(q, 3)
    assert p.prefetch() == 3 and len(p.buffer) == 3 and len(q) == 3
    assert [p.get_next() for _ in range(6)] == list(range(6))
    st = p.statistics()
    assert st.requests == 6 and st.hits == 6 and st.hit_rate == 1.0 and st.prefetched == 6
    with pytest.raises(TimeoutError):
        p.get_next(timeout_ms=10)
    assert p.statistics().misses == 1
    p.reset()
    assert p.statistics().requests == 0


def test_crash_detector_recovery_and_timeout_tracker():
    det = W.WorkerCrashDetector(heartbeat_timeout_s=0.05)
    seen = []
    det.on_crash.append(lambda w, why: seen.append((w, why.split(" for")[0])))
    t = threading.Thread(target=lambda: None)
    t.start()
    t.join()
    det.register_worker(0, t)                     # its thread is already gone
    det.register_worker(1)
    det.register_worker(2)
    time.sleep(0.08)
    det.update_heartbeat(2)
    assert det.time_since_last_heartbeat(2) < 0.05 and det.time_since_last_heartbeat(9) is None
    assert sorted(det.check_now()) == [(0, "thread ended"), (1, det.crashes[1][1])] and det.registered_worker_count() == 1
    assert seen == [(0, "thread ended"), (1, "no heartbeat")] and det.check_now() == []
    det.start_monitoring()
    det.stop_monitoring()

    slept = []
    rec = W.WorkerRecoveryService(max_retries=2, restart_delay_s=0.5, backoff=3.0, sleep=slept.append)
    started = []
    assert rec.try_restart(7, started.append) and rec.try_restart(7, started.append)
    assert slept == [0.5, 1.5] and started == [7, 7] and rec.remaining_retries(7) == 0 and not rec.can_restart(7)
    assert not rec.try_restart(7, started.append) and rec.is_worker_failed(7) and rec.failed_workers() == [7]

    def bad(_):
        raise OSError("no")
    assert not rec.try_restart(8, bad) and rec.retry_count(8) == 1 and not rec.is_worker_failed(8)
    assert not rec.try_restart(8, bad) and rec.is_worker_failed(8) and rec.failed_worker_count() == 2
    assert "2 failed for good: [7, 8]" in rec.recovery_summary()
    rec.reset_worker(7)
    assert rec.can_restart(7)
    rec.mark_worker_failed(3)
    rec.reset_all()
    assert rec.failed_workers() == []

    tr = W.WorkerTimeoutTracker(timeout_s=0.03)
    late = []
    tr.on_timeout.append(lambda w, el: late.append(w))
    tr.start_operation(1)
    tr.start_operation(2)
    assert tr.end_operation(2) < 0.03 and tr.end_operation(5) is None
    time.sleep(0.05)
    assert [w for w, _ in tr.check_now()] == [1] and tr.check_now() == [] and late == [1]
    assert tr.is_tracking(1) and tr.active_worker_count() == 1 and "worker 1" in tr.tracking_summary() and tr.elapsed(1) > 0.03
    tr.clear_all()
    assert tr.active_worker_count() == 0


def test_worker_pool_orders_results_retries_failures_and_reports_errors():
    inits = []
    with W.WorkerPool(lambda x, ctx: (x * x, ctx.worker_id), num_workers=3, init_fn=lambda c: inits.append(c.seed), seed=100) as pool:
        out = list(pool.map(range(20)))
    assert [v for v, _ in out] == [i * i for i in range(20)] and sorted(inits) == [100, 101, 102]
    assert sum(pool.completed_by_worker.values()) == 20

    flaky = {"n": 0}

    def sometimes(x, ctx):
        if x == 3 and flaky["n"] < 2:
            flaky["n"] += 1
            raise RuntimeError("transient")
        return x
    pool = W.WorkerPool(sometimes, num_workers=1, recovery=W.WorkerRecoveryService(max_retries=2))
    assert sorted(pool.map(range(5), ordered=False)) == [0, 1, 2, 3, 4] and flaky["n"] == 2
    pool.shutdown()

    def always(x, ctx):
        if x == 1:
            raise ValueError("bad sample")
        return x
    pool = W.WorkerPool(always, num_workers=2, recovery=W.WorkerRecoveryService(max_retries=1),
                        timeouts=W.WorkerTimeoutTracker(), crash_detector=W.WorkerCrashDetector())
    it = pool.map([0, 1, 2])
    assert next(it) == 0
    with pytest.raises(ValueError, match="bad sample"):
        next(it)
    pool.shutdown()
    assert pool.crash_detector.registered_worker_count() == 0
    empty = W.WorkerPool(lambda x, c: x, 1)
    empty.start()
    with pytest.raises(TimeoutError):
        next(empty.results(1, timeout_s=0.05))
    empty.shutdown()


def test_pools_reuse_and_report():
    made = []
    pool = W.ObjectPool(lambda: made.append(1) or [], reset=lambda l: l.clear(), max_size=1, initial=1)
    a = pool.rent()
    b = pool.rent()
    a.append(5)
    pool.give_back(a)
    pool.give_back(b)
    c = pool.rent()
    s = pool.statistics()
    assert c == [] and c is a and (s.rents, s.created, s.returns, s.discarded, s.available) == (3, 2, 2, 1, 0) and abs(s.hit_rate - 1 / 3) < 1e-9
    ap = W.ArrayPool(np.float32)
    x = ap.rent(100, clear=True)
    assert x.shape == (100,) and x.base.shape == (128,) and not x.any()
    ap.give_back(x)
    y = ap.rent(120)
    assert y.base is x.base and ap.statistics().created == 1
    ap.give_back(np.zeros(100, np.float32))       # not a pool array: discarded
    assert ap.statistics().discarded == 1
    tp = W.TensorPool(max_per_key=1)
    t1 = tp.rent((4, 8), torch.bfloat16)
    tp.give_back(t1)
    assert tp.rent((4, 8), torch.bfloat16) is t1 and tp.rent((4, 8), torch.float32) is not t1
    mgr = W.PoolManager()
    mgr.register("objs", pool)
    mgr.register("tensors", tp)
    assert mgr.get_or_create("arrays", lambda: ap) is ap and mgr.names() == ["arrays", "objs", "tensors"]
    with pytest.raises(KeyError):
        mgr.register("objs", pool)
    assert "tensors: 3 rents, 2 created" in mgr.report() and mgr.statistics()["objs"].rents == 3
    mgr.clear_all()
    assert mgr.remove("arrays") and not mgr.remove("arrays")


def test_array_and_in_memory_datasets_and_collates():
    ds = ArrayDataset(np.arange(12, dtype=np.float32).reshape(4, 3), np.array([0, 1, 0, 1]))
    x, y = ds[2]
    assert len(ds) == 4 and x.tolist() == [6.0, 7.0, 8.0] and int(y) == 0
    assert ArrayDataset(np.arange(3))[1].item() == 1
    with pytest.raises(ValueError):
        ArrayDataset(np.zeros(3), np.zeros(4))
    calls = []
    mem = InMemoryDataset((i for i in range(10)), transform=lambda v: calls.append(v) or v * 2, limit=4)
    assert len(mem) == 4 and mem[3] == 6 and mem[3] == 6 and calls == [0, 1, 2, 3]
    assert len(InMemoryDataset(TensorDataset(torch.arange(5)))) == 5
    assert stack_collate([torch.zeros(2), torch.ones(2)]).shape == (2, 2)
    with pytest.raises(ValueError):
        stack_collate([torch.zeros(2), torch.zeros(3)])
    with pytest.raises(TypeError):
        stack_collate([1, 2])
    d = dict_collate([{"x": torch.zeros(2), "id": 1}, {"x": torch.ones(2), "id": 2}], per_key={"id": list})
    assert d["x"].shape == (2, 2) and d["id"] == [1, 2]
    with pytest.raises(KeyError):
        dict_collate([{"a": 1}, {"b": 2}])


def test_advanced_loader_async_iteration():
    ds = TensorDataset(torch.arange(10).float())
    loader = AdvancedDataLoader(ds, DataLoaderConfig(batch_size=4, num_workers=2))

    async def run():
        sizes = [b[0].shape[0] async for b in loader]
        first = await loader.next_batch_async()
        rest = [await loader.next_batch_async() for _ in range(3)]
        return sizes, first, rest
    sizes, first, rest = asyncio.run(run())
    assert sizes == [4, 4, 2] and first[0].tolist() == [0.0, 1.0, 2.0, 3.0] and rest[2] is None and rest[1][0].shape[0] == 2


def test_performance_counter_scope_and_loading_metrics():
    c = PerformanceCounter("fetch")
    for v in (0.2, 0.1, 0.3):
        c.record(v)
    d = c.as_dict()
    assert d["count"] == 3 and abs(d["mean_s"] - 0.2) < 1e-9 and d["min_s"] == 0.1 and d["max_s"] == 0.3 and d["last_s"] == 0.3
    c.reset()
    assert c.as_dict()["min_s"] == 0.0
    with pytest.raises(ZeroDivisionError):
        with ProfilingScope(c):
            1 / 0
    assert c.count == 1
    col = MetricsCollector()
    with ProfilingScope(col, "blk") as sc:
        pass
    assert col.snapshot()["timings"]["blk"]["count"] == 1 and sc.elapsed_s >= 0
    m = DataLoadingMetrics()
    with m.scope("fetch"):
        time.sleep(0.01)
    with m.scope("wait"):
        time.sleep(0.03)
    m.record_batch(32, queue_depth=2)
    m.record_batch(32, queue_depth=4)
    snap = m.snapshot()
    assert snap["batches"] == 2 and snap["samples"] == 64 and snap["mean_queue_depth"] == 3.0 and snap["samples_per_second"] > 0
    assert snap["wait_fraction"] > 0.1 and snap["bottleneck"] == "loader:fetch"
    m.publish(col)
    s = col.snapshot()
    assert s["counters"]["data.batches"] == 2.0 and s["gauges"]["data.fetch_mean_ms"] >= 10.0
    idle = DataLoadingMetrics()
    assert idle.bottleneck() == "consumer"
