"""Error policies, device-side transforms, stream replication, prefetching iterable data sets, statistics, pinned memory."""
import io
import threading
import time

import pytest
import torch

from ml_framework_b200.data import extras as X


def test_error_policies():
    def flaky(n, fails={"left": 2}):
        if n == 3:
            raise ValueError("bad sample")
        if n == 5 and fails["left"] > 0:
            fails["left"] -= 1
            raise IOError("transient")
        return n * 10

    with pytest.raises(ValueError):
        list(X.ErrorPolicyHandler(X.ErrorPolicy.FAIL_FAST).map(flaky, range(6)))
    buf = io.StringIO()
    log = X.ConsoleErrorLogger(buf, clock=lambda: 0.0)
    h = X.ErrorPolicyHandler(X.ErrorPolicy.CONTINUE, logger=log)
    assert list(h.map(flaky, range(5))) == [0, 10, 20, 40] and h.skipped == 1 and h.errors[0][0] == 3
    assert "[1970-01-01 00:00:00] [data] ERROR: skipping item after error: bad sample (ValueError: bad sample)" in buf.getvalue()
    log.log_warning("slow", worker_id=2); log.log_info("ok")
    assert "[data worker 2] WARNING: slow" in buf.getvalue() and log.counts == {"error": 1, "warning": 1, "info": 1}
    ig = X.ErrorPolicyHandler(X.ErrorPolicy.IGNORE)
    assert list(ig.map(flaky, [2, 3, 4])) == [20, 40] and ig.errors == [] and ig.skipped == 1
    rs = X.ErrorPolicyHandler(X.ErrorPolicy.RESTART, max_restarts=3)
    assert rs.run(flaky, 5) == (True, 50) and rs.restarts == 2
    with pytest.raises(RuntimeError, match="failed 2 times"):
        X.ErrorPolicyHandler(X.ErrorPolicy.RESTART, max_restarts=1).run(flaky, 3)
    assert [s.value for s in X.DynamicBatchStrategy] == ["pad_to_max", "bucket", "dynamic"]


def test_device_transforms_and_lanczos():
    n = X.GpuNormalizeTransform([0.5, 0.25], [0.5, 0.25])
    x = torch.rand(2, 4, 4)
    torch.testing.assert_close(n(x)[1], (x[1] - 0.25) / 0.25)
    assert n(torch.rand(3, 2, 4, 4)).shape == (3, 2, 4, 4) and n(torch.ones(2, 4, 4, dtype=torch.uint8)).dtype == torch.float32
    n.set_gpu_device(1)
    assert n.gpu_device == 1 and n.gpu_available == (torch.cuda.is_available() and torch.cuda.device_count() > 1)
    for bad in (lambda: X.GpuNormalizeTransform([0.5], [0.0]), lambda: X.GpuNormalizeTransform([0.5], [1.0, 1.0]), lambda: n(torch.rand(3, 4, 4)),
                lambda: n.set_gpu_device(-1)):
        with pytest.raises(ValueError):
            bad()
    with pytest.raises(TypeError):
        n([1, 2])
    img = torch.rand(3, 16, 12)
    for mode in X.InterpolationMode:
        out = X.GpuResizeTransform(6, 8, mode)(img)
        assert out.shape == (3, 8, 6), mode
    assert X.GpuResizeTransform(24, 32)(img[None]).shape == (1, 3, 32, 24)
    # Lanczos: constants stay constant, the identity size is the identity, a smooth ramp stays a ramp when enlarged
    const = torch.full((1, 9, 7), 3.0)
    torch.testing.assert_close(X.lanczos_resize(const, (5, 11)), torch.full((1, 5, 11), 3.0))
    torch.testing.assert_close(X.lanczos_resize(img, (16, 12)), img, atol=1e-6, rtol=0)
    ramp = torch.arange(32, dtype=torch.float32).repeat(4, 1)[None]
    up = X.lanczos_resize(ramp, (4, 64))[0, 0]
    want = (torch.arange(64, dtype=torch.float32) + 0.5) / 2 - 0.5
    assert (up[8:-8] - want[8:-8]).abs().max() < 0.02
    # shrinking low-passes: an alternating pattern averages out instead of aliasing
    stripes = torch.tensor([0.0, 1.0] * 32).repeat(2, 1)[None]
    small = X.lanczos_resize(stripes, (2, 8))
    assert (small[..., 1:-1] - 0.5).abs().max() < 0.02 and (small - 0.5).abs().max() < 0.1     # the repeated border sample biases the ends
    with pytest.raises(ValueError):
        X.GpuResizeTransform(0, 4)
    with pytest.raises(TypeError):
        X.GpuResizeTransform(4, 4)(torch.rand(4, 4))


def test_stream_replicator_splits_by_stride_even_with_uneven_readers():
    rep = X.StreamReplicator(iter(range(20)), 3, max_buffered=2)
    streams = [rep.get_replica_stream(r) for r in range(3)]
    out = [[], [], []]

    def read(r, delay):
        for v in streams[r]:
            out[r].append(v)
            time.sleep(delay)
    ts = [threading.Thread(target=read, args=(r, d)) for r, d in enumerate((0.0, 0.002, 0.0005))]
    [t.start() for t in ts]; [t.join(20) for t in ts]
    assert out == [list(range(0, 20, 3)), list(range(1, 20, 3)), list(range(2, 20, 3))]
    with pytest.raises(RuntimeError):
        rep.get_replica_stream(0)
    with pytest.raises(IndexError):
        rep.get_replica_stream(3)
    with pytest.raises(ValueError):
        X.StreamReplicator(range(3), 0)
    one = X.StreamReplicator(range(4), 1)
    assert list(one.get_replica_stream(0)) == [0, 1, 2, 3]


def test_optimized_iterable_dataset_prefetches_batches_and_propagates_errors():
    ds = X.OptimizedIterableDataset(lambda: range(10), buffer_size=2, transform=lambda v: v * 2, batch_size=4, collate=torch.tensor)
    batches = list(ds)
    assert [b.tolist() for b in batches] == [[0, 2, 4, 6], [8, 10, 12, 14], [16, 18]] and ds.items_read == 10
    assert [b.tolist() for b in ds][0] == [0, 2, 4, 6] and ds.items_read == 20       # a second epoch restarts the source
    plain = X.OptimizedIterableDataset(lambda: iter("abc"))
    assert list(plain) == ["a", "b", "c"]

    def broken():
        yield 1
        raise OSError("disk gone")
    with pytest.raises(OSError, match="disk gone"):
        list(X.OptimizedIterableDataset(broken))
    # leaving early stops the producer
    started = threading.active_count()
    it = iter(X.OptimizedIterableDataset(lambda: iter(range(10 ** 9)), buffer_size=4))
    assert next(it) == 0
    it.close()
    time.sleep(0.2)
    assert threading.active_count() <= started
    for bad in (lambda: X.OptimizedIterableDataset(range, buffer_size=0), lambda: X.OptimizedIterableDataset(range, batch_size=0)):
        with pytest.raises(ValueError):
            bad()


def test_statistics_tracker():
    now = [0.0]

    def slow_batches():
        for i in range(4):
            now[0] += 0.010 if i % 2 else 0.0002          # every second batch makes the consumer wait
            yield torch.zeros(8, 3)
    tr = X.StatisticsTracker(clock=lambda: now[0])
    assert len(list(tr.track(slow_batches()))) == 4
    st = tr.statistics(X.QueueStatistics(capacity=4, average_depth=1.5))
    assert st.batches_loaded == 4 and st.total_samples == 32 and st.prefetch_statistics.hits == 2 and st.prefetch_statistics.hit_rate == 0.5
    assert st.average_batch_time_ms == pytest.approx((0.0002 * 2 + 0.010 * 2) / 4 * 1e3) and st.throughput_samples_per_second == pytest.approx(32 / 0.0204)
    assert "prefetch hit rate 50 %" in str(st) and "queue depth 1.5/4" in str(st)
    assert X.StatisticsTracker._guess({"ids": torch.zeros(5, 2)}) == 5 and X.StatisticsTracker._guess((torch.zeros(7), 1)) == 7
    assert X.StatisticsTracker._guess([1, 2, 3]) == 3 and X.StatisticsTracker().statistics().batches_loaded == 0


def test_worker_pool_factory():
    assert 1 <= X.WorkerPoolFactory.optimal_worker_count() <= 32
    pool = X.WorkerPoolFactory.create(lambda task, ctx: task + 1, 2)
    pool.start()
    for i in range(5):
        pool.submit(i)
    assert sorted(pool.results(5)) == [1, 2, 3, 4, 5]
    pool.shutdown()


def test_pinning_strategy_buffers_and_allocator():
    S, P = X.PinningStrategySelector, X.PinningStrategy
    assert S.select_strategy_by_byte_size(512, 100) is P.NONE and S.select_strategy_by_byte_size(4096, 1) is P.PIN_IN_PLACE
    assert S.select_strategy_by_byte_size(4096, 10) is P.PINNED_POOL and S.select_strategy_by_byte_size(2 << 20, 2) is P.ALLOCATE_PINNED
    assert S.select_strategy_by_byte_size(2 << 20, 50) is P.PINNED_POOL and S.select_strategy(1024, torch.float32, 0) is P.PIN_IN_PLACE
    for bad in (lambda: S.select_strategy_by_byte_size(0, 1), lambda: S.select_strategy_by_byte_size(10, -1), lambda: S.select_strategy(0, torch.float32, 1)):
        with pytest.raises(ValueError):
            bad()
    t = torch.arange(2048, dtype=torch.float32)
    assert S.create_pinned_memory(t, P.NONE) is None
    a = S.create_pinned_memory(t, P.PIN_IN_PLACE)
    b = S.create_pinned_memory(t, P.ALLOCATE_PINNED)
    assert torch.equal(a.tensor, t) and torch.equal(b.tensor, t) and b.tensor.data_ptr() != t.data_ptr()
    assert a.is_pinned == torch.cuda.is_available()
    from ml_framework_b200.data.loader import PinnedMemoryPool
    pool = PinnedMemoryPool()
    with S.create_pinned_memory(t, P.PINNED_POOL, pool) as c:
        assert torch.equal(c.tensor, t)
    again = S.create_pinned_memory(t * 2, P.PINNED_POOL, pool)
    assert pool.reuses == 1 and float(again.tensor[1]) == 2.0
    with pytest.raises(ValueError):
        S.create_pinned_memory(t, P.PINNED_POOL)
    buf = X.PinnedBuffer.allocate(8)
    buf.copy_from(torch.arange(20.0), source_offset=4)
    dst = torch.zeros(12)
    buf.copy_to(dst, destination_offset=2)
    assert dst.tolist() == [0, 0, 4, 5, 6, 7, 8, 9, 10, 11, 0, 0] and buf.length == 8 and buf.pointer != 0
    buf.fill(7.0)
    assert float(buf.to_device("cpu").sum()) == 56.0
    with pytest.raises(ValueError):
        buf.copy_from(torch.zeros(3))
    with pytest.raises(ValueError):
        buf.copy_to(torch.zeros(3))
    buf.release()
    with pytest.raises(RuntimeError):
        buf.tensor
    with X.PinnedMemoryAllocator() as alloc:
        m = alloc.allocate(16)
        alloc.copy_to_pinned_memory(m, b"hello world", offset=6)
        assert alloc.copy_from_pinned_memory(m, 5) == b"world" and alloc.live_buffers == 1 and alloc.total_allocated_bytes == 16
        with pytest.raises(ValueError):
            alloc.copy_to_pinned_memory(m, b"x" * 40)
        alloc.free(m)
        with pytest.raises(KeyError):
            alloc.free(m)
        alloc.allocate(4)
    assert alloc.live_buffers == 0
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            X.PinnedMemoryAllocator(force_pinned=True)
