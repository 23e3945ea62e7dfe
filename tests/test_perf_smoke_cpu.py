"""Throughput / latency smoke tests on the host with loose bounds: they assert that the measuring paths work and that
obviously wrong behaviour (serial instead of batched, quadratic instead of linear) shows up, not absolute speed."""
import time

import torch

from ml_framework_b200.data.loader import DataLoader, DataLoaderConfig, TensorDataset
from ml_framework_b200.data.workers import SharedQueue, WorkerPool
from ml_framework_b200.dist.algorithms import RabenseifnerAllReduce, RecursiveDoublingAllReduce
from ml_framework_b200.dist.process_group import run_fake_world
from ml_framework_b200.serving.scheduler import BatchOutput, ContinuousBatchScheduler, Request, SchedulerConfiguration


class _Exec:
    def __init__(self, step_s):
        self.step_s, self.calls = step_s, 0

    def execute_batch(self, batch):
        self.calls += 1
        time.sleep(self.step_s)                      # one model step costs the same for 1 or 8 requests
        out = {}
        for r in batch.requests:
            r.prefilled = len(r.prompt_tokens)
            out[r.id] = 2 if len(r.generated) + 1 >= 8 else 100
        return BatchOutput(out)


def test_continuous_batching_throughput_scales_with_batch_size():
    rates = {}
    for bs in (1, 8):
        ex = _Exec(0.002)
        s = ContinuousBatchScheduler(ex, None, SchedulerConfiguration(max_batch_size=bs))
        futs = [s.enqueue(Request([1, 2, 3], max_tokens=16)) for _ in range(16)]
        t0 = time.perf_counter()
        s.run_until_idle()
        dt = time.perf_counter() - t0
        res = [f.result(0) for f in futs]
        rates[bs] = sum(len(r.tokens) for r in res) / dt
        snap = s.metrics.snapshot()
        assert snap["completed"] == 16 and snap["iteration_ms_p50"] >= 2.0 and all(r.latency_s >= r.ttft_s > 0 for r in res)
    assert rates[8] > 3 * rates[1]


def test_loader_workers_hide_per_sample_latency():
    class Slow(TensorDataset):
        def __getitem__(self, i):
            time.sleep(0.002)
            return super().__getitem__(i)
    ds = Slow(torch.arange(64).float())
    times = {}
    for workers in (0, 4):
        loader = DataLoader(ds, DataLoaderConfig(batch_size=8, num_workers=workers))
        t0 = time.perf_counter()
        n = sum(b[0].shape[0] for b in loader)
        times[workers] = time.perf_counter() - t0
        assert n == 64
    assert times[4] < 0.7 * times[0]


def test_worker_pool_and_queue_sustain_a_reasonable_rate():
    q = SharedQueue(1024)
    t0 = time.perf_counter()
    for i in range(20_000):
        q.enqueue(i)
        q.dequeue()
    assert 20_000 / (time.perf_counter() - t0) > 20_000                 # > 20 K round trips per second on one thread
    with WorkerPool(lambda x, c: x + 1, num_workers=4) as pool:
        t0 = time.perf_counter()
        out = list(pool.map(range(2000)))
        assert out == list(range(1, 2001)) and 2000 / (time.perf_counter() - t0) > 1000


def test_bandwidth_optimal_algorithm_sends_fewer_bytes_than_the_latency_optimal_one():
    def run(pg):
        a, b = RecursiveDoublingAllReduce(pg), RabenseifnerAllReduce(pg)
        a.all_reduce(torch.ones(1 << 14))
        b.all_reduce(torch.ones(1 << 14))
        return a.bytes_sent, a.steps, b.bytes_sent, b.steps
    for rd_bytes, rd_steps, rab_bytes, rab_steps in run_fake_world(8, run):
        assert rd_steps == 3 and rab_steps == 6 and rab_bytes < 0.6 * rd_bytes
