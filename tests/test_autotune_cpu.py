"""Launch-configuration autotuning on a synthetic cost surface: strategies, cache, failures, records."""
import math

import pytest
import torch

from ml_framework_b200.compiler import autotune as AT


class FakeProfiler(AT.WallClockProfiler):
    """Reports the cost the operation computed for the configuration instead of a clock reading."""

    def __init__(self, box):
        super().__init__()
        self.box = box

    def measure_execution(self, action):
        action()
        return self.box["ms"]


def _op(box, calls, bad=()):
    def run(cfg, x):
        calls.append(cfg.key())
        if cfg.block_dim.x in bad:
            raise RuntimeError("too many resources requested for launch")
        # a bowl in log2 space with its minimum at 128 threads, y = 2, unroll 4
        box["ms"] = 1.0 + (math.log2(cfg.block_dim.x) - 7) ** 2 + 0.5 * (math.log2(cfg.block_dim.y) - 1) ** 2 \
            + 0.25 * (math.log2(cfg.parameter("unroll")) - 2) ** 2
    return AT.TunableOperation("bowl", 1 << 20, bytes_moved=8 << 20, input_shapes=((4,),), knobs={"unroll": (1, 2, 4, 8)}, run=run)


def _tuner(box):
    dev = AT.DeviceQuery.B200
    return AT.KernelAutotuner(benchmark_runner=AT.BenchmarkRunner(FakeProfiler(box), dev))


def test_device_query_and_configuration_records():
    d = AT.DeviceQuery().get_current_device_info()
    assert d.sm_count > 0 and d.key().count("|") == 2
    g = AT.SearchSpaceGenerator()
    op = AT.TunableOperation("x", 1000, shared_memory_bytes=1 << 30)
    c = g.create_configuration(op, 128, 2, 1, AT.DeviceQuery.B200, (("unroll", 2),))
    assert c.block_dim.total() == 256 and c.grid_dim.x == 4 and c.shared_memory_bytes == 227 * 1024 and c.parameter("unroll") == 2
    big = g.create_configuration(AT.TunableOperation("x", 1 << 40), 32, 1, 1, AT.DeviceQuery.B200)
    assert big.grid_dim.x == 148 * 32
    assert AT.KernelLaunchConfiguration.from_json(c.to_json()) == c
    space = g.full_grid(AT.TunableOperation("x", 10, knobs={"u": (1, 2)}), AT.DeviceQuery.B200)
    assert len(space) == (5 * 4 - 3) * 2                      # 256x8, 512x4, 512x8 exceed 1024 threads
    assert AT.WallClockProfiler.measure_sm_utilization(c, AT.DeviceQuery.B200) == 0
    assert AT.WallClockProfiler.measure_sm_utilization(big, AT.DeviceQuery.B200) == 50


def test_grid_search_finds_the_minimum_and_caches():
    box, calls = {}, []
    t = _tuner(box)
    op = _op(box, calls)
    r = t.tune(op, AT.AutotuningOptions(warmup_runs=1, measurement_runs=1))
    best = r.best_configuration
    assert (best.block_dim.x, best.block_dim.y, best.parameter("unroll")) == (128, 2, 4) and r.best_execution_time_ms == 1.0
    assert not r.cache_hit and len(r.benchmarks) == 68 and r.benchmarks[0].memory_bandwidth_gbps == pytest.approx(8 * 2 ** 20 / 1e-3 / 1e9)
    n = len(calls)
    again = t.tune(op)
    assert again.cache_hit and again.best_configuration == best and len(calls) == n
    assert t.cache.count == 1 and t.cache.contains(op, AT.DeviceQuery.B200) and t.cache.remove(op, AT.DeviceQuery.B200)
    with pytest.raises(ValueError):
        t.tune(AT.TunableOperation("norun", 1))


@pytest.mark.parametrize("strategy,budget,slack", [(AT.SearchStrategy.RANDOM_SEARCH, 20, 2.5),
                                                   (AT.SearchStrategy.BAYESIAN_OPTIMIZATION, 16, 0.26),
                                                   (AT.SearchStrategy.GENETIC_ALGORITHM, 24, 1.01)])
def test_budgeted_strategies_stay_within_budget_and_get_close(strategy, budget, slack):
    box, calls = {}, []
    t = _tuner(box)
    r = t.tune(_op(box, calls), AT.AutotuningOptions(max_iterations=budget, warmup_runs=0, measurement_runs=1, search_strategy=strategy, seed=3))
    assert len(r.benchmarks) <= budget and len(set(calls)) == len(r.benchmarks)
    assert r.best_execution_time_ms <= 1.0 + slack, (strategy, r.best_execution_time_ms)


def test_model_based_search_beats_random_on_average():
    def best_of(strategy, seed):
        box, calls = {}, []
        return _tuner(box).tune(_op(box, calls), AT.AutotuningOptions(max_iterations=12, warmup_runs=0, measurement_runs=1,
                                                                      search_strategy=strategy, seed=seed)).best_execution_time_ms
    model = sum(best_of(AT.SearchStrategy.BAYESIAN_OPTIMIZATION, s) for s in range(5)) / 5
    rand = sum(best_of(AT.SearchStrategy.RANDOM_SEARCH, s) for s in range(5)) / 5
    assert model < rand


def test_failing_configurations_are_skipped_and_all_failing_raises():
    box, calls = {}, []
    t = _tuner(box)
    r = t.tune(_op(box, calls, bad=(128, 256, 512)), AT.AutotuningOptions(warmup_runs=0, measurement_runs=1))
    assert r.best_configuration.block_dim.x == 64 and len(t.runner.failures) == (4 + 3 + 2) * 4
    with pytest.raises(RuntimeError, match="no configuration"):
        _tuner(box).tune(_op(box, [], bad=(32, 64, 128, 256, 512)))


def test_file_cache_survives_a_restart(tmp_path):
    box, calls = {}, []
    path = str(tmp_path / "tune.json")
    dev = AT.DeviceQuery.B200
    t1 = AT.KernelAutotuner(cache=AT.FileTuningCache(path), benchmark_runner=AT.BenchmarkRunner(FakeProfiler(box), dev))
    op = _op(box, calls)
    first = t1.tune(op, AT.AutotuningOptions(warmup_runs=0, measurement_runs=1))
    n = len(calls)
    t2 = AT.KernelAutotuner(cache=AT.FileTuningCache(path), benchmark_runner=AT.BenchmarkRunner(FakeProfiler(box), dev))
    second = t2.tune(op)
    assert second.cache_hit and second.best_configuration == first.best_configuration and len(calls) == n
    other = _op(box, calls)
    other.output_elements = 1 << 10                     # another size is another entry
    assert not t2.tune(other, AT.AutotuningOptions(warmup_runs=0, measurement_runs=1)).cache_hit and t2.cache.count == 2
    t2.cache.clear()
    assert AT.FileTuningCache(path).count == 0


def test_wall_clock_runner_on_a_real_callable_and_tensor_generator():
    gen = AT.TensorGenerator(seed=1)
    assert gen.generate_random_tensor((3, 2), torch.int32).dtype == torch.int32
    x = gen.generate_random_tensor((256, 256))

    def run(cfg, a):
        (a @ a) if cfg.block_dim.x == 32 else a.sum()
    op = AT.TunableOperation("real", x.numel(), bytes_moved=x.numel() * 4, input_shapes=((256, 256),), block_x=(32, 64), block_y=(1,), run=run)
    r = AT.KernelAutotuner().tune(op, AT.AutotuningOptions(warmup_runs=2, measurement_runs=5))
    assert r.best_configuration.block_dim.x == 64 and r.benchmarks[0].execution_time_ms > 0
    with pytest.raises(ValueError):
        AT.tune_fused_elementwise(None, [x])
