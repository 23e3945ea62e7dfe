"""Mobile runtime: extra tensor operators, per-operator profile, benchmark runner with monitors, profiler, exporters, comparator."""
import json

import pytest
import torch

from ml_framework_b200.mobile import benchmarking as MB
from ml_framework_b200.mobile.format import MobModel, MobOperator, MobTensor
from ml_framework_b200.mobile.runtime import MobileRuntime


def _model():
    ops = [MobOperator("matmul", ["x", "w"], ["h"]), MobOperator("sub", ["h", "b"], ["h2"]), MobOperator("abs", ["h2"], ["a"]),
           MobOperator("sqrt", ["a"], ["s"]), MobOperator("square", ["s"], ["q"]), MobOperator("transpose", ["q"], ["t"], {"perm": [1, 0]}),
           MobOperator("max", ["t"], ["m"], {"axis": 0, "keepdims": True}), MobOperator("div", ["t", "m"], ["d"]),
           MobOperator("mean", ["d"], ["mu"], {"axis": 1}), MobOperator("sum", ["mu"], ["tot"]), MobOperator("cast", ["tot"], ["i"], {"dtype": "int32"}),
           MobOperator("copy", ["d"], ["dc"]), MobOperator("exp", ["dc"], ["e"]), MobOperator("log", ["e"], ["l"]), MobOperator("min", ["l"], ["lo"], {"axis": 1})]
    return MobModel([{"name": "x", "shape": [3, 4]}], ["i", "l", "lo"], ops,
                    {"w": MobTensor("w", torch.arange(20.0).reshape(4, 5) / 10), "b": MobTensor("b", torch.full((5,), 0.5))})


def test_tensor_operator_set_matches_torch():
    rt = MobileRuntime("cpu").load_model(_model())
    x = torch.arange(12.0).reshape(3, 4) / 7
    i, l, lo = rt.predict(x)
    a = (x @ (torch.arange(20.0).reshape(4, 5) / 10) - 0.5).abs()
    t = a.sqrt().square().t()
    d = t / t.amax(0, keepdim=True)
    assert i.dtype == torch.int32 and int(i) == int(d.mean(1).sum()) and torch.allclose(l, d, atol=1e-6) and torch.allclose(lo, d.amin(1), atol=1e-6)
    prof = rt.profile_operators(x, iters=2)
    assert len(prof) == 15 and abs(sum(r["share"] for r in prof) - 1.0) < 1e-9 and prof[0]["mean_ms"] >= prof[-1]["mean_ms"]
    with pytest.raises(RuntimeError):
        MobileRuntime("cpu").profile_operators(x)


def test_runner_with_monitors_and_suite():
    mem_values = iter([100, 150, 400, 250, 250, 250, 250, 250, 250])
    mem = MB.MemoryMonitor(1000, reader=lambda: next(mem_values))
    t = {"now": 0.0}
    power = iter([100.0, 300.0, 200.0, 200.0, 200.0])

    def clock():
        t["now"] += 0.5
        return t["now"]
    en = MB.EnergyMonitor(1000, power_reader=lambda: next(power), clock=clock)
    calls = []
    r = MB.BenchmarkRunner(mem, en).run_benchmark("f", lambda: calls.append(1), iterations=4, warmup=2)
    assert len(calls) == 6 and len(r.times_ms) == 4 and r.min_ms <= r.median_ms <= r.max_ms and r.std_ms >= 0
    assert (r.memory.samples, r.memory.start_bytes, r.memory.peak_bytes, r.memory.end_bytes, r.memory.growth_bytes) == (2, 100, 150, 150, 50)
    assert r.energy.samples == 2 and r.energy.energy_joules == 0.5 * (100 + 300) * 0.5 and r.energy.average_power_w == 200.0 and r.energy.peak_power_w == 300.0
    assert r.energy_per_iteration_j == 25.0 and r.row()["energy_j"] == 100.0
    none = MB.EnergyMonitor(100, power_reader=None) if MB.nvml_power_reader() is None else None
    if none is not None:
        none.start_monitoring(); none.stop_monitoring()
        assert not none.available and none.snapshot().energy_joules == 0.0
    runner = MB.BenchmarkRunner(sync=lambda: calls.append("s"))
    import time
    suite = runner.run_benchmark_suite("ops", MB.BenchmarkConfig("fast", lambda: None, 3, 0), MB.BenchmarkConfig("slow", lambda: time.sleep(0.002), 3, 0))
    s = suite.summary()
    assert (s.total_benchmarks, s.fastest, s.slowest) == (2, "fast", "slow") and calls.count("s") == 12 and set(suite.by_name()) == {"fast", "slow"}
    assert len(runner.results().results) == 2
    runner.reset()
    assert runner.results().summary().total_benchmarks == 0
    with pytest.raises(ValueError):
        runner.run_benchmark("x", lambda: None, iterations=0)


def test_profiler_nests_scopes_by_path():
    t = {"now": 0.0}

    def clock():
        return t["now"]
    p = MB.Profiler(clock)
    for _ in range(2):
        with p.begin_scope("infer"):
            t["now"] += 0.001
            with p.begin_scope("conv"):
                t["now"] += 0.004
            p.profile("fc", lambda: t.__setitem__("now", t["now"] + 0.002))
    with p.begin_scope("post"):
        with p.begin_scope("conv"):
            t["now"] += 0.001
    r = p.report()
    e = r.by_name()
    assert set(e) == {"infer", "infer/conv", "infer/fc", "post", "post/conv"} and e["infer"].calls == 2 and abs(e["infer"].total_ms - 14.0) < 1e-9
    assert abs(e["infer/conv"].mean_ms - 4.0) < 1e-9 and e["infer/conv"].depth == 1 and abs(r.total_ms - 15.0) < 1e-9
    assert "  conv: 2 calls, 8.000 ms total" in p.render()
    with pytest.raises(RuntimeError):
        p.end_scope()
    p.reset()
    assert p.report().entries == []


def test_exporters_and_comparator(tmp_path):
    base = MB.BenchmarkResults("suite", [MB.BenchmarkResult("a", 3, [1.0, 1.0, 1.0]), MB.BenchmarkResult("b", 3, [2.0, 2.0, 2.0]), MB.BenchmarkResult("gone", 1, [1.0])])
    cur = MB.BenchmarkResults("suite", [MB.BenchmarkResult("a", 3, [1.2, 1.2, 1.2]), MB.BenchmarkResult("b", 3, [1.0, 1.0, 1.0]), MB.BenchmarkResult("new", 1, [1.0])])
    j = json.loads(MB.BenchmarkExporter.render(base))
    assert j["suite"] == "suite" and j["summary"]["slowest"] == "b" and j["results"][1]["median_ms"] == 2.0
    assert MB.BenchmarkExporter.render(base, "csv").splitlines()[0].startswith("name,iterations,mean_ms") and "| b | 3 | 2.000 |" in MB.BenchmarkExporter.render(base, "markdown")
    h = MB.BenchmarkExporter.render(MB.BenchmarkResults("<s>", base.results), "html")
    assert "&lt;s&gt;" in h and "<td>gone</td>" in h
    with pytest.raises(ValueError):
        MB.BenchmarkExporter.render(base, "pdf")
    MB.BenchmarkExporter.export(base, str(tmp_path / "r.md"), "markdown")
    assert open(tmp_path / "r.md").read().startswith("# suite")
    c = MB.PerformanceComparator(0.1).compare(base, cur)
    assert [e.name for e in c.regressions()] == ["a"] and [e.name for e in c.improvements()] == ["b"] and c.only_in_baseline == ["gone"] and c.only_in_current == ["new"]
    assert abs(c.entries[0].change - 0.2) < 1e-9 and c.entries[1].speedup == 2.0
    p1, p2 = MB.Profiler(), MB.Profiler()
    p1.profile("x", lambda: None)
    p2.profile("x", lambda: None)
    assert [e.name for e in MB.PerformanceComparator().compare_profiles(p1.report(), p2.report()).entries] == ["x"]
    p1.export_report(str(tmp_path / "p.json"))
    p1.export_report(str(tmp_path / "p.csv"), "csv")
    assert json.load(open(tmp_path / "p.json"))["entries"][0]["name"] == "x" and open(tmp_path / "p.csv").read().startswith("name,depth")


def test_constant_folder_evaluates_weight_only_subgraphs():
    from ml_framework_b200.mobile.runtime import fold_constants
    ops = [MobOperator("transpose", ["w"], ["wt"]), MobOperator("mul", ["wt", "two"], ["w2"]), MobOperator("matmul", ["x", "w2"], ["y"]),
           MobOperator("add", ["y", "b"], ["out"])]
    m = MobModel([{"name": "x", "shape": [2, 3]}], ["out"], ops,
                 {"w": MobTensor("w", torch.arange(12.0).reshape(4, 3)), "two": MobTensor("two", torch.tensor(2.0)), "b": MobTensor("b", torch.ones(4)),
                  "unused": MobTensor("unused", torch.zeros(1))})
    x = torch.randn(2, 3)
    ref = MobileRuntime("cpu").load_model(m).predict(x)[0]
    f = fold_constants(m)
    assert [o.type for o in f.operators] == ["matmul", "add"] and set(f.tensors) == {"w2", "b"} and f.metadata["constants_folded"] == 2
    assert f.validate() == [] and torch.allclose(MobileRuntime("cpu").load_model(f).predict(x)[0], ref)
