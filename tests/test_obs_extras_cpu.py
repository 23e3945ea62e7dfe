"""Histogram statistics and logger, computational graphs (module tree, autograd, IR), binary event files, GPU trackers on a fake NVML."""
import json
import os
import struct

import pytest
import torch
import torch.nn as nn

from ml_framework_b200.obs import event_file as ef
from ml_framework_b200.obs import gpu_trackers as gt
from ml_framework_b200.obs import graphs as G
from ml_framework_b200.obs import histograms as H
from ml_framework_b200.obs.events import EventFactory, EventSystem, EventType


def test_moments_quantiles_and_outliers():
    v = torch.tensor([1.0, 2.0, 3.0, 4.0, 100.0])
    assert H.QuantileCalculator.calculate(v, 0.5) == 3.0 and H.QuantileCalculator.calculate(v, 0.25) == 2.0
    assert H.QuantileCalculator.calculate_multiple([0.0, 10.0], [0.0, 0.3, 1.0]) == [0.0, 3.0, 10.0]
    with pytest.raises(ValueError):
        H.QuantileCalculator.calculate(v, 1.5)
    with pytest.raises(ValueError):
        H.QuantileCalculator.calculate([], 0.5)
    g = torch.Generator().manual_seed(0)
    n = torch.randn(200_000, generator=g)
    sk, ku = H.MomentsCalculator.both(n)
    assert abs(sk) < 0.03 and abs(ku) < 0.06
    assert H.MomentsCalculator.skewness(torch.cat([n.abs(), torch.zeros(10)])) > 0.5 and H.MomentsCalculator.kurtosis([1.0]) == 0.0
    assert H.MomentsCalculator.skewness(torch.ones(5)) == 0.0
    cnt, idx = H.OutlierDetector.by_iqr(v)
    assert (cnt, idx) == (1, [4]) and H.OutlierDetector.by_std(v, 1.5) == (1, [4]) and H.OutlierDetector.outlier_values(v, 1.5) == [100.0]
    lo, hi = H.OutlierDetector.bounds_by_std(torch.tensor([0.0, 2.0]), 2.0)
    assert (lo, hi) == (-1.0, 3.0) and H.OutlierDetector.by_std([]) == (0, [])
    assert H.OutlierDetector.count_dead_neurons(torch.tensor([0.0, 1e-4, -2.0, 0.0])) == 2
    assert H.OutlierDetector.count_dead_neurons(torch.tensor([0.0, 1e-4, -2.0, 0.0]), 1e-3) == 3


def test_histogram_and_distribution_logging():
    ev = EventSystem()
    got = []
    ev.subscribe(got.append, EventType.HISTOGRAM)
    log = H.HistogramLogger(ev, H.HistogramBinConfig(bin_count=4))
    h = log.log_histogram("w", torch.tensor([0.0, 1.0, 2.0, 3.0, 4.0, float("nan")]))
    assert h.step == 0 and h.count == 5 and h.bin_counts == [1, 1, 1, 2] and h.bin_edges == [0.0, 1.0, 2.0, 3.0, 4.0] and sum(h.normalized()) == 1.0
    assert h.mode_bin() == (3.0, 4.0) and log.log_histogram("w", torch.ones(3)).step == 1 and len(got) == 2
    fixed = log.log_histogram("f", torch.tensor([-5.0, 0.5, 9.0]), step=7, config=H.HistogramBinConfig(2, 0.0, 1.0))
    assert (fixed.underflow, fixed.overflow, fixed.bin_counts) == (1, 1, [0, 1]) and log.get_histogram("f", 7) is fixed
    lg = log.log_histogram("lg", torch.tensor([1e-3, 1e-2, 1.0, 10.0]), config=H.HistogramBinConfig(4, log_scale=True))
    assert lg.bin_edges[0] == -3.0 and lg.bin_counts == [1, 1, 0, 2]
    assert log.log_histogram("e", torch.tensor([float("inf")])).count == 0
    with pytest.raises(ValueError):
        H.HistogramBinConfig(0).validate()
    d = log.log_distribution("act", torch.tensor([0.0] * 6 + [1.0, 2.0, float("nan"), float("inf")]))
    assert d.count == 8 and d.dead == 6 and d.nan == 1 and d.inf == 1 and d.quantiles["p50"] == 0.0
    assert any("dead" in w for w in d.warnings()) and any("NaN" in w for w in d.warnings())
    assert "constant tensor" in H.build_distribution("c", torch.ones(4)).warnings()
    m = nn.Linear(3, 2)
    m(torch.randn(4, 3)).sum().backward()
    nn.init.zeros_(m.bias)
    warns = log.log_module(m, step=3)
    assert any(w.startswith("bias:") for w in warns) and "weight.grad" in log.distribution_names()
    assert [x.step for x in log.histograms_over_time("w")] == [0, 1] and log.distributions_over_time("weight")[0].step == 3
    small = H.HistogramLogger(max_steps_per_name=2)
    for i in range(4):
        small.log_distribution("x", torch.randn(4))
    assert [x.step for x in small.distributions_over_time("x")] == [2, 3]
    log.clear("w")
    assert "w" not in log.histogram_names()
    log.clear()
    assert log.histogram_names() == [] and log.get_distribution("act", 0) is None


class _Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(4, 4), nn.Linear(4, 4)

    def forward(self, x):
        return x + self.fc2(torch.relu(self.fc1(x)))


def test_graphs_from_module_autograd_and_ir_with_analysis_and_serialisation():
    model = nn.Sequential(_Block(), _Block())
    g = G.graph_from_module(model)
    a = G.GraphAnalyzer().analyze(g)
    assert a.total_parameters == 8 and a.parameter_elements == 4 * (16 + 4) and a.operation_counts["Linear"] == 4 and not g.has_cycle()
    x = torch.randn(2, 4, requires_grad=False)
    loss = model(x).sum()
    ag = G.graph_from_autograd(loss, dict(model.named_parameters()))
    aa = G.GraphAnalyzer().analyze(ag)
    assert aa.total_parameters == 8 and aa.operation_counts.get("Addmm", 0) == 4 and aa.operation_counts.get("Relu", 0) == 2
    assert aa.skip_connections >= 1 and any("skip connections" in r for r in aa.recommendations)
    assert {n.name for n in ag.nodes.values() if n.type == G.NodeType.PARAMETER} == set(dict(model.named_parameters()))
    assert [n.id for n in ag.outputs()] == ["output"] and ag.depth >= 8
    with pytest.raises(ValueError):
        G.graph_from_autograd(torch.zeros(1))
    from ml_framework_b200.compiler.ir import HLGraph
    hl = HLGraph("ir")
    xi = hl.input("x", (2, 3))
    hl.output(hl.op("relu", hl.op("add", xi, hl.constant(torch.ones(2, 3)))))
    ig = G.graph_from_ir(hl)
    assert [n.op_type for n in ig.topological_order() if n.type == G.NodeType.OPERATION] == ["add", "relu"] and ig.depth == 3
    back = G.GraphSerializer.from_json(G.GraphSerializer.to_json(ig))
    assert list(back.nodes) == list(ig.nodes) and back.edges == ig.edges and back.nodes["x"].shape == (2, 3)
    dot = G.GraphSerializer.to_dot(ig)
    assert dot.startswith('digraph "ir"') and '"x" -> ' in dot and "shape=ellipse" in dot
    c = G.ComputationalGraph("cyc")
    for k in "abc":
        c.add_node(G.GraphNode(k, k, G.NodeType.OPERATION, "op"))
    c.add_node(G.GraphNode("lonely", "lonely", G.NodeType.OPERATION, "op"))
    c.add_edge("a", "b"); c.add_edge("b", "c"); c.add_edge("c", "a"); c.add_edge("a", "b")
    ca = G.GraphAnalyzer().analyze(c)
    assert c.has_cycle() and len(c.edges) == 3 and c.depth == -1 and len(c.disconnected_components()) == 2
    assert any("cycles" in w for w in ca.warnings) and any("2 disconnected" in w for w in ca.warnings)
    with pytest.raises(KeyError):
        c.add_edge("a", "zzz")
    with pytest.raises(KeyError):
        c.add_node(G.GraphNode("a", "a", G.NodeType.INPUT))
    wide = G.ComputationalGraph("wide")
    wide.add_node(G.GraphNode("sink", "sink", G.NodeType.OPERATION, "cat"))
    for i in range(12):
        wide.add_node(G.GraphNode(f"i{i}", f"i{i}", G.NodeType.INPUT))
        wide.add_edge(f"i{i}", "sink")
    assert any("fan-in (max 12)" in w for w in G.GraphAnalyzer().analyze(wide).warnings)


def test_graph_logger_capture_records_execution_order():
    from ml_framework_b200.obs.events import MemoryStorageBackend
    store = MemoryStorageBackend()
    gl = G.GraphLogger(store)
    model = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 2))
    gl.log_graph(model, "tree")
    assert store.events[0].type == EventType.GRAPH and store.events[0].value["name"] == "tree"
    gl.start_graph_capture("run", model)
    with pytest.raises(RuntimeError):
        gl.start_graph_capture("again", model)
    model(torch.randn(3, 4))
    g = gl.stop_graph_capture()
    assert [n.op_type for n in g.topological_order()] == ["Linear", "ReLU", "Linear"] and g.nodes["2#2"].shape == (3, 2)
    model(torch.randn(3, 4))                        # hooks are gone
    assert len(g.nodes) == 3 and gl.captured_graph() is g
    assert gl.analyze_graph("run").graph_depth == 3 and set(gl.analyze_all_graphs()) == {"tree", "run"}
    with pytest.raises(KeyError):
        gl.analyze_graph("none")
    with pytest.raises(RuntimeError):
        gl.stop_graph_capture()
    gl.clear_graphs()
    assert gl.all_graphs() == {}


def test_event_file_round_trip_append_truncation_and_corruption(tmp_path):
    p = str(tmp_path / "sub" / "run.mlfevt")
    with ef.EventFileWriter(p) as w:
        for i in range(5):
            w.write_event(EventFactory.scalar("loss", 1.0 / (i + 1), i))
        assert w.records_written == 5
    with ef.EventFileWriter(p, append=True) as w:
        w.write_event(EventFactory.histogram("h", [1, 2, 3], 9))
    r = ef.EventFileReader(p)
    evs = r.read_all()
    assert [e.step for e in evs] == [0, 1, 2, 3, 4, 9] and evs[-1].type == EventType.HISTOGRAM and r.corrupt_records == 0 and not r.truncated
    size = os.path.getsize(p)
    with open(p, "r+b") as f:                        # damage one payload byte of the second record
        f.seek(len(ef.MAGIC))
        n0, = struct.unpack("<I", f.read(4))
        f.seek(len(ef.MAGIC) + 8 + n0 + 8 + 3)
        b = f.read(1)
        f.seek(-1, 1)
        f.write(bytes([b[0] ^ 0xFF]))
    assert [e.step for e in r.read_all()] == [0, 2, 3, 4, 9] and r.corrupt_records == 1
    with open(p, "r+b") as f:
        f.truncate(size - 5)
    assert r.count() == 4 and r.truncated
    with pytest.raises(ef.EventFileError):
        bad = tmp_path / "bad"
        bad.write_bytes(b"not an event file")
        ef.EventFileReader(str(bad)).read_all()
    with pytest.raises(ef.EventFileError):
        ef.EventFileWriter(str(bad), append=True)
    with pytest.raises(FileNotFoundError):
        ef.EventFileReader(str(tmp_path / "missing"))
    w = ef.EventFileWriter(str(tmp_path / "c"))
    w.close()
    with pytest.raises(ef.EventFileError):
        w.write_event(EventFactory.scalar("x", 1))
    be = ef.BinaryFileStorageBackend(str(tmp_path / "logs"), max_file_bytes=200)
    be.write([EventFactory.scalar("s", float(i), i) for i in range(10)])
    assert len(be.paths) > 1 and [e.step for e in be.read_all()] == list(range(10))
    be.close()


class _FakeNvml:
    NVML_CLOCK_SM, NVML_TEMPERATURE_GPU = 1, 0

    def __init__(self):
        self.t = 0

    def nvmlDeviceGetCount(self): return 2
    def nvmlDeviceGetHandleByIndex(self, i): return i
    def nvmlDeviceGetName(self, h): return b"NVIDIA B200"
    def nvmlDeviceGetCudaComputeCapability(self, h): return (10, 0)
    def nvmlSystemGetDriverVersion(self): return "580.00"

    def nvmlDeviceGetMemoryInfo(self, h):
        class M: used, total = (10 + h) << 30, 180 << 30
        return M()

    def nvmlDeviceGetUtilizationRates(self, h):
        self.t += 1

        class U: gpu = 50 + 10 * (self.t % 3)
        return U()

    def nvmlDeviceGetTemperature(self, h, k): return 61
    def nvmlDeviceGetPowerUsage(self, h): return 900_000
    def nvmlDeviceGetClockInfo(self, h, k): return 1500 + 100 * (self.t % 2)
    def nvmlDeviceGetMaxClockInfo(self, h, k): return 1965
    def nvmlDeviceGetCurrentClocksEventReasons(self, h): return 0x4 if h == 0 else 0x4 | 0x40


def test_gpu_trackers_on_a_fake_nvml():
    assert gt.decode_reasons(0x4 | 0x20) == ["sw_power_cap", "sw_thermal_slowdown"] and gt.decode_reasons(0) == []
    assert not gt.RocmGpuTracker().is_available() and gt.RocmGpuTracker().device_count() == 0
    tr = gt.GPUUtilizationTracker([gt.RocmGpuTracker(), gt.CudaGpuTracker(_FakeNvml())], sampling_interval_s=0.01)
    assert tr.is_available and tr.tracker.vendor == "nvidia"
    devs = tr.available_devices()
    assert [d.name for d in devs] == ["NVIDIA B200"] * 2 and devs[0].compute_capability == "10.0" and devs[0].driver_version == "580.00"
    with pytest.raises(IndexError):
        tr.device_info(5)
    tr._tracked = [0, 1]
    for _ in range(4):
        tr.sample_utilization()
    tr.disable()
    tr.sample_utilization()
    tr.enable()
    s0, s1 = tr.statistics(0), tr.statistics(1)
    assert s0.sample_count == 4 and 50 <= s0.average_utilization <= 70 and s0.peak_power_w == 900.0 and s0.peak_temperature_c == 61
    assert s0.reasons_seen == ["sw_power_cap"] and not s0.throttled() and s1.throttled() and s0.sm_clock_max_mhz == 1965
    assert s1.peak_memory_bytes == 11 << 30 and abs(tr.samples(0)[0].memory_percent - 100 * 10 / 180) < 1e-9
    assert set(tr.all_statistics()) == {0, 1} and tr.samples(0, start=1e18) == []
    tr.clear()
    tr.start_tracking(-1)
    import time
    time.sleep(0.08)
    tr.stop_tracking()
    assert tr.statistics(1).sample_count >= 2
    with pytest.raises(ValueError):
        tr.set_sampling_interval(0)
    none = gt.GPUUtilizationTracker([gt.RocmGpuTracker()])
    assert not none.is_available and none.available_devices() == [] and none.statistics(0).sample_count == 0
    none.start_tracking()
    with pytest.raises(RuntimeError):
        none.device_info(0)


def test_seed_manager_device_worker_seeds_scopes_registry_and_validation(tmp_path):
    import io
    import random

    from ml_framework_b200.obs.seed import DeterministicModeFlags as F, SeedManager
    sm = SeedManager()
    with pytest.raises(ValueError):
        sm.seed_workers(2)                                  # no base seed yet
    sm.set_global_seed(11)
    sm.seed_all_devices(device_count=3)
    assert len({sm.device_seed(d) for d in range(3)}) == 3 and sm.current_seed == 11
    with pytest.raises(KeyError):
        sm.device_seed(7)
    assert sm.seed_workers(2) == [sm.worker_seed(0), sm.worker_seed(1)]
    # a seeded scope repeats, and the outer stream continues as if the scope had not been there
    torch.manual_seed(5); random.seed(5)
    a0 = torch.rand(1)
    with sm.with_global_seed(99):
        inner1 = (torch.rand(2), random.random())
    a1 = torch.rand(1)
    with sm.with_global_seed(99):
        inner2 = (torch.rand(2), random.random())
    torch.manual_seed(5)
    assert torch.equal(torch.rand(1), a0) and torch.equal(torch.rand(1), a1)
    assert torch.equal(inner1[0], inner2[0]) and inner1[1] == inner2[1] and sm.current_seed == 11
    # snapshots survive a file
    snap = sm.capture_rng_state()
    x = torch.rand(3)
    sm.save_rng_snapshot(snap, str(tmp_path / "rng.pt"))
    torch.rand(10)
    sm.restore_rng_state(sm.load_rng_snapshot(str(tmp_path / "rng.pt")))
    assert torch.equal(torch.rand(3), x)
    # flags
    assert sm.check_performance_impact() is None and "no performance impact" in sm.performance_impact()
    with sm.with_deterministic_mode(F.NO_ATOMIC_REDUCTIONS):
        assert sm.is_deterministic_mode_enabled(F.NO_ATOMIC_REDUCTIONS) and "reported, not replaced" in sm.check_performance_impact()
        sm.register_non_deterministic_operation("matmul")
        sm.register_non_deterministic_operation("matmul")
        sm.register_non_deterministic_operation("scatter_add")
        res = sm.validate_configuration()
        assert not res.is_valid and len(res.errors) == 1 and "scatter_add" in res.errors[0]
        assert sum("matmul" in w for w in res.warnings) == 1 and any("flash_bwd" in w for w in res.warnings)
        assert "2 workers seeded" in res.messages and "3 devices seeded" in res.messages
    assert sm.flags == F.NONE and sm.validate_configuration().is_valid
    sm.enable_deterministic_mode(F.NO_TF32)
    sm.disable_deterministic_mode(F.NO_TF32)
    assert not sm.is_deterministic_mode_enabled(F.NO_TF32)
    assert sm.non_deterministic_operations() == ["matmul", "scatter_add"]
    assert sm.can_be_deterministic("dropout") and not sm.can_be_deterministic("atomic_add") and not sm.can_be_deterministic(" ")
    with pytest.raises(ValueError):
        sm.register_non_deterministic_operation("")
    buf = io.StringIO()
    sm.print_diagnostics(file=buf)
    assert "scatter_add (non-determinizable)" in buf.getvalue() and "current seed: 11" in buf.getvalue()
    info = sm.diagnostic_info()
    assert info.device_count == 3 and info.worker_count == 2
