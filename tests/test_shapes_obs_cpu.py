"""Symbolic shape inference (every rule, constraints, the static checker, report formats) and the visualizer's text /
image / export / builder / configuration paths, on CPU."""
import json

import pytest
import torch
import torch.nn as nn

from ml_framework_b200.compiler import shapes as S
from ml_framework_b200.obs import events, visualizer as V


def test_shape_rules_agree_with_torch_on_concrete_shapes():
    eng = S.ShapeInferenceEngine()
    x = torch.zeros(2, 3, 17, 20)
    w = torch.zeros(8, 3, 3, 5)
    want = torch.nn.functional.conv2d(x, w, stride=2, padding=1, dilation=1).shape
    assert eng.infer("conv2d", [x.shape, w.shape], stride=2, padding=1).concrete() == tuple(want)
    assert eng.infer("maxpool2d", [x.shape], kernel=3, stride=2, padding=1).concrete() == tuple(torch.nn.functional.max_pool2d(x, 3, 2, 1).shape)
    assert eng.infer("avgpool2d", [x.shape]).concrete() == tuple(torch.nn.functional.avg_pool2d(x, 2).shape)
    assert eng.infer("reshape", [(4, 6)], shape=[-1, 8]).concrete() == (3, 8)
    assert eng.infer("reshape", [(4, 6)], shape=[2, 12]).concrete() == (2, 12)
    assert eng.infer("transpose", [(2, 3, 4)]).concrete() == (2, 4, 3) and eng.infer("transpose", [(2, 3, 4)], dim0=0, dim1=2).concrete() == (4, 3, 2)
    assert eng.infer("concat", [(2, 3), (5, 3), (1, 3)], dim=0).concrete() == (8, 3)
    assert eng.infer("concat", [(2, 3), (2, 4)], dim=1).concrete() == (2, 7)
    assert eng.infer("sum", [(2, 3, 4)], dim=1).concrete() == (2, 4) and eng.infer("mean", [(2, 3, 4)], dim=-1, keepdim=True).concrete() == (2, 3, 1)
    assert eng.infer("max", [(2, 3)]).concrete() == ()
    assert eng.infer("matmul", [(5, 1, 2, 3), (7, 3, 4)]).concrete() == tuple((torch.zeros(5, 1, 2, 3) @ torch.zeros(7, 3, 4)).shape)
    assert eng.infer("linear", [(9, 2, 16), (32, 16)]).concrete() == (9, 2, 32)
    for bad in (("reshape", [(4, 6)], dict(shape=[5, -1])), ("reshape", [(4, 6)], dict(shape=[5, 5])),
                ("concat", [(2, 3), (2, 3, 1)], dict(dim=0)), ("concat", [(2, 3), (2, 4)], dict(dim=0)),
                ("conv2d", [(1, 4, 8, 8), (8, 3, 3, 3)], {}), ("matmul", [(3,), (3, 2)], {}), ("linear", [(2, 5), (4, 6)], {})):
        with pytest.raises(S.ShapeMismatchException):
            eng.infer(bad[0], bad[1], **bad[2])
    with pytest.raises(KeyError):
        eng.infer("fft", [(2,)])
    eng.register("double_rows", lambda s, a: S.SymbolicShape([2 * s[0][0].value] + list(s[0].dims[1:])))
    assert eng.infer("double_rows", [(3, 4)]).concrete() == (6, 4)


def test_symbolic_dimensions_bind_constraints_and_static_checker():
    B = S.SymbolicDimension("B", min_value=1, max_value=64)
    x = S.SymbolicShape([B, 3, 32, 32])
    assert not x.is_fully_known and x.rank == 4 and [str(d) for d in x] == ["B", "3", "32", "32"] and repr(x) == "[B, 3, 32, 32]"
    with pytest.raises(ValueError):
        x.concrete()
    assert x.bind({"B": 8}).concrete() == (8, 3, 32, 32) and x == S.SymbolicShape([B, 3, 32, 32]) and x != S.SymbolicShape([B, 3, 32, 31])
    with pytest.raises(ValueError):
        x.bind({"B": 65})
    out = S.ShapeInferenceEngine().infer("conv2d", [x, (16, 3, 3, 3)], padding=1)
    assert str(out[0]) == "B" and out.bind({"B": 2}).concrete() == (2, 16, 32, 32)
    H = S.SymbolicDimension("H")
    sym = S.ShapeInferenceEngine().infer("maxpool2d", [S.SymbolicShape([1, 1, H, 8])])
    assert not sym[2].is_known and "H" in sym[2].name and sym[3].value == 4
    assert S.EqualityConstraint("a", "b").check({"a": 2, "b": 2}) and not S.EqualityConstraint("a", "b").check({"a": 2, "b": 3})
    assert S.EqualityConstraint("a", "b").check({"a": 2})                               # unbound names constrain nothing
    assert S.ModuloConstraint("n", 8).check({"n": 64}) and not S.ModuloConstraint("n", 8, 1).check({"n": 64})
    assert S.RangeConstraint("n", 1, 10).check({"n": 10}) and not S.RangeConstraint("n", 1, 10).check({"n": 11})
    chk = S.StaticShapeChecker(constraints=[S.ModuloConstraint("B", 4), S.RangeConstraint("B", 1, 64)])
    prog = [("conv2d", ["x", "w"], "h", {"padding": 1}), ("maxpool2d", ["h"], "p", {}), ("reshape", ["p"], "f", {"shape": [-1, 16 * 16 * 16]}),
            ("linear", ["f", "fc"], "y", {})]
    shapes, errs = chk.check({"x": x, "w": (16, 3, 3, 3), "fc": (10, 4096)}, prog, {"B": 8})
    assert not errs and shapes["y"].concrete() == (8, 10) and shapes["p"].concrete() == (8, 16, 16, 16)
    _, errs = chk.check({"x": x, "w": (16, 3, 3, 3), "fc": (10, 4000)}, prog, {"B": 6})
    assert len(errs) == 2 and "constraint violated" in errs[0] and errs[1].startswith("op #3 (linear)")
    _, errs = chk.check({"x": x}, [("fft", ["x"], "y", {})], {"B": 4})
    assert errs and "op #0 (fft)" in errs[0]


def test_shape_mismatch_reports_in_three_formats():
    try:
        S.ShapeInferenceEngine().infer("matmul", [(4, 8), (16, 8)])
    except S.ShapeMismatchException as e:
        assert e.op == "matmul" and any("transpose" in s for s in e.suggestions)
        assert "suggestions" in S.ShapeReportFormatter.text(e)
        j = json.loads(S.ShapeReportFormatter.json(e))
        assert j["operation"] == "matmul" and j["shapes"] == ["[4, 8]", "[16, 8]"] and len(j["suggestions"]) == 2
        h = S.ShapeReportFormatter.html(e)
        assert h.startswith("<div class='shape-error'><b>matmul</b>") and h.count("<li>") == 2
    else:
        raise AssertionError("no mismatch raised")


def test_visualizer_text_image_export_builder_and_configuration(tmp_path):
    mem = events.MemoryStorageBackend()
    v = V.VisualizerBuilder().with_backend(mem).with_async(False).with_histogram_bins(5).with_storage("memory").enabled(True).build()
    v.log_text("note", "hello", 3)
    v.log_image("img", torch.rand(3, 200, 120), 1)
    v.log_histogram("h", torch.arange(100.0))
    v.log_scalar("loss", 0.5, 1)
    v.log_scalar("loss", 0.25, 2)
    v.record_instant("mark")
    with v.start_profile("step"):
        pass
    v.flush()
    kinds = [e.type for e in mem.events]
    assert kinds.count(events.EventType.TEXT) == 1 and kinds.count(events.EventType.IMAGE) == 1
    img = next(e for e in mem.events if e.type == events.EventType.IMAGE).value
    assert img["shape"] == [3, 200, 120] and len(img["thumb"]) == 3 and len(img["thumb"][0]) == 50 and len(img["thumb"][0][0]) == 30
    hist = next(e for e in mem.events if e.type == events.EventType.HISTOGRAM).value
    assert hist["count"] == 100 and len(hist["bins"]) == 5 and sum(hist["bins"]) == 100 and hist["quantiles"]["p50"] == pytest.approx(49.5)
    assert v.profiler.instants[0][0] == "mark"
    out = tmp_path / "export.json"
    v.export(str(out))
    d = json.loads(out.read_text())
    assert d["scalars"]["loss"] == {"steps": [1, 2], "values": [0.5, 0.25]} and d["profile"]["step"]["count"] == 1
    v.close()
    off = V.VisualizerBuilder().with_backend(events.MemoryStorageBackend()).with_async(False).enabled(False).build()
    off.log_scalar("x", 1.0)
    off.log_text("t", "x")
    off.log_image("i", torch.rand(1, 4, 4))
    off.log_graph(nn.Linear(1, 1))
    off.flush()
    assert off.backend.events == []
    off.close()
    assert V.histogram_summary(torch.empty(0)) == {"count": 0}
    g = V.module_graph(nn.Sequential(nn.Linear(2, 3), nn.ReLU()))
    assert [n["name"] for n in g["nodes"]] == ["<root>", "0", "1"] and g["nodes"][1]["params"] == 9 and g["edges"][0] == {"from": "<root>", "to": "0"}
    c = V.ConfigurationLoader.from_json('{"log_dir": "/tmp/x", "histogram_bins": 12, "storage": "memory"}')
    assert c.histogram_bins == 12 and c.storage == "memory"
    p = tmp_path / "viz.json"
    p.write_text('{"buffer_capacity": 7}')
    assert V.ConfigurationLoader.from_file(str(p)).buffer_capacity == 7
    for bad in ('{"histogram_bins": 0}', '{"storage": "s3"}', '{"flush_interval_s": 0}'):
        with pytest.raises(ValueError):
            V.ConfigurationLoader.from_json(bad)
    with pytest.raises(ValueError):
        V.ConfigurationLoader.from_environment(env={"MLFRAMEWORK_VISUALIZATION_BUFFER_CAPACITY": "0"})
