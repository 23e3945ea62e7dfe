"""Typed IR front door: types, attributes, operation classes, functions, modules, analysis."""
import pytest
import torch

from ml_framework_b200.compiler import ir_ops as O
from ml_framework_b200.compiler.ir import HLGraph

F32 = O.ScalarType.FLOAT32


def test_types_and_attributes():
    t = O.TensorType(F32, (2, 3, 4))
    assert t.rank == 3 and t.num_elements == 24 and t.size_in_bytes == 96 and str(t) == "tensor<2x3x4xfloat32>"
    assert t.with_shape((6, 4)).shape == (6, 4) and O.ScalarType.of(torch.bfloat16) is O.ScalarType.BFLOAT16
    assert O.ScalarType.BFLOAT16.size_in_bytes == 2 and not O.ScalarType.INT32.is_floating_point
    with pytest.raises(TypeError):
        O.ScalarType.of(torch.complex64)
    assert O.IntAttribute(3).value == 3 and O.FloatAttribute(2).value == 2.0 and O.BoolAttribute(True).value is True
    assert O.ArrayAttribute([O.IntAttribute(1), 2]).value == (1, 2) and len(O.ArrayAttribute([1, 2, 3])) == 3
    assert O.TensorAttribute(torch.zeros(2, 2)).type == O.TensorType(F32, (2, 2))
    for bad in (lambda: O.IntAttribute(True), lambda: O.IntAttribute(1.5), lambda: O.BoolAttribute(1), lambda: O.TensorAttribute([1])):
        with pytest.raises(TypeError):
            bad()


def test_typed_ops_build_an_executable_function():
    f = O.HLIRFunction("mlp", [("x", O.TensorType(F32, (4, 8))), ("w", O.TensorType(F32, (16, 8))), ("b", O.TensorType(F32, (16,)))])
    x, w, b = f.parameters
    h = O.GELUOp(f.graph, O.LinearOp(f.graph, x, w, b).result).result
    half = O.MulOp(f.graph, h, O.ConstantOp(f.graph, 0.5).result).result
    s = O.SliceOp(f.graph, half, [0, 4], [4, 12], [2, 1]).result
    assert s.shape == (2, 8) and str(s.type) == "tensor<2x8xfloat32>"
    r = O.ReduceSumOp(f.graph, O.SoftmaxOp(f.graph, s, dim=-1).result, dim=-1, keepdim=True).result
    c = O.ConcatOp(f.graph, r, O.ReduceMaxOp(f.graph, s, dim=1, keepdim=True).result, dim=1).result
    out = O.CastOp(f.graph, O.TransposeOp(f.graph, O.ReshapeOp(f.graph, c, (2, 2)).result).result, O.ScalarType.FLOAT64)
    f.set_results(out.result)
    assert f.verify() == [] and "@mlp(x: tensor<4x8xfloat32>" in f.signature and "-> (tensor<2x2xfloat64>)" in f.signature
    assert "slice" in str(O.SliceOp(f.graph, half, [0], [2])) and "hl.slice" in f.dump()
    torch.manual_seed(0)
    X, W, B = torch.randn(4, 8), torch.randn(16, 8), torch.randn(16)
    hh = torch.nn.functional.gelu(torch.nn.functional.linear(X, W, B), approximate="tanh") * 0.5
    ss = hh[0:4:2, 4:12]
    want = torch.cat([torch.softmax(ss, -1).sum(-1, keepdim=True), ss.amax(1, keepdim=True)], 1).reshape(2, 2).t().double()
    torch.testing.assert_close(f(X, W, B), want)
    with pytest.raises(ValueError, match="expected"):
        f(X.t(), W, B)
    with pytest.raises(ValueError, match="arguments"):
        f(X)


def test_operation_checks():
    g = HLGraph("g")
    a = O.IRValue(g, g.input("a", (2, 3)))
    img = O.IRValue(g, g.input("img", (1, 3, 8, 8)))
    k = O.IRValue(g, g.input("k", (4, 3, 3, 3)))
    other = HLGraph("other")
    foreign = O.IRValue(other, other.input("z", (2, 3)))
    assert O.Conv2DOp(g, img, k, padding=1, activation="relu").result.shape == (1, 4, 8, 8)
    assert O.MaxPool2DOp(g, img).result.shape == (1, 3, 4, 4) and O.AvgPool2DOp(g, img, kernel=4, stride=4).result.shape == (1, 3, 2, 2)
    assert O.BroadcastToOp(g, O.ReshapeOp(g, a, (2, 1, 3)).result, (2, 5, 3)).result.shape == (2, 5, 3)
    assert O.ReduceMeanOp(g, a, dim=(0, 1)).result.shape == ()
    for bad in (lambda: O.AddOp(g, a), lambda: O.AddOp(g, a, foreign), lambda: O.MatMulOp(g, a, O.IRValue(g, g.input("v", (3,)))),
                lambda: O.Conv2DOp(g, a, k), lambda: O.MaxPool2DOp(g, a), lambda: O.ReduceSumOp(g, a, dim=2),
                lambda: O.BroadcastToOp(g, a, (2, 4)), lambda: O.ConcatOp(g, a), lambda: O.LinearOp(g, a),
                lambda: O.Conv2DOp(g, img, k, groups=0)):
        with pytest.raises(ValueError):
            bad()
    assert {o.value for o in O.IROpcode} >= {"add", "slice", "if", "loop", "constant"}


def test_control_flow_ops_and_module():
    m = O.HLIRModule("demo")
    T = O.TensorType(F32, (3,))
    double = m.create_function("double", [("v", T)])
    double.set_results(O.AddOp(double.graph, double.parameters[0], double.parameters[0]).result)
    negate = m.create_function("negate", [("v", T)])
    negate.set_results(O.NegOp(negate.graph, negate.parameters[0]).result)
    main = m.create_function("main", [("p", O.TensorType(F32, ())), ("x", T)])
    p, x = main.parameters
    picked = O.IfOp(main.graph, p, double, negate, x).result
    grown = O.LoopOp(main.graph, 3, double, picked).result
    main.set_results(grown)
    assert m.verify() == [] and "module @demo" in m.dump() and m.get_function("double") is double
    v = torch.tensor([1.0, 2.0, 3.0])
    torch.testing.assert_close(main(torch.tensor(1.0), v), v * 16)
    torch.testing.assert_close(main(torch.tensor(0.0), v), -v * 8)
    m.optimize()
    torch.testing.assert_close(main(torch.tensor(1.0), v), v * 16)
    with pytest.raises(ValueError):
        m.create_function("main")
    with pytest.raises(KeyError):
        m.get_function("nope")
    with pytest.raises(ValueError):
        O.LoopOp(main.graph, -1, double, picked)
    empty = m.create_function("empty", [("v", T)])
    assert any("returns nothing" in e for e in m.verify())
    assert m.remove_function("empty") and not m.remove_function("empty")
    with pytest.raises(ValueError):
        double.add_parameter("v", T)


def test_graph_analyzer_counts_depth_flops_and_memory():
    f = O.HLIRFunction("net", [("x", O.TensorType(F32, (8, 32)))])
    x = f.parameters[0]
    w1 = O.ConstantOp(f.graph, torch.zeros(32, 64)).result
    w2 = O.ConstantOp(f.graph, torch.zeros(64, 16)).result
    h = O.ReLUOp(f.graph, O.MatMulOp(f.graph, x, w1).result).result
    side = O.ReduceSumOp(f.graph, x, dim=1, keepdim=True).result
    y = O.AddOp(f.graph, O.MatMulOp(f.graph, h, w2).result, side).result
    f.set_results(y)
    st = O.HLIRGraphAnalyzer.analyze(f)
    assert st.operation_count == 5 and st.operations_by_kind == {"matmul": 2, "relu": 1, "sum": 1, "add": 1} and st.depth == 4
    assert st.flops == 2 * 8 * 64 * 32 + 8 * 64 + 8 * 32 + 2 * 8 * 16 * 64 + 8 * 16
    assert st.parameter_bytes == (32 * 64 + 64 * 16) * 4 and st.activation_bytes == (8 * 64 * 2 + 8 + 8 * 16 * 2) * 4
    assert st.peak_live_bytes >= (8 * 32 + 8 * 64 * 2) * 4 and st.peak_live_bytes <= st.activation_bytes + 8 * 32 * 4
    path = O.HLIRGraphAnalyzer.critical_path(f)
    assert len(path) == 4 and path[-1] == y.name and path[0].startswith("%matmul")
    assert O.HLIRGraphAnalyzer.critical_path(HLGraph("e")) == [] and O.HLIRGraphAnalyzer.analyze(HLGraph("e")).depth == 0
    body = O.HLIRFunction("body", [("c", O.TensorType(F32, (4, 4)))])
    body.set_results(O.MatMulOp(body.graph, body.parameters[0], body.parameters[0]).result)
    outer = O.HLIRFunction("outer", [("c", O.TensorType(F32, (4, 4)))])
    outer.set_results(O.LoopOp(outer.graph, 5, body, outer.parameters[0]).result)
    assert O.HLIRGraphAnalyzer.analyze(outer).flops == 5 * 2 * 4 * 4 * 4
