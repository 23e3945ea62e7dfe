"""IR verifier, rewriter, constant passes, instrumented pass manager, control flow, back-end registry / compiler."""
import pytest
import torch

from ml_framework_b200.compiler import ir_infra as ii
from ml_framework_b200.compiler.ir import CompilationOptions, HLGraph, Op, Value


def test_verifier_finds_structural_and_shape_errors():
    g = HLGraph("f")
    x = g.input("x", (2, 3))
    y = g.op("relu", x)
    g.output(y)
    v = ii.IRVerifier()
    assert v.errors(g) == []
    g.ops.append(Op("tanh", ["%nope"], "%t"))
    g.values["%t"] = Value("%t", (2, 3))
    g.ops.append(Op("add", [x, y], y))                         # second definition of y
    g.values[y] = Value(y, (5, 5))                              # and a wrong shape for it
    msgs = [d.message for d in v.verify(g)]
    assert any("undefined value %nope" in m for m in msgs) and any("defined twice" in m for m in msgs)
    assert any("result shape (5, 5), operands give (2, 3)" in m for m in msgs)
    assert any(d.severity == "warning" and "%t is never read" in d.message for d in v.verify(g))
    with pytest.raises(RuntimeError, match="IR verification failed"):
        v.check(g)
    bad = HLGraph()
    a = bad.input("a", (2, 3))
    b = bad.input("b", (4, 5))
    bad.ops.append(Op("matmul", [a, b], "%m"))
    bad.values["%m"] = Value("%m", (2, 5))
    bad.output("%m")
    assert any("operands rejected" in d.message for d in v.errors(bad))


def test_control_flow_ops_run_at_every_level_and_are_verified():
    then_g, else_g = HLGraph("then"), HLGraph("else")
    t = then_g.input("v", (3,))
    then_g.output(then_g.op("mul", t, then_g.constant(torch.tensor(2.0))))
    e = else_g.input("v", (3,))
    else_g.output(else_g.op("neg", e))
    body = HLGraph("body")
    c = body.input("c", (3,))
    s = body.input("step", (3,))
    body.output(body.op("add", c, s))

    g = HLGraph("main")
    p = g.input("p", ())
    x = g.input("x", (3,))
    st = g.input("st", (3,))
    y = g.cond(p, then_g, else_g, x)
    z = g.loop(4, body, y, st)
    g.output(z)
    x0, s0 = torch.tensor([1.0, 2.0, 3.0]), torch.tensor([0.5, 0.5, 0.5])
    assert torch.equal(g.run({"p": torch.tensor(1.0), "x": x0, "st": s0})[0], x0 * 2 + 2.0)
    assert torch.equal(g.run({"p": torch.tensor(0.0), "x": x0, "st": s0})[0], -x0 + 2.0)
    assert ii.IRVerifier().errors(g) == []
    prog = ii.BackendCompiler().compile(g, "cpu", CompilationOptions(optimization_level=1))
    assert torch.equal(prog.run({"p": torch.tensor(1.0), "x": x0, "st": s0})[0], x0 * 2 + 2.0) and prog.level == "ml"
    with pytest.raises(ValueError, match="branches disagree"):
        w = HLGraph()
        q = w.input("v", (3,))
        w.output(w.op("sum", q))
        g.cond(p, then_g, w, x)
    with pytest.raises(ValueError, match="loop body"):
        g.loop(2, then_g, y, st)
    g.ops[0].attrs["else"] = body                               # wrong arity for a branch
    assert any("takes 2 inputs, op passes 1" in d.message for d in ii.IRVerifier().errors(g))


def test_rewriter_applies_rules_to_a_fixed_point():
    g = HLGraph()
    x = g.input("x", (4,))
    a = g.op("neg", g.op("neg", g.op("neg", g.op("neg", x))))
    b = g.op("sub", a, a)
    g.output(g.op("add", a, b))

    def double_neg(graph, o):
        prod = {q.output: q for q in graph.ops}.get(o.inputs[0])
        return prod.inputs[0] if prod is not None and prod.kind == "neg" else None

    def sub_self(graph, o):
        if o.inputs[0] == o.inputs[1]:
            zero = graph.constant(torch.zeros(graph.values[o.output].shape))
            return [Op("mul", [o.inputs[0], zero], o.output)]
        return None

    rw = ii.OperationRewriter().add_rule("neg", double_neg).add_rule("sub", sub_self)
    n = rw.run(g)
    assert n >= 3 and rw.applied["double_neg"] >= 2 and rw.applied["sub_self"] == 1
    from ml_framework_b200.compiler.ir import DeadCodeElimination
    DeadCodeElimination().run(g)
    assert [o.kind for o in g.ops] == ["mul", "add"] and g.ops[1].inputs[0] == "x"
    xv = torch.randn(4)
    assert torch.equal(g.run({"x": xv})[0], xv)
    with pytest.raises(ValueError):
        ii.OperationRewriter().add_rule("mul", lambda gr, o: [Op("mul", o.inputs, "%other")]).run(g)
    assert ii.RewritePass(ii.OperationRewriter()).run(g) is False


def test_inline_constants_dedups_drops_and_inlines_scalars():
    g = HLGraph()
    x = g.input("x", (2, 2))
    c1, c2 = g.constant(torch.ones(2, 2)), g.constant(torch.ones(2, 2))
    g.constant(torch.zeros(3))                                   # nobody reads it
    half = g.constant(torch.tensor(0.5))
    y = g.op("add", g.op("add", x, c1), c2)
    z = g.op("mul", y, half)
    w = g.op("sub", g.constant(torch.tensor(1.0)), z)
    g.output(w)
    xv = torch.randn(2, 2)
    ref = g.run({"x": xv})[0]
    assert ii.InlineConstants().run(g)
    consts = [n for n, v in g.values.items() if v.const is not None]
    assert len(consts) == 1 and g.ops[0].inputs[1] == g.ops[1].inputs[1]
    assert [o.kind for o in g.ops] == ["add", "add", "mul_scalar", "sub_scalar"]
    assert g.ops[2].attrs["scalar"] == 0.5 and g.ops[3].attrs["scalar_side"] == "lhs"
    assert torch.equal(g.run({"x": xv})[0], ref) and g.verify() == []
    assert not ii.InlineConstants().run(g)
    ev = ii.ConstantEvaluator(max_result_elems=8)
    h = HLGraph()
    a, b = h.constant(torch.ones(2, 2)), h.constant(torch.full((2, 2), 3.0))
    s = h.op("add", a, b)
    big = h.op("matmul", h.constant(torch.ones(4, 1)), h.constant(torch.ones(1, 4)))
    assert ev.can_evaluate(h, h.ops[0]) and torch.equal(ev.evaluate(h, h.ops[0]), torch.full((2, 2), 4.0))
    assert not ev.can_evaluate(h, h.ops[1]) and s and big


def test_instrumented_pass_manager_records_and_verifies():
    g = HLGraph()
    x = g.input("x", (4,))
    a = g.op("add", x, g.constant(torch.tensor(0.0)))
    b = g.op("relu", a)
    g.op("tanh", a)                                              # dead
    g.output(g.op("add", b, g.op("relu", a)))                    # CSE candidate
    seen = []
    instr = ii.PassInstrumentation()
    instr.before.append(lambda name, gr: seen.append(("before", name)))
    instr.after.append(lambda rec, gr: seen.append(("after", rec.name, rec.changed)))
    pm = ii.InstrumentedPassManager(instrumentation=instr, verifier=ii.IRVerifier())
    pm.run(g)
    assert [o.kind for o in g.ops] == ["relu", "add"]
    s = instr.summary()
    assert s["dce"]["ops_removed"] >= 1 and s["cse"]["changed"] >= 1 and s["simplify"]["changed"] >= 1
    assert seen[0] == ("before", "constant-folding") and "dce:" in instr.render()

    class Breaks(ii.Pass):
        name = "breaks"

        def run(self, gr):
            gr.ops.append(Op("relu", ["%missing"], "%x9"))
            gr.values["%x9"] = Value("%x9", (4,))
            return True
    with pytest.raises(RuntimeError, match="invalid after pass breaks"):
        ii.InstrumentedPassManager([Breaks()], verifier=ii.IRVerifier()).run(g)


def test_backend_registry_compiler_levels_and_capabilities():
    reg = ii.default_backend_registry()
    assert reg.names() == ["b200", "cpu"]
    with pytest.raises(KeyError, match="unknown back-end"):
        reg.get("tpu")
    cc = ii.ComputeCapability.SM_100A
    assert cc.arch == "sm_100a" and cc.has_tcgen05 and cc.has_tma and cc.gencode() == "arch=compute_100a,code=sm_100a"
    assert not ii.ComputeCapability.SM_80.has_tma and not ii.ComputeCapability.SM_90A.has_tcgen05 and ii.ComputeCapability.SM_90.has_tma

    def build():
        g = HLGraph("net")
        x = g.input("x", (4, 8))
        w = g.constant(torch.randn(8, 8) * 0.3)
        h = g.op("gelu", g.op("linear", x, w))
        g.output(g.op("exp", g.op("tanh", g.op("relu", h))))
        return g
    torch.manual_seed(0)
    g0 = build()
    xv = torch.randn(4, 8)
    ref = g0.run({"x": xv})[0]
    comp = ii.BackendCompiler()
    p3 = comp.compile(g0, "b200", CompilationOptions(optimization_level=3))
    assert [o.kind for o in p3.graph.ops] == ["linear", "fused_elementwise"] and p3.target == "sm_100a"
    assert len(p3.sources) == 1 and "__global__" in next(iter(p3.sources.values()))
    assert [k for _, k, _ in p3.plan] == ["linear", "fused_elementwise"]
    assert torch.allclose(p3.run({"x": xv})[0], ref, atol=1e-5)
    torch.manual_seed(0)
    p0 = comp.compile(build(), "cpu", CompilationOptions(optimization_level=0), cpu_level="ll")
    assert p0.level == "ll" and len(p0.graph.ops) == 5
    small = HLGraph()
    q = small.input("q", (3,))
    small.output(small.op("relu", small.op("neg", q)))
    pl = comp.compile(small, "cpu", CompilationOptions(optimization_level=1), cpu_level="ll")
    assert torch.equal(pl.run({"q": torch.tensor([1.0, -2.0, 3.0])})[0], torch.tensor([0.0, 2.0, 0.0]))
    ml = ii.HLToMLLowering().run(small)
    assert ii.MLToLLLowering().run(ml).verify() == []
