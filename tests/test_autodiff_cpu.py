"""Gradient graphs built from IR graphs agree with PyTorch's autograd."""
import pytest
import torch
import torch.nn.functional as F

from ml_framework_b200.compiler import autodiff as AD
from ml_framework_b200.compiler.ir import HLGraph, Op, Value


def _check(build, feeds, wrt, torch_fn, atol=1e-10):
    g, out = build()
    bg, names = AD.build_backward(g, out, wrt)
    got = bg.run({k: v.clone() for k, v in feeds.items()})
    leaves = {k: v.clone().requires_grad_(True) for k, v in feeds.items()}
    torch_fn(leaves).sum().backward()
    for w, gr in zip(wrt, got):
        want = leaves[w].grad if leaves[w].grad is not None else torch.zeros_like(leaves[w])
        assert gr.shape == want.shape and torch.allclose(gr, want, atol=atol), w
    return bg


def test_elementwise_chain_with_broadcasting_and_reuse():
    def build():
        g = HLGraph()
        x, b = g.input("x", (3, 4), torch.float64), g.input("b", (4,), torch.float64)
        s = g.op("add", x, b)
        t = g.op("tanh", s)
        u = g.op("mul", t, s)                       # s used twice: gradients accumulate
        v = g.op("div", g.op("exp", u), g.op("sigmoid", x))
        w = g.op("sub", g.op("sqrt", g.op("exp", v)), g.op("log", g.op("exp", b)))
        out = g.op("neg", g.op("relu", w))
        g.output(out)
        return g, out
    feeds = {"x": torch.randn(3, 4, dtype=torch.float64) * 0.3, "b": torch.randn(4, dtype=torch.float64) * 0.3}

    def ref(l):
        s = l["x"] + l["b"]
        v = torch.exp(torch.tanh(s) * s) / torch.sigmoid(l["x"])
        return -torch.relu(torch.sqrt(torch.exp(v)) - torch.log(torch.exp(l["b"])))
    bg = _check(build, feeds, ["x", "b"], ref)
    assert any(o.kind == "sum_to" for o in bg.ops) and len(bg.outputs) == 2


def test_reductions_linear_matmul_gelu_and_shape_ops():
    torch.manual_seed(0)

    def build():
        g = HLGraph()
        x, w, bias = g.input("x", (2, 3, 4), torch.float64), g.input("w", (5, 4), torch.float64), g.input("bias", (5,), torch.float64)
        m = g.input("m", (5, 6), torch.float64)
        h = g.op("gelu", g.op("linear", x, w, bias))                    # [2, 3, 5]
        h2 = g.op("reshape", h, shape=(6, 5))
        y = g.op("matmul", h2, m)                                       # [6, 6]
        yt = g.op("transpose", y, dim0=0, dim1=1)
        r = g.op("mean", yt, dim=1, keepdim=True)                       # [6, 1]
        s = g.op("sum", g.op("mul", yt, r), dim=0)                      # [6]
        out = g.op("mean", s)
        g.output(out)
        return g, out
    feeds = {"x": torch.randn(2, 3, 4, dtype=torch.float64), "w": torch.randn(5, 4, dtype=torch.float64), "bias": torch.randn(5, dtype=torch.float64),
             "m": torch.randn(5, 6, dtype=torch.float64)}

    def ref(l):
        h = F.gelu(F.linear(l["x"], l["w"], l["bias"]), approximate="tanh").reshape(6, 5)
        yt = (h @ l["m"]).t()
        return ((yt * yt.mean(1, keepdim=True)).sum(0)).mean()
    _check(build, feeds, ["x", "w", "bias", "m"], ref, atol=1e-9)


def test_pow_scale_cast_unused_inputs_and_errors():
    def build():
        g = HLGraph()
        x, unused = g.input("x", (4,), torch.float64), g.input("unused", (2,), torch.float64)
        p = g.op("cast", x, dtype=torch.float64)
        g.ops.append(Op("pow", [p], "%p3", {"exponent": 3}))
        g.values["%p3"] = Value("%p3", (4,), torch.float64)
        g.ops.append(Op("scale", ["%p3"], "%sc", {"factor": 0.5}))
        g.values["%sc"] = Value("%sc", (4,), torch.float64)
        side = g.op("exp", unused)                                      # not on the path to the output
        g.output("%sc", side)
        return g, "%sc"
    feeds = {"x": torch.tensor([0.5, -1.0, 2.0, 3.0], dtype=torch.float64), "unused": torch.zeros(2, dtype=torch.float64)}
    bg = _check(build, feeds, ["x", "unused"], lambda l: 0.5 * l["x"] ** 3)
    assert not any(o.kind == "exp" and o.output in bg.outputs for o in bg.ops)
    g, out = build()
    both, names = AD.build_backward(g, out, ["x"], keep_forward_outputs=True)
    assert len(both.outputs) == 3 and both.outputs[-1] == names[0]
    fn = AD.gradient_function(g, out, ["x"])
    assert torch.allclose(fn(feeds)[0], 1.5 * feeds["x"] ** 2)
    with pytest.raises(KeyError):
        AD.build_backward(g, "nope", ["x"])
    with pytest.raises(KeyError):
        AD.build_backward(g, out, ["nope"])
    h = HLGraph()
    a = h.input("a", (2, 2))
    o = h.op("softmax", a)
    h.output(o)
    with pytest.raises(NotImplementedError, match="softmax"):
        AD.build_backward(h, o, ["a"])
    reg = AD.default_registry()
    reg.register("softmax", lambda b, op, g: [g])
    assert reg.has("softmax") and AD.build_backward(h, o, ["a"], reg)[1]


def test_gradient_graph_can_be_fused():
    from ml_framework_b200.compiler.fusion_passes import FusionVerifier, GraphTransformer
    g = HLGraph()
    x = g.input("x", (64,))
    c = g.input("c", (64,))
    out = g.op("neg", g.op("sub", g.op("neg", x), c))
    g.output(out)
    bg, _ = AD.build_backward(g, out, ["x"])                # d out / d x = neg(neg(ones)): a chain of single-use element-wise ops
    fused = GraphTransformer().transform(bg)
    assert len(fused.ops) < len(bg.ops) and any(o.kind == "fused_elementwise" for o in fused.ops) and FusionVerifier().verify(bg, fused).passed
