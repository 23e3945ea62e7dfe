"""Reverse-mode differentiation of a high-level IR graph: the gradient is itself a graph.

Reference: the explicit-graph autograd engine - src/MLFramework/Autograd/BackwardPass.cs:44-64 (reverse topological
order, each operation's ``BackwardFn(gradOut)``, gradient accumulation with a broadcast reduce), GraphBuilder.cs,
OperationContext.cs, and the per-operation rules ``Autograd/Operations/{Add,Sub,Mul,Div,Pow,Exp,Log,Sqrt,Relu,Sigmoid,
Tanh,Sum,Mean}Grad.cs`` behind ``IOperationGrad.ComputeGrad`` (Operations/IOperationGrad.cs:9).

Tensors in this package are differentiated by PyTorch's autograd; this module does the same job for GRAPHS: given a
graph and one of its values it appends the operations that compute d value / d input for the requested inputs, so
that the result can be optimised (CSE, fusion of the element-wise gradient chains) and compiled like any other graph.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .ir import HLGraph, Op, Value

GradRule = Callable[["_Builder", Op, str], List[Optional[str]]]


class _Builder:
    """Appends ops to a graph with explicit result shapes (gradient ops are created directly, not through shape
    inference)."""

    def __init__(self, g: HLGraph):
        self.g = g

    def emit(self, kind: str, inputs: Sequence[str], out_shape: Sequence[int], out_dtype: torch.dtype, /, **attrs) -> str:
        out = self.g._fresh("d_" + kind)
        self.g.values[out] = Value(out, tuple(out_shape), out_dtype)
        self.g.ops.append(Op(kind, list(inputs), out, attrs))
        return out

    def like(self, kind: str, inputs: Sequence[str], ref: str, /, **attrs) -> str:
        v = self.g.values[ref]
        return self.emit(kind, inputs, v.shape, v.dtype, **attrs)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.g.values[name].shape)

    def reduce_to(self, grad: str, target: str) -> str:
        """Sums a gradient over the dimensions along which ``target`` was broadcast."""
        if self.shape(grad) == self.shape(target):
            return grad
        v = self.g.values[target]
        return self.emit("sum_to", [grad], v.shape, v.dtype, shape=tuple(v.shape))


class OperationGradRegistry:
    """``rule(builder, op, upstream) -> [gradient value or None per input]``."""

    def __init__(self):
        self.rules: Dict[str, GradRule] = {}

    def register(self, kind: str, rule: GradRule):
        self.rules[kind] = rule

    def has(self, kind: str) -> bool:
        return kind in self.rules

    def get(self, kind: str) -> GradRule:
        if kind not in self.rules:
            raise NotImplementedError(f"no gradient rule for operation {kind!r}; registered: {sorted(self.rules)}")
        return self.rules[kind]


def _binary(fa, fb):
    def rule(b: _Builder, o: Op, g: str):
        x, y = o.inputs
        ga, gb = fa(b, o, g, x, y), fb(b, o, g, x, y)
        return [b.reduce_to(ga, x) if ga is not None else None, b.reduce_to(gb, y) if gb is not None else None]
    return rule


def default_registry() -> OperationGradRegistry:
    r = OperationGradRegistry()
    r.register("add", _binary(lambda b, o, g, x, y: g, lambda b, o, g, x, y: g))
    r.register("sub", _binary(lambda b, o, g, x, y: g, lambda b, o, g, x, y: b.like("neg", [g], g)))
    r.register("mul", _binary(lambda b, o, g, x, y: b.like("mul", [g, y], o.output), lambda b, o, g, x, y: b.like("mul", [g, x], o.output)))

    def div_b(b, o, g, x, y):               # -g * (x / y) / y
        q = b.like("div", [o.output, y], o.output)
        return b.like("neg", [b.like("mul", [g, q], o.output)], o.output)
    r.register("div", _binary(lambda b, o, g, x, y: b.like("div", [g, y], o.output), div_b))
    r.register("neg", lambda b, o, g: [b.like("neg", [g], g)])
    r.register("exp", lambda b, o, g: [b.like("mul", [g, o.output], o.output)])
    r.register("log", lambda b, o, g: [b.like("div", [g, o.inputs[0]], o.output)])

    def sqrt_rule(b, o, g):                 # g / (2 sqrt(x))
        return [b.like("div", [b.like("scale", [g], g, factor=0.5), o.output], o.output)]
    r.register("sqrt", sqrt_rule)

    def pow_rule(b, o, g):                  # g * p * x^(p-1)
        p = o.attrs["exponent"]
        xp = b.like("pow", [o.inputs[0]], o.output, exponent=p - 1)
        return [b.like("scale", [b.like("mul", [g, xp], o.output)], o.output, factor=float(p))]
    r.register("pow", pow_rule)
    r.register("scale", lambda b, o, g: [b.like("scale", [g], g, factor=o.attrs["factor"])])
    r.register("relu", lambda b, o, g: [b.like("relu_grad", [g, o.inputs[0]], o.output)])
    r.register("sigmoid", lambda b, o, g: [b.like("sigmoid_grad", [g, o.output], o.output)])
    r.register("tanh", lambda b, o, g: [b.like("tanh_grad", [g, o.output], o.output)])
    r.register("gelu", lambda b, o, g: [b.like("gelu_grad", [g, o.inputs[0]], o.output)])

    def reduce_rule(mean: bool):
        def rule(b: _Builder, o: Op, g: str):
            x = o.inputs[0]
            shp = b.shape(x)
            n = 1
            if "dim" in o.attrs:
                ax = o.attrs["dim"] % len(shp)
                n = shp[ax]
                view = list(shp)
                view[ax] = 1
                attrs = {"shape": shp} if o.attrs.get("keepdim", False) else {"shape": shp, "view": tuple(view)}
            else:
                for d in shp:
                    n *= d
                attrs = {"shape": shp, "view": (1,) * len(shp)}
            e = b.like("broadcast_to", [g], x, **attrs)
            return [b.like("scale", [e], x, factor=1.0 / n) if mean else e]
        return rule
    r.register("sum", reduce_rule(False))
    r.register("mean", reduce_rule(True))

    def matmul_rule(b, o, g):               # dA = g B^T, dB = A^T g (2-D operands)
        a, w = o.inputs
        if len(b.shape(a)) != 2 or len(b.shape(w)) != 2:
            raise NotImplementedError("matmul gradients are implemented for 2-D operands")
        wt = b.emit("transpose", [w], b.shape(w)[::-1], b.g.values[w].dtype, dim0=-2, dim1=-1)
        at = b.emit("transpose", [a], b.shape(a)[::-1], b.g.values[a].dtype, dim0=-2, dim1=-1)
        return [b.like("matmul", [g, wt], a), b.like("matmul", [at, g], w)]
    r.register("matmul", matmul_rule)

    def linear_rule(b, o, g):               # y = x W^T + bias, x [..., in], W [out, in]
        x, w = o.inputs[0], o.inputs[1]
        xs, ws = b.shape(x), b.shape(w)
        rows = 1
        for d in xs[:-1]:
            rows *= d
        g2 = g if len(xs) == 2 else b.emit("reshape", [g], (rows, ws[0]), b.g.values[g].dtype, shape=(rows, ws[0]))
        x2 = x if len(xs) == 2 else b.emit("reshape", [x], (rows, xs[-1]), b.g.values[x].dtype, shape=(rows, xs[-1]))
        dx2 = b.emit("matmul", [g2, w], (rows, xs[-1]), b.g.values[x].dtype)
        dx = dx2 if len(xs) == 2 else b.emit("reshape", [dx2], xs, b.g.values[x].dtype, shape=xs)
        g2t = b.emit("transpose", [g2], (ws[0], rows), b.g.values[g].dtype, dim0=-2, dim1=-1)
        dw = b.emit("matmul", [g2t, x2], ws, b.g.values[w].dtype)
        out = [dx, dw]
        if len(o.inputs) > 2:
            out.append(b.emit("sum", [g2], (ws[0],), b.g.values[g].dtype, dim=0))
        return out
    r.register("linear", linear_rule)
    r.register("reshape", lambda b, o, g: [b.like("reshape", [g], o.inputs[0], shape=b.shape(o.inputs[0]))])
    r.register("transpose", lambda b, o, g: [b.like("transpose", [g], o.inputs[0], **o.attrs)])
    r.register("cast", lambda b, o, g: [b.like("cast", [g], o.inputs[0], dtype=b.g.values[o.inputs[0]].dtype)])
    return r


def build_backward(graph: HLGraph, output: str, wrt: Sequence[str], registry: Optional[OperationGradRegistry] = None,
                   keep_forward_outputs: bool = False) -> Tuple[HLGraph, List[str]]:
    """A copy of ``graph`` extended by the operations that compute d sum(``output``) / d ``w`` for every ``w`` in ``wrt``;
    returns it with the names of the gradient values (which are the new graph's outputs, after the forward outputs
    when ``keep_forward_outputs``). A value that does not influence the output gets a zero gradient."""
    from .fusion_passes import clone_graph
    reg = registry or default_registry()
    g = clone_graph(graph)
    if output not in g.values:
        raise KeyError(f"unknown value {output!r}")
    for w in wrt:
        if w not in g.values:
            raise KeyError(f"unknown value {w!r}")
    b = _Builder(g)
    forward_ops = list(g.ops)
    producer = {o.output: o for o in forward_ops}
    # only ops that lie on a path to ``output``
    needed, stack = set(), [output]
    while stack:
        n = stack.pop()
        o = producer.get(n)
        if o is not None and o.output not in needed:
            needed.add(o.output)
            stack.extend(o.inputs)
    grads: Dict[str, str] = {output: b.like("ones_like", [output], output)}
    for o in reversed(forward_ops):
        if o.output not in needed or o.output not in grads:
            continue
        ups = reg.get(o.kind)(b, o, grads[o.output])
        if len(ups) != len(o.inputs):
            raise RuntimeError(f"gradient rule of {o.kind!r} returned {len(ups)} gradients for {len(o.inputs)} inputs")
        for name, gi in zip(o.inputs, ups):
            if gi is None or g.values[name].const is not None and name not in wrt:
                continue
            grads[name] = gi if name not in grads else b.like("add", [grads[name], gi], name)      # accumulation
    outs = []
    for w in wrt:
        if w in grads:
            outs.append(grads[w])
        else:
            v = g.values[w]
            outs.append(g.constant(torch.zeros(v.shape, dtype=v.dtype)))
    g.outputs = (list(g.outputs) if keep_forward_outputs else []) + outs
    errs = g.verify()
    if errs:
        raise RuntimeError(f"gradient graph is invalid: {errs}")
    return g, outs


def gradient_function(graph: HLGraph, output: str, wrt: Sequence[str], optimize: bool = True) -> Callable[[Dict[str, torch.Tensor]], List[torch.Tensor]]:
    """``feeds -> [gradients]``: builds the gradient graph once (optionally running the optimisation passes over it)."""
    bg, _ = build_backward(graph, output, wrt)
    if optimize:
        from .ir import CommonSubexpressionElimination, DeadCodeElimination
        CommonSubexpressionElimination().run(bg)
        DeadCodeElimination().run(bg)
    return bg.run
