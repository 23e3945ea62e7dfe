"""Typed construction of the high-level IR: types, attributes, one class per operation, modules of
functions, and a graph analyser.

Reference: src/MLFramework/IR — Types/{TensorType.cs, ScalarType.cs}, Attributes/{TensorAttribute.cs,
FloatAttribute.cs, IntAttribute.cs, BoolAttribute.cs, ArrayAttribute.cs}, Operations/** (AddOp, SubOp,
MulOp, DivOp, MatMulOp, Conv2DOp, MaxPool2DOp, AvgPool2DOp, ReLUOp, SigmoidOp, TanhOp, GELUOp,
ReduceSumOp, ReduceMeanOp, ReduceMaxOp, ReshapeOp, TransposeOp, BroadcastToOp, SliceOp, CastOp,
ConstantOp, IfOp, LoopOp), HLIR/{HLIRModule.cs, HLIRFunction.cs, HLIRGraphAnalyzer.cs}, IROpcode.cs.

The executable IR of this package names operations by strings (``compiler.ir.HLGraph.op``); the classes
here are the typed front door to it: each checks its own operands and attributes, then emits exactly
one graph operation, so everything downstream (passes, lowering, differentiation, execution) is shared.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from .ir import HLGraph, PassManager

__all__ = [
    "ScalarType", "TensorType", "Attribute", "IntAttribute", "FloatAttribute", "BoolAttribute", "ArrayAttribute",
    "TensorAttribute", "IROpcode", "IRValue", "Operation", "AddOp", "SubOp", "MulOp", "DivOp", "MatMulOp", "LinearOp", "Conv2DOp",
    "MaxPool2DOp", "AvgPool2DOp", "ReLUOp", "SigmoidOp", "TanhOp", "GELUOp", "ExpOp", "LogOp", "SqrtOp", "NegOp", "SoftmaxOp",
    "ReduceSumOp", "ReduceMeanOp", "ReduceMaxOp", "ReshapeOp", "TransposeOp", "BroadcastToOp", "SliceOp", "CastOp", "ConcatOp",
    "ConstantOp", "IfOp", "LoopOp", "HLIRFunction", "HLIRModule", "HLIRGraphAnalyzer", "GraphStatistics",
]


class ScalarType(enum.Enum):
    FLOAT32 = torch.float32
    FLOAT16 = torch.float16
    BFLOAT16 = torch.bfloat16
    FLOAT64 = torch.float64
    INT8 = torch.int8
    INT32 = torch.int32
    INT64 = torch.int64
    BOOL = torch.bool

    @property
    def size_in_bytes(self) -> int:
        return torch.empty((), dtype=self.value).element_size()

    @property
    def is_floating_point(self) -> bool:
        return self.value.is_floating_point

    @classmethod
    def of(cls, dtype: torch.dtype) -> "ScalarType":
        for s in cls:
            if s.value == dtype:
                return s
        raise TypeError(f"{dtype} has no IR scalar type")


@dataclass(frozen=True)
class TensorType:
    element_type: ScalarType
    shape: Tuple[int, ...]

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def num_elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def size_in_bytes(self) -> int:
        return self.num_elements * self.element_type.size_in_bytes

    def with_shape(self, shape: Sequence[int]) -> "TensorType":
        return TensorType(self.element_type, tuple(shape))

    def __str__(self):
        return f"tensor<{'x'.join(map(str, self.shape)) or 'scalar'}x{self.element_type.name.lower()}>"


# ---- attributes: compile-time constants attached to an operation
@dataclass(frozen=True)
class Attribute:
    value: object


class IntAttribute(Attribute):
    def __init__(self, value: int):
        if isinstance(value, bool) or not isinstance(value, int):
            raise TypeError("an integer attribute needs an int")
        super().__init__(value)


class FloatAttribute(Attribute):
    def __init__(self, value: float):
        super().__init__(float(value))


class BoolAttribute(Attribute):
    def __init__(self, value: bool):
        if not isinstance(value, bool):
            raise TypeError("a boolean attribute needs a bool")
        super().__init__(value)


class ArrayAttribute(Attribute):
    def __init__(self, values: Sequence):
        super().__init__(tuple(v.value if isinstance(v, Attribute) else v for v in values))

    def __len__(self):
        return len(self.value)


class TensorAttribute(Attribute):
    def __init__(self, value: torch.Tensor):
        if not isinstance(value, torch.Tensor):
            raise TypeError("a tensor attribute needs a tensor")
        super().__init__(value)

    @property
    def type(self) -> TensorType:
        return TensorType(ScalarType.of(self.value.dtype), tuple(self.value.shape))

    def __hash__(self):
        return id(self.value)


class IROpcode(enum.Enum):
    ADD = "add"; SUB = "sub"; MUL = "mul"; DIV = "div"; MATMUL = "matmul"; LINEAR = "linear"; CONV2D = "conv2d"      # noqa: E702
    MAXPOOL2D = "maxpool2d"; AVGPOOL2D = "avgpool2d"; RELU = "relu"; SIGMOID = "sigmoid"; TANH = "tanh"; GELU = "gelu"  # noqa: E702
    EXP = "exp"; LOG = "log"; SQRT = "sqrt"; NEG = "neg"; SOFTMAX = "softmax"; REDUCE_SUM = "sum"; REDUCE_MEAN = "mean"  # noqa: E702
    REDUCE_MAX = "max"; RESHAPE = "reshape"; TRANSPOSE = "transpose"; BROADCAST_TO = "broadcast_to"; SLICE = "slice"    # noqa: E702
    CAST = "cast"; CONCAT = "concat"; CONSTANT = "constant"; IF = "if"; LOOP = "loop"                                    # noqa: E702


@dataclass(frozen=True)
class IRValue:
    """A value of a graph: its name there and its type."""
    graph: HLGraph
    name: str

    @property
    def type(self) -> TensorType:
        v = self.graph.values[self.name]
        return TensorType(ScalarType.of(v.dtype), tuple(v.shape))

    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(self.graph.values[self.name].shape)

    def __str__(self):
        return f"{self.name}: {self.type}"


def _plain(v):
    return v.value if isinstance(v, Attribute) else v


class Operation:
    """Base of the typed operations: ``XOp(graph, operands..., attributes...)`` checks, emits one graph
    operation and exposes ``result``."""

    opcode: IROpcode
    arity: Optional[int] = None

    def __init__(self, graph: HLGraph, *operands: IRValue, **attrs):
        if self.arity is not None and len(operands) != self.arity:
            raise ValueError(f"{type(self).__name__} takes {self.arity} operand(s), got {len(operands)}")
        for o in operands:
            if not isinstance(o, IRValue) or o.graph is not graph:
                raise ValueError(f"{type(self).__name__}: operands must be values of the same graph")
        self.graph, self.operands = graph, tuple(operands)
        self.attributes: Dict[str, object] = {k: _plain(v) for k, v in attrs.items() if v is not None}
        self.validate()
        self.result = IRValue(graph, graph.op(self.opcode.value, *(o.name for o in operands), **self.attributes))

    def validate(self) -> None:
        pass

    def __str__(self):
        a = f" {self.attributes}" if self.attributes else ""
        return f"{self.result.name} = {self.opcode.value}({', '.join(o.name for o in self.operands)}){a} : {self.result.type}"


def _binary(code):
    return type(f"_{code.name}", (Operation,), {"opcode": code, "arity": 2})


class AddOp(_binary(IROpcode.ADD)): pass                  # noqa: E701
class SubOp(_binary(IROpcode.SUB)): pass                  # noqa: E701
class MulOp(_binary(IROpcode.MUL)): pass                  # noqa: E701
class DivOp(_binary(IROpcode.DIV)): pass                  # noqa: E701


class MatMulOp(Operation):
    opcode, arity = IROpcode.MATMUL, 2

    def validate(self):
        a, b = self.operands
        if len(a.shape) < 2 or len(b.shape) < 2:
            raise ValueError("MatMulOp: both operands need at least two dimensions")


class LinearOp(Operation):
    """``x @ w^T (+ bias)`` with ``w`` as [out, in]."""
    opcode = IROpcode.LINEAR

    def validate(self):
        if len(self.operands) not in (2, 3):
            raise ValueError("LinearOp takes (input, weight) or (input, weight, bias)")


def _unary(code):
    return type(f"_{code.name}", (Operation,), {"opcode": code, "arity": 1})


class ReLUOp(_unary(IROpcode.RELU)): pass                 # noqa: E701
class SigmoidOp(_unary(IROpcode.SIGMOID)): pass           # noqa: E701
class TanhOp(_unary(IROpcode.TANH)): pass                 # noqa: E701
class GELUOp(_unary(IROpcode.GELU)): pass                 # noqa: E701
class ExpOp(_unary(IROpcode.EXP)): pass                   # noqa: E701
class LogOp(_unary(IROpcode.LOG)): pass                   # noqa: E701
class SqrtOp(_unary(IROpcode.SQRT)): pass                 # noqa: E701
class NegOp(_unary(IROpcode.NEG)): pass                   # noqa: E701


class SoftmaxOp(Operation):
    opcode, arity = IROpcode.SOFTMAX, 1

    def __init__(self, graph, x, dim: int = -1):
        super().__init__(graph, x, dim=dim)


class Conv2DOp(Operation):
    opcode = IROpcode.CONV2D

    def __init__(self, graph, x, weight, bias: Optional[IRValue] = None, stride=1, padding=0, dilation=1, groups: int = 1,
                 activation: Optional[str] = None):
        ops = (x, weight) if bias is None else (x, weight, bias)
        super().__init__(graph, *ops, stride=stride, padding=padding, dilation=dilation, groups=groups, activation=activation)

    def validate(self):
        x, w = self.operands[0], self.operands[1]
        if len(x.shape) != 4 or len(w.shape) != 4:
            raise ValueError("Conv2DOp: input [N, C, H, W] and weight [O, C/groups, kh, kw]")
        if self.attributes.get("groups", 1) <= 0:
            raise ValueError("Conv2DOp: groups must be positive")


class _Pool(Operation):
    arity = 1

    def __init__(self, graph, x, kernel=2, stride=None, padding=0):
        super().__init__(graph, x, kernel=kernel, stride=stride if stride is not None else kernel, padding=padding)

    def validate(self):
        if len(self.operands[0].shape) != 4:
            raise ValueError(f"{type(self).__name__}: the input must be [N, C, H, W]")


class MaxPool2DOp(_Pool):
    opcode = IROpcode.MAXPOOL2D


class AvgPool2DOp(_Pool):
    opcode = IROpcode.AVGPOOL2D


class _Reduce(Operation):
    arity = 1

    def __init__(self, graph, x, dim: Union[int, Sequence[int]], keepdim: bool = False):
        super().__init__(graph, x, dim=dim if isinstance(dim, int) else tuple(dim), keepdim=keepdim)

    def validate(self):
        rank = len(self.operands[0].shape)
        dims = self.attributes["dim"]
        for d in ((dims,) if isinstance(dims, int) else dims):
            if not -rank <= d < rank:
                raise ValueError(f"{type(self).__name__}: dimension {d} out of range for rank {rank}")


class ReduceSumOp(_Reduce):
    opcode = IROpcode.REDUCE_SUM


class ReduceMeanOp(_Reduce):
    opcode = IROpcode.REDUCE_MEAN


class ReduceMaxOp(_Reduce):
    opcode = IROpcode.REDUCE_MAX


class ReshapeOp(Operation):
    opcode, arity = IROpcode.RESHAPE, 1

    def __init__(self, graph, x, shape: Sequence[int]):
        super().__init__(graph, x, shape=tuple(_plain(shape)))


class TransposeOp(Operation):
    opcode, arity = IROpcode.TRANSPOSE, 1

    def __init__(self, graph, x, dim0: int = -2, dim1: int = -1):
        super().__init__(graph, x, dim0=dim0, dim1=dim1)


class BroadcastToOp(Operation):
    opcode, arity = IROpcode.BROADCAST_TO, 1

    def __init__(self, graph, x, shape: Sequence[int]):
        super().__init__(graph, x, shape=tuple(_plain(shape)))

    def validate(self):
        src, dst = self.operands[0].shape, self.attributes["shape"]
        if len(src) > len(dst):
            raise ValueError("BroadcastToOp: the target has fewer dimensions than the input")
        for s, d in zip(src[::-1], dst[::-1]):
            if s != d and s != 1:
                raise ValueError(f"BroadcastToOp: {src} cannot be broadcast to {tuple(dst)}")


class SliceOp(Operation):
    opcode, arity = IROpcode.SLICE, 1

    def __init__(self, graph, x, starts: Sequence[int], ends: Sequence[int], steps: Optional[Sequence[int]] = None):
        super().__init__(graph, x, starts=tuple(_plain(starts)), ends=tuple(_plain(ends)),
                         steps=tuple(_plain(steps)) if steps is not None else None)


class CastOp(Operation):
    opcode, arity = IROpcode.CAST, 1

    def __init__(self, graph, x, target: Union[ScalarType, torch.dtype]):
        super().__init__(graph, x, dtype=target.value if isinstance(target, ScalarType) else target)


class ConcatOp(Operation):
    opcode = IROpcode.CONCAT

    def __init__(self, graph, *values: IRValue, dim: int = 0):
        if len(values) < 2:
            raise ValueError("ConcatOp needs at least two values")
        super().__init__(graph, *values, dim=dim)


class ConstantOp:
    """A compile-time tensor: becomes a constant value of the graph (no operation is emitted)."""
    opcode = IROpcode.CONSTANT

    def __init__(self, graph: HLGraph, value: Union[torch.Tensor, TensorAttribute, float, int], name: Optional[str] = None):
        t = value.value if isinstance(value, TensorAttribute) else value
        if not isinstance(t, torch.Tensor):
            t = torch.tensor(t, dtype=torch.float32 if isinstance(t, float) else None)
        self.graph, self.value = graph, t
        self.result = IRValue(graph, graph.constant(t, name))


class IfOp:
    """``then(*args)`` where the scalar predicate is non-zero, else ``otherwise(*args)``."""
    opcode = IROpcode.IF

    def __init__(self, graph: HLGraph, predicate: IRValue, then: "HLIRFunction", otherwise: "HLIRFunction", *args: IRValue):
        self.graph = graph
        self.result = IRValue(graph, graph.cond(predicate.name, then.graph, otherwise.graph, *(a.name for a in args)))


class LoopOp:
    """``carry = body(carry, *invariants)`` repeated ``count`` times."""
    opcode = IROpcode.LOOP

    def __init__(self, graph: HLGraph, count: int, body: "HLIRFunction", init: IRValue, *invariants: IRValue):
        if count < 0:
            raise ValueError("the trip count cannot be negative")
        self.graph = graph
        self.result = IRValue(graph, graph.loop(count, body.graph, init.name, *(v.name for v in invariants)))


# ------------------------------------------------------------------ functions and modules
class HLIRFunction:
    """One graph with a typed signature."""

    def __init__(self, name: str, parameters: Sequence[Tuple[str, TensorType]] = ()):
        self.name, self.graph = name, HLGraph(name)
        self.parameters: List[IRValue] = []
        for n, t in parameters:
            self.add_parameter(n, t)

    def add_parameter(self, name: str, type: TensorType) -> IRValue:
        if name in self.graph.values:
            raise ValueError(f"parameter {name!r} already exists")
        v = IRValue(self.graph, self.graph.input(name, type.shape, type.element_type.value))
        self.parameters.append(v)
        return v

    def set_results(self, *values: IRValue) -> None:
        self.graph.outputs.clear()
        self.graph.output(*(v.name for v in values))

    @property
    def results(self) -> List[IRValue]:
        return [IRValue(self.graph, n) for n in self.graph.outputs]

    @property
    def signature(self) -> str:
        ins = ", ".join(str(p) for p in self.parameters)
        outs = ", ".join(str(r.type) for r in self.results)
        return f"@{self.name}({ins}) -> ({outs})"

    def verify(self) -> List[str]:
        errs = self.graph.verify()
        if not self.graph.outputs:
            errs.append(f"function {self.name} returns nothing")
        return errs

    def optimize(self) -> "HLIRFunction":
        PassManager().run(self.graph)
        return self

    def __call__(self, *tensors: torch.Tensor):
        if len(tensors) != len(self.parameters):
            raise ValueError(f"{self.name} takes {len(self.parameters)} arguments, got {len(tensors)}")
        for p, t in zip(self.parameters, tensors):
            if tuple(t.shape) != p.shape:
                raise ValueError(f"{self.name}: argument {p.name} has shape {tuple(t.shape)}, expected {p.shape}")
        out = self.graph.run({p.name: t for p, t in zip(self.parameters, tensors)})
        return out[0] if len(out) == 1 else tuple(out)

    def dump(self) -> str:
        return self.graph.dump()


class HLIRModule:
    """Named functions compiled together."""

    def __init__(self, name: str = "module"):
        self.name = name
        self.functions: Dict[str, HLIRFunction] = {}

    def add_function(self, fn: HLIRFunction) -> HLIRFunction:
        if fn.name in self.functions:
            raise ValueError(f"function {fn.name!r} already exists in module {self.name!r}")
        self.functions[fn.name] = fn
        return fn

    def create_function(self, name: str, parameters: Sequence[Tuple[str, TensorType]] = ()) -> HLIRFunction:
        return self.add_function(HLIRFunction(name, parameters))

    def get_function(self, name: str) -> HLIRFunction:
        if name not in self.functions:
            raise KeyError(f"module {self.name!r} has no function {name!r}")
        return self.functions[name]

    def remove_function(self, name: str) -> bool:
        return self.functions.pop(name, None) is not None

    def verify(self) -> List[str]:
        return [f"{n}: {e}" for n, f in self.functions.items() for e in f.verify()]

    def optimize(self) -> "HLIRModule":
        for f in self.functions.values():
            f.optimize()
        return self

    def dump(self) -> str:
        return f"module @{self.name} {{\n" + "\n\n".join(f.dump() for f in self.functions.values()) + "\n}"


# ------------------------------------------------------------------ analysis
@dataclass
class GraphStatistics:
    operation_count: int
    operations_by_kind: Dict[str, int]
    depth: int                        # longest chain of dependent operations
    flops: int
    parameter_bytes: int              # constants held by the graph
    activation_bytes: int             # every produced value, once
    peak_live_bytes: int              # largest set of values alive at one point of the program order


class HLIRGraphAnalyzer:
    """Counts, critical-path depth, arithmetic and memory of a graph."""

    @staticmethod
    def _numel(shape) -> int:
        n = 1
        for d in shape:
            n *= int(d)
        return n

    @classmethod
    def _flops(cls, g: HLGraph, o) -> int:
        out = cls._numel(g.values[o.output].shape)
        if o.kind in ("matmul", "linear"):
            return 2 * out * int(g.values[o.inputs[0]].shape[-1])
        if o.kind == "conv2d":
            w = g.values[o.inputs[1]].shape
            return 2 * out * int(w[1]) * int(w[2]) * int(w[3])
        if o.kind in ("sum", "mean", "max", "softmax", "layer_norm"):
            return cls._numel(g.values[o.inputs[0]].shape) * (5 if o.kind in ("softmax", "layer_norm") else 1)
        if o.kind in ("reshape", "transpose", "slice", "concat", "broadcast_to", "cast"):
            return 0
        if o.kind == "loop":
            return o.attrs["count"] * cls.analyze(o.attrs["body"]).flops
        if o.kind == "if":
            return max(cls.analyze(o.attrs["then"]).flops, cls.analyze(o.attrs["else"]).flops)
        return out

    @classmethod
    def analyze(cls, graph: Union[HLGraph, HLIRFunction]) -> GraphStatistics:
        g = graph.graph if isinstance(graph, HLIRFunction) else graph

        def nbytes(name):
            v = g.values[name]
            return cls._numel(v.shape) * torch.empty((), dtype=v.dtype).element_size()
        kinds: Dict[str, int] = {}
        depth: Dict[str, int] = {}
        last_use: Dict[str, int] = {}
        for i, o in enumerate(g.ops):
            kinds[o.kind] = kinds.get(o.kind, 0) + 1
            depth[o.output] = 1 + max((depth.get(n, 0) for n in o.inputs), default=0)
            for n in o.inputs:
                last_use[n] = i
        for n in g.outputs:
            last_use[n] = len(g.ops)
        live = sum(nbytes(n) for n in g.inputs)
        peak = live
        for i, o in enumerate(g.ops):
            live += nbytes(o.output)
            peak = max(peak, live)
            for n in set(o.inputs) | {o.output}:
                if last_use.get(n, -1) <= i and g.values[n].const is None and (n in g.inputs or n in depth):
                    live -= nbytes(n)
        return GraphStatistics(len(g.ops), kinds, max(depth.values(), default=0), sum(cls._flops(g, o) for o in g.ops),
                               sum(nbytes(n) for n, v in g.values.items() if v.const is not None),
                               sum(nbytes(o.output) for o in g.ops), peak)

    @classmethod
    def critical_path(cls, graph: Union[HLGraph, HLIRFunction]) -> List[str]:
        """Output names of the operations on one longest dependency chain, in order."""
        g = graph.graph if isinstance(graph, HLIRFunction) else graph
        depth: Dict[str, int] = {}
        best_in: Dict[str, Optional[str]] = {}
        for o in g.ops:
            prev = max((n for n in o.inputs if n in depth), key=lambda n: depth[n], default=None)
            depth[o.output] = 1 + (depth[prev] if prev else 0)
            best_in[o.output] = prev
        if not depth:
            return []
        cur: Optional[str] = max(depth, key=lambda n: depth[n])
        path = []
        while cur is not None:
            path.append(cur)
            cur = best_in[cur]
        return path[::-1]
