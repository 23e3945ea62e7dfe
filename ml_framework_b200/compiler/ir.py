"""Three-level IR with lowering and optimisation passes.

Reference: high-level ops (src/MLFramework/IR/HLIR/**, Graph/HLIRBuilder.cs) -> mid level with explicit
broadcasts, loops and allocation (IR/MLIR/**, Lowering/HLIRtoMLIRLoweringPass.cs) -> low level scalar /
vector ops with loads and stores (IR/LLIR/**, MLIRtoLLIRLoweringPass.cs); passes CSE, constant folding,
dead-code elimination, constant inlining, operation simplification (IR/Passes/*.cs); pass manager and
verifier (IR/Transformations/IRPassManager.cs, IRVerifier.cs); back-ends (IR/Backend/GPU/CUDABackend.cs
targets SM_80 and emits only a PTX header).

Here the high-level graph is the useful level: it is what the fusion planner reads (``fusion.py``) and
it can be executed directly (``HLGraph.run``), with ops mapped to this package's kernels on a B200.
The two lowerings produce inspectable loop-nest and instruction listings; the accelerator back-end's
target is sm_100a and "code generation" for it means choosing among the hand-written kernels.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .shapes import ShapeInferenceEngine, SymbolicShape

ELEMENTWISE = {"add", "sub", "mul", "div", "maximum", "minimum"}
UNARY = {"relu", "gelu", "sigmoid", "tanh", "exp", "log", "sqrt", "neg"}


@dataclass
class Value:
    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
    const: Optional[torch.Tensor] = None


@dataclass
class Op:
    kind: str
    inputs: List[str]
    output: str
    attrs: dict = field(default_factory=dict)


class HLGraph:
    def __init__(self, name: str = "main"):
        self.name = name
        self.values: Dict[str, Value] = {}
        self.ops: List[Op] = []
        self.inputs: List[str] = []
        self.outputs: List[str] = []
        self._ids = itertools.count()
        self._shape = ShapeInferenceEngine()

    # ---- builder
    def _fresh(self, hint: str) -> str:
        return f"%{hint}{next(self._ids)}"

    def input(self, name: str, shape: Sequence[int], dtype=torch.float32) -> str:
        self.values[name] = Value(name, tuple(shape), dtype)
        self.inputs.append(name)
        return name

    def constant(self, t: torch.Tensor, name: Optional[str] = None) -> str:
        name = name or self._fresh("c")
        self.values[name] = Value(name, tuple(t.shape), t.dtype, t)
        return name

    def op(self, kind: str, *inputs: str, **attrs) -> str:
        out = self._fresh(kind)
        shp = self._shape.infer(kind, [SymbolicShape(self.values[i].shape) for i in inputs], **attrs).concrete()
        dtype = attrs.get("dtype", self.values[inputs[0]].dtype)
        self.values[out] = Value(out, shp, dtype)
        self.ops.append(Op(kind, list(inputs), out, attrs))
        return out

    def output(self, *names: str):
        self.outputs.extend(names)

    # ---- analysis
    def users(self) -> Dict[str, List[int]]:
        u: Dict[str, List[int]] = {}
        for i, o in enumerate(self.ops):
            for n in o.inputs:
                u.setdefault(n, []).append(i)
        return u

    def verify(self) -> List[str]:
        errs, defined = [], set(self.inputs) | {n for n, v in self.values.items() if v.const is not None}
        for i, o in enumerate(self.ops):
            for n in o.inputs:
                if n not in defined:
                    errs.append(f"op #{i} {o.kind}: use of undefined value {n}")
            if o.output in defined:
                errs.append(f"op #{i} {o.kind}: value {o.output} defined twice")
            defined.add(o.output)
        errs += [f"output {n} undefined" for n in self.outputs if n not in defined]
        return errs

    # ---- execution
    def run(self, feeds: Dict[str, torch.Tensor]) -> List[torch.Tensor]:
        env = {n: v.const for n, v in self.values.items() if v.const is not None}
        env.update(feeds)
        for o in self.ops:
            env[o.output] = _execute(o, [env[n] for n in o.inputs])
        return [env[n] for n in self.outputs]

    def dump(self) -> str:
        lines = [f"func @{self.name}({', '.join(f'{n}: {self.values[n].shape}' for n in self.inputs)}) {{"]
        for o in self.ops:
            a = f" {o.attrs}" if o.attrs else ""
            lines.append(f"  {o.output} = hl.{o.kind}({', '.join(o.inputs)}){a} : {self.values[o.output].shape}")
        lines.append(f"  return {', '.join(self.outputs)}\n}}")
        return "\n".join(lines)


def _execute(o: Op, x: List[torch.Tensor]) -> torch.Tensor:
    import torch.nn.functional as F
    k, a = o.kind, o.attrs
    if k == "add": return x[0] + x[1]
    if k == "sub": return x[0] - x[1]
    if k == "mul": return x[0] * x[1]
    if k == "div": return x[0] / x[1]
    if k == "maximum": return torch.maximum(x[0], x[1])
    if k == "minimum": return torch.minimum(x[0], x[1])
    if k == "relu": return torch.relu(x[0])
    if k == "gelu": return F.gelu(x[0], approximate="tanh")
    if k == "sigmoid": return torch.sigmoid(x[0])
    if k == "tanh": return torch.tanh(x[0])
    if k == "exp": return torch.exp(x[0])
    if k == "log": return torch.log(x[0])
    if k == "sqrt": return torch.sqrt(x[0])
    if k == "neg": return -x[0]
    if k == "cast": return x[0].to(a["dtype"])
    if k == "softmax": return torch.softmax(x[0], a.get("dim", -1))
    if k == "matmul":
        if x[0].is_cuda and x[0].dtype == torch.bfloat16 and x[0].dim() == 2 and x[1].dim() == 2:
            from ..ops.gemm import gemm
            return gemm(x[0], x[1], b_mn=True)
        return x[0] @ x[1]
    if k == "linear":
        if x[0].is_cuda and x[0].dtype == torch.bfloat16:
            from ..ops import functional as Fn
            return Fn.linear(x[0], x[1], x[2] if len(x) > 2 else None)
        return F.linear(x[0], x[1], x[2] if len(x) > 2 else None)
    if k == "conv2d": return F.conv2d(x[0], x[1], x[2] if len(x) > 2 else None, a.get("stride", 1), a.get("padding", 0), a.get("dilation", 1), a.get("groups", 1))
    if k == "maxpool2d": return F.max_pool2d(x[0], a.get("kernel", 2), a.get("stride", a.get("kernel", 2)), a.get("padding", 0))
    if k == "avgpool2d": return F.avg_pool2d(x[0], a.get("kernel", 2), a.get("stride", a.get("kernel", 2)), a.get("padding", 0))
    if k == "reshape": return x[0].reshape(a["shape"])
    if k == "transpose": return x[0].transpose(a.get("dim0", -2), a.get("dim1", -1))
    if k == "concat": return torch.cat(x, a.get("dim", 0))
    if k in ("sum", "mean", "max"):
        if "dim" not in a:
            return getattr(x[0], k)()
        r = getattr(x[0], "amax" if k == "max" else k)(a["dim"], keepdim=a.get("keepdim", False))
        return r
    if k == "layer_norm": return F.layer_norm(x[0], x[0].shape[-1:], x[1] if len(x) > 1 else None, x[2] if len(x) > 2 else None, a.get("eps", 1e-5))
    if k == "fused_elementwise":
        v = x[0]
        rest = iter(x[1:])
        for kind, binary in a["chain"]:
            v = _execute(Op(kind, [], ""), [v, next(rest)] if binary else [v])
        return v
    raise NotImplementedError(k)


# ------------------------------------------------------------------ passes
class Pass:
    name = "pass"

    def run(self, g: HLGraph) -> bool:
        raise NotImplementedError


class DeadCodeElimination(Pass):
    name = "dce"

    def run(self, g):
        live, keep = set(g.outputs), []
        for o in reversed(g.ops):
            if o.output in live:
                keep.append(o)
                live.update(o.inputs)
        keep.reverse()
        changed = len(keep) != len(g.ops)
        g.ops = keep
        return changed


class CommonSubexpressionElimination(Pass):
    name = "cse"

    def run(self, g):
        seen: Dict[Tuple, str] = {}
        rename: Dict[str, str] = {}
        out, changed = [], False
        for o in g.ops:
            ins = [rename.get(n, n) for n in o.inputs]
            if o.kind in ("add", "mul", "maximum", "minimum"):
                key_ins = tuple(sorted(ins))
            else:
                key_ins = tuple(ins)
            key = (o.kind, key_ins, repr(sorted(o.attrs.items(), key=lambda kv: kv[0])))
            if key in seen:
                rename[o.output] = seen[key]
                changed = True
                continue
            seen[key] = o.output
            out.append(Op(o.kind, ins, o.output, o.attrs))
        g.ops = out
        g.outputs = [rename.get(n, n) for n in g.outputs]
        return changed


class ConstantFolding(Pass):
    name = "constant-folding"

    def run(self, g):
        changed, out = False, []
        for o in g.ops:
            if o.inputs and all(g.values[n].const is not None for n in o.inputs):
                g.values[o.output].const = _execute(o, [g.values[n].const for n in o.inputs])
                changed = True
            else:
                out.append(o)
        g.ops = out
        return changed


class OperationSimplification(Pass):
    """x + 0, x * 1, x / 1, neg(neg x), transpose(transpose x) with equal axes, reshape to the same shape."""
    name = "simplify"

    @staticmethod
    def _is_scalar(g, n, v):
        c = g.values[n].const
        return c is not None and c.numel() == 1 and float(c) == v

    def run(self, g):
        rename: Dict[str, str] = {}
        producer = {o.output: o for o in g.ops}
        out, changed = [], False
        for o in g.ops:
            ins = [rename.get(n, n) for n in o.inputs]
            rep = None
            if o.kind in ("add", "sub") and self._is_scalar(g, ins[1], 0.0): rep = ins[0]
            elif o.kind == "add" and self._is_scalar(g, ins[0], 0.0): rep = ins[1]
            elif o.kind in ("mul", "div") and self._is_scalar(g, ins[1], 1.0): rep = ins[0]
            elif o.kind == "mul" and self._is_scalar(g, ins[0], 1.0): rep = ins[1]
            elif o.kind == "neg" and ins[0] in producer and producer[ins[0]].kind == "neg": rep = rename.get(producer[ins[0]].inputs[0], producer[ins[0]].inputs[0])
            elif o.kind == "transpose" and ins[0] in producer and producer[ins[0]].kind == "transpose" and producer[ins[0]].attrs == o.attrs:
                rep = rename.get(producer[ins[0]].inputs[0], producer[ins[0]].inputs[0])
            elif o.kind == "reshape" and tuple(o.attrs["shape"]) == g.values[ins[0]].shape: rep = ins[0]
            if rep is not None and g.values[rep].shape == g.values[o.output].shape:
                rename[o.output] = rep
                changed = True
            else:
                out.append(Op(o.kind, ins, o.output, o.attrs))
        g.ops = out
        g.outputs = [rename.get(n, n) for n in g.outputs]
        return changed


class PassManager:
    def __init__(self, passes: Optional[Sequence[Pass]] = None, verify: bool = True, max_iterations: int = 8):
        self.passes = list(passes) if passes is not None else [ConstantFolding(), OperationSimplification(),
                                                               CommonSubexpressionElimination(), DeadCodeElimination()]
        self.verify, self.max_iterations = verify, max_iterations
        self.log: List[Tuple[str, bool, int]] = []

    def run(self, g: HLGraph) -> HLGraph:
        for _ in range(self.max_iterations):
            any_change = False
            for p in self.passes:
                ch = p.run(g)
                self.log.append((p.name, ch, len(g.ops)))
                any_change |= ch
                if self.verify:
                    errs = g.verify()
                    if errs:
                        raise RuntimeError(f"IR invalid after pass {p.name}: {errs}")
            if not any_change:
                break
        return g


# ------------------------------------------------------------------ lowering
def lower_to_loops(g: HLGraph) -> List[str]:
    """Mid-level listing: explicit allocation, loop nests and broadcasts."""
    out = []
    for o in g.ops:
        shp = g.values[o.output].shape
        out.append(f"{o.output} = ml.alloc {shp}")
        idx = [f"i{k}" for k in range(len(shp))]
        if o.kind in ELEMENTWISE or o.kind in UNARY:
            out.append(f"ml.parallel_for ({', '.join(idx)}) in {shp} {{ {o.output}[{', '.join(idx)}] = {o.kind}("
                       + ", ".join(f"ml.broadcast({n})[{', '.join(idx)}]" for n in o.inputs) + ") }")
        elif o.kind == "matmul":
            k = g.values[o.inputs[0]].shape[-1]
            out.append(f"ml.parallel_for ({', '.join(idx)}) in {shp} {{ acc = 0; ml.for k in {k} {{ acc += {o.inputs[0]}[.., k] * {o.inputs[1]}[k, ..] }}; {o.output}[{', '.join(idx)}] = acc }}")
        elif o.kind in ("sum", "mean", "max"):
            out.append(f"ml.reduce<{o.kind}> {o.inputs[0]} over {o.attrs.get('dim', 'all')} -> {o.output}")
        else:
            out.append(f"ml.call @{o.kind}({', '.join(o.inputs)}) -> {o.output}")
    return out


def lower_to_instructions(loops: Sequence[str]) -> List[str]:
    """Low-level listing: loads, arithmetic, stores, branches per loop body."""
    out = []
    for i, l in enumerate(loops):
        if l.lstrip().startswith("ml.parallel_for"):
            out += [f"L{i}: %tid = ll.thread_index", f"    br.ge %tid, %n, L{i}.end", "    %v = ll.vload.128 [%src + %tid * 16]",
                    "    %r = ll.vop %v", "    ll.vstore.128 [%dst + %tid * 16], %r", f"L{i}.end:"]
        elif "ml.alloc" in l:
            out.append(f"    %buf{i} = ll.alloca_global")
        else:
            out.append(f"    ll.call {l.split('@')[-1] if '@' in l else l}")
    return out


@dataclass
class CompilationOptions:
    optimization_level: int = 2
    target: str = "sm_100a"
    fast_math: bool = True


class B200Backend:
    """Kernel selection for the accelerator: every high-level op maps to a hand-written kernel family
    (or to a library call where the op is outside the hot path)."""
    triple = "nvptx64-nvidia-cuda"
    compute_capability = "sm_100a"
    KERNELS = {"matmul": "gemm_tcgen05", "linear": "gemm_tcgen05 (+bias epilogue)", "gelu": "GEMM epilogue / ew_unary",
               "relu": "ew_unary", "add": "ew_binary / GEMM residual epilogue", "mul": "ew_binary", "sub": "ew_binary", "div": "ew_binary",
               "layer_norm": "norm_fwd", "softmax": "flash_fwd (inside attention) / torch", "sum": "reduce_all / colsum",
               "conv2d": "mobile conv2d (direct) / torch cuDNN", "maxpool2d": "mobile pool2d"}

    def compile(self, g: HLGraph, options: Optional[CompilationOptions] = None) -> Dict[str, object]:
        PassManager().run(g) if (options or CompilationOptions()).optimization_level > 0 else None
        plan = [(o.output, o.kind, self.KERNELS.get(o.kind, "torch")) for o in g.ops]
        return {"target": self.compute_capability, "plan": plan, "run": g.run}
