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
from typing import Dict, List, Optional, Sequence, Tuple

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
        self._next_id = 0
        self._shape = ShapeInferenceEngine()

    # ---- builder
    def _fresh(self, hint: str) -> str:
        self._next_id += 1
        return f"%{hint}{self._next_id - 1}"

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

    # ---- structured control flow (the reference's high-level If / Loop ops, IR/HLIR/ControlFlow/*.cs)
    def cond(self, pred: str, then_graph: "HLGraph", else_graph: "HLGraph", *args: str) -> str:
        """``then_graph(*args)`` where the scalar ``pred`` is non-zero, else ``else_graph(*args)``. Both branches take
        ``args`` as their inputs (in order) and return one value of the same shape and dtype."""
        for b in (then_graph, else_graph):
            if len(b.inputs) != len(args) or len(b.outputs) != 1:
                raise ValueError("a branch takes the op's arguments and returns one value")
        t, e = then_graph.values[then_graph.outputs[0]], else_graph.values[else_graph.outputs[0]]
        if t.shape != e.shape or t.dtype != e.dtype:
            raise ValueError(f"branches disagree: {t.shape} {t.dtype} vs {e.shape} {e.dtype}")
        out = self._fresh("if")
        self.values[out] = Value(out, t.shape, t.dtype)
        self.ops.append(Op("if", [pred, *args], out, {"then": then_graph, "else": else_graph}))
        return out

    def loop(self, count: int, body: "HLGraph", init: str, *invariants: str) -> str:
        """``carry = body(carry, *invariants)`` repeated ``count`` times, starting from ``init``."""
        if len(body.inputs) != 1 + len(invariants) or len(body.outputs) != 1:
            raise ValueError("a loop body takes (carry, *invariants) and returns the next carry")
        c0, c1 = self.values[init], body.values[body.outputs[0]]
        if c0.shape != c1.shape or c0.dtype != c1.dtype:
            raise ValueError(f"the body changes the carried value: {c0.shape} {c0.dtype} -> {c1.shape} {c1.dtype}")
        out = self._fresh("loop")
        self.values[out] = Value(out, c0.shape, c0.dtype)
        self.ops.append(Op("loop", [init, *invariants], out, {"count": int(count), "body": body}))
        return out

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
    if k == "if":
        br = a["then"] if bool(x[0].reshape(-1)[0] != 0) else a["else"]
        return br.run(dict(zip(br.inputs, x[1:])))[0]
    if k == "loop":
        body, carry = a["body"], x[0]
        for _ in range(a["count"]):
            carry = body.run(dict(zip(body.inputs, [carry, *x[1:]])))[0]
        return carry
    if k.endswith("_scalar"):     # a binary op whose constant scalar operand was inlined into the attributes
        c = torch.tensor(a["scalar"], dtype=x[0].dtype, device=x[0].device)
        return _execute(Op(k[:-7], [], ""), [c, x[0]] if a.get("scalar_side") == "lhs" else [x[0], c])
    # ---- ops that only gradient graphs produce (compiler/autodiff.py)
    if k == "ones_like": return torch.ones_like(x[0])
    if k == "broadcast_to": return x[0].reshape(a["view"]).expand(a["shape"]).contiguous() if "view" in a else x[0].expand(a["shape"]).contiguous()
    if k == "sum_to": return x[0].sum_to_size(a["shape"]) if tuple(x[0].shape) != tuple(a["shape"]) else x[0]
    if k == "scale": return x[0] * a["factor"]
    if k == "pow": return torch.pow(x[0], a["exponent"])
    if k == "relu_grad": return x[0] * (x[1] > 0).to(x[0].dtype)
    if k == "sigmoid_grad": return x[0] * x[1] * (1 - x[1])                    # (upstream, sigmoid output)
    if k == "tanh_grad": return x[0] * (1 - x[1] * x[1])                        # (upstream, tanh output)
    if k == "gelu_grad":
        g, t = x[0], x[1].detach().clone().requires_grad_(True)
        with torch.enable_grad():
            (d,) = torch.autograd.grad(F.gelu(t, approximate="tanh").sum(), t)
        return g * d
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
    if k in ("matmul", "linear"):
        # ``epilogue`` (set by the fusion rewrite): "gelu", or "residual" with the residual as the LAST input
        epi = a.get("epilogue")
        res = x[-1] if epi == "residual" else None
        if res is not None:
            x = x[:-1]
        bias = x[2] if k == "linear" and len(x) > 2 else None
        if epi is None and k == "linear" and x[0].is_cuda and x[0].dtype == torch.bfloat16:
            from ..ops import functional as Fn
            return Fn.linear(x[0], x[1], bias)
        if x[0].is_cuda and x[0].dtype == torch.bfloat16 and x[1].dim() == 2 and (k == "linear" or x[0].dim() == 2):
            # one tensor-core GEMM whose epilogue applies bias / GELU / residual
            from ..ops.gemm import EPI_BIAS, EPI_GELU, EPI_RESIDUAL, gemm
            x2 = x[0].reshape(-1, x[0].shape[-1])
            flags = (EPI_BIAS if bias is not None else 0) | (EPI_GELU if epi == "gelu" else 0) | (EPI_RESIDUAL if res is not None else 0)
            n_out = x[1].shape[0] if k == "linear" else x[1].shape[1]
            y = gemm(x2, x[1], b_mn=(k == "matmul"), bias=bias, flags=flags,
                     aux_in=res.reshape(-1, n_out).contiguous() if res is not None else None)
            return y.reshape(*x[0].shape[:-1], n_out)
        y = F.linear(x[0], x[1], bias) if k == "linear" else x[0] @ x[1]
        if epi == "gelu":
            y = F.gelu(y, approximate="tanh")
        return y + res if res is not None else y
    if k == "conv2d":
        y = F.conv2d(x[0], x[1], x[2] if len(x) > 2 else None, a.get("stride", 1), a.get("padding", 0), a.get("dilation", 1), a.get("groups", 1))
        act = a.get("activation")
        return _execute(Op(act, [], ""), [y]) if act else y
    if k == "batchnorm":      # inputs: x, gamma, beta, running mean, running variance (inference form)
        return F.batch_norm(x[0], x[3], x[4], x[1], x[2], False, 0.0, a.get("eps", 1e-5))
    if k == "maxpool2d": return F.max_pool2d(x[0], a.get("kernel", 2), a.get("stride", a.get("kernel", 2)), a.get("padding", 0))
    if k == "avgpool2d": return F.avg_pool2d(x[0], a.get("kernel", 2), a.get("stride", a.get("kernel", 2)), a.get("padding", 0))
    if k == "reshape": return x[0].reshape(a["shape"])
    if k == "transpose": return x[0].transpose(a.get("dim0", -2), a.get("dim1", -1))
    if k == "concat": return torch.cat(x, a.get("dim", 0))
    if k == "slice":
        steps = a.get("steps", [1] * len(a["starts"]))
        return x[0][tuple(slice(b, e, st) for b, e, st in zip(a["starts"], a["ends"], steps))].contiguous()
    if k in ("sum", "mean", "max"):
        if "dim" not in a:
            return getattr(x[0], k)()
        r = getattr(x[0], "amax" if k == "max" else k)(a["dim"], keepdim=a.get("keepdim", False))
        return r
    if k == "layer_norm": return F.layer_norm(x[0], x[0].shape[-1:], x[1] if len(x) > 1 else None, x[2] if len(x) > 2 else None, a.get("eps", 1e-5))
    if k == "fused_elementwise":
        if x[0].is_cuda and a.get("jit", True) and all(t.shape == x[0].shape and t.dtype == x[0].dtype for t in x[1:]) \
                and x[0].dtype in (torch.bfloat16, torch.float16, torch.float32):
            # one generated kernel for the whole chain (compiled on first use, cached per chain and dtype)
            from .jit_cuda import SNIPPETS, CompileError, compile_chain
            kinds = tuple(kind for kind, _ in a["chain"])
            if all(kd in SNIPPETS for kd in kinds) and _JIT_CHAINS.get(kinds) is not False:
                fn = _JIT_CHAINS.get(kinds)
                if fn is None:
                    fn = _JIT_CHAINS[kinds] = compile_chain(kinds)
                try:
                    return fn(*x)
                except CompileError:
                    _JIT_CHAINS[kinds] = False       # no compiler here: this chain runs op by op from now on
        v = x[0]
        rest = iter(x[1:])
        for kind, binary in a["chain"]:
            v = _execute(Op(kind, [], ""), [v, next(rest)] if binary else [v])
        return v
    raise NotImplementedError(k)


_JIT_CHAINS: Dict[tuple, object] = {}       # fused element-wise chains compiled at run time, by op-name tuple


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


# ------------------------------------------------------------------ mid level: buffers, explicit broadcasts, loop nests
@dataclass
class MLStmt:
    """One statement of the mid-level IR. ``kind``:
    ``alloc`` (dst), ``broadcast`` (src -> dst of the statement's shape), ``map`` (element-wise ``fn`` over sources that
    all have the destination's shape: broadcasting is explicit at this level), ``contract`` (dst[.., m, n] = sum_k
    lhs[.., m, k] * rhs[.., k, n]), ``reduce`` (``fn`` over ``dims``), ``call`` (an op kept whole: conv, pool, norm,
    softmax, reshape ...)."""
    kind: str
    dst: str
    srcs: List[str] = field(default_factory=list)
    fn: str = ""
    attrs: dict = field(default_factory=dict)


class MLProgram:
    def __init__(self, name: str):
        self.name = name
        self.buffers: Dict[str, Tuple[Tuple[int, ...], torch.dtype]] = {}
        self.consts: Dict[str, torch.Tensor] = {}
        self.inputs: List[str] = []
        self.outputs: List[str] = []
        self.stmts: List[MLStmt] = []

    def verify(self) -> List[str]:
        errs, ready = [], set(self.inputs) | set(self.consts)
        allocated = set(ready)
        for i, st in enumerate(self.stmts):
            if st.kind == "alloc":
                if st.dst in allocated:
                    errs.append(f"stmt #{i}: buffer {st.dst} allocated twice")
                allocated.add(st.dst)
                continue
            for n in st.srcs:
                if n not in ready:
                    errs.append(f"stmt #{i} {st.kind}: read of {n} before it is written")
            if st.dst not in allocated:
                errs.append(f"stmt #{i} {st.kind}: write to unallocated buffer {st.dst}")
            if st.kind == "map":
                for n in st.srcs:
                    if self.buffers[n][0] != self.buffers[st.dst][0]:
                        errs.append(f"stmt #{i} map: operand {n} {self.buffers[n][0]} differs from {st.dst} {self.buffers[st.dst][0]}"
                                    " (broadcasts are explicit at this level)")
            ready.add(st.dst)
        errs += [f"output {n} never written" for n in self.outputs if n not in ready]
        return errs

    def run(self, feeds: Dict[str, torch.Tensor]) -> List[torch.Tensor]:
        env: Dict[str, torch.Tensor] = dict(self.consts)
        env.update(feeds)
        for st in self.stmts:
            if st.kind == "alloc":
                continue
            x = [env[n] for n in st.srcs]
            if st.kind == "broadcast":
                env[st.dst] = x[0].expand(self.buffers[st.dst][0]).contiguous()
            elif st.kind == "map":
                env[st.dst] = _execute(Op(st.fn, [], "", st.attrs), x)
            elif st.kind == "contract":
                env[st.dst] = torch.einsum("...mk,...kn->...mn", x[0], x[1])
            elif st.kind == "reduce":
                env[st.dst] = _execute(Op(st.fn, [], "", st.attrs), x)
            else:
                env[st.dst] = _execute(Op(st.fn, [], "", st.attrs), x)
        return [env[n] for n in self.outputs]

    def dump(self) -> List[str]:
        out = []
        for st in self.stmts:
            shp = self.buffers[st.dst][0]
            idx = ", ".join(f"i{k}" for k in range(len(shp)))
            if st.kind == "alloc":
                out.append(f"{st.dst} = ml.alloc {shp}")
            elif st.kind == "broadcast":
                out.append(f"ml.parallel_for ({idx}) in {shp} {{ {st.dst}[{idx}] = ml.broadcast({st.srcs[0]})[{idx}] }}")
            elif st.kind == "map":
                out.append(f"ml.parallel_for ({idx}) in {shp} {{ {st.dst}[{idx}] = {st.fn}(" + ", ".join(f"{n}[{idx}]" for n in st.srcs) + ") }")
            elif st.kind == "contract":
                k = self.buffers[st.srcs[0]][0][-1]
                out.append(f"ml.parallel_for ({idx}) in {shp} {{ acc = 0; ml.for k in {k} {{ acc += {st.srcs[0]}[.., k] * {st.srcs[1]}[k, ..] }}; {st.dst}[{idx}] = acc }}")
            elif st.kind == "reduce":
                out.append(f"ml.reduce<{st.fn}> {st.srcs[0]} over {st.attrs.get('dim', 'all')} -> {st.dst}")
            else:
                out.append(f"ml.call @{st.fn}({', '.join(st.srcs)}) -> {st.dst}")
        return out


def lower_to_ml(g: HLGraph) -> MLProgram:
    """High level -> mid level: every value becomes a buffer with an allocation, broadcasting operands of element-wise
    ops get explicit broadcast statements, matmul becomes a contraction loop nest, reductions are marked as such
    (the reference's HLIRtoMLIRLoweringPass)."""
    p = MLProgram(g.name)
    p.inputs, p.outputs = list(g.inputs), list(g.outputs)
    for n, v in g.values.items():
        p.buffers[n] = (tuple(v.shape), v.dtype)
        if v.const is not None:
            p.consts[n] = v.const
    tmp = itertools.count()
    for o in g.ops:
        shp = tuple(g.values[o.output].shape)
        p.stmts.append(MLStmt("alloc", o.output))
        if o.kind in ELEMENTWISE or o.kind in UNARY:
            srcs = []
            for n in o.inputs:
                if tuple(g.values[n].shape) != shp:
                    b = f"%bc{next(tmp)}"
                    p.buffers[b] = (shp, g.values[n].dtype)
                    p.stmts.append(MLStmt("alloc", b))
                    p.stmts.append(MLStmt("broadcast", b, [n]))
                    srcs.append(b)
                else:
                    srcs.append(n)
            p.stmts.append(MLStmt("map", o.output, srcs, o.kind, dict(o.attrs)))
        elif o.kind == "matmul" and len(g.values[o.inputs[0]].shape) >= 2 and len(g.values[o.inputs[1]].shape) >= 2:
            p.stmts.append(MLStmt("contract", o.output, list(o.inputs)))
        elif o.kind in ("sum", "mean", "max"):
            p.stmts.append(MLStmt("reduce", o.output, list(o.inputs), o.kind, dict(o.attrs)))
        else:
            p.stmts.append(MLStmt("call", o.output, list(o.inputs), o.kind, dict(o.attrs)))
    return p


# ------------------------------------------------------------------ low level: scalar instructions over flat buffers
@dataclass
class LLInstr:
    """``op``: loop / endloop (counted loops with an index register), load / store (flat address = sum of index
    registers times strides), const, the scalar arithmetic of the element-wise ops, fma, and ``call`` for statements
    kept whole. Registers are named strings; buffers are flat arrays."""
    op: str
    dst: str = ""
    args: Tuple = ()


class LLProgram:
    def __init__(self, ml: MLProgram):
        self.ml = ml
        self.instrs: List[LLInstr] = []

    def dump(self) -> List[str]:
        out, depth = [], 0
        for ins in self.instrs:
            if ins.op == "endloop":
                depth -= 1
            out.append("    " * depth + (f"{ins.dst} = " if ins.dst else "") + f"ll.{ins.op} " + ", ".join(str(a) for a in ins.args))
            if ins.op == "loop":
                depth += 1
        return out

    def verify(self) -> List[str]:
        errs, depth, defined = [], 0, set()
        for i, ins in enumerate(self.instrs):
            if ins.op == "loop":
                depth += 1
                defined.add(ins.dst)
            elif ins.op == "endloop":
                depth -= 1
                if depth < 0:
                    errs.append(f"instr #{i}: endloop without loop")
            elif ins.op in ("load", "const", "acc0"):
                defined.add(ins.dst)
            elif ins.op == "call":
                pass
            else:
                regs = [a for a in ins.args if isinstance(a, str) and a.startswith("%r")]
                for r in regs:
                    if r not in defined:
                        errs.append(f"instr #{i} {ins.op}: register {r} used before definition")
                if ins.dst:
                    defined.add(ins.dst)
        if depth != 0:
            errs.append("unbalanced loops")
        return errs

    def run(self, feeds: Dict[str, torch.Tensor]) -> List[torch.Tensor]:
        """Scalar interpreter (the CPU back-end of last resort: exact, slow; meant for small shapes and for checking
        the lowering)."""
        import math
        ml = self.ml
        mem: Dict[str, list] = {n: t.detach().double().reshape(-1).tolist() for n, t in ml.consts.items()}
        for n, t in feeds.items():
            mem[n] = t.detach().double().reshape(-1).tolist()
        reg: Dict[str, float] = {}
        tens: Dict[str, torch.Tensor] = {}
        unary = {"relu": lambda v: max(v, 0.0), "neg": lambda v: -v, "exp": math.exp, "log": math.log, "sqrt": math.sqrt,
                 "tanh": math.tanh, "sigmoid": lambda v: 1.0 / (1.0 + math.exp(-v)),
                 "gelu": lambda v: 0.5 * v * (1.0 + math.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))}
        binary = {"add": lambda a, b: a + b, "sub": lambda a, b: a - b, "mul": lambda a, b: a * b, "div": lambda a, b: a / b,
                  "maximum": max, "minimum": min}
        # match loops
        stack, jump = [], {}
        for i, ins in enumerate(self.instrs):
            if ins.op == "loop":
                stack.append(i)
            elif ins.op == "endloop":
                j = stack.pop()
                jump[i], jump[j] = j, i
        pc = 0

        def addr(terms):
            return int(sum(reg[r] * s for r, s in terms))
        while pc < len(self.instrs):
            ins = self.instrs[pc]
            o = ins.op
            if o == "alloc":
                shp = ml.buffers[ins.dst][0]
                n = 1
                for d in shp:
                    n *= d
                mem[ins.dst] = [0.0] * n
            elif o == "loop":
                reg[ins.dst] = 0.0
                if ins.args[0] <= 0:
                    pc = jump[pc]
            elif o == "endloop":
                j = jump[pc]
                r, n = self.instrs[j].dst, self.instrs[j].args[0]
                reg[r] += 1.0
                if reg[r] < n:
                    pc = j
            elif o == "load":
                reg[ins.dst] = mem[ins.args[0]][addr(ins.args[1])]
            elif o == "store":
                mem[ins.args[0]][addr(ins.args[1])] = reg[ins.args[2]]
            elif o == "const" or o == "acc0":
                reg[ins.dst] = float(ins.args[0]) if ins.args else 0.0
            elif o == "fma":
                reg[ins.dst] = reg[ins.args[0]] * reg[ins.args[1]] + reg[ins.args[2]]
            elif o in unary:
                reg[ins.dst] = unary[o](reg[ins.args[0]])
            elif o in binary:
                reg[ins.dst] = binary[o](reg[ins.args[0]], reg[ins.args[1]])
            elif o == "call":
                st = ins.args[0]
                x = []
                for n in st.srcs:
                    shp, dt = ml.buffers[n]
                    x.append(torch.tensor(mem[n], dtype=torch.float64).reshape(shp))
                if st.kind == "broadcast":
                    y = x[0].expand(ml.buffers[st.dst][0]).contiguous()
                else:
                    y = _execute(Op(st.fn, [], "", st.attrs), x)
                mem[st.dst] = y.double().reshape(-1).tolist()
            else:
                raise NotImplementedError(o)
            pc += 1
        outs = []
        for n in ml.outputs:
            shp, dt = ml.buffers[n]
            outs.append(torch.tensor(mem[n], dtype=torch.float64).reshape(shp).to(dt))
        return outs


def _strides(shape):
    st, acc = [], 1
    for d in reversed(shape):
        st.append(acc)
        acc *= d
    return list(reversed(st))


def lower_to_ll(ml: MLProgram) -> LLProgram:
    """Mid level -> low level: maps become counted loops with loads, scalar ops and stores; contractions become the
    three-deep loop nest with a fused multiply-add; everything else stays a call (the reference's
    MLIRtoLLIRLoweringPass)."""
    p = LLProgram(ml)
    ids = itertools.count()
    r = lambda: f"%r{next(ids)}"  # noqa: E731
    for st in ml.stmts:
        if st.kind == "alloc":
            p.instrs.append(LLInstr("alloc", st.dst))
            continue
        shp = ml.buffers[st.dst][0]
        if st.kind == "map" and st.fn in (ELEMENTWISE | UNARY) and not st.attrs:
            n = 1
            for d in shp:
                n *= d
            i = r()
            p.instrs.append(LLInstr("loop", i, (n,)))
            vals = []
            for s in st.srcs:
                v = r()
                p.instrs.append(LLInstr("load", v, (s, ((i, 1),))))
                vals.append(v)
            o = r()
            p.instrs.append(LLInstr(st.fn, o, tuple(vals)))
            p.instrs.append(LLInstr("store", "", (st.dst, ((i, 1),), o)))
            p.instrs.append(LLInstr("endloop"))
        elif st.kind == "contract" and len(shp) == 2 and len(ml.buffers[st.srcs[0]][0]) == 2 and len(ml.buffers[st.srcs[1]][0]) == 2:
            M, N = shp
            K = ml.buffers[st.srcs[0]][0][1]
            im, in_, ik, acc, a, b = r(), r(), r(), r(), r(), r()
            p.instrs += [LLInstr("loop", im, (M,)), LLInstr("loop", in_, (N,)), LLInstr("acc0", acc), LLInstr("loop", ik, (K,)),
                         LLInstr("load", a, (st.srcs[0], ((im, K), (ik, 1)))), LLInstr("load", b, (st.srcs[1], ((ik, N), (in_, 1)))),
                         LLInstr("fma", acc, (a, b, acc)), LLInstr("endloop"),
                         LLInstr("store", "", (st.dst, ((im, N), (in_, 1)), acc)), LLInstr("endloop"), LLInstr("endloop")]
        else:
            p.instrs.append(LLInstr("call", st.dst, (st,)))
    return p


def lower_to_loops(g: HLGraph) -> List[str]:
    """Listing of the mid-level program of ``g``."""
    return lower_to_ml(g).dump()


def lower_to_instructions(loops_or_graph) -> List[str]:
    """Listing of the low-level program (accepts a graph, a mid-level program, or - for callers that only want a
    listing of a listing - the lines of ``lower_to_loops``)."""
    if isinstance(loops_or_graph, HLGraph):
        return lower_to_ll(lower_to_ml(loops_or_graph)).dump()
    if isinstance(loops_or_graph, MLProgram):
        return lower_to_ll(loops_or_graph).dump()
    out = []
    for i, l in enumerate(loops_or_graph):
        if l.lstrip().startswith("ml.parallel_for"):
            out += [f"%i{i} = ll.loop n", "    %v = ll.load", "    %r = ll.op %v", "    ll.store %r", "ll.endloop"]
        elif "ml.alloc" in l:
            out.append(f"%buf{i} = ll.alloc")
        else:
            out.append(f"ll.call {l.split('@')[-1] if '@' in l else l}")
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


class CPUBackend:
    """Host back-end: runs a graph through all three levels. ``compile`` optimises the high-level graph, lowers it to
    the mid level (buffers, explicit broadcasts, loop nests) and verifies it; the returned ``run`` executes the
    mid-level program with vectorised host kernels. ``level="ll"`` lowers once more and runs the scalar instruction
    interpreter instead (exact and slow: for checking the lowering on small shapes). The reference's CPU back-end is
    src/MLFramework/IR/Backend/CPU/*."""
    triple = "x86_64-unknown-linux-gnu"

    def compile(self, g: HLGraph, options: Optional[CompilationOptions] = None, level: str = "ml") -> Dict[str, object]:
        if (options or CompilationOptions()).optimization_level > 0:
            PassManager().run(g)
        ml = lower_to_ml(g)
        errs = ml.verify()
        if errs:
            raise RuntimeError(f"mid-level IR invalid: {errs}")
        if level == "ml":
            return {"target": "cpu", "level": "ml", "program": ml, "run": ml.run}
        ll = lower_to_ll(ml)
        errs = ll.verify()
        if errs:
            raise RuntimeError(f"low-level IR invalid: {errs}")
        return {"target": "cpu", "level": "ll", "program": ll, "run": ll.run}
