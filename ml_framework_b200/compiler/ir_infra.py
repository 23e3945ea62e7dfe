"""Infrastructure around the IR: verifier, rewriter, instrumented pass runs, constant handling, back-end registry.

Reference: src/MLFramework/IR/Transformations/{IRVerifier.cs, OperationRewriter.cs, PassInstrumentation.cs,
IRPassManager.cs, LoweringPassBase.cs}, IR/Passes/{InlineConstantsPass.cs, ConstantEvaluator.cs},
IR/Backend/{BackendRegistry.cs, BackendCompiler.cs, CompilationOptions.cs, OptimizationLevel.cs},
IR/Backend/GPU/{ComputeCapability.cs (SM_70 .. SM_90), CUDABackend.cs (default SM_80, emits a PTX header only)}.
Here the accelerator target is sm_100a and "emitting code" for it means: the kernel plan of the graph plus the CUDA
source of every fused element-wise op (compiled at run time by :mod:`ml_framework_b200.compiler.jit_cuda`).
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .ir import (B200Backend, CompilationOptions, CPUBackend, HLGraph, Op, Pass, PassManager, _execute, lower_to_ll, lower_to_ml)
from .shapes import ShapeInferenceEngine, SymbolicShape


# ------------------------------------------------------------------ verifier
@dataclass
class VerifierDiagnostic:
    severity: str          # "error" | "warning"
    where: str
    message: str


class IRVerifier:
    """Structural and type checks of a high-level graph: single definition, definition before use, declared outputs,
    shapes and dtypes that agree with what shape inference derives from the operands, branch / body signatures of
    control-flow ops (checked recursively), and - as warnings - values that nothing reads."""

    def __init__(self, check_shapes: bool = True):
        self.check_shapes = check_shapes
        self._infer = ShapeInferenceEngine()

    def verify(self, g: HLGraph, _path: str = "") -> List[VerifierDiagnostic]:
        d: List[VerifierDiagnostic] = []
        where = lambda i, o: f"{_path}{g.name}#{i}:{o.kind}"      # noqa: E731
        defined = set(g.inputs) | {n for n, v in g.values.items() if v.const is not None}
        for n in g.inputs:
            if n not in g.values:
                d.append(VerifierDiagnostic("error", f"{_path}{g.name}", f"input {n} has no value record"))
        for i, o in enumerate(g.ops):
            for n in o.inputs:
                if n not in defined:
                    d.append(VerifierDiagnostic("error", where(i, o), f"use of undefined value {n}"))
            if o.output in defined:
                d.append(VerifierDiagnostic("error", where(i, o), f"value {o.output} defined twice"))
            defined.add(o.output)
            if o.output not in g.values:
                d.append(VerifierDiagnostic("error", where(i, o), f"result {o.output} has no value record"))
                continue
            if o.kind in ("if", "loop"):
                subs = [o.attrs["then"], o.attrs["else"]] if o.kind == "if" else [o.attrs["body"]]
                n_args = len(o.inputs) - 1 if o.kind == "if" else len(o.inputs)
                for sub in subs:
                    if len(sub.inputs) != n_args:
                        d.append(VerifierDiagnostic("error", where(i, o), f"sub-graph {sub.name} takes {len(sub.inputs)} inputs, op passes {n_args}"))
                    d += self.verify(sub, f"{_path}{g.name}#{i}/")
                continue
            if self.check_shapes and o.kind in self._infer.rules and all(n in g.values for n in o.inputs):
                try:
                    want = self._infer.infer(o.kind, [SymbolicShape(g.values[n].shape) for n in o.inputs], **o.attrs).concrete()
                    if tuple(want) != tuple(g.values[o.output].shape):
                        d.append(VerifierDiagnostic("error", where(i, o), f"result shape {g.values[o.output].shape}, operands give {tuple(want)}"))
                except Exception as e:       # noqa: BLE001 - a shape rule that rejects the operands is the finding
                    d.append(VerifierDiagnostic("error", where(i, o), f"operands rejected: {e}"))
        for n in g.outputs:
            if n not in defined:
                d.append(VerifierDiagnostic("error", f"{_path}{g.name}", f"output {n} undefined"))
        used = {n for o in g.ops for n in o.inputs} | set(g.outputs)
        for o in g.ops:
            if o.output not in used:
                d.append(VerifierDiagnostic("warning", f"{_path}{g.name}", f"value {o.output} is never read"))
        return d

    def errors(self, g: HLGraph) -> List[VerifierDiagnostic]:
        return [x for x in self.verify(g) if x.severity == "error"]

    def check(self, g: HLGraph):
        e = self.errors(g)
        if e:
            raise RuntimeError("IR verification failed:\n" + "\n".join(f"  {x.where}: {x.message}" for x in e))


# ------------------------------------------------------------------ rewriter
RewriteFn = Callable[[HLGraph, Op], Optional[object]]


class OperationRewriter:
    """Rule-driven local rewrites. A rule is ``(kind, fn)``; ``fn(graph, op)`` returns ``None`` (no change), a value
    name (the op's result is replaced by that existing value), or a list of ops (the op is replaced by them; the last
    one must define the original result name). Rules are applied to a fixed point, at most ``max_rounds`` sweeps."""

    def __init__(self, max_rounds: int = 8):
        self.rules: List[Tuple[str, RewriteFn, str]] = []
        self.max_rounds = max_rounds
        self.applied: Dict[str, int] = {}

    def add_rule(self, kind: str, fn: RewriteFn, name: Optional[str] = None):
        self.rules.append((kind, fn, name or getattr(fn, "__name__", "rule")))
        return self

    def run(self, g: HLGraph) -> int:
        total = 0
        for _ in range(self.max_rounds):
            rename: Dict[str, str] = {}
            out: List[Op] = []
            n = 0
            for o in g.ops:
                o = Op(o.kind, [rename.get(x, x) for x in o.inputs], o.output, o.attrs)
                rep = None
                for kind, fn, name in self.rules:
                    if kind in (o.kind, "*"):
                        rep = fn(g, o)
                        if rep is not None:
                            self.applied[name] = self.applied.get(name, 0) + 1
                            break
                if rep is None:
                    out.append(o)
                elif isinstance(rep, str):
                    rename[o.output] = rename.get(rep, rep)      # the rule may have read a name this sweep already replaced
                    n += 1
                else:
                    rep = list(rep)
                    if not rep or rep[-1].output != o.output:
                        raise ValueError("a replacement sequence must end by defining the replaced result")
                    out.extend(rep)
                    n += 1
            g.ops = out
            g.outputs = [rename.get(x, x) for x in g.outputs]
            total += n
            if n == 0:
                break
        return total


class RewritePass(Pass):
    def __init__(self, rewriter: OperationRewriter, name: str = "rewrite"):
        self.rewriter, self.name = rewriter, name

    def run(self, g):
        return self.rewriter.run(g) > 0


# ------------------------------------------------------------------ constants
class ConstantEvaluator:
    """Evaluates an op whose operands are all constants, within a size budget (folding must not materialise a
    large tensor that the program would otherwise compute lazily)."""

    def __init__(self, max_result_elems: int = 1 << 22):
        self.max_result_elems = max_result_elems

    def can_evaluate(self, g: HLGraph, o: Op) -> bool:
        if o.kind in ("if", "loop") or not o.inputs:
            return False
        if any(g.values[n].const is None for n in o.inputs):
            return False
        n = 1
        for dim in g.values[o.output].shape:
            n *= int(dim)
        return n <= self.max_result_elems

    def evaluate(self, g: HLGraph, o: Op) -> torch.Tensor:
        return _execute(o, [g.values[n].const for n in o.inputs])


class InlineConstants(Pass):
    """Constant hygiene: (1) identical constants (same dtype, shape and bytes) become one value; (2) constants nobody
    reads are dropped; (3) with ``inline_scalars``, a binary element-wise op with a one-element constant operand
    becomes ``<op>_scalar`` with the number in its attributes, so the kernel takes an immediate instead of a pointer."""
    name = "inline-constants"
    _BIN = ("add", "sub", "mul", "div", "maximum", "minimum")

    def __init__(self, inline_scalars: bool = True):
        self.inline_scalars = inline_scalars

    def run(self, g):
        changed = False
        seen: Dict[tuple, str] = {}
        rename: Dict[str, str] = {}
        for n, v in g.values.items():
            if v.const is None or n in g.inputs:
                continue
            key = (str(v.const.dtype), tuple(v.const.shape), v.const.detach().cpu().contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()
                   if v.const.numel() <= 4096 else id(v.const))
            if key in seen:
                rename[n] = seen[key]
            else:
                seen[key] = n
        if rename:
            changed = True
            for o in g.ops:
                o.inputs = [rename.get(x, x) for x in o.inputs]
            g.outputs = [rename.get(x, x) for x in g.outputs]
        if self.inline_scalars:
            for o in g.ops:
                if o.kind in self._BIN and len(o.inputs) == 2:
                    for side, idx in (("rhs", 1), ("lhs", 0)):
                        c = g.values[o.inputs[idx]].const
                        other = g.values[o.inputs[1 - idx]]
                        if c is not None and c.numel() == 1 and other.const is None and tuple(other.shape) == tuple(g.values[o.output].shape):
                            o.attrs = {**o.attrs, "scalar": float(c.reshape(-1)[0]), "scalar_side": side}
                            o.inputs = [o.inputs[1 - idx]]
                            o.kind = o.kind + "_scalar"
                            changed = True
                            break
        used = {x for o in g.ops for x in o.inputs} | set(g.outputs)
        dead = [n for n, v in g.values.items() if v.const is not None and n not in used and n not in g.inputs]
        for n in dead:
            del g.values[n]
            changed = True
        return changed


# ------------------------------------------------------------------ instrumented pass runs
@dataclass
class PassRecord:
    name: str
    changed: bool
    ops_before: int
    ops_after: int
    ms: float


class PassInstrumentation:
    """Callbacks and records around every pass of an ``InstrumentedPassManager``."""

    def __init__(self):
        self.records: List[PassRecord] = []
        self.before: List[Callable[[str, HLGraph], None]] = []
        self.after: List[Callable[[PassRecord, HLGraph], None]] = []

    def summary(self) -> Dict[str, Dict[str, float]]:
        out: Dict[str, Dict[str, float]] = {}
        for r in self.records:
            s = out.setdefault(r.name, {"runs": 0, "changed": 0, "ms": 0.0, "ops_removed": 0})
            s["runs"] += 1
            s["changed"] += int(r.changed)
            s["ms"] += r.ms
            s["ops_removed"] += r.ops_before - r.ops_after
        return out

    def render(self) -> str:
        return "\n".join(f"{k}: {v['runs']} runs, {v['changed']} with changes, {v['ops_removed']} ops removed, {v['ms']:.3f} ms"
                         for k, v in self.summary().items())


class InstrumentedPassManager(PassManager):
    def __init__(self, passes: Optional[Sequence[Pass]] = None, instrumentation: Optional[PassInstrumentation] = None,
                 verifier: Optional[IRVerifier] = None, max_iterations: int = 8):
        super().__init__(passes, verify=False, max_iterations=max_iterations)
        self.instr = instrumentation or PassInstrumentation()
        self.verifier = verifier

    def run(self, g: HLGraph) -> HLGraph:
        for _ in range(self.max_iterations):
            any_change = False
            for p in self.passes:
                for cb in self.instr.before:
                    cb(p.name, g)
                n0, t0 = len(g.ops), time.perf_counter()
                ch = p.run(g)
                rec = PassRecord(p.name, ch, n0, len(g.ops), (time.perf_counter() - t0) * 1e3)
                self.instr.records.append(rec)
                self.log.append((p.name, ch, len(g.ops)))
                for cb in self.instr.after:
                    cb(rec, g)
                if self.verifier is not None:
                    errs = self.verifier.errors(g)
                    if errs:
                        raise RuntimeError(f"IR invalid after pass {p.name}: " + "; ".join(e.message for e in errs))
                any_change |= ch
            if not any_change:
                break
        return g


# ------------------------------------------------------------------ lowering passes as objects
class LoweringPass:
    """One step down the level stack; ``run`` returns the lower program and verifies it."""
    source, target = "", ""

    def run(self, program):
        raise NotImplementedError


class HLToMLLowering(LoweringPass):
    source, target = "hl", "ml"

    def run(self, program: HLGraph):
        ml = lower_to_ml(program)
        errs = ml.verify()
        if errs:
            raise RuntimeError(f"mid-level IR invalid: {errs}")
        return ml


class MLToLLLowering(LoweringPass):
    source, target = "ml", "ll"

    def run(self, program):
        ll = lower_to_ll(program)
        errs = ll.verify()
        if errs:
            raise RuntimeError(f"low-level IR invalid: {errs}")
        return ll


# ------------------------------------------------------------------ back-ends
class OptimizationLevel(enum.IntEnum):
    NONE = 0
    BASIC = 1          # folding, simplification, CSE, DCE
    STANDARD = 2       # + constant hygiene
    AGGRESSIVE = 3     # + fusion rewrites (checked by the verifier when one is configured)


class ComputeCapability(enum.Enum):
    SM_70 = (7, 0, "")
    SM_75 = (7, 5, "")
    SM_80 = (8, 0, "")
    SM_90 = (9, 0, "")
    SM_90A = (9, 0, "a")
    SM_100 = (10, 0, "")
    SM_100A = (10, 0, "a")

    @property
    def arch(self) -> str:
        return f"sm_{self.value[0]}{self.value[1]}{self.value[2]}"

    @property
    def has_tcgen05(self) -> bool:
        return self.value[0] == 10 and self.value[2] == "a"

    @property
    def has_tma(self) -> bool:
        return self.value[0] >= 9

    def gencode(self) -> str:
        c = f"{self.value[0]}{self.value[1]}{self.value[2]}"
        return f"arch=compute_{c},code=sm_{c}"


@dataclass
class CompiledProgram:
    target: str
    run: Callable[[Dict[str, torch.Tensor]], List[torch.Tensor]]
    plan: List[tuple] = field(default_factory=list)
    sources: Dict[str, str] = field(default_factory=dict)      # result name -> CUDA source of a generated kernel
    graph: Optional[HLGraph] = None
    level: str = "hl"


class BackendRegistry:
    def __init__(self):
        self._b: Dict[str, Callable[[], object]] = {}

    def register(self, name: str, factory: Callable[[], object]):
        self._b[name] = factory

    def get(self, name: str):
        if name not in self._b:
            raise KeyError(f"unknown back-end {name!r}; registered: {sorted(self._b)}")
        return self._b[name]()

    def names(self) -> List[str]:
        return sorted(self._b)


def default_backend_registry() -> BackendRegistry:
    r = BackendRegistry()
    r.register("b200", B200Backend)
    r.register("cpu", CPUBackend)
    return r


class BackendCompiler:
    """``compile(graph, target, options)``: optimise at the requested level, then hand the graph to the back-end."""

    def __init__(self, registry: Optional[BackendRegistry] = None, verifier: Optional[IRVerifier] = None):
        self.registry, self.verifier = registry or default_backend_registry(), verifier or IRVerifier()

    def optimize(self, g: HLGraph, level: OptimizationLevel) -> HLGraph:
        if level >= OptimizationLevel.BASIC:
            InstrumentedPassManager(verifier=self.verifier).run(g)
        if level >= OptimizationLevel.STANDARD:
            InlineConstants(inline_scalars=False).run(g)
        if level >= OptimizationLevel.AGGRESSIVE:
            from .fusion_passes import FusionFallbackHandler, FusionVerifier
            g = FusionFallbackHandler(verifier=FusionVerifier(trials=1)).compile(g)
        return g

    def compile(self, g: HLGraph, target: str = "b200", options: Optional[CompilationOptions] = None, cpu_level: str = "ml") -> CompiledProgram:
        opts = options or CompilationOptions()
        self.verifier.check(g)
        g = self.optimize(g, OptimizationLevel(min(int(opts.optimization_level), 3)))
        be = self.registry.get(target)
        no_opt = CompilationOptions(optimization_level=0, target=opts.target, fast_math=opts.fast_math)
        if isinstance(be, CPUBackend):
            r = be.compile(g, no_opt, level=cpu_level)
            return CompiledProgram("cpu", r["run"], graph=g, level=r["level"])
        r = be.compile(g, no_opt)
        sources = {}
        if isinstance(be, B200Backend):
            from .fusion_passes import FusionKernelGenerator
            gen = FusionKernelGenerator()
            for o in g.ops:
                if o.kind == "fused_elementwise":
                    sources[o.output] = gen.source(o, g.values[o.output].dtype if g.values[o.output].dtype != torch.float64 else torch.float32,
                                                   "k_" + o.output.strip("%"))
        return CompiledProgram(r.get("target", target), r["run"], r.get("plan", []), sources, g)
