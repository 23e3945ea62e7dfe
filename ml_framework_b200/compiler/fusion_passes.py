"""Fusion as a checked graph transformation: detect -> validate -> rewrite -> verify -> (fall back).

:mod:`ml_framework_b200.compiler.fusion` finds the patterns; this module is the machinery around a rewrite that the
reference spreads over its fusion directory:

* ``GraphAnalyzer`` / ``OperationCompatibilityChecker`` - access pattern of an op (element-wise, reduction, spatial,
  contraction, gather / scatter, reshape), producers / consumers, pairwise compatibility
  (src/MLFramework/Fusion/Patterns/GraphAnalyzer.cs, OperationCompatibilityChecker.cs);
* pattern detectors as objects with ``detect(graph) -> [FusionPatternMatch]``: element-wise chains, conv + activation,
  conv + batch-norm, linear + bias / GELU / residual (Patterns/*PatternDetector.cs; the last one is this package's GEMM
  epilogue set), each match carrying a ``FusionStrategy`` (FusionStrategy.cs: merge, fold, replace, in-place);
* constraints with violations of a severity: memory layout, numerical precision, side effects, control flow, memory
  access pattern, and the launch-resource constraint, which here knows a B200 SM (1024 threads, 64 K registers,
  227 KB shared memory per CTA, kernel parameter space) instead of a bare thread count
  (Validation/Constraints/*.cs, FusionConstraintsValidator.cs);
* ``GraphTransformer`` - applies accepted matches to a copy of the graph (GraphTransformer.cs);
* ``FusionVerifier`` - runs both graphs on random inputs and compares (Validation/FusionVerifier.cs);
* ``FusionFallbackHandler`` - the fused graph if it verifies and runs, the original otherwise
  (Validation/FusionFallbackHandler.cs);
* ``FusionStatisticsCollector``, ``FusionDecisionLogger``, ``FusionProfiler`` with a timing instrument and a report
  (FusionStatisticsCollector.cs, Profiling/*.cs);
* run-time shape fusion: ``FusionBenefit``, ``FusionCandidateAnalyzer`` (a traffic and launch model with this device's
  measured numbers), ``RuntimeShapeInjector`` (specialises a graph with symbolic sizes for the shapes of a call and
  caches per shape signature), ``FusionKernelGenerator`` (CUDA source of an accepted chain through the run-time
  compiler's renderer) (Dynamic/*.cs);
* the code generator's planning helpers: ``TilingConfiguration``, ``SharedMemoryPlanner``, ``MemoryAccessOptimizer``,
  ``LoopUnrollingOptimizer``, ``CudaTypeMapper`` (KernelCode/Cuda/*.cs).
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .fusion import FusionConstraints, FusionEngine, FusionRegistry
from .ir import ELEMENTWISE, UNARY, HLGraph, Op, Value

ACTIVATIONS = ("relu", "gelu", "sigmoid", "tanh")


# ------------------------------------------------------------------ analysis
class MemoryAccessPattern(enum.Enum):
    ELEMENT_WISE = "element_wise"
    REDUCTION = "reduction"
    SPATIAL = "spatial"            # convolution / pooling windows
    CONTRACTION = "contraction"    # matmul / linear
    GATHER = "gather"
    SCATTER = "scatter"
    RESHAPE = "reshape"            # metadata only
    UNKNOWN = "unknown"


_PATTERN_OF = {**{k: MemoryAccessPattern.ELEMENT_WISE for k in ELEMENTWISE | UNARY | {"cast", "fused_elementwise", "batchnorm"}},
               **{k: MemoryAccessPattern.REDUCTION for k in ("sum", "mean", "max", "softmax", "layer_norm")},
               **{k: MemoryAccessPattern.SPATIAL for k in ("conv2d", "maxpool2d", "avgpool2d")},
               **{k: MemoryAccessPattern.CONTRACTION for k in ("matmul", "linear")},
               "gather": MemoryAccessPattern.GATHER, "embedding": MemoryAccessPattern.GATHER, "scatter": MemoryAccessPattern.SCATTER,
               **{k: MemoryAccessPattern.RESHAPE for k in ("reshape", "transpose", "concat")}}

SIDE_EFFECT_OPS = {"print", "assert", "random", "dropout", "all_reduce", "send", "recv", "copy_"}
CONTROL_FLOW_OPS = {"if", "loop", "while", "cond"}


class GraphAnalyzer:
    def access_pattern(self, op: Op) -> MemoryAccessPattern:
        return _PATTERN_OF.get(op.kind, MemoryAccessPattern.UNKNOWN)

    def producers(self, g: HLGraph) -> Dict[str, int]:
        return {o.output: i for i, o in enumerate(g.ops)}

    def consumers(self, g: HLGraph) -> Dict[str, List[int]]:
        return g.users()

    def single_use(self, g: HLGraph, value: str) -> bool:
        return len(g.users().get(value, ())) == 1 and value not in g.outputs

    def intermediate_bytes(self, g: HLGraph, op_indices: Sequence[int]) -> int:
        """Bytes of the values produced AND consumed inside the group: what a fusion keeps out of memory."""
        inside = set(op_indices)
        users = g.users()
        n = 0
        for i in op_indices:
            v = g.values[g.ops[i].output]
            u = users.get(v.name, [])
            if u and all(k in inside for k in u) and v.name not in g.outputs:
                n += _numel(v.shape) * _itemsize(v.dtype)
        return n

    def external_inputs(self, g: HLGraph, op_indices: Sequence[int]) -> List[str]:
        made = {g.ops[i].output for i in op_indices}
        seen, out = set(), []
        for i in op_indices:
            for n in g.ops[i].inputs:
                if n not in made and n not in seen:
                    seen.add(n)
                    out.append(n)
        return out


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


def _itemsize(dt: torch.dtype) -> int:
    return torch.empty(0, dtype=dt).element_size()


class OperationCompatibilityChecker:
    """Pairwise rule for producer -> consumer fusion."""

    _OK = {(MemoryAccessPattern.ELEMENT_WISE, MemoryAccessPattern.ELEMENT_WISE),
           (MemoryAccessPattern.ELEMENT_WISE, MemoryAccessPattern.REDUCTION),
           (MemoryAccessPattern.SPATIAL, MemoryAccessPattern.ELEMENT_WISE),
           (MemoryAccessPattern.CONTRACTION, MemoryAccessPattern.ELEMENT_WISE)}

    def __init__(self, analyzer: Optional[GraphAnalyzer] = None):
        self.an = analyzer or GraphAnalyzer()

    def patterns_compatible(self, a: MemoryAccessPattern, b: MemoryAccessPattern) -> bool:
        return (a, b) in self._OK

    def can_fuse(self, g: HLGraph, producer: Op, consumer: Op) -> Tuple[bool, str]:
        if producer.output not in consumer.inputs:
            return False, "consumer does not read the producer"
        if not self.an.single_use(g, producer.output):
            return False, "intermediate has other readers"
        pa, pb = self.an.access_pattern(producer), self.an.access_pattern(consumer)
        if not self.patterns_compatible(pa, pb):
            return False, f"access patterns {pa.value} -> {pb.value} do not fuse"
        va, vb = g.values[producer.output], g.values[consumer.output]
        if pb == MemoryAccessPattern.ELEMENT_WISE and va.shape != vb.shape:
            return False, f"shape changes {va.shape} -> {vb.shape}"
        return True, ""


# ------------------------------------------------------------------ matches
class FusionStrategy(enum.Enum):
    MERGE = "merge"        # several ops become one kernel
    FOLD = "fold"          # an op disappears into another one's constants
    REPLACE = "replace"    # the group is replaced by a library / hand-written fused op
    INPLACE = "inplace"    # the consumer overwrites the producer's buffer


@dataclass
class FusionPatternMatch:
    pattern: str
    op_indices: List[int]
    strategy: FusionStrategy
    detail: dict = field(default_factory=dict)

    def ops(self, g: HLGraph) -> List[Op]:
        return [g.ops[i] for i in self.op_indices]


class FusionPatternDetector:
    name = "pattern"
    priority = 0                      # higher first: a GEMM epilogue takes an activation before a chain does

    def detect(self, g: HLGraph) -> List[FusionPatternMatch]:
        raise NotImplementedError


class ElementWisePatternDetector(FusionPatternDetector):
    name, priority = "elementwise_chain", 0

    def __init__(self, registry: Optional[FusionRegistry] = None, constraints: Optional[FusionConstraints] = None):
        self._eng = FusionEngine(registry, constraints)

    def detect(self, g):
        return [FusionPatternMatch(self.name, c, FusionStrategy.MERGE) for c in self._eng.find_elementwise_chains(g)]


class ConvActivationPatternDetector(FusionPatternDetector):
    name, priority = "conv_activation", 2

    def detect(self, g):
        users, out = g.users(), []
        for i, o in enumerate(g.ops):
            if o.kind != "conv2d" or o.output in g.outputs or o.attrs.get("activation"):
                continue
            u = users.get(o.output, [])
            if len(u) == 1 and g.ops[u[0]].kind in ACTIVATIONS:
                out.append(FusionPatternMatch(self.name, [i, u[0]], FusionStrategy.MERGE, {"activation": g.ops[u[0]].kind}))
        return out


class ConvBatchNormPatternDetector(FusionPatternDetector):
    """conv2d -> batchnorm with constant statistics (inference): the normalisation folds into weights and bias."""
    name, priority = "conv_batchnorm", 3

    def detect(self, g):
        users, out = g.users(), []
        for i, o in enumerate(g.ops):
            if o.kind != "conv2d" or o.output in g.outputs:
                continue
            u = users.get(o.output, [])
            if len(u) != 1 or g.ops[u[0]].kind != "batchnorm":
                continue
            bn = g.ops[u[0]]
            consts = [g.values[n].const is not None for n in list(o.inputs[1:]) + list(bn.inputs[1:])]
            if all(consts) and not bn.attrs.get("training", False):
                out.append(FusionPatternMatch(self.name, [i, u[0]], FusionStrategy.FOLD, {"eps": bn.attrs.get("eps", 1e-5)}))
        return out


class LinearEpiloguePatternDetector(FusionPatternDetector):
    """linear / matmul followed by GELU or by a same-shape add: epilogues of the tensor-core GEMM."""
    name, priority = "gemm_epilogue", 4

    def detect(self, g):
        out = []
        for i, j, kind in FusionEngine().find_gemm_epilogues(g):
            mm, nxt = g.ops[i], g.ops[j]
            if mm.attrs.get("epilogue"):
                continue                      # one epilogue per product
            if kind == "residual":
                other = [n for n in nxt.inputs if n != mm.output]
                if len(other) != 1 or g.values[other[0]].shape != g.values[mm.output].shape:
                    continue                  # a broadcast operand is a bias, not a residual
            out.append(FusionPatternMatch(self.name, [i, j], FusionStrategy.REPLACE, {"epilogue": kind}))
        return out


def default_detectors() -> List[FusionPatternDetector]:
    return [LinearEpiloguePatternDetector(), ConvBatchNormPatternDetector(), ConvActivationPatternDetector(), ElementWisePatternDetector()]


# ------------------------------------------------------------------ constraints
class Severity(enum.Enum):
    INFO = 0
    WARNING = 1
    ERROR = 2


@dataclass
class ConstraintViolation:
    constraint: str
    message: str
    severity: Severity = Severity.ERROR


class FusionConstraint:
    name = "constraint"

    def violations(self, g: HLGraph, ops: Sequence[Op]) -> List[ConstraintViolation]:
        raise NotImplementedError

    def satisfies(self, g: HLGraph, ops: Sequence[Op]) -> bool:
        return not any(v.severity == Severity.ERROR for v in self.violations(g, ops))


class MemoryLayoutConstraint(FusionConstraint):
    """All operands of a merged kernel are walked with one index: layouts (``attrs['layout']``, default row-major
    contiguous) must agree."""
    name = "MemoryLayout"

    def violations(self, g, ops):
        layouts = {o.attrs.get("layout", "contiguous") for o in ops}
        if len(layouts) > 1:
            return [ConstraintViolation(self.name, f"mixed layouts {sorted(layouts)}")]
        return []


class NumericalPrecisionConstraint(FusionConstraint):
    """Merged element-wise math runs in fp32 registers, so mixing 16-bit types with fp32 is fine; fp64 or integer
    values inside a floating-point group are not."""
    name = "NumericalPrecision"

    def violations(self, g, ops):
        dts = {g.values[o.output].dtype for o in ops}
        out = []
        if torch.float64 in dts and len(dts) > 1:
            out.append(ConstraintViolation(self.name, "fp64 values inside a lower-precision group"))
        ints = {d for d in dts if not d.is_floating_point}
        if ints and len(dts) > len(ints):
            out.append(ConstraintViolation(self.name, f"integer and floating-point results mixed: {sorted(map(str, dts))}"))
        if len({d for d in dts if d in (torch.float16, torch.bfloat16)}) == 2:
            out.append(ConstraintViolation(self.name, "fp16 and bf16 results in one group", Severity.WARNING))
        return out


class SideEffectConstraint(FusionConstraint):
    name = "SideEffect"

    def violations(self, g, ops):
        bad = [o.kind for o in ops if o.kind in SIDE_EFFECT_OPS or o.attrs.get("side_effect")]
        return [ConstraintViolation(self.name, f"ops with side effects: {bad}")] if bad else []


class ControlFlowConstraint(FusionConstraint):
    name = "ControlFlow"

    def violations(self, g, ops):
        bad = [o.kind for o in ops if o.kind in CONTROL_FLOW_OPS]
        return [ConstraintViolation(self.name, f"control flow inside the group: {bad}")] if bad else []


class MemoryAccessPatternConstraint(FusionConstraint):
    name = "MemoryAccessPattern"

    def __init__(self):
        self._chk = OperationCompatibilityChecker()

    def violations(self, g, ops):
        an, out = self._chk.an, []
        pats = [an.access_pattern(o) for o in ops]
        for a, b in zip(pats, pats[1:]):
            if not self._chk.patterns_compatible(a, b):
                out.append(ConstraintViolation(self.name, f"incompatible access patterns: {a.value} then {b.value}"))
        if any(p in (MemoryAccessPattern.GATHER, MemoryAccessPattern.SCATTER) for p in pats):
            out.append(ConstraintViolation(self.name, "gather / scatter ops rarely fuse efficiently", Severity.WARNING))
        return out


@dataclass
class LaunchLimits:
    """One B200 SM."""
    max_threads_per_cta: int = 1024
    registers_per_sm: int = 65536
    max_registers_per_thread: int = 255
    shared_bytes_per_cta: int = 227 * 1024
    max_pointer_args: int = 16


class LaunchResourceConstraint(FusionConstraint):
    """Can ONE kernel hold the group? Registers per thread are estimated as 24 + vector width x (live inputs + 2) for a
    merged element-wise kernel; a spatial or contraction producer brings its own kernel, whose epilogue adds 8."""
    name = "LaunchResources"

    def __init__(self, limits: Optional[LaunchLimits] = None, threads: int = 256, vector: int = 8):
        self.lim, self.threads, self.vector = limits or LaunchLimits(), threads, vector

    def estimate_registers(self, g: HLGraph, ops: Sequence[Op]) -> int:
        an = GraphAnalyzer()
        idx = [g.ops.index(o) for o in ops if o in g.ops]
        n_in = len(an.external_inputs(g, idx)) if idx else sum(len(o.inputs) for o in ops)
        heavy = any(an.access_pattern(o) in (MemoryAccessPattern.SPATIAL, MemoryAccessPattern.CONTRACTION) for o in ops)
        return (96 if heavy else 24) + self.vector * (min(n_in, 4) + 2) + (8 if heavy else 0)

    def violations(self, g, ops):
        out = []
        if self.threads > self.lim.max_threads_per_cta:
            out.append(ConstraintViolation(self.name, f"{self.threads} threads exceed {self.lim.max_threads_per_cta} per CTA"))
        regs = self.estimate_registers(g, ops)
        if regs > self.lim.max_registers_per_thread:
            out.append(ConstraintViolation(self.name, f"about {regs} registers per thread exceed {self.lim.max_registers_per_thread}"))
        elif regs * self.threads > self.lim.registers_per_sm:
            out.append(ConstraintViolation(self.name, f"{regs} registers x {self.threads} threads exceed the register file"))
        idx = [g.ops.index(o) for o in ops if o in g.ops]
        n_ptr = len(GraphAnalyzer().external_inputs(g, idx)) + 1
        if n_ptr > self.lim.max_pointer_args:
            out.append(ConstraintViolation(self.name, f"{n_ptr} pointer arguments exceed {self.lim.max_pointer_args}"))
        smem = sum(int(o.attrs.get("shared_bytes", 0)) for o in ops)
        if smem > self.lim.shared_bytes_per_cta:
            out.append(ConstraintViolation(self.name, f"{smem} bytes of shared memory exceed {self.lim.shared_bytes_per_cta}"))
        return out


class FusionConstraintsValidator:
    def __init__(self, constraints: Optional[Sequence[FusionConstraint]] = None):
        self.constraints = list(constraints) if constraints is not None else [
            MemoryLayoutConstraint(), NumericalPrecisionConstraint(), SideEffectConstraint(), ControlFlowConstraint(),
            MemoryAccessPatternConstraint(), LaunchResourceConstraint()]

    def validate(self, g: HLGraph, match: FusionPatternMatch) -> List[ConstraintViolation]:
        ops = match.ops(g)
        return [v for c in self.constraints for v in c.violations(g, ops)]

    def accepts(self, g: HLGraph, match: FusionPatternMatch) -> bool:
        return not any(v.severity == Severity.ERROR for v in self.validate(g, match))


# ------------------------------------------------------------------ statistics and decision log
@dataclass
class FusionStatistics:
    total_ops_before: int = 0
    total_ops_after: int = 0
    fused_groups: int = 0
    fused_ops: int = 0
    rejected: int = 0
    by_pattern: Dict[str, int] = field(default_factory=dict)
    rejection_reasons: Dict[str, int] = field(default_factory=dict)

    @property
    def fusion_ratio(self) -> float:
        return self.fused_ops / self.total_ops_before if self.total_ops_before else 0.0


class FusionStatisticsCollector:
    def __init__(self):
        self.stats = FusionStatistics()

    def record_fusion(self, pattern: str, n_ops: int):
        s = self.stats
        s.fused_groups += 1
        s.fused_ops += n_ops
        s.by_pattern[pattern] = s.by_pattern.get(pattern, 0) + 1

    def record_rejection(self, pattern: str, reason: str):
        s = self.stats
        s.rejected += 1
        s.rejection_reasons[reason] = s.rejection_reasons.get(reason, 0) + 1

    def reset(self):
        self.stats = FusionStatistics()


@dataclass
class FusionDecisionRecord:
    pattern: str
    ops: List[str]
    accepted: bool
    reason: str
    timestamp: float = field(default_factory=time.time)


class FusionDecisionLogger:
    def __init__(self, capacity: int = 10_000):
        self.capacity, self.records = capacity, []

    def log(self, pattern: str, ops: Sequence[str], accepted: bool, reason: str = ""):
        if len(self.records) < self.capacity:
            self.records.append(FusionDecisionRecord(pattern, list(ops), accepted, reason))

    def accepted(self) -> List[FusionDecisionRecord]:
        return [r for r in self.records if r.accepted]

    def rejected(self) -> List[FusionDecisionRecord]:
        return [r for r in self.records if not r.accepted]

    def render(self) -> str:
        return "\n".join(f"[{'fuse' if r.accepted else 'skip'}] {r.pattern}: {' -> '.join(r.ops)}" + (f"  ({r.reason})" if r.reason else "")
                         for r in self.records)


# ------------------------------------------------------------------ transformer
def clone_graph(g: HLGraph) -> HLGraph:
    h = HLGraph(g.name)
    h.values = {k: Value(v.name, v.shape, v.dtype, v.const) for k, v in g.values.items()}
    h.ops = [Op(o.kind, list(o.inputs), o.output, dict(o.attrs)) for o in g.ops]
    h.inputs, h.outputs = list(g.inputs), list(g.outputs)
    h._next_id = g._next_id
    return h


class GraphTransformer:
    """Applies matches (highest detector priority first; a match touching an op that an earlier match took is dropped)
    to a COPY of the graph. The rewritten ops stay executable by the graph executor:

    * element-wise chain -> one ``fused_elementwise`` op (a run-time compiled kernel on the GPU);
    * conv2d + activation -> ``conv2d`` with ``activation`` attribute;
    * conv2d + batchnorm -> ``conv2d`` with folded constant weights and bias;
    * linear / matmul + GELU or residual add -> ``linear`` / ``matmul`` with ``epilogue`` attribute (and the residual as
      an extra input), which the executor maps to the GEMM's epilogue flags."""

    def __init__(self, detectors: Optional[Sequence[FusionPatternDetector]] = None, validator: Optional[FusionConstraintsValidator] = None,
                 stats: Optional[FusionStatisticsCollector] = None, logger: Optional[FusionDecisionLogger] = None):
        self.detectors = sorted(detectors if detectors is not None else default_detectors(), key=lambda d: -d.priority)
        self.validator = validator or FusionConstraintsValidator()
        self.stats = stats or FusionStatisticsCollector()
        self.logger = logger or FusionDecisionLogger()
        self._rejected: set = set()          # (pattern, value names) already logged as rejected

    def transform(self, g: HLGraph) -> HLGraph:
        h = clone_graph(g)
        self.stats.stats.total_ops_before += len(h.ops)
        for det in self.detectors:
            # one detector at a time: indices are valid until the graph is rewritten, so re-detect after every rewrite
            while True:
                applied = False
                for m in det.detect(h):
                    names = [h.ops[i].output for i in m.op_indices]
                    viol = self.validator.validate(h, m)
                    errs = [v for v in viol if v.severity == Severity.ERROR]
                    if errs:
                        key = (m.pattern, tuple(names))
                        if key not in self._rejected:
                            self._rejected.add(key)
                            self.stats.record_rejection(m.pattern, errs[0].constraint)
                            self.logger.log(m.pattern, names, False, errs[0].message)
                        continue
                    self._apply(h, m)
                    self.stats.record_fusion(m.pattern, len(m.op_indices))
                    self.logger.log(m.pattern, names, True)
                    applied = True
                    break
                if not applied:
                    break
        self.stats.stats.total_ops_after += len(h.ops)
        errs = h.verify()
        if errs:
            raise RuntimeError(f"graph invalid after fusion: {errs}")
        return h

    # ---- rewrites
    def _apply(self, g: HLGraph, m: FusionPatternMatch):
        if m.pattern == "elementwise_chain":
            self._merge_chain(g, m.op_indices)
        elif m.pattern == "conv_activation":
            i, j = m.op_indices
            conv, act = g.ops[i], g.ops[j]
            g.ops[j] = Op("conv2d", list(conv.inputs), act.output, {**conv.attrs, "activation": act.kind})
            del g.ops[i]
        elif m.pattern == "conv_batchnorm":
            self._fold_bn(g, m)
        elif m.pattern == "gemm_epilogue":
            i, j = m.op_indices
            mm, nxt = g.ops[i], g.ops[j]
            if m.detail["epilogue"] == "gelu":
                g.ops[j] = Op(mm.kind, list(mm.inputs), nxt.output, {**mm.attrs, "epilogue": "gelu"})
            else:
                other = [n for n in nxt.inputs if n != mm.output][0]
                g.ops[j] = Op(mm.kind, list(mm.inputs), nxt.output, {**mm.attrs, "epilogue": "residual", "residual": other})
                g.ops[j].inputs.append(other)
            del g.ops[i]
        else:
            raise KeyError(f"no rewrite for pattern {m.pattern!r}")

    @staticmethod
    def _merge_chain(g: HLGraph, chain: Sequence[int]):
        first, last = g.ops[chain[0]], g.ops[chain[-1]]
        spec, extra = [], []
        for n, k in enumerate(chain):
            o = g.ops[k]
            binary = len(o.inputs) == 2
            spec.append((o.kind, binary))
            if n == 0:
                extra.extend(o.inputs[1:])
            elif binary:
                extra.append(o.inputs[1])
        g.ops[chain[-1]] = Op("fused_elementwise", [first.inputs[0]] + extra, last.output, {"chain": spec})
        drop = set(chain[:-1])
        g.ops = [o for i, o in enumerate(g.ops) if i not in drop]

    @staticmethod
    def _fold_bn(g: HLGraph, m: FusionPatternMatch):
        i, j = m.op_indices
        conv, bn = g.ops[i], g.ops[j]
        w = g.values[conv.inputs[1]].const
        b = g.values[conv.inputs[2]].const if len(conv.inputs) > 2 else None
        gamma, beta, mean, var = (g.values[n].const for n in bn.inputs[1:5])
        w2, b2 = FusionEngine.fold_conv_batchnorm(w, b, gamma, beta, mean, var, m.detail.get("eps", 1e-5))
        wn, bname = g.constant(w2), g.constant(b2)
        g.ops[j] = Op("conv2d", [conv.inputs[0], wn, bname], bn.output, dict(conv.attrs))
        del g.ops[i]


# ------------------------------------------------------------------ verification and fall-back
@dataclass
class VerificationTestResult:
    trial: int
    max_abs_error: float
    max_rel_error: float
    passed: bool


@dataclass
class VerificationResult:
    passed: bool
    trials: List[VerificationTestResult]
    message: str = ""

    @property
    def worst_abs_error(self) -> float:
        return max((t.max_abs_error for t in self.trials), default=0.0)


class FusionVerifier:
    """Both graphs on the same random feeds; every output within ``atol + rtol * |reference|``."""

    def __init__(self, trials: int = 3, atol: float = 1e-4, rtol: float = 1e-4, seed: int = 0, device: str = "cpu"):
        self.trials, self.atol, self.rtol, self.seed, self.device = trials, atol, rtol, seed, device

    def _feeds(self, g: HLGraph, gen: torch.Generator) -> Dict[str, torch.Tensor]:
        f = {}
        for n in g.inputs:
            v = g.values[n]
            t = torch.randn(v.shape, generator=gen, dtype=torch.float32) if v.dtype.is_floating_point else \
                torch.randint(0, 8, v.shape, generator=gen)
            f[n] = t.to(v.dtype).to(self.device)
        return f

    def verify(self, original: HLGraph, fused: HLGraph) -> VerificationResult:
        if original.inputs != fused.inputs or len(original.outputs) != len(fused.outputs):
            return VerificationResult(False, [], "graphs differ in their interface")
        gen = torch.Generator().manual_seed(self.seed)
        res = []
        for t in range(self.trials):
            feeds = self._feeds(original, gen)
            try:
                a, b = original.run(dict(feeds)), fused.run(dict(feeds))
            except Exception as e:       # noqa: BLE001 - any failure of the fused graph is a verification failure
                return VerificationResult(False, res, f"execution failed: {e}")
            worst_abs = worst_rel = 0.0
            ok = True
            for x, y in zip(a, b):
                if x.shape != y.shape:
                    return VerificationResult(False, res, f"output shape {tuple(y.shape)} differs from {tuple(x.shape)}")
                x, y = x.double(), y.double()
                d = (x - y).abs()
                worst_abs = max(worst_abs, float(d.max()) if d.numel() else 0.0)
                worst_rel = max(worst_rel, float((d / x.abs().clamp_min(1e-12)).max()) if d.numel() else 0.0)
                ok &= bool((d <= self.atol + self.rtol * x.abs()).all())
            res.append(VerificationTestResult(t, worst_abs, worst_rel, ok))
        passed = all(r.passed for r in res)
        return VerificationResult(passed, res, "" if passed else "outputs differ beyond tolerance")


class FusionFallbackHandler:
    """``compile(graph)`` returns the graph to run: the fused one when the transformation succeeded and verified, the
    original otherwise. ``run`` additionally falls back at execution time (once a fused graph raised, it stays off)."""

    def __init__(self, transformer: Optional[GraphTransformer] = None, verifier: Optional[FusionVerifier] = None):
        self.transformer, self.verifier = transformer or GraphTransformer(), verifier
        self.fallbacks: List[str] = []
        self._disabled: set = set()

    def compile(self, g: HLGraph) -> HLGraph:
        try:
            fused = self.transformer.transform(g)
        except Exception as e:           # noqa: BLE001
            self.fallbacks.append(f"transform: {e}")
            return g
        if self.verifier is not None:
            r = self.verifier.verify(g, fused)
            if not r.passed:
                self.fallbacks.append(f"verify: {r.message}")
                return g
        return fused

    def run(self, original: HLGraph, fused: HLGraph, feeds: Dict[str, torch.Tensor]) -> List[torch.Tensor]:
        if id(fused) not in self._disabled:
            try:
                return fused.run(feeds)
            except Exception as e:       # noqa: BLE001
                self._disabled.add(id(fused))
                self.fallbacks.append(f"run: {e}")
        return original.run(feeds)


# ------------------------------------------------------------------ profiling
@dataclass
class KernelTiming:
    name: str
    samples_ms: List[float] = field(default_factory=list)

    @property
    def mean_ms(self) -> float:
        return sum(self.samples_ms) / len(self.samples_ms) if self.samples_ms else 0.0

    @property
    def min_ms(self) -> float:
        return min(self.samples_ms) if self.samples_ms else 0.0


class KernelTimingInstrument:
    """Times a callable: CUDA events on the current stream when ``device`` is a GPU, the host clock otherwise."""

    def __init__(self, device: Optional[torch.device] = None, warmup: int = 3, iters: int = 10):
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.warmup, self.iters = warmup, iters

    def time(self, name: str, fn: Callable[[], object]) -> KernelTiming:
        for _ in range(self.warmup):
            fn()
        t = KernelTiming(name)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            for _ in range(self.iters):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                b.synchronize()
                t.samples_ms.append(a.elapsed_time(b))
        else:
            for _ in range(self.iters):
                t0 = time.perf_counter()
                fn()
                t.samples_ms.append((time.perf_counter() - t0) * 1e3)
        return t


@dataclass
class FusionProfilingReport:
    original: KernelTiming
    fused: KernelTiming
    ops_before: int
    ops_after: int

    @property
    def speedup(self) -> float:
        return self.original.min_ms / self.fused.min_ms if self.fused.min_ms > 0 else 0.0

    def render(self) -> str:
        return (f"fusion: {self.ops_before} ops -> {self.ops_after} ops; "
                f"{self.original.min_ms:.3f} ms -> {self.fused.min_ms:.3f} ms ({self.speedup:.2f}x)")


class FusionProfiler:
    def __init__(self, instrument: Optional[KernelTimingInstrument] = None):
        self.instrument = instrument or KernelTimingInstrument()
        self.reports: List[FusionProfilingReport] = []

    def compare(self, original: HLGraph, fused: HLGraph, feeds: Dict[str, torch.Tensor]) -> FusionProfilingReport:
        a = self.instrument.time("original", lambda: original.run(dict(feeds)))
        b = self.instrument.time("fused", lambda: fused.run(dict(feeds)))
        r = FusionProfilingReport(a, b, len(original.ops), len(fused.ops))
        self.reports.append(r)
        return r


# ------------------------------------------------------------------ run-time (dynamic-shape) fusion
@dataclass
class FusionBenefit:
    estimated_speedup: float
    memory_saved: int
    kernel_count_reduction: int
    complexity_score: float

    def should_fuse(self, threshold: float = 1.1) -> bool:
        return self.estimated_speedup >= threshold and self.kernel_count_reduction > 0

    @staticmethod
    def none() -> "FusionBenefit":
        return FusionBenefit(1.0, 0, 0, float("inf"))


@dataclass
class DeviceModel:
    """What a kernel costs here: a fixed launch and ramp cost plus its traffic at the copy bandwidth."""
    hbm_bytes_per_s: float = 6.6e12
    launch_s: float = 4e-6

    def kernel_s(self, nbytes: int) -> float:
        return self.launch_s + nbytes / self.hbm_bytes_per_s


class FusionCandidateAnalyzer:
    """Benefit of merging a group: every op alone reads its inputs and writes its output; merged, only the group's
    external inputs are read and the last value is written."""

    def __init__(self, device: Optional[DeviceModel] = None):
        self.dev, self.an = device or DeviceModel(), GraphAnalyzer()

    def _bytes(self, g: HLGraph, name: str) -> int:
        v = g.values[name]
        return _numel(v.shape) * _itemsize(v.dtype)

    def analyze(self, g: HLGraph, op_indices: Sequence[int]) -> FusionBenefit:
        if len(op_indices) < 2:
            return FusionBenefit.none()
        separate = sum(self.dev.kernel_s(sum(self._bytes(g, n) for n in g.ops[i].inputs) + self._bytes(g, g.ops[i].output)) for i in op_indices)
        ext = self.an.external_inputs(g, op_indices)
        merged = self.dev.kernel_s(sum(self._bytes(g, n) for n in ext) + self._bytes(g, g.ops[op_indices[-1]].output))
        return FusionBenefit(separate / merged, self.an.intermediate_bytes(g, op_indices), len(op_indices) - 1,
                             float(len(op_indices) + len(ext)))


class RuntimeShapeInjector:
    """A graph builder with symbolic sizes, specialised per call. ``build(shapes) -> HLGraph`` is called once per
    distinct shape signature; the fused graph of a signature is cached (least recently used beyond ``capacity``)."""

    def __init__(self, build: Callable[[Dict[str, Tuple[int, ...]]], HLGraph], handler: Optional[FusionFallbackHandler] = None, capacity: int = 32):
        self.build, self.handler, self.capacity = build, handler or FusionFallbackHandler(), capacity
        self._cache: Dict[tuple, Tuple[HLGraph, HLGraph]] = {}
        self.hits = self.misses = 0

    @staticmethod
    def signature(feeds: Dict[str, torch.Tensor]) -> tuple:
        return tuple(sorted((k, tuple(v.shape), str(v.dtype)) for k, v in feeds.items()))

    def specialize(self, feeds: Dict[str, torch.Tensor]) -> Tuple[HLGraph, HLGraph]:
        sig = self.signature(feeds)
        hit = self._cache.pop(sig, None)
        if hit is None:
            self.misses += 1
            g = self.build({k: tuple(v.shape) for k, v in feeds.items()})
            hit = (g, self.handler.compile(g))
            if len(self._cache) >= self.capacity:
                self._cache.pop(next(iter(self._cache)))
        else:
            self.hits += 1
        self._cache[sig] = hit
        return hit

    def __call__(self, **feeds: torch.Tensor) -> List[torch.Tensor]:
        g, fused = self.specialize(feeds)
        return self.handler.run(g, fused, feeds)


class CudaTypeMapper:
    _MAP = {torch.float32: "float", torch.float16: "__half", torch.bfloat16: "__nv_bfloat16", torch.float64: "double",
            torch.int32: "int", torch.int64: "long long", torch.int8: "signed char", torch.uint8: "unsigned char", torch.bool: "bool"}

    @classmethod
    def cuda_type(cls, dt: torch.dtype) -> str:
        if dt not in cls._MAP:
            raise KeyError(f"no CUDA type for {dt}")
        return cls._MAP[dt]

    @classmethod
    def vector_elems(cls, dt: torch.dtype, access_bytes: int = 16) -> int:
        return max(1, access_bytes // _itemsize(dt))


class FusionKernelGenerator:
    """CUDA source (and, on demand, the compiled kernel) of a ``fused_elementwise`` op."""

    def source(self, op: Op, dtype: torch.dtype = torch.bfloat16, name: str = "fused_chain") -> str:
        if op.kind != "fused_elementwise":
            raise ValueError("not a fused element-wise op")
        from .jit_cuda import CudaChainSource, KernelConfig
        return CudaChainSource().render(name, [k for k, _ in op.attrs["chain"]], dtype, KernelConfig())

    def compile(self, op: Op, **kw):
        from .jit_cuda import compile_chain
        return compile_chain([k for k, _ in op.attrs["chain"]], **kw)


# ------------------------------------------------------------------ code generator planning helpers
@dataclass
class TilingConfiguration:
    tile_m: int = 128
    tile_n: int = 128
    tile_k: int = 64
    stages: int = 4
    elem_bytes: int = 2

    def shared_bytes(self) -> int:
        return self.stages * (self.tile_m + self.tile_n) * self.tile_k * self.elem_bytes

    def fits(self, limit: int = 227 * 1024) -> bool:
        return self.shared_bytes() <= limit

    @staticmethod
    def for_gemm(m: int, n: int, k: int, elem_bytes: int = 2, limit: int = 227 * 1024) -> "TilingConfiguration":
        """128-row tiles (one tensor-core instruction's M); the widest N tile that divides the work into at least one
        wave of 148 SMs, else 64; as many 64-deep stages as fit, at most 8."""
        tn = 64
        for cand in (256, 128):
            if -(-m // 128) * -(-n // cand) >= 148:
                tn = cand
                break
        t = TilingConfiguration(128, tn, 64, 8, elem_bytes)
        while t.stages > 2 and not t.fits(limit):
            t.stages -= 1
        return t


@dataclass
class SharedBuffer:
    name: str
    rows: int
    row_bytes: int
    offset: int = 0
    padded_row_bytes: int = 0

    @property
    def size(self) -> int:
        return self.rows * self.padded_row_bytes


class SharedMemoryPlanner:
    """Lays out the shared buffers of a generated kernel: rows whose pitch is a multiple of 128 bytes (all 32 banks)
    get 16 bytes of padding so that column walks do not hit one bank; buffers start 128-byte aligned (1024 for
    buffers a TMA copy with 128-byte swizzle fills)."""

    def __init__(self, limit: int = 227 * 1024):
        self.limit = limit

    def plan(self, buffers: Sequence[Tuple[str, int, int]], swizzled: Sequence[str] = ()) -> List[SharedBuffer]:
        out, off = [], 0
        for name, rows, row_bytes in buffers:
            sw = name in swizzled
            pitch = row_bytes if sw or row_bytes % 128 else row_bytes + 16
            align = 1024 if sw else 128
            off = (off + align - 1) // align * align
            b = SharedBuffer(name, rows, row_bytes, off, pitch)
            off += b.size
            out.append(b)
        if off > self.limit:
            raise ValueError(f"shared-memory plan needs {off} bytes, limit {self.limit}")
        return out

    @staticmethod
    def total(plan: Sequence[SharedBuffer]) -> int:
        return max((b.offset + b.size for b in plan), default=0)


class MemoryAccessOptimizer:
    """Widest vector access every operand allows: 16 bytes when all base offsets and the row length are 16-byte
    multiples, else 8, 4, or scalar."""

    def vector_bytes(self, elem_bytes: int, row_elems: int, base_offsets_bytes: Sequence[int] = (0,)) -> int:
        for vb in (16, 8, 4):
            if vb < elem_bytes:
                break
            if (row_elems * elem_bytes) % vb == 0 and all(o % vb == 0 for o in base_offsets_bytes):
                return vb
        return elem_bytes

    def vector_elems(self, elem_bytes: int, row_elems: int, base_offsets_bytes: Sequence[int] = (0,)) -> int:
        return self.vector_bytes(elem_bytes, row_elems, base_offsets_bytes) // elem_bytes


class LoopUnrollingOptimizer:
    """Vectors in flight per thread: enough loads outstanding to cover memory latency (about 8 x 16 bytes per thread at
    256 threads x 2 CTAs per SM) without pushing the kernel over the register budget."""

    def unroll_factor(self, n_inputs: int, vector_elems: int, register_budget: int = 128, base_registers: int = 24) -> int:
        per_iter = vector_elems * (n_inputs + 1)
        best = 1
        for u in (2, 4, 8):
            if base_registers + u * per_iter <= register_budget and u * n_inputs <= 8:
                best = u
        return best
