"""CUDA graphs: capture after warm-up, validate, replay, fall back to eager.

Covers the reference's graph manager (src/MLFramework/HAL/CUDA/Graphs/CUDAGraphManager.cs:40-109:
3 warm-up iterations, 512 MB pool, GetOrCaptureGraph, ExecuteGraphOrFallback), capture object
(CUDAGraphCapture.cs:30-57), validation rules (Validation/Rules/*: control flow, dynamic memory,
empty graph, I/O, synchronisation), fallback handler (Fallback/CUDAGraphFallbackHandler.cs:56),
weight updater (ICUDAGraphWeightUpdater.cs) and the capture-safe fixed-address pool
(HAL/CUDA/Memory/CUDAGraphMemoryPool.cs:24-98, 256-byte alignment).

Launch-bound loops here (one decode iteration is ~300 launches of a few microseconds each) are the
target: a captured decode step replays as one graph launch. Inputs live in static buffers from the
pool; ``replay`` copies new inputs in, launches and returns the static outputs.
"""
from __future__ import annotations

import contextlib
import enum
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch


class GraphMemoryPool:
    """Bump allocator over one device slab; addresses stay fixed for the life of the pool so that a
    captured graph's pointers stay valid. ``reset`` rewinds; blocks may be returned in LIFO order."""

    ALIGN = 256

    def __init__(self, capacity_bytes: int = 512 << 20, device: Optional[torch.device] = None):
        self.capacity = capacity_bytes
        self.device = device if device is not None else (torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu"))
        self._slab: Optional[torch.Tensor] = None
        self._off = 0
        self.peak = 0
        self._blocks: List[Tuple[int, int]] = []

    def _ensure(self):
        if self._slab is None:
            self._slab = torch.empty(self.capacity, dtype=torch.uint8, device=self.device)

    def allocate(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        self._ensure()
        esz = torch.empty((), dtype=dtype).element_size()
        n = 1
        for s in shape:
            n *= s
        nbytes = (n * esz + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        if self._off + nbytes > self.capacity:
            raise MemoryError(f"graph memory pool exhausted: {self._off + nbytes} > {self.capacity} bytes")
        t = self._slab[self._off:self._off + n * esz].view(dtype).view(*shape)
        self._blocks.append((self._off, nbytes))
        self._off += nbytes
        self.peak = max(self.peak, self._off)
        return t

    def return_block(self, t: torch.Tensor) -> bool:
        if not self._blocks:
            return False
        off, nbytes = self._blocks[-1]
        if self._slab.data_ptr() + off == t.data_ptr():
            self._blocks.pop()
            self._off = off
            return True
        return False

    def reset(self):
        self._off = 0
        self._blocks.clear()

    def stats(self) -> Dict[str, int]:
        return {"capacity": self.capacity, "used": self._off, "peak": self.peak, "blocks": len(self._blocks)}


class ValidationSeverity(enum.Enum):
    WARNING = 1
    ERROR = 2


@dataclass
class ValidationIssue:
    rule: str
    message: str
    severity: ValidationSeverity = ValidationSeverity.ERROR


@dataclass
class CapturedOp:
    """What a capture recorded about one operation, for validation."""
    name: str
    kind: str = "kernel"      # kernel | memcpy | memset | host | alloc | free | sync | io | branch


# node kinds of a real capture (ml_framework_b200.hal.cuda_rt.NODE_KINDS) -> the kinds the rules speak about
_NODE_TO_OP = {"kernel": "kernel", "memcpy": "memcpy", "memset": "memset", "host": "host", "graph": "kernel", "empty": "empty",
               "wait_event": "event", "event_record": "event", "ext_semaphore_signal": "sync", "ext_semaphore_wait": "sync",
               "mem_alloc": "alloc", "mem_free": "free", "batch_mem_op": "memset", "conditional": "branch"}


class ValidationRule:
    """One check over the operations of a capture (Graphs/Validation/IValidationRule.cs)."""

    rule_name = "rule"
    description = ""

    def validate(self, ops: Sequence[CapturedOp]) -> List[ValidationIssue]:
        raise NotImplementedError

    def _each(self, ops, kinds, message: str, severity=ValidationSeverity.ERROR) -> List[ValidationIssue]:
        return [ValidationIssue(self.rule_name, f"{op.name}: {message}", severity) for op in ops if op.kind in kinds]


class EmptyGraphRule(ValidationRule):
    rule_name, description = "EmptyGraph", "a capture must record at least one operation"

    def validate(self, ops):
        return [] if ops else [ValidationIssue(self.rule_name, "capture recorded no operations")]


class DynamicMemoryRule(ValidationRule):
    rule_name, description = "DynamicMemory", "device memory may not be allocated or freed inside a capture"

    def validate(self, ops):
        return self._each(ops, ("alloc", "free"), "device memory management inside a capture")


class ControlFlowRule(ValidationRule):
    rule_name, description = "ControlFlow", "host control flow on device data cannot be replayed"

    def validate(self, ops):
        return self._each(ops, ("branch",), "data-dependent host control flow cannot be replayed")


class IOOperationRule(ValidationRule):
    rule_name, description = "IOOperation", "host input / output does not belong in a capture"

    def validate(self, ops):
        return self._each(ops, ("io",), "host I/O inside a capture")


class SynchronizationRule(ValidationRule):
    rule_name, description = "Synchronization", "device or stream synchronisation ends a capture"

    def validate(self, ops):
        return self._each(ops, ("sync",), "device / stream synchronisation inside a capture")


class HostCallbackRule(ValidationRule):
    rule_name, description = "HostCallback", "host callbacks serialise the replay on the CPU"

    def validate(self, ops):
        return self._each(ops, ("host",), "host callback", ValidationSeverity.WARNING)


class CrossStreamEventRule(ValidationRule):
    rule_name, description = "CrossStreamEvent", "event nodes show that a side stream joined the capture"

    def validate(self, ops):
        return self._each(ops, ("event",), "event node (a side stream joined the capture)", ValidationSeverity.WARNING)


def default_validation_rules() -> List[ValidationRule]:
    return [EmptyGraphRule(), DynamicMemoryRule(), ControlFlowRule(), IOOperationRule(), SynchronizationRule(),
            HostCallbackRule(), CrossStreamEventRule()]


@dataclass
class CUDAGraphValidationResult:
    is_valid: bool
    errors: List[str]
    warnings: List[str]
    operation_count: int = 0

    @classmethod
    def success(cls, operation_count: int):
        return cls(True, [], [], operation_count)

    @classmethod
    def failure(cls, errors: Sequence[str], operation_count: int = 0):
        return cls(False, list(errors), [], operation_count)


class CUDAGraphValidationContext:
    """Collects what a capture does while it is being described: operation names with their kinds and the
    addresses it allocates (Graphs/Validation/CUDAGraphValidationContext.cs); ``ops()`` feeds a validator."""

    def __init__(self):
        self._ops: List[CapturedOp] = []
        self._memory: set = set()
        self._counts: Dict[str, int] = {}

    def record_operation(self, name: str, kind: str = "kernel") -> None:
        if not name:
            return
        self._ops.append(CapturedOp(name, kind))
        self._counts[name] = self._counts.get(name, 0) + 1

    def record_memory_allocation(self, ptr: int) -> None:
        if ptr:
            self._memory.add(int(ptr))
            self._ops.append(CapturedOp(f"alloc@{int(ptr):#x}", "alloc"))

    @property
    def captured_operations(self) -> List[str]:
        return [o.name for o in self._ops if o.kind != "alloc" or not o.name.startswith("alloc@")]

    @property
    def allocated_memory(self) -> frozenset:
        return frozenset(self._memory)

    @property
    def operation_counts(self) -> Dict[str, int]:
        return dict(self._counts)

    def get_operation_count(self, name: str) -> int:
        return self._counts.get(name, 0)

    def has_operation(self, name: str) -> bool:
        return name in self._counts

    def ops(self) -> List[CapturedOp]:
        return list(self._ops)

    def clear(self) -> None:
        self._ops.clear(); self._memory.clear(); self._counts.clear()


class GraphPhase(enum.Enum):
    """Which part of a training step a capture covers (Graphs/GraphPhase.cs)."""
    FORWARD = "forward"
    BACKWARD = "backward"
    OPTIMIZER_STEP = "optimizer_step"
    FORWARD_BACKWARD = "forward_backward"
    FULL_TRAINING_STEP = "full_training_step"


class CUDAGraphState(enum.Enum):
    CREATED = "created"
    CAPTURING = "capturing"
    READY = "ready"
    EXECUTING = "executing"
    INVALIDATED = "invalidated"
    DISPOSED = "disposed"


class CUDAGraphFallbackStrategy(enum.Enum):
    NEVER_CAPTURE = "never_capture"                    # always the eager path
    CAPTURE_OR_FALLBACK = "capture_or_fallback"        # try the graph every call; on failure run eagerly
    CAPTURE_ONLY = "capture_only"                      # failures propagate
    TRY_ONCE_THEN_FALLBACK = "try_once_then_fallback"  # one failure switches to eager for good
    RETRY_THEN_FALLBACK = "retry_then_fallback"        # ``max_failures`` consecutive failures switch to eager


class CUDAGraphCaptureException(RuntimeError):
    def __init__(self, message: str, graph_name: str = "", cause: Optional[BaseException] = None):
        super().__init__(f"{graph_name}: {message}" if graph_name else message)
        self.graph_name, self.cause = graph_name, cause


class GraphValidator:
    """Rules over the operations of a capture: a graph must not be empty, allocate or free device memory,
    depend on host-side control flow, perform host I/O, or synchronise the device.

    ``validate_graph`` reads the node list of a REAL captured ``cudaGraph_t`` through the native runtime binding
    (``cudaGraphGetNodes`` + ``cudaGraphNodeGetType``, the reference's CudaGraphGetNodes,
    src/MLFramework/HAL/CUDA/CudaApi.cs:184, feeding src/MLFramework/HAL/CUDA/Graphs/Validation/CUDAGraphValidator.cs)
    and applies the same rules to what was actually recorded; ``validate`` takes a declared list, for callers that
    describe a capture before making it."""

    def ops_of_graph(self, graph) -> List["CapturedOp"]:
        """``graph``: a :class:`ml_framework_b200.hal.cuda_rt.Graph` or a raw ``cudaGraph_t`` address."""
        from . import cuda_rt
        g = graph if isinstance(graph, cuda_rt.Graph) else cuda_rt.Graph(int(graph), owned=False)
        return [CapturedOp(f"node{i}:{k}", _NODE_TO_OP.get(k, "kernel")) for i, k in enumerate(g.node_kinds())]

    def validate_graph(self, graph) -> List[ValidationIssue]:
        ops = self.ops_of_graph(graph)
        issues = self.validate([o for o in ops if o.kind != "empty"])
        if not any(o.kind in ("kernel", "memcpy", "memset") for o in ops) and not any(i.rule == "EmptyGraph" for i in issues):
            issues.append(ValidationIssue("EmptyGraph", "capture holds no kernel, copy or memset node"))
        return issues

    def __init__(self, rules: Optional[Sequence["ValidationRule"]] = None):
        self.rules: List[ValidationRule] = list(rules) if rules is not None else default_validation_rules()

    def add_rule(self, rule: "ValidationRule") -> None:
        if any(r.rule_name == rule.rule_name for r in self.rules):
            raise ValueError(f"a rule named {rule.rule_name!r} is already installed")
        self.rules.append(rule)

    def remove_rule(self, rule_name: str) -> bool:
        n = len(self.rules)
        self.rules = [r for r in self.rules if r.rule_name != rule_name]
        return len(self.rules) < n

    def validate(self, ops: Sequence[CapturedOp]) -> List[ValidationIssue]:
        issues: List[ValidationIssue] = []
        for rule in self.rules:
            issues += rule.validate(ops)
        return issues

    def validation_result(self, ops: Sequence[CapturedOp]) -> "CUDAGraphValidationResult":
        """Errors and warnings as text, with the operation count (CUDAGraphValidationResult.cs)."""
        issues = self.validate(ops)
        errors = [f"[{i.rule}] {i.message}" for i in issues if i.severity == ValidationSeverity.ERROR]
        warnings = [f"[{i.rule}] {i.message}" for i in issues if i.severity == ValidationSeverity.WARNING]
        return CUDAGraphValidationResult(not errors, errors, warnings, len(ops))

    def is_valid(self, ops: Sequence[CapturedOp]) -> bool:
        return not any(i.severity == ValidationSeverity.ERROR for i in self.validate(ops))


@dataclass
class CaptureOptions:
    warmup_iterations: int = 3
    pool_bytes: int = 512 << 20
    enable_fallback: bool = True
    max_capture_failures: int = 3
    validate: bool = True             # inspect the captured graph's nodes; errors make the capture fail (-> fallback)


class GraphValidationError(RuntimeError):
    def __init__(self, issues: List[ValidationIssue]):
        super().__init__("; ".join(f"{i.rule}: {i.message}" for i in issues))
        self.issues = issues


class CapturedGraph:
    def __init__(self, graph, static_inputs: List[torch.Tensor], static_outputs, name: str,
                 node_kinds: Optional[List[str]] = None, issues: Optional[List[ValidationIssue]] = None):
        self.graph, self.static_inputs, self.static_outputs, self.name = graph, static_inputs, static_outputs, name
        self.replays = 0
        self.node_kinds = node_kinds or []        # node types of the captured cudaGraph_t
        self.issues = issues or []                # validator findings (warnings; errors abort the capture)

    def replay(self, *inputs: torch.Tensor):
        for dst, src in zip(self.static_inputs, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        return self.static_outputs

    def update_weights(self, pairs: Sequence[Tuple[torch.Tensor, torch.Tensor]]):
        """In-place weight refresh: the graph holds addresses, so new values are copied into the old
        storage (the reference's weight-updater contract)."""
        with torch.no_grad():
            for old, new in pairs:
                old.copy_(new)


class CUDAGraphManager:
    """``run(name, fn, *inputs)``: eager for the first ``warmup_iterations`` calls, then captured once
    per (name, input signature) and replayed; capture failures fall back to eager permanently after
    ``max_capture_failures``."""

    def __init__(self, options: Optional[CaptureOptions] = None):
        self.opt = options or CaptureOptions()
        self._graphs: Dict[Tuple, CapturedGraph] = {}
        self._calls: Dict[Tuple, int] = {}
        self._failures: Dict[str, int] = {}
        self._pool_handle = None
        self.fallbacks = 0
        self.validator = GraphValidator()

    @staticmethod
    def _sig(name: str, inputs: Sequence[torch.Tensor]) -> Tuple:
        return (name,) + tuple((tuple(t.shape), t.dtype, t.device.index) for t in inputs)

    def capture(self, name: str, fn: Callable, inputs: Sequence[torch.Tensor]) -> CapturedGraph:
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA graphs need a CUDA device")
        static_in = [t.clone() for t in inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn(*static_in)                                   # settle lazy initialisation off the main stream
        torch.cuda.current_stream().wait_stream(side)
        inspect = self.opt.validate and hasattr(torch.cuda.CUDAGraph, "raw_cuda_graph")
        g = torch.cuda.CUDAGraph(keep_graph=True) if inspect else torch.cuda.CUDAGraph()
        if self._pool_handle is None:
            self._pool_handle = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(g, pool=self._pool_handle):
            out = fn(*static_in)
        kinds, issues = [], []
        if inspect:
            # the cudaGraph_t is kept until instantiation: read its nodes back and check what was recorded
            from . import cuda_rt
            raw = cuda_rt.Graph(int(g.raw_cuda_graph()), owned=False)
            kinds = raw.node_kinds()
            issues = self.validator.validate_graph(raw)
            errors = [i for i in issues if i.severity == ValidationSeverity.ERROR]
            if errors:
                raise GraphValidationError(errors)
            g.instantiate()
        cg = CapturedGraph(g, static_in, out, name, kinds, issues)
        self._graphs[self._sig(name, inputs)] = cg
        return cg

    def run(self, name: str, fn: Callable, *inputs: torch.Tensor):
        key = self._sig(name, inputs)
        cg = self._graphs.get(key)
        if cg is not None:
            return cg.replay(*inputs)
        n = self._calls.get(key, 0)
        self._calls[key] = n + 1
        can_capture = torch.cuda.is_available() and all(t.is_cuda for t in inputs) \
            and self._failures.get(name, 0) < self.opt.max_capture_failures
        if n < self.opt.warmup_iterations or not can_capture:
            if n >= self.opt.warmup_iterations:
                self.fallbacks += 1
            return fn(*inputs)
        try:
            cg = self.capture(name, fn, inputs)
            return cg.replay(*inputs)
        except Exception:
            self._failures[name] = self._failures.get(name, 0) + 1
            if not self.opt.enable_fallback:
                raise
            self.fallbacks += 1
            return fn(*inputs)

    def stats(self) -> Dict[str, int]:
        return {"graphs": len(self._graphs), "fallbacks": self.fallbacks,
                "replays": sum(g.replays for g in self._graphs.values())}

    def clear(self):
        self._graphs.clear()
        self._calls.clear()


def capture_graph(manager: CUDAGraphManager, name: Optional[str] = None):
    """Decorator form (the reference's ``[CaptureGraph]`` attribute and proxy)."""
    def deco(fn):
        def wrapped(*inputs):
            return manager.run(name or fn.__name__, fn, *inputs)
        wrapped.__wrapped__ = fn
        return wrapped
    return deco


# ------------------------------------------------------------------ fall-back handler, proxy, allocator, static facade
class CUDAGraphFallbackHandler:
    """``execute_with_fallback(graph_fn, eager_fn)``: try the graph path; on an exception run the eager path, count the
    failure by exception type, and stop trying the graph path after ``max_failures`` consecutive failures
    (src/MLFramework/HAL/CUDA/Graphs/Fallback/CUDAGraphFallbackHandler.cs:56)."""

    def __init__(self, max_failures: int = 3, on_fallback: Optional[Callable[[BaseException], None]] = None,
                 strategy: CUDAGraphFallbackStrategy = CUDAGraphFallbackStrategy.RETRY_THEN_FALLBACK):
        self.strategy = strategy
        if strategy is CUDAGraphFallbackStrategy.TRY_ONCE_THEN_FALLBACK:
            max_failures = 1
        self.max_failures, self.on_fallback = max_failures, on_fallback
        self.consecutive_failures = 0
        self.total_fallbacks = 0
        self.successes = 0
        self.by_type: Dict[str, int] = {}
        self.last_error: Optional[BaseException] = None

    @property
    def graph_path_enabled(self) -> bool:
        S = CUDAGraphFallbackStrategy
        if self.strategy is S.NEVER_CAPTURE:
            return False
        if self.strategy in (S.CAPTURE_OR_FALLBACK, S.CAPTURE_ONLY):
            return True
        return self.consecutive_failures < self.max_failures

    def execute_with_fallback(self, graph_fn: Callable, eager_fn: Callable):
        if self.graph_path_enabled:
            try:
                out = graph_fn()
                self.successes += 1
                if self.strategy is not CUDAGraphFallbackStrategy.TRY_ONCE_THEN_FALLBACK:
                    self.consecutive_failures = 0
                return out
            except Exception as e:       # noqa: BLE001 - any capture / replay failure goes to the eager path
                if self.strategy is CUDAGraphFallbackStrategy.CAPTURE_ONLY:
                    raise CUDAGraphCaptureException(str(e), cause=e) from e
                self.consecutive_failures += 1
                self.by_type[type(e).__name__] = self.by_type.get(type(e).__name__, 0) + 1
                self.last_error = e
                if self.on_fallback is not None:
                    self.on_fallback(e)
        self.total_fallbacks += 1
        return eager_fn()

    def reset(self):
        self.consecutive_failures = 0
        self.last_error = None

    def stats(self) -> Dict[str, object]:
        return {"successes": self.successes, "fallbacks": self.total_fallbacks, "consecutive_failures": self.consecutive_failures,
                "graph_path_enabled": self.graph_path_enabled, "by_type": dict(self.by_type)}


class CUDAGraphProxy:
    """A callable (function or module) behind a graph manager: calls go through capture-and-replay per input signature,
    with the eager callable as the fall-back (Graphs/Proxies/CUDAGraphProxy.cs). ``invalidate()`` drops the captures
    (after a shape-changing edit of the module); ``update_weights`` refreshes parameters in place so captures stay
    valid (ICUDAGraphWeightUpdater.cs)."""

    def __init__(self, fn: Callable, manager: Optional["CUDAGraphManager"] = None, name: Optional[str] = None, enabled: bool = True):
        self.fn, self.manager = fn, manager or CUDAGraphManager()
        self.name = name or getattr(fn, "__name__", type(fn).__name__)
        self.enabled = enabled
        self.calls = 0

    def __call__(self, *inputs: torch.Tensor):
        self.calls += 1
        if not self.enabled:
            return self.fn(*inputs)
        return self.manager.run(self.name, self.fn, *inputs)

    @property
    def captured_signatures(self) -> int:
        return sum(1 for k in self.manager._graphs if k[0] == self.name)

    @property
    def is_captured(self) -> bool:
        return self.captured_signatures > 0

    def invalidate(self):
        for k in [k for k in self.manager._graphs if k[0] == self.name]:
            del self.manager._graphs[k]
        for k in [k for k in self.manager._calls if k[0] == self.name]:
            del self.manager._calls[k]

    def update_weights(self, new_state: Dict[str, torch.Tensor]) -> int:
        """Copies ``new_state`` into the wrapped module's parameters / buffers in place; returns how many were written."""
        if not isinstance(self.fn, torch.nn.Module):
            raise TypeError("update_weights needs a module")
        own, n = self.fn.state_dict(), 0
        with torch.no_grad():
            for k, v in new_state.items():
                if k in own:
                    if own[k].shape != v.shape:
                        raise ValueError(f"{k}: shape {tuple(v.shape)} does not match {tuple(own[k].shape)}; invalidate() and recapture instead")
                    own[k].copy_(v)
                    n += 1
        return n


@dataclass
class MemoryUsageStats:
    pool_capacity: int = 0
    pool_used: int = 0
    pool_peak: int = 0
    pool_blocks: int = 0
    pool_allocations: int = 0
    fallback_allocations: int = 0
    fallback_bytes: int = 0

    @property
    def pool_utilization(self) -> float:
        return self.pool_used / self.pool_capacity if self.pool_capacity else 0.0


class GraphCompatibleMemoryAllocator:
    """Allocation front for code that may run under capture: inside ``capture_scope()`` tensors come from the
    fixed-address pool (their addresses are what the graph records); outside they come from the caching allocator
    (Memory/GraphCompatibleMemoryAllocator.cs). A pool that is full raises inside a capture (a silent fall-back
    allocation there would be freed and reused under the graph's feet)."""

    def __init__(self, pool: Optional[GraphMemoryPool] = None):
        self.pool = pool or GraphMemoryPool()
        self._in_capture = 0
        self._s = MemoryUsageStats()

    @contextlib.contextmanager
    def capture_scope(self):
        self._in_capture += 1
        try:
            yield self
        finally:
            self._in_capture -= 1

    @property
    def in_capture(self) -> bool:
        return self._in_capture > 0

    def allocate(self, shape: Sequence[int], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        if self.in_capture:
            t = self.pool.allocate(shape, dtype)
            self._s.pool_allocations += 1
            return t
        t = torch.empty(tuple(shape), dtype=dtype, device=self.pool.device)
        self._s.fallback_allocations += 1
        self._s.fallback_bytes += t.numel() * t.element_size()
        return t

    def free(self, t: torch.Tensor) -> bool:
        """Returns a pool block when it is the most recent one; other tensors are left to the caching allocator."""
        return self.pool.return_block(t) if self.pool._slab is not None else False

    def reset_pool(self):
        if self.in_capture:
            raise RuntimeError("the pool cannot be rewound during a capture")
        self.pool.reset()

    def stats(self) -> MemoryUsageStats:
        p = self.pool.stats()
        s = MemoryUsageStats(**{**self._s.__dict__})
        s.pool_capacity, s.pool_used, s.pool_peak, s.pool_blocks = p["capacity"], p["used"], p["peak"], p["blocks"]
        return s


class CUDAGraphStatic:
    """Process-wide default manager for code that does not carry one around (Graphs/CUDAGraphStatic.cs)."""
    _manager: Optional[CUDAGraphManager] = None
    enabled = True

    @classmethod
    def manager(cls) -> CUDAGraphManager:
        if cls._manager is None:
            cls._manager = CUDAGraphManager()
        return cls._manager

    @classmethod
    def configure(cls, options: CaptureOptions):
        cls._manager = CUDAGraphManager(options)

    @classmethod
    def run(cls, name: str, fn: Callable, *inputs: torch.Tensor):
        return cls.manager().run(name, fn, *inputs) if cls.enabled else fn(*inputs)

    @classmethod
    def proxy(cls, fn: Callable, name: Optional[str] = None) -> CUDAGraphProxy:
        return CUDAGraphProxy(fn, cls.manager(), name)

    @classmethod
    def stats(cls) -> Dict[str, int]:
        return cls.manager().stats()

    @classmethod
    def reset(cls):
        cls._manager = None
        cls.enabled = True
