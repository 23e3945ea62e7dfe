"""Functional transforms: vmap, pmap, jit, grad composition.

Reference: src/MLFramework/Functional/** (``VMapTransform`` with per-argument axes, ``PMapTransform`` over a device
mesh with named axes and collectives, ``JITTransform`` with tracing and a per-signature cache, ``compose``).

* ``vmap`` batches a function over chosen axes of its arguments. Functions made of plain tensor operations go through
  ``torch.func.vmap`` (one batched launch); functions that cannot be batched that way (the native autograd functions
  of this package, data-dependent Python) fall back to an explicit loop, optionally in chunks to bound memory.
* ``pmap`` splits the mapped axis over the ranks of a process group (or one dimension of a ``DeviceMesh``), runs the
  function on each rank's slice with the axis name bound, so that ``psum`` / ``pmean`` / ``pmax`` / ``all_gather``
  inside the function reduce over the mapped ranks, and gathers the outputs.
* ``jit`` traces a function of tensors into the high-level IR (``compiler.ir.HLGraph``) by running it on tracer
  objects, optimises the graph with the pass manager and executes the optimised graph, cached per input signature.
  What cannot be traced (unsupported operations, control flow on values) falls back to CUDA-graph capture on CUDA
  inputs and to plain execution otherwise: launch overhead is what a captured graph removes, kernels stay hand-written.
"""
from __future__ import annotations

import contextlib
import enum
import threading
import weakref
from typing import Callable, Dict, Optional, Sequence, Tuple, Union

import torch
import torch.func as tf

from ..hal.cuda_graphs import CUDAGraphManager

grad = tf.grad
grad_and_value = tf.grad_and_value


def compose(*fns: Callable) -> Callable:
    def run(x):
        for f in fns:
            x = f(x)
        return x
    return run


# ------------------------------------------------------------------ combinators (Functional/Composition.cs:11-334)
def pipe(value, *fns: Callable):
    """``pipe(x, f, g)`` = ``g(f(x))``."""
    for f in fns:
        value = f(value)
    return value


def partial(fn: Callable, first) -> Callable:
    """Fixes the first argument."""
    return lambda *rest, **kw: fn(first, *rest, **kw)


def partial_second(fn: Callable, second) -> Callable:
    """Fixes the second argument."""
    return lambda first, *rest, **kw: fn(first, second, *rest, **kw)


def curry(fn: Callable, arity: int = 2) -> Callable:
    """``curry(f)(a)(b) == f(a, b)`` (``arity`` arguments, one call each)."""
    if arity < 1:
        raise ValueError("arity must be at least 1")

    def take(args):
        return (lambda x: take(args + (x,))) if len(args) + 1 < arity else (lambda x: fn(*args, x))
    return take(())


def uncurry(fn: Callable) -> Callable:
    def run(*args):
        out = fn
        for a in args:
            out = out(a)
        return out
    return run


def identity(value):
    return value


def constant(value) -> Callable:
    return lambda *a, **k: value


def tap(value, action: Callable):
    """Runs ``action(value)`` for its side effect (logging, a check) and passes the value on."""
    action(value)
    return value


def tap_if(value, condition: bool, action: Callable):
    if condition:
        action(value)
    return value


# ------------------------------------------------------------------ transformation bookkeeping
class TransformationType(enum.Enum):
    VECTORIZATION = "vectorization"
    PARALLELIZATION = "parallelization"
    COMPILATION = "compilation"
    COMPOSITION = "composition"


class MeshAxisNames:
    """Conventional axis names of a device mesh (Functional/Distributed/MeshAxisNames.cs)."""
    DATA = "data"
    MODEL = "model"
    PIPELINE = "pipeline"


class TransformationContext:
    """Settings shared by nested transformations; a child sees its parents' metadata
    (Functional/TransformationContext.cs:6-90)."""

    def __init__(self, parent: Optional["TransformationContext"] = None):
        self.parent = parent
        self.metadata: Dict[str, object] = {}
        self.debug_mode = parent.debug_mode if parent is not None else False

    def get_metadata(self, key: str, default=None, search_parents: bool = True):
        if key in self.metadata:
            return self.metadata[key]
        if search_parents and self.parent is not None:
            return self.parent.get_metadata(key, default, True)
        return default

    def set_metadata(self, key: str, value) -> None:
        self.metadata[key] = value

    def create_child_context(self) -> "TransformationContext":
        return TransformationContext(self)


def tensor_function(fn: Optional[Callable] = None, *, is_pure: bool = True, input_shapes: Optional[Sequence[str]] = None,
                    output_shape: Optional[str] = None, description: str = ""):
    """Marks a function of tensors: whether it is pure (no side effects: transformations may re-run,
    reorder or cache it) and, optionally, its symbolic shapes (Functional/TensorFunctionAttribute.cs)."""
    def mark(f):
        f.__tensor_function__ = {"is_pure": is_pure, "input_shapes": tuple(input_shapes or ()),
                                 "output_shape": output_shape, "description": description}
        return f
    return mark(fn) if fn is not None else mark


def is_function_pure(fn: Callable) -> bool:
    """Unmarked functions are taken to be pure, as the reference does."""
    return getattr(fn, "__tensor_function__", {"is_pure": True})["is_pure"]


class BaseTransformation:
    """A named transformation of a function; ``__call__`` applies it and records the fact in the
    registry (Functional/BaseTransformation.cs:8-110)."""

    def __init__(self, name: str, type: TransformationType, context: Optional[TransformationContext] = None):
        self.name, self.type = name, type
        self.context = context or TransformationContext()

    def transform(self, original: Callable) -> Callable:
        raise NotImplementedError

    def validate(self, fn: Callable) -> None:
        if not callable(fn):
            raise TypeError(f"{self.name}: expected a function, got {type(fn).__name__}")
        if self.type is not TransformationType.COMPOSITION and not is_function_pure(fn):
            raise ValueError(f"{self.name}: function {getattr(fn, '__name__', fn)!r} is marked impure and cannot be transformed")

    def __call__(self, fn: Callable) -> Callable:
        self.validate(fn)
        out = self.transform(fn)
        TransformationRegistry.register(fn, self)
        if self.context.debug_mode:
            self.context.set_metadata("last_applied", (self.name, getattr(fn, "__name__", repr(fn))))
        return out


class VMapTransformation(BaseTransformation):
    def __init__(self, in_axes=0, out_axes: int = 0, chunk_size: Optional[int] = None, context=None):
        super().__init__("vmap", TransformationType.VECTORIZATION, context)
        self.in_axes, self.out_axes, self.chunk_size = in_axes, out_axes, chunk_size

    def transform(self, original):
        return vmap(original, self.in_axes, self.out_axes, self.chunk_size)


class PMapTransformation(BaseTransformation):
    def __init__(self, pg=None, axis_name: str = MeshAxisNames.DATA, in_axes=0, context=None):
        super().__init__("pmap", TransformationType.PARALLELIZATION, context)
        self.pg, self.axis_name, self.in_axes = pg, axis_name, in_axes

    def transform(self, original):
        return pmap(original, self.pg, self.axis_name, self.in_axes)


class JITTransformation(BaseTransformation):
    def __init__(self, optimize: bool = True, context=None):
        super().__init__("jit", TransformationType.COMPILATION, context)
        self.optimize = optimize

    def transform(self, original):
        return jit(original, optimize=self.optimize)


class TransformationRegistry:
    """Which transformations have been applied to which function (Functional/TransformationRegistry.cs).
    Functions are held weakly where they allow it, so the registry does not keep closures alive."""

    _lock = threading.Lock()
    _by_id: Dict[int, Tuple[object, list]] = {}

    @classmethod
    def _key(cls, fn) -> int:
        return id(fn)

    @classmethod
    def register(cls, original: Callable, transform: BaseTransformation) -> None:
        if original is None or transform is None:
            raise ValueError("function and transformation are required")
        with cls._lock:
            k = cls._key(original)
            if k not in cls._by_id:
                try:
                    ref = weakref.ref(original, lambda _r, k=k: cls._by_id.pop(k, None))
                except TypeError:
                    ref = lambda o=original: o                       # noqa: E731 - objects without weak references stay alive
                cls._by_id[k] = (ref, [])
            lst = cls._by_id[k][1]
            if not any(t.name == transform.name and t.type == transform.type for t in lst):
                lst.append(transform)

    @classmethod
    def get_transformations(cls, original: Callable) -> list:
        with cls._lock:
            e = cls._by_id.get(cls._key(original))
            return list(e[1]) if e is not None and e[0]() is original else []

    @classmethod
    def get_transformations_by_type(cls, original: Callable, type: TransformationType) -> list:
        return [t for t in cls.get_transformations(original) if t.type == type]

    @classmethod
    def has_transformations(cls, original: Callable) -> bool:
        return bool(cls.get_transformations(original))

    @classmethod
    def has_transformation_of_type(cls, original: Callable, type: TransformationType) -> bool:
        return bool(cls.get_transformations_by_type(original, type))

    @classmethod
    def unregister(cls, original: Callable) -> bool:
        with cls._lock:
            return cls._by_id.pop(cls._key(original), None) is not None

    @classmethod
    def clear(cls) -> None:
        with cls._lock:
            cls._by_id.clear()

    @classmethod
    def count(cls) -> int:
        return len(cls._by_id)

    @classmethod
    def total_transformation_count(cls) -> int:
        with cls._lock:
            return sum(len(e[1]) for e in cls._by_id.values())


def vectorize(fn: Callable, in_axes=0, out_axes: int = 0) -> Callable:
    """``vmap`` that also records itself in the registry."""
    return VMapTransformation(in_axes, out_axes)(fn)


def parallelize(fn: Callable, pg=None, axis_name: str = MeshAxisNames.DATA, in_axes=0) -> Callable:
    return PMapTransformation(pg, axis_name, in_axes)(fn)


def compile_function(fn: Callable, optimize: bool = True) -> Callable:
    return JITTransformation(optimize)(fn)


# ------------------------------------------------------------------ vmap
def _norm_axes(axes, n) -> Tuple:
    if isinstance(axes, (tuple, list)):
        if len(axes) != n:
            raise ValueError(f"in_axes has {len(axes)} entries for {n} arguments")
        return tuple(axes)
    return (axes,) * n


def vmap(fn: Callable, in_axes: Union[int, None, Sequence] = 0, out_axes: int = 0, chunk_size: Optional[int] = None,
         fallback: str = "auto") -> Callable:
    """``vmap(fn, in_axes, out_axes)(*args)``. ``in_axes[i] = None`` passes argument i unchanged to every call.
    ``fallback``: "auto" tries ``torch.func.vmap`` and loops when that fails, "loop" always loops, "never" raises."""
    def run(*args):
        axes = _norm_axes(in_axes, len(args))
        sizes = {a.shape[ax] for a, ax in zip(args, axes) if ax is not None}
        if len(sizes) != 1:
            raise ValueError(f"mapped axes disagree on their size: {sorted(sizes)}")
        n = sizes.pop()
        if fallback != "loop":
            try:
                return tf.vmap(fn, in_dims=axes, out_dims=out_axes, chunk_size=chunk_size)(*args)
            except Exception:
                if fallback == "never":
                    raise
        outs = []
        for i in range(n):
            outs.append(fn(*[a.select(ax, i) if ax is not None else a for a, ax in zip(args, axes)]))
        if isinstance(outs[0], (tuple, list)):
            return type(outs[0])(torch.stack([o[k] for o in outs], out_axes) for k in range(len(outs[0])))
        return torch.stack(outs, out_axes)
    run.__wrapped__ = fn
    return run


# ------------------------------------------------------------------ pmap and its collectives
_axis_env = threading.local()


def _axes() -> Dict[str, object]:
    if not hasattr(_axis_env, "d"):
        _axis_env.d = {}
    return _axis_env.d


@contextlib.contextmanager
def _bind_axis(name: str, pg):
    env = _axes()
    old = env.get(name)
    env[name] = pg
    try:
        yield
    finally:
        if old is None:
            env.pop(name, None)
        else:
            env[name] = old


def _group(axis_name: str):
    pg = _axes().get(axis_name)
    if pg is None and axis_name not in _axes():
        raise NameError(f"axis {axis_name!r} is not bound: psum / pmean / all_gather must run inside pmap(..., axis_name={axis_name!r})")
    return pg


def psum(x: torch.Tensor, axis_name: str) -> torch.Tensor:
    pg = _group(axis_name)
    if pg is None or pg.world_size == 1:
        return x
    from ..dist.process_group import ReduceOp
    return pg.all_reduce(x.clone(), ReduceOp.SUM)


def pmean(x: torch.Tensor, axis_name: str) -> torch.Tensor:
    pg = _group(axis_name)
    return psum(x, axis_name) / (pg.world_size if pg is not None else 1)


def pmax(x: torch.Tensor, axis_name: str) -> torch.Tensor:
    pg = _group(axis_name)
    if pg is None or pg.world_size == 1:
        return x
    from ..dist.process_group import ReduceOp
    return pg.all_reduce(x.clone(), ReduceOp.MAX)


def all_gather(x: torch.Tensor, axis_name: str, axis: int = 0) -> torch.Tensor:
    pg = _group(axis_name)
    if pg is None or pg.world_size == 1:
        return x
    return pg.all_gather(x, dim=axis)


def axis_index(axis_name: str) -> int:
    pg = _group(axis_name)
    return 0 if pg is None else pg.rank


def pmap(fn: Callable, pg=None, axis_name: str = "i", in_axes: Union[int, None, Sequence] = 0, out_axis: int = 0,
         mesh=None, mesh_dim: Optional[str] = None, gather: bool = True) -> Callable:
    """``pmap(fn, pg)(x, ...)``: every mapped argument is split along its axis over the ranks; each rank applies ``fn``
    to its slice with ``axis_name`` bound to the group; with ``gather`` the outputs are all-gathered along ``out_axis``
    so that every rank returns the full result. ``mesh`` + ``mesh_dim`` map over one dimension of a ``DeviceMesh``.
    Without a group the function runs once on the whole input (one "device")."""
    group = pg
    if mesh is not None:
        group = mesh.process_group(mesh_dim)

    def run(*args):
        axes = _norm_axes(in_axes, len(args))
        W = group.world_size if group is not None else 1
        r = group.rank if group is not None else 0
        local = []
        for a, ax in zip(args, axes):
            if ax is None or W == 1:
                local.append(a)
                continue
            if a.shape[ax] % W:
                raise ValueError(f"mapped dimension {a.shape[ax]} not divisible by the {W} ranks of axis {axis_name!r}")
            n = a.shape[ax] // W
            local.append(a.narrow(ax, r * n, n))
        with _bind_axis(axis_name, group):
            y = fn(*local)
        if W == 1 or not gather:
            return y
        if isinstance(y, (tuple, list)):
            return type(y)(group.all_gather(t.contiguous(), dim=out_axis) for t in y)
        return group.all_gather(y.contiguous(), dim=out_axis)
    run.__wrapped__ = fn
    return run


# ------------------------------------------------------------------ jit: tracing into the high-level IR
class TraceError(RuntimeError):
    pass


class Tracer:
    """Stands for a tensor while a function is traced: operations on it append to an ``HLGraph``."""
    __array_priority__ = 1000

    def __init__(self, graph, name: str):
        self.g, self.name = graph, name

    @property
    def shape(self):
        return self.g.values[self.name].shape

    @property
    def dtype(self):
        return self.g.values[self.name].dtype

    def _lift(self, other) -> str:
        if isinstance(other, Tracer):
            return other.name
        if isinstance(other, torch.Tensor):
            return self.g.constant(other)
        if isinstance(other, (int, float)):
            return self.g.constant(torch.tensor(float(other), dtype=self.dtype))
        raise TraceError(f"cannot trace an operand of type {type(other).__name__}")

    def _bin(self, kind, other, swap=False):
        a, b = self.name, self._lift(other)
        return Tracer(self.g, self.g.op(kind, *((b, a) if swap else (a, b))))

    def __add__(self, o): return self._bin("add", o)
    def __radd__(self, o): return self._bin("add", o, True)
    def __sub__(self, o): return self._bin("sub", o)
    def __rsub__(self, o): return self._bin("sub", o, True)
    def __mul__(self, o): return self._bin("mul", o)
    def __rmul__(self, o): return self._bin("mul", o, True)
    def __truediv__(self, o): return self._bin("div", o)
    def __rtruediv__(self, o): return self._bin("div", o, True)
    def __matmul__(self, o): return self._bin("matmul", o)
    def __neg__(self): return Tracer(self.g, self.g.op("neg", self.name))

    def __bool__(self):
        raise TraceError("the truth value of a traced tensor is not known while tracing (data-dependent control flow)")

    def _compare(self, other):
        raise TraceError("comparisons of traced tensors are not traceable (their result would steer Python control flow)")

    __lt__ = __le__ = __gt__ = __ge__ = _compare

    def _concrete(self, *a, **k):
        raise TraceError("the value of a traced tensor is not known while tracing")

    __float__ = __int__ = __index__ = item = tolist = numpy = _concrete

    def _un(self, kind, **attrs):
        return Tracer(self.g, self.g.op(kind, self.name, **attrs))

    def relu(self): return self._un("relu")
    def exp(self): return self._un("exp")
    def log(self): return self._un("log")
    def sqrt(self): return self._un("sqrt")
    def tanh(self): return self._un("tanh")
    def sigmoid(self): return self._un("sigmoid")
    def sum(self, dim=None, keepdim=False): return self._un("sum", **({} if dim is None else {"dim": dim, "keepdim": keepdim}))
    def mean(self, dim=None, keepdim=False): return self._un("mean", **({} if dim is None else {"dim": dim, "keepdim": keepdim}))
    def reshape(self, *shape): return self._un("reshape", shape=tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else tuple(shape))
    def transpose(self, d0, d1): return self._un("transpose", dim0=d0, dim1=d1)

    @property
    def T(self):
        return self.transpose(-2, -1)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        name = getattr(func, "__name__", "")
        table = {"relu": "relu", "exp": "exp", "log": "log", "sqrt": "sqrt", "tanh": "tanh", "sigmoid": "sigmoid", "neg": "neg",
                 "add": "add", "sub": "sub", "mul": "mul", "div": "div", "true_divide": "div", "matmul": "matmul", "maximum": "maximum",
                 "minimum": "minimum"}
        t = next(a for a in args if isinstance(a, Tracer))
        if name == "gelu":
            return t._un("gelu")
        if name == "softmax":
            return t._un("softmax", dim=kwargs.get("dim", args[1] if len(args) > 1 else -1))
        if name in ("sum", "mean"):
            return getattr(t, name)(*args[1:], **kwargs)
        if name in table:
            kind = table[name]
            if len(args) == 1:
                return t._un(kind)
            a, b = args[0], args[1]
            return a._bin(kind, b) if isinstance(a, Tracer) else b._bin(kind, a, True)
        raise TraceError(f"operation {name!r} is not traceable")


_live_jit_functions: "weakref.WeakSet" = weakref.WeakSet()


def clear_jit_cache() -> int:
    """Clears the caches of all live jitted functions (Functional.ClearJITCache); returns how many."""
    fns = list(_live_jit_functions)
    for f in fns:
        f.clear_cache()
    return len(fns)


class JitFunction:
    """Result of ``jit(fn)``: per input signature either a traced + optimised graph, a CUDA-graph capture, or ``fn`` itself."""

    def __init__(self, fn: Callable, name: Optional[str] = None, optimize: bool = True):
        self.fn, self.name, self.optimize = fn, name or getattr(fn, "__name__", "jit_fn"), optimize
        self._cache: Dict[Tuple, Tuple[str, object]] = {}
        self.stats = {"traced": 0, "captured": 0, "eager": 0, "hits": 0}
        self.__wrapped__ = fn
        _live_jit_functions.add(self)

    def clear_cache(self) -> None:
        """Forgets every traced graph and capture: the next call of each signature traces again."""
        self._cache.clear()

    @staticmethod
    def _sig(inputs) -> Tuple:
        return tuple((tuple(t.shape), t.dtype, t.device.type) for t in inputs)

    def _trace(self, inputs):
        from . import ir
        g = ir.HLGraph(self.name)
        tracers = [Tracer(g, g.input(f"arg{i}", t.shape, t.dtype)) for i, t in enumerate(inputs)]
        out = self.fn(*tracers)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        if not all(isinstance(o, Tracer) for o in outs):
            raise TraceError("the function returned something that was not computed from its tensor arguments")
        g.output(*[o.name for o in outs])
        if self.optimize:
            ir.PassManager().run(g)
        return g, isinstance(out, (tuple, list))

    def graph(self, *inputs):
        """The optimised graph for these inputs (traces if needed); None when the function is not traceable."""
        self(*inputs)
        kind, obj = self._cache[self._sig(inputs)]
        return obj[0] if kind == "graph" else None

    def __call__(self, *inputs: torch.Tensor):
        key = self._sig(inputs)
        ent = self._cache.get(key)
        if ent is None:
            try:
                g, many = self._trace(inputs)
                ent = ("graph", (g, many))
                self.stats["traced"] += 1
            except (TraceError, TypeError, AttributeError, NotImplementedError):
                # not expressible in the IR (an operation or a method the tracer does not know, control flow on values)
                if all(t.is_cuda for t in inputs) and torch.cuda.is_available():
                    ent = ("capture", _graph_manager())
                    self.stats["captured"] += 1
                else:
                    ent = ("eager", None)
                    self.stats["eager"] += 1
            self._cache[key] = ent
        else:
            self.stats["hits"] += 1
        kind, obj = ent
        if kind == "graph":
            g, many = obj
            res = g.run({f"arg{i}": t for i, t in enumerate(inputs)})
            return tuple(res) if many else res[0]
        if kind == "capture":
            return obj.run(self.name, self.fn, *inputs)
        return self.fn(*inputs)


_manager: Optional[CUDAGraphManager] = None


def _graph_manager() -> CUDAGraphManager:
    global _manager
    if _manager is None:
        _manager = CUDAGraphManager()
    return _manager


def jit(fn: Optional[Callable] = None, name: Optional[str] = None, optimize: bool = True):
    if fn is None:
        return lambda f: JitFunction(f, name, optimize)
    return JitFunction(fn, name, optimize)
