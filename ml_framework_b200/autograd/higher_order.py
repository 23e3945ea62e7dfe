"""Higher-order derivative toolkit beyond the basic calls: options and results, sparse / partial / regularised Hessians,
eigenvalues, batched and numerical Hessian-vector products with validation, numerical gradients, a function registry,
and a context that tracks differentiation order.

Reference (src/MLFramework/Autograd/): Hessian.cs:233-470 (Compute with options, ComputeDiagonal,
ComputeVectorHessianProduct, ComputeNumerical, ComputeWithRegularization), Jacobian.cs:183-698 (options with modes
Auto / Forward / Reverse, numerical, Validate), HessianVectorProduct.cs:105-484 (batch, checkpointing, numerical,
Validate), HigherOrderExtensions.cs:95-193 (HessianWithEigenvalues, SparseHessian, PartialHessian, GradOfGrad),
HigherOrderContext.cs, GradientComputer.cs:90-276 (numerical gradients, error measures), FunctionRegistry.cs:26-182.

All of it is built on ``torch.func`` transforms, so every call works on GPU tensors and composes with this
package's custom autograd functions (which define ``setup_context`` where needed).
"""
from __future__ import annotations

import contextlib
import enum
import threading
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Type

import torch
import torch.func as tf

from .functional import CustomFunction, hvp as _hvp


# ------------------------------------------------------------------ options / results
class JacobianMode(enum.Enum):
    AUTO = "auto"
    FORWARD = "forward"
    REVERSE = "reverse"


@dataclass
class JacobianOptions:
    mode: JacobianMode = JacobianMode.AUTO
    chunk_size: Optional[int] = None         # rows (reverse) or columns (forward) per vectorised sweep; None = all at once
    validate: bool = False
    tolerance: float = 1e-4


@dataclass
class JacobianResult:
    jacobian: torch.Tensor
    mode_used: JacobianMode
    sweeps: int
    max_numerical_error: Optional[float] = None


@dataclass
class HessianOptions:
    sparse: bool = False
    sparsity_threshold: float = 1e-8         # |entry| <= threshold counts as zero
    symmetrize: bool = True
    eigenvalues: bool = False
    regularization: float = 0.0
    indices: Optional[Sequence[int]] = None  # partial Hessian over these flat coordinates only


@dataclass
class HessianResult:
    hessian: torch.Tensor                    # dense, or a sparse COO tensor when ``sparse``
    is_sparse: bool
    nonzeros: int
    density: float
    eigenvalues: Optional[torch.Tensor] = None

    @property
    def condition_number(self) -> Optional[float]:
        if self.eigenvalues is None:
            return None
        a = self.eigenvalues.abs()
        return float(a.max() / a.min().clamp_min(1e-30))

    @property
    def is_positive_definite(self) -> Optional[bool]:
        return None if self.eigenvalues is None else bool((self.eigenvalues > 0).all())


# ------------------------------------------------------------------ Jacobian
def jacobian_with_options(f: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, options: Optional[JacobianOptions] = None) -> JacobianResult:
    o = options or JacobianOptions()
    y = f(x)
    n_in, n_out = x.numel(), y.numel()
    mode = o.mode
    if mode == JacobianMode.AUTO:                       # one sweep per input (forward) or per output (reverse)
        mode = JacobianMode.FORWARD if n_in <= n_out else JacobianMode.REVERSE
    if mode == JacobianMode.FORWARD:
        J = tf.jacfwd(f, chunk_size=o.chunk_size)(x) if o.chunk_size else tf.jacfwd(f)(x)
        sweeps = -(-n_in // o.chunk_size) if o.chunk_size else 1
    else:
        J = tf.jacrev(f, chunk_size=o.chunk_size)(x) if o.chunk_size else tf.jacrev(f)(x)
        sweeps = -(-n_out // o.chunk_size) if o.chunk_size else 1
    err = None
    if o.validate:
        num = numerical_jacobian(f, x)
        err = float((J.reshape(n_out, n_in) - num).abs().max())
        if err > o.tolerance * max(1.0, float(num.abs().max())):
            raise ArithmeticError(f"Jacobian differs from finite differences by {err:.3e}")
    return JacobianResult(J, mode, sweeps, err)


def numerical_jacobian(f: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, eps: Optional[float] = None) -> torch.Tensor:
    """Central differences; ``[outputs, inputs]``. The step defaults to eps^(1/3) of the dtype times the input scale."""
    x = x.detach()
    h = eps if eps is not None else float(torch.finfo(x.dtype).eps) ** (1 / 3)
    flat = x.reshape(-1)
    cols = []
    for i in range(flat.numel()):
        s = h * max(1.0, abs(float(flat[i])))
        e = torch.zeros_like(flat)
        e[i] = s
        cols.append(((f((flat + e).view_as(x)) - f((flat - e).view_as(x))) / (2 * s)).reshape(-1))
    return torch.stack(cols, 1)


def numerical_gradient(f: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, eps: Optional[float] = None) -> torch.Tensor:
    return numerical_jacobian(lambda t: f(t).reshape(1), x, eps).reshape(x.shape)


def numerical_gradients(f: Callable[..., torch.Tensor], inputs: Sequence[torch.Tensor], eps: Optional[float] = None) -> List[torch.Tensor]:
    out = []
    for k in range(len(inputs)):
        def fk(t, k=k):
            args = list(inputs)
            args[k] = t
            return f(*args)
        out.append(numerical_gradient(fk, inputs[k], eps))
    return out


def relative_error(analytical: torch.Tensor, numerical: torch.Tensor) -> float:
    d = (analytical - numerical).norm()
    return float(d / (analytical.norm() + numerical.norm()).clamp_min(1e-30))


def mean_squared_error(analytical: torch.Tensor, numerical: torch.Tensor) -> float:
    return float(((analytical - numerical) ** 2).mean())


def validate_gradient(analytical: torch.Tensor, numerical: torch.Tensor, tolerance: float = 1e-4) -> bool:
    return analytical.shape == numerical.shape and relative_error(analytical, numerical) <= tolerance


# ------------------------------------------------------------------ Hessian
def hessian_with_options(f: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, options: Optional[HessianOptions] = None) -> HessianResult:
    o = options or HessianOptions()
    n = x.numel()
    if o.indices is not None:
        H = partial_hessian(f, x, o.indices)
    else:
        H = tf.hessian(f)(x).reshape(n, n)
    if o.symmetrize:
        H = 0.5 * (H + H.t())
    if o.regularization:
        H = H + o.regularization * torch.eye(H.shape[0], dtype=H.dtype, device=H.device)
    ev = torch.linalg.eigvalsh(H) if o.eigenvalues else None
    mask = H.abs() > o.sparsity_threshold
    nnz = int(mask.sum())
    out = H
    if o.sparse:
        idx = mask.nonzero().t()
        out = torch.sparse_coo_tensor(idx, H[mask], H.shape, check_invariants=False).coalesce()
    return HessianResult(out, o.sparse, nnz, nnz / max(H.numel(), 1), ev)


def partial_hessian(f: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, indices: Sequence[int]) -> torch.Tensor:
    """The rows and columns ``indices`` (flat coordinates of ``x``) of the Hessian: one Hessian-vector product per index."""
    idx = list(indices)
    n = x.numel()
    if any(not (0 <= i < n) for i in idx):
        raise IndexError("index outside the input")
    rows = []
    for i in idx:
        e = torch.zeros(n, dtype=x.dtype, device=x.device)
        e[i] = 1.0
        rows.append(_hvp(f, x, e.view_as(x)).reshape(-1)[idx])
    return torch.stack(rows)


def hessian_with_eigenvalues(f, x) -> Tuple[torch.Tensor, torch.Tensor]:
    r = hessian_with_options(f, x, HessianOptions(eigenvalues=True))
    return r.hessian, r.eigenvalues


def sparse_hessian(f, x, threshold: float = 1e-8) -> HessianResult:
    return hessian_with_options(f, x, HessianOptions(sparse=True, sparsity_threshold=threshold))


def regularized_hessian(f, x, regularization: float = 1e-6) -> torch.Tensor:
    return hessian_with_options(f, x, HessianOptions(regularization=regularization)).hessian


def top_eigenvalue(f, x, iters: int = 50, tol: float = 1e-6, seed: int = 0) -> Tuple[float, torch.Tensor]:
    """Largest-magnitude Hessian eigenvalue by power iteration on Hessian-vector products (no Hessian is formed)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    v = torch.randn(x.shape, generator=g, dtype=x.dtype).to(x.device)
    v = v / v.norm()
    lam = 0.0
    for _ in range(iters):
        w = _hvp(f, x, v)
        new = float((v * w).sum())
        nw = w.norm()
        if float(nw) == 0.0:
            return 0.0, v
        v = w / nw
        if abs(new - lam) <= tol * max(1.0, abs(new)):
            lam = new
            break
        lam = new
    return lam, v


def grad_of_grad(f: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor) -> torch.Tensor:
    """d/dx of sum(df/dx): the row sums of the Hessian, in one extra backward pass."""
    return tf.grad(lambda t: tf.grad(f)(t).sum())(x)


# ------------------------------------------------------------------ Hessian-vector products
@dataclass
class HVPOptions:
    checkpoint: bool = False         # recompute the gradient graph per product instead of holding it for the batch
    validate: bool = False
    tolerance: float = 1e-3


def hvp_batch(f, x: torch.Tensor, vectors: Sequence[torch.Tensor], options: Optional[HVPOptions] = None) -> List[torch.Tensor]:
    """Products with several vectors. Without ``checkpoint`` they are one vectorised sweep (``vmap`` over the tangent);
    with it they run one at a time, holding one gradient graph at most."""
    o = options or HVPOptions()
    if not vectors:
        return []
    if o.checkpoint:
        out = [_hvp(f, x, v) for v in vectors]
    else:
        V = torch.stack(list(vectors))
        out = list(torch.vmap(lambda v: tf.jvp(tf.grad(f), (x,), (v,))[1])(V))
    if o.validate:
        for v, r in zip(vectors, out):
            if not validate_hvp(f, x, v, o.tolerance, analytical=r):
                raise ArithmeticError("Hessian-vector product differs from finite differences")
    return out


def numerical_hvp(f, x: torch.Tensor, v: torch.Tensor, eps: Optional[float] = None) -> torch.Tensor:
    """(grad f(x + h v) - grad f(x - h v)) / 2h."""
    h = eps if eps is not None else float(torch.finfo(x.dtype).eps) ** (1 / 3)
    g = tf.grad(f)
    return (g(x + h * v) - g(x - h * v)) / (2 * h)


def validate_hvp(f, x, v, tolerance: float = 1e-3, analytical: Optional[torch.Tensor] = None) -> bool:
    a = analytical if analytical is not None else _hvp(f, x, v)
    return relative_error(a, numerical_hvp(f, x, v)) <= tolerance


# ------------------------------------------------------------------ Jacobian-vector and vector-Jacobian products
@dataclass
class JVPOptions:
    """Options of ``JacobianVectorProduct`` (JacobianVectorProduct.cs:31-70)."""
    exploit_sparsity: bool = True        # a zero tangent gives a zero product after one plain forward pass (for the shape)
    cache_tangents: bool = False         # remember products per (function, point, tangent)
    sparsity_threshold: float = 1e-10
    enable_parallel: bool = True         # batches as one vectorised sweep instead of a loop
    max_parallel_tasks: int = -1         # chunk size of that sweep; -1 = everything at once
    output_buffer: Optional[torch.Tensor] = None
    clear_cache: bool = False


@dataclass
class VJPOptions:
    """Options of ``VectorJacobianProduct`` (VectorJacobianProduct.cs:31-70)."""
    exploit_sparsity: bool = True
    cache_gradients: bool = False
    sparsity_threshold: float = 1e-10
    enable_parallel: bool = True
    max_parallel_tasks: int = -1
    output_buffer: Optional[torch.Tensor] = None
    clear_cache: bool = False


def _cache_key(f, x: torch.Tensor, v: torch.Tensor):
    return (id(f), tuple(x.shape), x.dtype, hash(x.detach().cpu().numpy().tobytes()), hash(v.detach().cpu().numpy().tobytes()))


def _emit(result: torch.Tensor, buffer: Optional[torch.Tensor]) -> torch.Tensor:
    if buffer is None:
        return result
    if buffer.shape != result.shape:
        raise ValueError(f"output buffer has shape {list(buffer.shape)}, the product {list(result.shape)}")
    buffer.copy_(result)
    return buffer


class JacobianVectorProduct:
    """``J(x) v`` by forward-mode differentiation: one pass, no Jacobian (JacobianVectorProduct.cs:14-460)."""

    _cache: Dict[tuple, torch.Tensor] = {}
    _lock = threading.Lock()

    @classmethod
    def compute(cls, f, x: torch.Tensor, v: torch.Tensor, options: Optional[JVPOptions] = None) -> torch.Tensor:
        o = options or JVPOptions()
        if v.shape != x.shape:
            raise ValueError(f"the tangent has shape {list(v.shape)}, the point {list(x.shape)}")
        if o.clear_cache:
            cls.clear_tangent_cache()
        if o.exploit_sparsity and (v.numel() == 0 or float(v.abs().max()) <= o.sparsity_threshold):
            with torch.no_grad():                                        # a plain forward pass gives the output's shape
                y = f(x.detach())
            return _emit(torch.zeros_like(y), o.output_buffer)
        key = _cache_key(f, x, v) if o.cache_tangents else None
        if key is not None:
            with cls._lock:
                hit = cls._cache.get(key)
            if hit is not None:
                return _emit(hit.clone(), o.output_buffer)
        res = tf.jvp(f, (x,), (v,))[1]
        if key is not None:
            with cls._lock:
                cls._cache[key] = res.detach().clone()
        return _emit(res, o.output_buffer)

    @classmethod
    def compute_batch(cls, f, x: torch.Tensor, vectors: Sequence[torch.Tensor], options: Optional[JVPOptions] = None) -> List[torch.Tensor]:
        o = options or JVPOptions()
        if not len(vectors):
            return []
        if not o.enable_parallel:
            return [cls.compute(f, x, v, o) for v in vectors]
        V = torch.stack(list(vectors))
        chunk = None if o.max_parallel_tasks <= 0 else o.max_parallel_tasks
        return list(torch.vmap(lambda v: tf.jvp(f, (x,), (v,))[1], chunk_size=chunk)(V))

    @classmethod
    def compute_multiple(cls, f, inputs: Sequence[torch.Tensor], v: torch.Tensor, input_index: int = 0,
                         options: Optional[JVPOptions] = None) -> torch.Tensor:
        """Product with respect to ``inputs[input_index]`` of a function of several tensors (given as a list)."""
        if not 0 <= input_index < len(inputs):
            raise IndexError(f"input index {input_index} of {len(inputs)} inputs")
        inputs = list(inputs)

        def g(xi):
            return f(inputs[:input_index] + [xi] + inputs[input_index + 1:])
        return cls.compute(g, inputs[input_index], v, options)

    @classmethod
    def clear_tangent_cache(cls) -> None:
        with cls._lock:
            cls._cache.clear()

    @classmethod
    def get_cache_size(cls) -> int:
        return len(cls._cache)

    @staticmethod
    def compute_numerical(f, x: torch.Tensor, v: torch.Tensor, epsilon: Optional[float] = None) -> torch.Tensor:
        h = epsilon if epsilon is not None else float(torch.finfo(x.dtype).eps) ** (1 / 3)
        return (f(x + h * v) - f(x - h * v)) / (2 * h)

    @classmethod
    def validate(cls, f, x, v, tolerance: float = 1e-3, epsilon: Optional[float] = None) -> bool:
        return relative_error(cls.compute(f, x, v, JVPOptions(exploit_sparsity=False)), cls.compute_numerical(f, x, v, epsilon)) <= tolerance

    @classmethod
    def compute_jacobian(cls, f, x: torch.Tensor) -> torch.Tensor:
        """The Jacobian column by column: one product per input element ([*out, *in])."""
        eye = torch.eye(x.numel(), dtype=x.dtype, device=x.device).view(x.numel(), *x.shape)
        cols = torch.vmap(lambda e: tf.jvp(f, (x,), (e,))[1])(eye)
        return cols.movedim(0, -1).reshape(*cols.shape[1:], *x.shape)


class VectorJacobianProduct:
    """``v^T J(x)`` by reverse-mode differentiation (VectorJacobianProduct.cs:14-500)."""

    _cache: Dict[tuple, torch.Tensor] = {}
    _lock = threading.Lock()

    @classmethod
    def compute(cls, f, x: torch.Tensor, v: torch.Tensor, options: Optional[VJPOptions] = None) -> torch.Tensor:
        o = options or VJPOptions()
        if o.clear_cache:
            cls.clear_gradient_cache()
        if o.exploit_sparsity and (v.numel() == 0 or float(v.abs().max()) <= o.sparsity_threshold):
            return _emit(torch.zeros_like(x), o.output_buffer)
        key = _cache_key(f, x, v) if o.cache_gradients else None
        if key is not None:
            with cls._lock:
                hit = cls._cache.get(key)
            if hit is not None:
                return _emit(hit.clone(), o.output_buffer)
        y, pull = tf.vjp(f, x)
        if v.shape != y.shape:
            raise ValueError(f"the cotangent has shape {list(v.shape)}, the output {list(y.shape)}")
        res = pull(v)[0]
        if key is not None:
            with cls._lock:
                cls._cache[key] = res.detach().clone()
        return _emit(res, o.output_buffer)

    @classmethod
    def compute_batch(cls, f, x: torch.Tensor, vectors: Sequence[torch.Tensor], options: Optional[VJPOptions] = None) -> List[torch.Tensor]:
        o = options or VJPOptions()
        if not len(vectors):
            return []
        if not o.enable_parallel:
            return [cls.compute(f, x, v, o) for v in vectors]
        _, pull = tf.vjp(f, x)                                           # one forward pass serves every cotangent
        chunk = None if o.max_parallel_tasks <= 0 else o.max_parallel_tasks
        return list(torch.vmap(lambda v: pull(v)[0], chunk_size=chunk)(torch.stack(list(vectors))))

    @classmethod
    def compute_multiple(cls, f, inputs: Sequence[torch.Tensor], v: torch.Tensor, options: Optional[VJPOptions] = None) -> List[torch.Tensor]:
        """One pull-back gives the product for every input of ``f(list_of_tensors)``."""
        _, pull = tf.vjp(lambda *xs: f(list(xs)), *inputs)
        return list(pull(v))

    @classmethod
    def clear_gradient_cache(cls) -> None:
        with cls._lock:
            cls._cache.clear()

    @classmethod
    def get_cache_size(cls) -> int:
        return len(cls._cache)

    @staticmethod
    def compute_numerical(f, x: torch.Tensor, v: torch.Tensor, epsilon: Optional[float] = None) -> torch.Tensor:
        """Element ``i`` is ``v . (f(x + h e_i) - f(x - h e_i)) / 2h``."""
        h = epsilon if epsilon is not None else float(torch.finfo(x.dtype).eps) ** (1 / 3)
        out = torch.zeros_like(x)
        flat = out.view(-1)
        for i in range(x.numel()):
            e = torch.zeros_like(x).view(-1)
            e[i] = h
            e = e.view_as(x)
            flat[i] = ((f(x + e) - f(x - e)) * v).sum() / (2 * h)
        return out

    @classmethod
    def validate(cls, f, x, v, tolerance: float = 1e-3, epsilon: Optional[float] = None) -> bool:
        return relative_error(cls.compute(f, x, v, VJPOptions(exploit_sparsity=False)), cls.compute_numerical(f, x, v, epsilon)) <= tolerance


# ------------------------------------------------------------------ order tracking
class HigherOrderContext:
    """Tracks how deeply differentiation is nested on this thread (``with ctx.order():`` around each level) and caps it;
    ``create_graph`` is what a backward call inside the block needs: True below the top level."""
    _tls = threading.local()

    def __init__(self, max_order: int = 4):
        if max_order < 1:
            raise ValueError("max_order must be at least 1")
        self.max_order = max_order

    @property
    def current_order(self) -> int:
        return getattr(self._tls, "depth", 0)

    @property
    def create_graph(self) -> bool:
        return self.current_order < self.max_order and getattr(self._tls, "want", 1) > self.current_order

    @contextlib.contextmanager
    def order(self, target_order: Optional[int] = None):
        d = self.current_order + 1
        if d > self.max_order:
            raise RecursionError(f"differentiation order {d} exceeds the limit {self.max_order}")
        prev_want = getattr(self._tls, "want", 1)
        if target_order is not None:
            if target_order > self.max_order:
                raise RecursionError(f"requested order {target_order} exceeds the limit {self.max_order}")
            self._tls.want = target_order
        self._tls.depth = d
        try:
            yield d
        finally:
            self._tls.depth = d - 1
            self._tls.want = prev_want

    def nth_derivative(self, f: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, n: int) -> torch.Tensor:
        """n-th derivative of a scalar-to-scalar function applied element-wise (sum trick), n <= max_order."""
        if n < 0 or n > self.max_order:
            raise RecursionError(f"order {n} outside [0, {self.max_order}]")
        g = f
        for _ in range(n):
            g = (lambda h: (lambda t: tf.grad(lambda u: h(u).sum())(t)))(g)
        return g(x)


# ------------------------------------------------------------------ function registry
class FunctionRegistry:
    """Named custom-function TYPES; ``create_instance`` builds a fresh one per use (functions may keep state)."""
    _types: Dict[str, Type[CustomFunction]] = {}
    _lock = threading.Lock()

    @classmethod
    def register(cls, name: str, fn_type: Type[CustomFunction], overwrite: bool = False):
        if not (isinstance(fn_type, type) and issubclass(fn_type, CustomFunction)):
            raise TypeError("expected a CustomFunction subclass")
        with cls._lock:
            if name in cls._types and not overwrite:
                raise KeyError(f"function {name!r} is already registered")
            cls._types[name] = fn_type

    @classmethod
    def is_registered(cls, name: str) -> bool:
        return name in cls._types

    @classmethod
    def get_function_type(cls, name: str) -> Type[CustomFunction]:
        if name not in cls._types:
            raise KeyError(f"no function named {name!r}; registered: {sorted(cls._types)}")
        return cls._types[name]

    @classmethod
    def create_instance(cls, name: str, *a, **k) -> CustomFunction:
        return cls.get_function_type(name)(*a, **k)

    @classmethod
    def unregister(cls, name: str) -> bool:
        with cls._lock:
            return cls._types.pop(name, None) is not None

    @classmethod
    def names(cls) -> List[str]:
        return sorted(cls._types)

    @classmethod
    def clear_all(cls):
        with cls._lock:
            cls._types.clear()

    @classmethod
    def apply_function(cls, name: str, *inputs, init_args: Sequence = ()):
        return cls.create_instance(name, *init_args).apply(*inputs)
