"""Autograd functions for tensors whose extents are only known at run time.

Reference: src/MLFramework/Autograd/{IDynamicGradientFunction.cs, DynamicAutogradContext.cs:9-372,
DynamicGradientTensor.cs:8-221} and Autograd/Operations/{DynamicSlice.cs, DynamicPad.cs,
DynamicMask.cs, DynamicGather.cs, DynamicBroadcastBackward.cs, DynamicReshapeBackward.cs,
DynamicMatMulBackward.cs, DynamicConv2DBackward.cs}.

Every function states its shape rule on symbolic shapes (``compiler.shapes.SymbolicShape``: a
dimension is a number or a name such as ``batch`` or ``seq``), checks the incoming gradient
against the shape it promised, and computes real gradients. ``fn(*tensors)`` runs it inside
torch's autograd, so the shape checks fire during ``backward()``; ``fn.compute_grad`` is the
gradient rule on its own, for the IR-level differentiation and for tests against autograd.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..compiler.shapes import SymbolicDimension, SymbolicShape

__all__ = [
    "DynamicAutogradContext", "DynamicGradientTensor", "DynamicGradientFunction", "DynamicSlice", "DynamicPad",
    "DynamicMask", "DynamicGather", "DynamicBroadcastBackward", "DynamicReshapeBackward", "DynamicMatMulBackward",
    "DynamicConv2DBackward", "shape_of", "matches",
]


def shape_of(t: torch.Tensor, names: Optional[Sequence[Optional[str]]] = None) -> SymbolicShape:
    """The tensor's shape; ``names[i]`` makes dimension ``i`` a named symbol bound to its current size."""
    if names is None:
        return SymbolicShape(list(t.shape))
    if len(names) != t.dim():
        raise ValueError(f"{len(names)} names for a tensor of rank {t.dim()}")
    return SymbolicShape([SymbolicDimension(n, s) if n else s for n, s in zip(names, t.shape)])


def matches(symbolic: SymbolicShape, concrete: Sequence[int], env: Optional[Dict[str, int]] = None) -> bool:
    """Whether ``concrete`` is an instance of ``symbolic``: known dimensions equal, each name bound to
    one value throughout (``env`` carries bindings in and out)."""
    if symbolic.rank != len(concrete):
        return False
    env = {} if env is None else env
    for d, c in zip(symbolic.dims, concrete):
        if d.is_known:
            if d.value != c:
                return False
        elif env.setdefault(d.name, int(c)) != c:
            return False
        elif c < d.min_value or (d.max_value is not None and c > d.max_value):
            return False
    return True


class DynamicAutogradContext:
    """What a dynamic function keeps between forward and backward: tensors, the symbolic shapes of
    its inputs and outputs, and the gradient shape it expects per output."""

    def __init__(self):
        self._saved: List[torch.Tensor] = []
        self._in: List[SymbolicShape] = []
        self._out: List[SymbolicShape] = []
        self._grad: Dict[int, SymbolicShape] = {}
        self._disposed = False

    def _alive(self):
        if self._disposed:
            raise RuntimeError("the context has been disposed")

    @property
    def saved_tensors(self) -> Tuple[torch.Tensor, ...]:
        return tuple(self._saved)

    @property
    def input_shapes(self) -> Tuple[SymbolicShape, ...]:
        return tuple(self._in)

    @property
    def output_shapes(self) -> Tuple[SymbolicShape, ...]:
        return tuple(self._out)

    saved_tensor_count = property(lambda self: len(self._saved))
    input_shape_count = property(lambda self: len(self._in))
    output_shape_count = property(lambda self: len(self._out))

    def save_for_backward(self, *tensors: torch.Tensor) -> None:
        self._alive()
        for t in tensors:
            if t is None:
                raise ValueError("cannot save None")
            self._saved.append(t)

    def get_saved_tensor(self, index: int) -> torch.Tensor:
        self._alive()
        if not 0 <= index < len(self._saved):
            raise IndexError(f"saved tensor {index} of {len(self._saved)}")
        return self._saved[index]

    def save_input_shape(self, *shapes: SymbolicShape) -> None:
        self._alive()
        self._in.extend(shapes)

    def save_output_shape(self, *shapes: SymbolicShape) -> None:
        self._alive()
        self._out.extend(shapes)

    def get_input_shape(self, index: int) -> SymbolicShape:
        return self._in[index]

    def get_output_shape(self, index: int) -> SymbolicShape:
        return self._out[index]

    def register_gradient_shape(self, index: int, shape: SymbolicShape) -> None:
        self._alive()
        if index < 0:
            raise IndexError("gradient index must be non-negative")
        self._grad[index] = shape

    def get_gradient_shape(self, index: int) -> SymbolicShape:
        if index not in self._grad:
            raise KeyError(f"no gradient shape registered for output {index}")
        return self._grad[index]

    def validate_gradient(self, index: int, grad_shape) -> None:
        """``grad_shape`` (symbolic or concrete) must be an instance of the registered shape."""
        want = self.get_gradient_shape(index)
        ok = want == grad_shape if isinstance(grad_shape, SymbolicShape) else matches(want, tuple(grad_shape))
        if not ok:
            raise ValueError(f"gradient {index} has shape {list(grad_shape) if not isinstance(grad_shape, SymbolicShape) else grad_shape}, expected {want}")

    def clear(self) -> None:
        self._saved.clear(); self._in.clear(); self._out.clear(); self._grad.clear()

    def dispose(self) -> None:
        self.clear()
        self._disposed = True

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.dispose()

    def __repr__(self):
        return f"DynamicAutogradContext(saved={len(self._saved)}, inputs={self._in}, outputs={self._out})"


class DynamicGradientTensor:
    """A tensor with its symbolic shape and an accumulated gradient that must keep that shape."""

    def __init__(self, tensor: torch.Tensor, shape: SymbolicShape, gradient_required: bool = True,
                 gradient: Optional[torch.Tensor] = None):
        if not matches(shape, tuple(tensor.shape)):
            raise ValueError(f"tensor of shape {list(tensor.shape)} is not an instance of {shape}")
        self.tensor, self.shape, self.gradient_required = tensor, shape, gradient_required
        self._gradient = gradient

    @property
    def gradient(self) -> Optional[torch.Tensor]:
        return self._gradient

    @property
    def has_gradient(self) -> bool:
        return self._gradient is not None

    def accumulate_gradient(self, grad: torch.Tensor) -> None:
        if not self.gradient_required:
            raise RuntimeError("this tensor does not require a gradient")
        if tuple(grad.shape) != tuple(self.tensor.shape):
            raise ValueError(f"gradient of shape {list(grad.shape)} for a tensor of shape {list(self.tensor.shape)} ({self.shape})")
        self._gradient = grad.clone() if self._gradient is None else self._gradient + grad

    def get_gradient(self) -> Optional[torch.Tensor]:
        return self._gradient

    def clear_gradient(self) -> None:
        self._gradient = None

    reset = clear_gradient

    def detach(self) -> "DynamicGradientTensor":
        return DynamicGradientTensor(self.tensor.detach(), self.shape, False)

    def __repr__(self):
        return f"DynamicGradientTensor(shape={self.shape}, requires_grad={self.gradient_required}, has_grad={self.has_gradient})"


class _Bridge(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, n_inputs, *inputs):
        ctx.fn = fn
        ctx.is_tensor = [isinstance(x, torch.Tensor) for x in inputs]
        ctx.others = [None if t else x for t, x in zip(ctx.is_tensor, inputs)]
        ctx.save_for_backward(*[x for x in inputs if isinstance(x, torch.Tensor)])
        with torch.no_grad():
            out = fn.forward(*inputs)
        ctx.out_shape = tuple(out.shape)
        return out

    @staticmethod
    def backward(ctx, grad):
        fn = ctx.fn
        if tuple(grad.shape) != ctx.out_shape:
            raise ValueError(f"{fn.operation_name}: gradient of shape {list(grad.shape)}, output was {list(ctx.out_shape)}")
        fn.validate_gradient_shape(tuple(grad.shape))
        saved = iter(ctx.saved_tensors)
        inputs = [next(saved) if t else o for t, o in zip(ctx.is_tensor, ctx.others)]
        grads = list(fn.compute_grad(grad, inputs))
        grads += [None] * (len(inputs) - len(grads))
        out = []
        for i, (g, x) in enumerate(zip(grads, inputs)):
            wanted = ctx.needs_input_grad[2 + i] and isinstance(x, torch.Tensor) and x.is_floating_point()
            out.append(g if (g is not None and wanted) else None)
        return (None, None, *out)


class DynamicGradientFunction:
    """Shape rule + forward + gradient rule of one operation."""

    operation_name = "dynamic"

    def get_output_shape(self, input_shapes: Sequence[SymbolicShape]) -> SymbolicShape:
        raise NotImplementedError

    def get_output_shapes(self, input_shapes: Sequence[SymbolicShape]) -> List[SymbolicShape]:
        return [self.get_output_shape(input_shapes)]

    def expected_gradient_shape(self) -> Optional[SymbolicShape]:
        return None

    def validate_gradient_shape(self, gradient_shape) -> None:
        want = self.expected_gradient_shape()
        if gradient_shape is None:
            raise ValueError("the gradient shape is required")
        if want is None:
            return
        ok = want == gradient_shape if isinstance(gradient_shape, SymbolicShape) else matches(want, tuple(gradient_shape))
        if not ok:
            shown = gradient_shape if isinstance(gradient_shape, SymbolicShape) else list(gradient_shape)
            raise ValueError(f"{self.operation_name}: gradient shape {shown} does not match {want}")

    def forward(self, *inputs: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def compute_grad(self, grad_output: torch.Tensor, inputs: Sequence[torch.Tensor], context=None) -> List[Optional[torch.Tensor]]:
        raise NotImplementedError

    def __call__(self, *inputs: torch.Tensor) -> torch.Tensor:
        return _Bridge.apply(self, len(inputs), *inputs)

    @staticmethod
    def _need(input_shapes, n: int, name: str):
        if input_shapes is None or len(input_shapes) != n:
            raise ValueError(f"{name} requires exactly {n} input shape{'s' if n != 1 else ''}")


class DynamicSlice(DynamicGradientFunction):
    """``x[start : start + size]`` per dimension; the gradient is the slice's gradient set into zeros of
    the input's shape."""

    operation_name = "DynamicSlice"

    def __init__(self, start_indices: Sequence[int], slice_shape: SymbolicShape):
        if not len(start_indices):
            raise ValueError("start indices must be non-empty")
        if slice_shape is None or slice_shape.rank != len(start_indices):
            raise ValueError("the slice shape needs one dimension per start index")
        self.start_indices, self.slice_shape = [int(s) for s in start_indices], slice_shape

    def get_output_shape(self, input_shapes):
        self._need(input_shapes, 1, self.operation_name)
        if input_shapes[0].rank != self.slice_shape.rank:
            raise ValueError(f"{self.operation_name}: input rank {input_shapes[0].rank}, slice rank {self.slice_shape.rank}")
        return self.slice_shape

    def expected_gradient_shape(self):
        return self.slice_shape

    def _index(self, x: torch.Tensor):
        sizes = []
        for d, (start, dim) in enumerate(zip(self.start_indices, self.slice_shape.dims)):
            size = dim.value if dim.is_known else x.shape[d] - start          # an unknown extent runs to the end
            if start < 0 or size < 0 or start + size > x.shape[d]:
                raise IndexError(f"{self.operation_name}: [{start}, {start + size}) is outside dimension {d} of size {x.shape[d]}")
            sizes.append(size)
        return tuple(slice(s, s + n) for s, n in zip(self.start_indices, sizes))

    def forward(self, x):
        return x[self._index(x)].clone()

    def compute_grad(self, grad_output, inputs, context=None):
        x = inputs[0]
        dx = torch.zeros_like(x, dtype=grad_output.dtype)
        dx[self._index(x)] = grad_output
        return [dx]


class DynamicPad(DynamicGradientFunction):
    """Zero padding ``(before_0, after_0, before_1, after_1, ...)`` in dimension order; the gradient is
    the interior of the output's gradient."""

    operation_name = "DynamicPad"

    def __init__(self, padding: Sequence[int], target_shape: Optional[SymbolicShape] = None):
        if not len(padding) or len(padding) % 2:
            raise ValueError("padding needs a (before, after) pair per padded dimension")
        if any(p < 0 for p in padding):
            raise ValueError("padding cannot be negative")
        self.padding, self.target_shape = [int(p) for p in padding], target_shape

    def get_output_shape(self, input_shapes):
        self._need(input_shapes, 1, self.operation_name)
        s = input_shapes[0]
        if s.rank < len(self.padding) // 2:
            raise ValueError(f"{self.operation_name}: {len(self.padding) // 2} padded dimensions for rank {s.rank}")
        if self.target_shape is not None:
            return self.target_shape
        dims = []
        for i, d in enumerate(s.dims):
            extra = self.padding[2 * i] + self.padding[2 * i + 1] if 2 * i + 1 < len(self.padding) else 0
            if d.is_known:
                dims.append(d.value + extra)
            else:
                dims.append(d if extra == 0 else SymbolicDimension(f"{d.name}+{extra}", None, d.min_value + extra,
                                                                   None if d.max_value is None else d.max_value + extra))
        return SymbolicShape(dims)

    def expected_gradient_shape(self):
        return self.target_shape

    def _torch_pad(self, rank: int) -> List[int]:
        pairs = [(self.padding[2 * i], self.padding[2 * i + 1]) if 2 * i + 1 < len(self.padding) else (0, 0) for i in range(rank)]
        flat: List[int] = []
        for b, a in reversed(pairs):                       # torch pads from the last dimension backwards
            flat += [b, a]
        return flat

    def forward(self, x):
        return F.pad(x, self._torch_pad(x.dim()))

    def compute_grad(self, grad_output, inputs, context=None):
        x = inputs[0]
        idx = tuple(slice(self.padding[2 * i], self.padding[2 * i] + x.shape[i]) if 2 * i + 1 < len(self.padding) else slice(None)
                    for i in range(x.dim()))
        return [grad_output[idx].clone()]


class DynamicMask(DynamicGradientFunction):
    """Zeroes positions at or beyond each row's length along the sequence axis (axis 1):
    ``forward(x [B, S, ...], lengths [B])``. The gradient passes where the mask is one."""

    operation_name = "DynamicMask"

    def __init__(self, sequence_length: SymbolicDimension):
        if sequence_length is None:
            raise ValueError("the sequence-length dimension is required")
        self.sequence_length = sequence_length

    def get_output_shape(self, input_shapes):
        if input_shapes is None or len(input_shapes) not in (1, 2):
            raise ValueError(f"{self.operation_name} requires the input shape (and optionally the lengths' shape)")
        s = input_shapes[0]
        if s.rank < 2:
            raise ValueError(f"{self.operation_name}: the input needs a batch and a sequence axis")
        return s

    @staticmethod
    def mask(x: torch.Tensor, lengths: torch.Tensor) -> torch.Tensor:
        pos = torch.arange(x.shape[1], device=x.device)
        m = pos[None, :] < lengths.to(x.device)[:, None]
        return m.view(*m.shape, *([1] * (x.dim() - 2)))

    def forward(self, x, lengths):
        if self.sequence_length.is_known and x.shape[1] != self.sequence_length.value:
            raise ValueError(f"{self.operation_name}: sequence axis is {x.shape[1]}, expected {self.sequence_length.value}")
        if self.sequence_length.max_value is not None and x.shape[1] > self.sequence_length.max_value:
            raise ValueError(f"{self.operation_name}: sequence axis {x.shape[1]} exceeds {self.sequence_length.max_value}")
        return x * self.mask(x, lengths).to(x.dtype)

    def compute_grad(self, grad_output, inputs, context=None):
        x, lengths = inputs
        return [grad_output * self.mask(x, lengths).to(grad_output.dtype), None]


class DynamicGather(DynamicGradientFunction):
    """``index_select`` along ``axis`` with a 1-D index tensor; the gradient scatter-adds back (repeated
    indices accumulate)."""

    operation_name = "DynamicGather"

    def __init__(self, axis: int):
        self.axis = int(axis)

    def get_output_shape(self, input_shapes):
        self._need(input_shapes, 2, self.operation_name)
        data, idx = input_shapes
        if idx.rank != 1:
            raise ValueError(f"{self.operation_name}: indices must be one-dimensional")
        ax = self.axis % data.rank if -data.rank <= self.axis < data.rank else None
        if ax is None:
            raise ValueError(f"{self.operation_name}: axis {self.axis} out of range for rank {data.rank}")
        dims = list(data.dims)
        dims[ax] = idx.dims[0]
        return SymbolicShape(dims)

    def forward(self, x, index):
        return x.index_select(self.axis, index)

    def compute_grad(self, grad_output, inputs, context=None):
        x, index = inputs
        dx = torch.zeros_like(x, dtype=grad_output.dtype)
        dx.index_add_(self.axis % x.dim(), index, grad_output)
        return [dx, None]


class DynamicBroadcastBackward(DynamicGradientFunction):
    """Broadcast of ``input_shape`` to ``output_shape``; the gradient sums over the broadcast axes
    (given, or found by aligning the shapes from the right)."""

    operation_name = "Broadcast"

    def __init__(self, input_shape: SymbolicShape, output_shape: SymbolicShape, broadcast_axes: Optional[Sequence[int]] = None):
        if input_shape is None or output_shape is None:
            raise ValueError("input and output shapes are required")
        if input_shape.rank > output_shape.rank:
            raise ValueError("a broadcast cannot lower the rank")
        self.input_shape, self.output_shape = input_shape, output_shape
        self.broadcast_axes = list(broadcast_axes) if broadcast_axes is not None else self._axes()

    def _axes(self) -> List[int]:
        lead = self.output_shape.rank - self.input_shape.rank
        axes = list(range(lead))
        for i, d in enumerate(self.input_shape.dims):
            o = self.output_shape.dims[lead + i]
            if d.is_known and d.value == 1 and not (o.is_known and o.value == 1):
                axes.append(lead + i)
        return axes

    def get_output_shape(self, input_shapes):
        self._need(input_shapes, 1, self.operation_name)
        return self.output_shape

    def expected_gradient_shape(self):
        return self.output_shape

    def forward(self, x, like: Optional[torch.Tensor] = None):
        target = tuple(like.shape) if like is not None else self.output_shape.concrete()
        return x.expand(target).clone()

    def compute_grad(self, grad_output, inputs, context=None):
        x = inputs[0]
        lead = grad_output.dim() - x.dim()
        g = grad_output
        keep = [a for a in self.broadcast_axes if a >= lead]
        if keep:
            g = g.sum(dim=keep, keepdim=True)
        if lead:
            g = g.sum(dim=list(range(lead)))
        return [g.reshape(x.shape)] + [None] * (len(inputs) - 1)


class DynamicReshapeBackward(DynamicGradientFunction):
    """Reshape to ``new_shape`` (one entry may be -1); the gradient is reshaped back to the original
    shape, whose element count the incoming gradient must have."""

    operation_name = "Reshape"

    def __init__(self, original_shape: SymbolicShape, new_shape: Optional[Sequence[int]] = None):
        if original_shape is None:
            raise ValueError("the original shape is required")
        self.original_shape, self.new_shape = original_shape, None if new_shape is None else tuple(new_shape)

    def get_output_shape(self, input_shapes):
        self._need(input_shapes, 1, self.operation_name)
        if self.new_shape is None:
            return input_shapes[0]
        s = input_shapes[0]
        if -1 in self.new_shape and s.is_fully_known:
            total = 1
            for d in s.concrete():
                total *= d
            rest = 1
            for d in self.new_shape:
                rest *= d if d != -1 else 1
            return SymbolicShape([total // rest if d == -1 else d for d in self.new_shape])
        return SymbolicShape([SymbolicDimension("inferred") if d == -1 else d for d in self.new_shape])

    def validate_gradient_shape(self, gradient_shape) -> None:
        if gradient_shape is None:
            raise ValueError("the gradient shape is required")
        if self.original_shape.is_fully_known and not isinstance(gradient_shape, SymbolicShape):
            n = 1
            for d in gradient_shape:
                n *= int(d)
            m = 1
            for d in self.original_shape.concrete():
                m *= d
            if n != m:
                raise ValueError(f"{self.operation_name}: gradient has {n} elements, the original shape {self.original_shape} has {m}")

    def forward(self, x):
        if not matches(self.original_shape, tuple(x.shape)):
            raise ValueError(f"{self.operation_name}: input {list(x.shape)} is not an instance of {self.original_shape}")
        return x.reshape(self.new_shape if self.new_shape is not None else x.shape).clone()

    def compute_grad(self, grad_output, inputs, context=None):
        return [grad_output.reshape(inputs[0].shape)]


class DynamicMatMulBackward(DynamicGradientFunction):
    """``a @ b`` with batch dimensions broadcast; ``dA = dC @ B^T`` and ``dB = A^T @ dC``, each summed
    back over the batch axes its operand was broadcast along."""

    operation_name = "MatMul"

    def get_output_shape(self, input_shapes):
        self._need(input_shapes, 2, self.operation_name)
        a, b = input_shapes
        if a.rank < 2 or b.rank < 2:
            raise ValueError(f"{self.operation_name}: both operands need at least two dimensions")
        ka, kb = a.dims[-1], b.dims[-2]
        if ka.is_known and kb.is_known and ka.value != kb.value:
            raise ValueError(f"{self.operation_name}: inner dimensions {ka} and {kb} differ")
        if not ka.is_known and not kb.is_known and ka.name != kb.name:
            raise ValueError(f"{self.operation_name}: inner dimensions {ka.name} and {kb.name} are different symbols")
        from ..compiler.shapes import broadcast_shapes
        batch = broadcast_shapes(SymbolicShape(a.dims[:-2]), SymbolicShape(b.dims[:-2]))
        return SymbolicShape([*batch.dims, a.dims[-2], b.dims[-1]])

    def forward(self, a, b):
        return a @ b

    @staticmethod
    def _unbroadcast(g: torch.Tensor, shape) -> torch.Tensor:
        lead = g.dim() - len(shape)
        if lead:
            g = g.sum(dim=list(range(lead)))
        axes = [i for i, (gs, s) in enumerate(zip(g.shape, shape)) if s == 1 and gs != 1]
        return g.sum(dim=axes, keepdim=True) if axes else g

    def compute_grad(self, grad_output, inputs, context=None):
        a, b = inputs
        da = self._unbroadcast(grad_output @ b.transpose(-1, -2).to(grad_output.dtype), a.shape)
        db = self._unbroadcast(a.transpose(-1, -2).to(grad_output.dtype) @ grad_output, b.shape)
        return [da, db]


def _pair(v) -> Tuple[int, int]:
    return (int(v[0]), int(v[1])) if isinstance(v, (tuple, list)) else (int(v), int(v))


class DynamicConv2DBackward(DynamicGradientFunction):
    """2-D convolution of [N, C, H, W] (any of N, H, W symbolic) with [O, C, kh, kw]; gradients for the
    input, the kernel and the optional bias."""

    operation_name = "Conv2D"

    def __init__(self, kernel_size, stride=1, padding=0, dilation=1):
        self.kernel_size, self.stride = _pair(kernel_size), _pair(stride)
        self.padding, self.dilation = _pair(padding), _pair(dilation)
        if min(self.kernel_size) <= 0 or min(self.stride) <= 0 or min(self.dilation) <= 0 or min(self.padding) < 0:
            raise ValueError("kernel, stride and dilation must be positive and padding non-negative")

    def _out(self, d: SymbolicDimension, i: int):
        k, s, p, dl = self.kernel_size[i], self.stride[i], self.padding[i], self.dilation[i]
        f = lambda n: (n + 2 * p - dl * (k - 1) - 1) // s + 1                     # noqa: E731
        if d.is_known:
            if f(d.value) <= 0:
                raise ValueError(f"{self.operation_name}: extent {d.value} is too small for kernel {k} (dilation {dl}, padding {p})")
            return f(d.value)
        return SymbolicDimension(f"conv({d.name})", None, max(1, f(d.min_value)), None if d.max_value is None else f(d.max_value))

    def get_output_shape(self, input_shapes):
        if input_shapes is None or len(input_shapes) not in (2, 3):
            raise ValueError(f"{self.operation_name} requires the input and kernel shapes (and optionally the bias shape)")
        x, w = input_shapes[0], input_shapes[1]
        if x.rank != 4 or w.rank != 4:
            raise ValueError(f"{self.operation_name}: input and kernel must have four dimensions")
        if x.dims[1].is_known and w.dims[1].is_known and x.dims[1].value != w.dims[1].value:
            raise ValueError(f"{self.operation_name}: input channels {x.dims[1]} do not match kernel channels {w.dims[1]}")
        for i in (0, 1):
            if w.dims[2 + i].is_known and w.dims[2 + i].value != self.kernel_size[i]:
                raise ValueError(f"{self.operation_name}: kernel shape {w} disagrees with kernel size {self.kernel_size}")
        return SymbolicShape([x.dims[0], w.dims[0], self._out(x.dims[2], 0), self._out(x.dims[3], 1)])

    def forward(self, x, w, bias=None):
        return F.conv2d(x, w, bias, self.stride, self.padding, self.dilation)

    def compute_grad(self, grad_output, inputs, context=None):
        x, w = inputs[0], inputs[1]
        g = grad_output
        dx = torch.nn.grad.conv2d_input(x.shape, w.to(g.dtype), g, self.stride, self.padding, self.dilation)
        dw = torch.nn.grad.conv2d_weight(x.to(g.dtype), w.shape, g, self.stride, self.padding, self.dilation)
        out: List[Optional[torch.Tensor]] = [dx, dw]
        if len(inputs) > 2:
            out.append(g.sum(dim=(0, 2, 3)) if inputs[2] is not None else None)
        return out
