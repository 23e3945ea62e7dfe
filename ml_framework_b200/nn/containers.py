"""Containers and module-tree utilities: editable sequential container, hierarchical access by path, wrappers,
parameter gradient hooks that fire, and the 2-D convolution layer.

Reference: src/MLFramework/NN/{SequentialModule.cs:20-155 (add / insert / remove / get), HierarchicalModule.cs:16-176
(named children, replace child, module container), HierarchicalWrapper.cs:19-226 (any module as a tree node with a
parent), Parameter.cs:41-67 (gradient hooks, stored but never invoked there)}, src/MLFramework/Modules/Conv2d.cs.
The tree is PyTorch's own module tree; these helpers give it the reference's vocabulary and add what is missing
(paths, parents, replacement by path). Hooks are installed with ``register_post_accumulate_grad_hook`` /
``register_hook`` and therefore run during backward.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class SequentialModule(nn.Module):
    """An ordered list of modules applied one after the other, editable in place."""

    def __init__(self, modules: Iterable[nn.Module] = (), name: str = "Sequential"):
        super().__init__()
        self.name = name
        self.layers = nn.ModuleList(list(modules))

    @property
    def count(self) -> int:
        return len(self.layers)

    def add(self, module: nn.Module) -> "SequentialModule":
        if not isinstance(module, nn.Module):
            raise TypeError("expected a module")
        self.layers.append(module)
        return self

    add_module_fluent = add

    def insert(self, index: int, module: nn.Module):
        if not (0 <= index <= len(self.layers)):
            raise IndexError(f"index {index} outside [0, {len(self.layers)}]")
        self.layers.insert(index, module)

    def get_module(self, index: int) -> nn.Module:
        return self.layers[index]

    def get_modules(self) -> List[nn.Module]:
        return list(self.layers)

    def remove_at(self, index: int) -> nn.Module:
        if not (0 <= index < len(self.layers)):
            raise IndexError(f"index {index} outside [0, {len(self.layers)})")
        m = self.layers[index]
        del self.layers[index]
        return m

    def clear(self):
        self.layers = nn.ModuleList()

    def forward(self, x):
        for m in self.layers:
            x = m(x)
        return x

    def __len__(self):
        return len(self.layers)

    def __iter__(self) -> Iterator[nn.Module]:
        return iter(self.layers)


# ------------------------------------------------------------------ tree access
def get_child(root: nn.Module, path: str) -> nn.Module:
    """Sub-module by dotted path (``"blocks.3.attn"``); the empty path is the root."""
    m = root
    for part in filter(None, path.split(".")):
        if part not in m._modules:
            raise KeyError(f"{type(m).__name__} has no child {part!r} (path {path!r})")
        m = m._modules[part]
    return m


def replace_child(root: nn.Module, path: str, new: nn.Module) -> nn.Module:
    """Replaces the sub-module at ``path``; returns the old one."""
    if not path:
        raise ValueError("the root cannot be replaced")
    parent_path, _, leaf = path.rpartition(".")
    parent = get_child(root, parent_path)
    if leaf not in parent._modules:
        raise KeyError(f"no child {leaf!r} under {parent_path or '<root>'}")
    old = parent._modules[leaf]
    parent._modules[leaf] = new
    return old


def parent_of(root: nn.Module, path: str) -> Optional[nn.Module]:
    return None if not path else get_child(root, path.rpartition(".")[0])


def depth_of(path: str) -> int:
    return 0 if not path else path.count(".") + 1


def walk(root: nn.Module, max_depth: Optional[int] = None) -> Iterator[Tuple[str, nn.Module, int]]:
    """(path, module, depth) in pre-order."""
    for n, m in root.named_modules():
        d = depth_of(n)
        if max_depth is None or d <= max_depth:
            yield n, m, d


def set_requires_grad(root: nn.Module, flag: bool, path: str = "") -> int:
    n = 0
    for p in get_child(root, path).parameters():
        p.requires_grad_(flag)
        n += 1
    return n


class HierarchicalWrapper(nn.Module):
    """Any module as a named tree node with a parent pointer and children that can be added or replaced by name."""

    def __init__(self, module: nn.Module, name: str):
        super().__init__()
        self.module, self.name = module, name
        self._parent: List[Optional["HierarchicalWrapper"]] = [None]     # in a list: not a registered sub-module
        self.extra = nn.ModuleDict()

    @property
    def module_type(self) -> str:
        return type(self.module).__name__

    @property
    def parent(self) -> Optional["HierarchicalWrapper"]:
        return self._parent[0]

    @property
    def path(self) -> str:
        return self.name if self.parent is None else f"{self.parent.path}.{self.name}"

    def children_nodes(self) -> List["HierarchicalWrapper"]:
        return list(self.extra.values())

    def add_child(self, child: "HierarchicalWrapper"):
        if child.name in self.extra:
            raise KeyError(f"{self.name} already has a child {child.name!r}")
        child._parent[0] = self
        self.extra[child.name] = child

    def get_child(self, name: str) -> "HierarchicalWrapper":
        if name not in self.extra:
            raise KeyError(f"{self.name} has no child {name!r}")
        return self.extra[name]

    def replace_child(self, name: str, new: "HierarchicalWrapper"):
        if name not in self.extra:
            raise KeyError(f"{self.name} has no child {name!r}")
        self.extra[name]._parent[0] = None
        new._parent[0] = self
        new.name = name
        self.extra[name] = new

    def forward(self, *a, **k):
        return self.module(*a, **k)


class ModuleContainer(HierarchicalWrapper):
    """A node without a computation of its own: forward runs its children in insertion order."""

    def __init__(self, name: str):
        super().__init__(nn.Identity(), name)

    def forward(self, x):
        for c in self.extra.values():
            x = c(x)
        return x


# ------------------------------------------------------------------ gradient hooks
class GradientHookRegistry:
    """``register(param, hook)``: ``hook(grad) -> grad or None`` runs when autograd produces the parameter's gradient
    (before accumulation; a returned tensor replaces it). ``register_ready(param, fn)``: ``fn(param)`` runs after the
    gradient was accumulated into ``param.grad`` - what bucketed gradient reduction listens to."""

    def __init__(self):
        self._handles: Dict[int, List] = {}
        self._names: Dict[int, str] = {}

    def register(self, param: torch.Tensor, hook: Callable[[torch.Tensor], Optional[torch.Tensor]], name: str = ""):
        if not param.requires_grad:
            raise ValueError("parameter does not require grad")
        self._handles.setdefault(id(param), []).append(param.register_hook(hook))
        self._names[id(param)] = name

    def register_ready(self, param: torch.Tensor, fn: Callable[[torch.Tensor], None], name: str = ""):
        if not param.requires_grad:
            raise ValueError("parameter does not require grad")
        self._handles.setdefault(id(param), []).append(param.register_post_accumulate_grad_hook(fn))
        self._names[id(param)] = name

    def has_hook(self, param: torch.Tensor) -> bool:
        return bool(self._handles.get(id(param)))

    def remove(self, param: torch.Tensor) -> int:
        hs = self._handles.pop(id(param), [])
        for h in hs:
            h.remove()
        self._names.pop(id(param), None)
        return len(hs)

    def clear(self):
        for hs in self._handles.values():
            for h in hs:
                h.remove()
        self._handles.clear()
        self._names.clear()

    def __len__(self):
        return sum(len(v) for v in self._handles.values())


# ------------------------------------------------------------------ conv layer
class Conv2d(nn.Module):
    """2-D convolution, weight ``[out, in / groups, kh, kw]``, Kaiming-uniform initialisation like ``Linear``. Runs
    cuDNN through PyTorch (convolutions are outside this package's transformer hot paths; the direct fp32 kernel of
    the mobile runtime serves inference there)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1, groups: int = 1, bias: bool = True,
                 dtype=None, device=None):
        super().__init__()
        if in_channels % groups or out_channels % groups:
            raise ValueError("channels must be divisible by groups")
        k = (kernel_size, kernel_size) if isinstance(kernel_size, int) else tuple(kernel_size)
        self.in_channels, self.out_channels, self.kernel_size = in_channels, out_channels, k
        self.stride, self.padding, self.dilation, self.groups = stride, padding, dilation, groups
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels // groups, *k, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_channels, dtype=dtype, device=device)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        with torch.no_grad():
            nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
            if self.bias is not None:
                self.bias.zero_()

    def output_shape(self, h: int, w: int) -> Tuple[int, int]:
        def one(n, k, s, p, d):
            return (n + 2 * p - d * (k - 1) - 1) // s + 1
        s = (self.stride, self.stride) if isinstance(self.stride, int) else self.stride
        p = (self.padding, self.padding) if isinstance(self.padding, int) else self.padding
        d = (self.dilation, self.dilation) if isinstance(self.dilation, int) else self.dilation
        return one(h, self.kernel_size[0], s[0], p[0], d[0]), one(w, self.kernel_size[1], s[1], p[1], d[1])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() != 4 or x.shape[1] != self.in_channels:
            raise ValueError(f"expected [N, {self.in_channels}, H, W], got {tuple(x.shape)}")
        return F.conv2d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)
