"""Transfer learning: heads, freezing, layer selection, parameter groups, layer-wise rates.

Reference: src/ModelZoo/TransferLearning — HeadAdapter.cs:19-255, HeadBuilder.cs:12-338,
HeadExtensions.cs:20-243, WeightInitializationStrategy.cs:8-85, FreezeExtensions.cs:12-305,
LayerSelectionHelper.cs:12-236, ParameterGroup.cs:10-169, ParameterGroupBuilder.cs:13-394,
LayerWiseLrScheduler.cs:11-520, LayerWiseLrExtensions.cs:13-339,
GradualUnfreezingScheduler.cs:12-242.

A "layer" is a leaf of the container tree: ``nn.Sequential`` and ``nn.ModuleList`` are looked
through, any other child module counts as one layer under its dotted name. The convolutional,
pooling and attention heads, which the reference stands in for with linear layers, are real
here. Frozen means ``requires_grad == False`` on every parameter of the layer.
"""
from __future__ import annotations

import enum
import math
import re
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple, Type

import torch
import torch.nn as nn

__all__ = [
    "WeightInitializationStrategy", "initialize_weights", "LinearHead", "MLPHead", "ConvHead",
    "AdaptiveAvgPoolHead", "AttentionHead", "HeadBuilder", "HeadAdapter", "HeadAdapterError",
    "HeadReplacementError", "remove_last_layer", "remove_last_n_layers", "add_head", "replace_head",
    "get_head", "get_heads", "head_input_dimension", "validate_head_replacement", "head_summary",
    "layers", "LayerSelection", "freeze", "unfreeze", "freeze_except_last", "freeze_by_name",
    "unfreeze_by_name", "freeze_by_pattern", "unfreeze_by_pattern", "frozen_layers", "unfrozen_layers",
    "FrozenStateSummary", "frozen_state_summary", "ParameterGroup", "ParameterGroupBuilder",
    "ScheduleType", "LayerWiseLrScheduler", "set_layer_wise_lrs", "clear_layer_wise_lrs",
    "apply_parameter_groups", "parameter_groups_of", "create_discriminative_groups",
    "GradualUnfreezingScheduler",
]


# ------------------------------------------------------------------ weight initialisation
class WeightInitializationStrategy(enum.Enum):
    XAVIER = "xavier"
    KAIMING = "kaiming"
    UNIFORM = "uniform"
    NORMAL = "normal"
    TRUNCATED_NORMAL = "truncated_normal"
    ORTHOGONAL = "orthogonal"

    def default_parameters(self) -> Tuple[float, float]:
        """(gain, std) of WeightInitializationStrategy.cs:54-67."""
        if self in (WeightInitializationStrategy.XAVIER, WeightInitializationStrategy.ORTHOGONAL):
            return 1.0, 1.0
        if self is WeightInitializationStrategy.KAIMING:
            return math.sqrt(2.0), 1.0
        return 1.0, 0.02

    def is_recommended_for(self, activation: str) -> bool:
        a = activation.lower()
        if self is WeightInitializationStrategy.XAVIER:
            return a in ("sigmoid", "tanh", "tanh_shrink")
        if self is WeightInitializationStrategy.KAIMING:
            return "relu" in a or a == "elu"
        return True


def initialize_weights(module: nn.Module, strategy: WeightInitializationStrategy,
                       generator: Optional[torch.Generator] = None) -> None:
    """Re-draws every weight matrix of ``module`` by ``strategy``; biases and vectors become zero
    (norm scales become one)."""
    gain, std = strategy.default_parameters()
    S = WeightInitializationStrategy
    with torch.no_grad():
        for m in module.modules():
            if isinstance(m, (nn.LayerNorm, nn.BatchNorm1d, nn.BatchNorm2d, nn.GroupNorm)):
                if m.weight is not None:
                    m.weight.fill_(1.0)
                if m.bias is not None:
                    m.bias.zero_()
                continue
            for name, p in m.named_parameters(recurse=False):
                if p.dim() < 2:
                    p.zero_()
                elif strategy is S.XAVIER:
                    nn.init.xavier_uniform_(p, gain=gain, generator=generator)
                elif strategy is S.KAIMING:
                    nn.init.kaiming_normal_(p, nonlinearity="relu", generator=generator)
                elif strategy is S.UNIFORM:
                    nn.init.uniform_(p, -std, std, generator=generator)
                elif strategy is S.NORMAL:
                    nn.init.normal_(p, 0.0, std, generator=generator)
                elif strategy is S.TRUNCATED_NORMAL:
                    nn.init.trunc_normal_(p, 0.0, std, -2 * std, 2 * std, generator=generator)
                else:
                    nn.init.orthogonal_(p, gain=gain, generator=generator)


# ------------------------------------------------------------------ heads
class LinearHead(nn.Module):
    """Affine classifier, optionally behind dropout (HeadBuilder.cs:12-118)."""

    def __init__(self, input_dim: int, output_dim: int, bias: bool = True, dropout: float = 0.0):
        super().__init__()
        if input_dim <= 0 or output_dim <= 0:
            raise ValueError("head dimensions must be positive")
        self.input_dim, self.output_dim = input_dim, output_dim
        self.drop = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        self.fc = nn.Linear(input_dim, output_dim, bias=bias)

    def forward(self, x):
        return self.fc(self.drop(x))

    def initialize_weights(self, strategy: WeightInitializationStrategy, generator=None):
        initialize_weights(self, strategy, generator)


class MLPHead(nn.Module):
    """Linear / ReLU stack ending in a linear layer (HeadBuilder.cs:124-180)."""

    def __init__(self, input_dim: int, hidden_dims: Sequence[int], output_dim: int):
        super().__init__()
        dims = [input_dim, *hidden_dims]
        if any(d <= 0 for d in dims) or output_dim <= 0:
            raise ValueError("head dimensions must be positive")
        body: List[nn.Module] = []
        for a, b in zip(dims[:-1], dims[1:]):
            body += [nn.Linear(a, b), nn.ReLU()]
        self.input_dim, self.output_dim = input_dim, output_dim
        self.net = nn.Sequential(*body, nn.Linear(dims[-1], output_dim))

    def forward(self, x):
        return self.net(x)

    def initialize_weights(self, strategy: WeightInitializationStrategy, generator=None):
        initialize_weights(self, strategy, generator)


class ConvHead(nn.Module):
    """Conv / BatchNorm / ReLU stages over [B, C, H, W], global average pool, linear classifier."""

    def __init__(self, input_channels: int, num_classes: int, kernel_sizes: Sequence[int] = (3,),
                 width: Optional[int] = None):
        super().__init__()
        width = width or input_channels
        stages, c = [], input_channels
        for k in kernel_sizes:
            stages += [nn.Conv2d(c, width, k, padding=k // 2, bias=False), nn.BatchNorm2d(width), nn.ReLU()]
            c = width
        self.input_dim, self.output_dim = input_channels, num_classes
        self.features = nn.Sequential(*stages)
        self.fc = nn.Linear(c, num_classes)

    def forward(self, x):
        return self.fc(self.features(x).mean(dim=(2, 3)))


class AdaptiveAvgPoolHead(nn.Module):
    """Pools [B, C, H, W] to ``output_size`` x ``output_size`` cells and classifies the flattened cells."""

    def __init__(self, channels: int, output_size: int, num_classes: int):
        super().__init__()
        self.input_dim, self.output_dim = channels, num_classes
        self.pool = nn.AdaptiveAvgPool2d(output_size)
        self.fc = nn.Linear(channels * output_size * output_size, num_classes)

    def forward(self, x):
        return self.fc(self.pool(x).flatten(1))


class AttentionHead(nn.Module):
    """One learned query attends over the tokens [B, T, D]; the pooled vector is classified."""

    def __init__(self, input_dim: int, num_classes: int, num_heads: int = 8):
        super().__init__()
        if input_dim % num_heads != 0:
            raise ValueError(f"input dim {input_dim} is not divisible by {num_heads} heads")
        self.input_dim, self.output_dim = input_dim, num_classes
        self.query = nn.Parameter(torch.zeros(1, 1, input_dim))
        self.attn = nn.MultiheadAttention(input_dim, num_heads, batch_first=True)
        self.fc = nn.Linear(input_dim, num_classes)

    def forward(self, x):
        if x.dim() == 2:
            x = x[:, None, :]
        pooled, _ = self.attn(self.query.expand(x.shape[0], -1, -1), x, x, need_weights=False)
        return self.fc(pooled[:, 0])


class HeadBuilder:
    """Factories of HeadBuilder.cs:185-338."""

    @staticmethod
    def linear_head(input_dim, num_classes, include_dropout: bool = False, dropout_rate: float = 0.5):
        return LinearHead(input_dim, num_classes, True, dropout_rate if include_dropout else 0.0)

    @staticmethod
    def mlp_head(input_dim, hidden_dims, output_dim):
        return MLPHead(input_dim, hidden_dims, output_dim)

    @staticmethod
    def conv_head(input_channels, num_classes, kernel_sizes: Optional[Sequence[int]] = None):
        return ConvHead(input_channels, num_classes, tuple(kernel_sizes or (3,)))

    @staticmethod
    def adaptive_avg_pool_head(channels, output_size, num_classes):
        return AdaptiveAvgPoolHead(channels, output_size, num_classes)

    @staticmethod
    def attention_head(input_dim, num_classes, num_heads: int = 8):
        return AttentionHead(input_dim, num_classes, num_heads)

    @staticmethod
    def initialize_head(head: nn.Module, strategy: WeightInitializationStrategy, generator=None):
        initialize_weights(head, strategy, generator)

    @staticmethod
    def create_default_head(input_dim: int, num_classes: int, head_type: str = "linear") -> nn.Module:
        t = head_type.lower()
        if t == "linear":
            return LinearHead(input_dim, num_classes)
        if t == "mlp":
            return MLPHead(input_dim, [max(1, input_dim // 2), max(1, input_dim // 4)], num_classes)
        if t == "conv":
            return ConvHead(input_dim, num_classes)
        if t == "attention":
            heads = next(h for h in (8, 4, 2, 1) if input_dim % h == 0)
            return AttentionHead(input_dim, num_classes, heads)
        raise ValueError(f"unknown head type: {head_type}")


class HeadAdapterError(RuntimeError):
    pass


class HeadReplacementError(RuntimeError):
    pass


def _in_features(m: nn.Module) -> Optional[int]:
    if hasattr(m, "input_dim"):
        return int(m.input_dim)
    for sub in m.modules():
        if isinstance(sub, nn.Linear):
            return sub.in_features
        if isinstance(sub, nn.Conv2d):
            return sub.in_channels
    return None


def _out_features(m: nn.Module) -> Optional[int]:
    if hasattr(m, "output_dim"):
        return int(m.output_dim)
    last = None
    for sub in m.modules():
        if isinstance(sub, nn.Linear):
            last = sub.out_features
    return last


# ---- operations on a sequential model (HeadExtensions.cs:20-243)
def _need_sequential(model) -> nn.Sequential:
    if not isinstance(model, nn.Sequential):
        raise HeadReplacementError(f"expected nn.Sequential, got {type(model).__name__}")
    return model


def remove_last_layer(model: nn.Sequential) -> nn.Module:
    _need_sequential(model)
    if len(model) == 0:
        raise HeadReplacementError("the model has no layers")
    key = list(model._modules)[-1]
    return model._modules.pop(key)


def remove_last_n_layers(model: nn.Sequential, n: int) -> List[nn.Module]:
    _need_sequential(model)
    if n < 0 or n > len(model):
        raise HeadReplacementError(f"cannot remove {n} of {len(model)} layers")
    return [remove_last_layer(model) for _ in range(n)][::-1]


def add_head(model: nn.Sequential, head: nn.Module) -> None:
    _need_sequential(model).append(head)


def replace_head(model: nn.Sequential, new_head: nn.Module) -> nn.Module:
    """Swaps the last layer for ``new_head``; returns the old one."""
    old = remove_last_layer(model)
    model.append(new_head)
    return old


def get_head(model: nn.Sequential) -> Optional[nn.Module]:
    _need_sequential(model)
    return model[-1] if len(model) else None


def get_heads(model: nn.Sequential, max_count: int = 3) -> List[nn.Module]:
    _need_sequential(model)
    return list(model)[-max_count:] if max_count > 0 else []


def head_input_dimension(model: nn.Sequential) -> Optional[int]:
    h = get_head(model)
    return _in_features(h) if h is not None else None


def validate_head_replacement(model: nn.Sequential, new_head: nn.Module, expected_input_dim: Optional[int] = None) -> bool:
    want = expected_input_dim if expected_input_dim is not None else head_input_dimension(model)
    got = _in_features(new_head)
    return want is None or got is None or want == got


def head_summary(model: nn.Sequential) -> str:
    h = get_head(model)
    if h is None:
        return "no head"
    n = sum(p.numel() for p in h.parameters())
    return f"{type(h).__name__}: in={_in_features(h)} out={_out_features(h)} parameters={n}"


class HeadAdapter:
    """Replaces the classification head of a sequential model (HeadAdapter.cs:19-255)."""

    def __init__(self, model: nn.Sequential, input_dim: int = -1):
        _need_sequential(model)
        if len(model) == 0:
            raise HeadAdapterError("the model has no layers")
        self.model = model
        self._original = model[-1]
        self.input_dim = input_dim if input_dim > 0 else (_in_features(model[-1]) or -1)
        self.num_classes = _out_features(model[-1]) or -1

    @property
    def current_head(self) -> nn.Module:
        return self.model[-1]

    def set_number_of_classes(self, num_classes: int, head_type: str = "linear",
                              initialize_strategy: WeightInitializationStrategy = WeightInitializationStrategy.KAIMING):
        if num_classes <= 0:
            raise ValueError("the number of classes must be positive")
        if self.input_dim <= 0:
            raise HeadAdapterError("the head's input dimension is unknown: call set_input_dim first")
        head = HeadBuilder.create_default_head(self.input_dim, num_classes, head_type)
        initialize_weights(head, initialize_strategy)
        self.replace_head(head, validate_dimensions=False)
        self.num_classes = num_classes

    def replace_head(self, new_head: nn.Module, validate_dimensions: bool = True):
        if validate_dimensions and self.input_dim > 0:
            got = _in_features(new_head)
            if got is not None and got != self.input_dim:
                raise HeadAdapterError(f"the new head expects {got} inputs, the body gives {self.input_dim}")
        ref = next(self.model[-1].parameters(), None)
        if ref is not None:
            new_head.to(device=ref.device)
        replace_head(self.model, new_head)
        self.num_classes = _out_features(new_head) or self.num_classes

    def initialize_weights(self, strategy: WeightInitializationStrategy):
        initialize_weights(self.current_head, strategy)

    def set_input_dim(self, input_dim: int):
        if input_dim <= 0:
            raise ValueError("the input dimension must be positive")
        self.input_dim = input_dim

    def reset(self):
        """Puts the head back that the model had when the adapter was made."""
        replace_head(self.model, self._original)
        self.num_classes = _out_features(self._original) or -1

    @classmethod
    def adapt_pretrained(cls, model: nn.Sequential, num_classes: int, head_type: str = "linear",
                         freeze_body: bool = True, input_dim: int = -1) -> "HeadAdapter":
        """New head for ``num_classes``; the body frozen unless told otherwise (HeadAdapter.cs:212-240)."""
        a = cls(model, input_dim)
        a.set_number_of_classes(num_classes, head_type)
        if freeze_body:
            for layer in list(model)[:-1]:
                freeze(layer)
            unfreeze(model[-1])
        return a

    def summary(self) -> str:
        return f"HeadAdapter(input_dim={self.input_dim}, num_classes={self.num_classes}, head={head_summary(self.model)})"


# ------------------------------------------------------------------ layers, selection, freezing
def layers(module: nn.Module, prefix: str = "") -> List[Tuple[str, nn.Module]]:
    """(dotted name, layer) in definition order; sequential and list containers are looked through."""
    out: List[Tuple[str, nn.Module]] = []
    for name, child in module.named_children():
        full = f"{prefix}{name}"
        if isinstance(child, (nn.Sequential, nn.ModuleList)):
            out += layers(child, full + ".")
        else:
            out.append((full, child))
    if not out and not prefix:
        out.append(("", module))
    return out


class LayerSelection:
    """Selectors of LayerSelectionHelper.cs:12-236; each returns [(name, layer)]."""

    @staticmethod
    def by_name(module, *names: str):
        want = set(names)
        return [(n, m) for n, m in layers(module) if n in want]

    @staticmethod
    def by_pattern(module, pattern: str):
        rx = re.compile(pattern)
        return [(n, m) for n, m in layers(module) if rx.search(n)]

    @staticmethod
    def by_index(module, index: int):
        ls = layers(module)
        if not -len(ls) <= index < len(ls):
            raise IndexError(f"layer index {index} out of range for {len(ls)} layers")
        return ls[index]

    @staticmethod
    def by_range(module, start: int, end: int):
        ls = layers(module)
        if start < 0 or end > len(ls) or start > end:
            raise IndexError(f"layer range [{start}, {end}) out of range for {len(ls)} layers")
        return ls[start:end]

    @staticmethod
    def by_type(module, layer_type: Type[nn.Module]):
        return [(n, m) for n, m in layers(module) if isinstance(m, layer_type)]

    @staticmethod
    def last_n(module, count: int):
        if count < 0:
            raise ValueError("count must be non-negative")
        ls = layers(module)
        return ls[len(ls) - min(count, len(ls)):]

    @staticmethod
    def first_n(module, count: int):
        if count < 0:
            raise ValueError("count must be non-negative")
        return layers(module)[:count]

    @staticmethod
    def trainable(module):
        return [(n, m) for n, m in layers(module) if _has_params(m) and not _is_frozen(m)]

    @staticmethod
    def frozen(module):
        return [(n, m) for n, m in layers(module) if _has_params(m) and _is_frozen(m)]


def _has_params(m: nn.Module) -> bool:
    return next(m.parameters(), None) is not None


def _is_frozen(m: nn.Module) -> bool:
    return all(not p.requires_grad for p in m.parameters())


def freeze(module: nn.Module) -> None:
    for p in module.parameters():
        p.requires_grad_(False)


def unfreeze(module: nn.Module) -> None:
    for p in module.parameters():
        p.requires_grad_(True)


def freeze_except_last(module: nn.Module, except_last_n: int) -> None:
    """Freezes everything, then thaws the last ``except_last_n`` layers that have parameters."""
    if except_last_n < 0:
        raise ValueError("except_last_n must be non-negative")
    freeze(module)
    with_params = [(n, m) for n, m in layers(module) if _has_params(m)]
    for _, m in with_params[len(with_params) - min(except_last_n, len(with_params)):]:
        unfreeze(m)


def freeze_by_name(module, *names: str) -> int:
    sel = LayerSelection.by_name(module, *names)
    for _, m in sel:
        freeze(m)
    return len(sel)


def unfreeze_by_name(module, *names: str) -> int:
    sel = LayerSelection.by_name(module, *names)
    for _, m in sel:
        unfreeze(m)
    return len(sel)


def freeze_by_pattern(module, pattern: str) -> int:
    sel = LayerSelection.by_pattern(module, pattern)
    for _, m in sel:
        freeze(m)
    return len(sel)


def unfreeze_by_pattern(module, pattern: str) -> int:
    sel = LayerSelection.by_pattern(module, pattern)
    for _, m in sel:
        unfreeze(m)
    return len(sel)


def frozen_layers(module):
    return LayerSelection.frozen(module)


def unfrozen_layers(module):
    return LayerSelection.trainable(module)


@dataclass
class FrozenStateSummary:
    total_parameters: int = 0
    frozen_parameters: int = 0
    total_layers: int = 0
    frozen_layer_names: List[str] = field(default_factory=list)
    unfrozen_layer_names: List[str] = field(default_factory=list)

    @property
    def unfrozen_parameters(self) -> int:
        return self.total_parameters - self.frozen_parameters

    @property
    def frozen_layers(self) -> int:
        return len(self.frozen_layer_names)

    @property
    def unfrozen_layers(self) -> int:
        return len(self.unfrozen_layer_names)

    @property
    def frozen_parameter_percentage(self) -> float:
        return 100.0 * self.frozen_parameters / self.total_parameters if self.total_parameters else 0.0

    @property
    def unfrozen_parameter_percentage(self) -> float:
        return 100.0 * self.unfrozen_parameters / self.total_parameters if self.total_parameters else 0.0

    def __str__(self):
        return (f"{self.frozen_layers}/{self.total_layers} layers frozen, "
                f"{self.frozen_parameters}/{self.total_parameters} parameters ({self.frozen_parameter_percentage:.1f} %)")


def frozen_state_summary(module: nn.Module) -> FrozenStateSummary:
    s = FrozenStateSummary()
    for name, m in layers(module):
        if not _has_params(m):
            continue
        s.total_layers += 1
        (s.frozen_layer_names if _is_frozen(m) else s.unfrozen_layer_names).append(name)
    for p in module.parameters():
        s.total_parameters += p.numel()
        if not p.requires_grad:
            s.frozen_parameters += p.numel()
    return s


# ------------------------------------------------------------------ parameter groups
class ParameterGroup:
    """Named parameters that share optimiser settings (ParameterGroup.cs:10-169)."""

    def __init__(self, name: str, learning_rate: float, weight_decay: float = 0.0, momentum: Optional[float] = None):
        if not name:
            raise ValueError("a group needs a name")
        self.name = name
        self._params: Dict[str, torch.Tensor] = {}
        self.learning_rate = learning_rate
        self.weight_decay = weight_decay
        self.momentum = momentum

    @property
    def learning_rate(self) -> float:
        return self._lr

    @learning_rate.setter
    def learning_rate(self, v: float):
        if v < 0:
            raise ValueError("the learning rate cannot be negative")
        self._lr = float(v)

    @property
    def weight_decay(self) -> float:
        return self._wd

    @weight_decay.setter
    def weight_decay(self, v: float):
        if v < 0:
            raise ValueError("weight decay cannot be negative")
        self._wd = float(v)

    @property
    def parameters(self) -> List[torch.Tensor]:
        return list(self._params.values())

    @property
    def parameter_names(self) -> List[str]:
        return list(self._params)

    @property
    def parameter_count(self) -> int:
        return len(self._params)

    @property
    def total_elements(self) -> int:
        return sum(p.numel() for p in self._params.values())

    def add_parameter(self, parameter: torch.Tensor, name: str):
        if name in self._params:
            raise ValueError(f"parameter {name!r} is already in group {self.name!r}")
        self._params[name] = parameter

    def add_parameters(self, named: Dict[str, torch.Tensor]):
        for n, p in named.items():
            self.add_parameter(p, n)

    def clear(self):
        self._params.clear()

    def to_parameter_dictionary(self) -> Dict[str, torch.Tensor]:
        return dict(self._params)

    def as_optimizer_group(self) -> Dict[str, object]:
        g: Dict[str, object] = {"params": self.parameters, "lr": self.learning_rate,
                                "weight_decay": self.weight_decay, "name": self.name}
        if self.momentum is not None:
            g["momentum"] = self.momentum
        return g

    def __repr__(self):
        return (f"ParameterGroup({self.name!r}, lr={self.learning_rate:g}, wd={self.weight_decay:g}, "
                f"{self.parameter_count} tensors, {self.total_elements} elements)")


class ParameterGroupBuilder:
    """Fluent construction of groups; the ``add_*`` calls fill the group opened last
    (ParameterGroupBuilder.cs:13-394). A parameter enters at most one group."""

    def __init__(self):
        self._groups: List[ParameterGroup] = []
        self._seen: set = set()

    @property
    def group_count(self) -> int:
        return len(self._groups)

    def new_group(self, name: str, learning_rate: float, weight_decay: float = 0.0, momentum: Optional[float] = None):
        if any(g.name == name for g in self._groups):
            raise ValueError(f"group {name!r} already exists")
        self._groups.append(ParameterGroup(name, learning_rate, weight_decay, momentum))
        return self

    def _cur(self) -> ParameterGroup:
        if not self._groups:
            raise RuntimeError("open a group with new_group first")
        return self._groups[-1]

    def _add_named(self, named: Iterable[Tuple[str, torch.Tensor]]):
        g = self._cur()
        for n, p in named:
            if id(p) in self._seen:
                continue
            self._seen.add(id(p))
            g.add_parameter(p, n)
        return self

    def _add_layers(self, sel):
        return self._add_named((f"{ln}.{pn}" if ln else pn, p) for ln, m in sel for pn, p in m.named_parameters())

    def add_frozen_parameters(self, module):
        return self._add_named((n, p) for n, p in module.named_parameters() if not p.requires_grad)

    def add_unfrozen_parameters(self, module):
        return self._add_named((n, p) for n, p in module.named_parameters() if p.requires_grad)

    def add_layer(self, layer_name: str, module):
        sel = LayerSelection.by_name(module, layer_name)
        if not sel:
            raise KeyError(f"no layer named {layer_name!r}")
        return self._add_layers(sel)

    def add_layers_by_pattern(self, pattern: str, module):
        return self._add_layers(LayerSelection.by_pattern(module, pattern))

    def add_first_n_layers(self, count: int, module):
        return self._add_layers(LayerSelection.first_n(module, count))

    def add_last_n_layers(self, count: int, module):
        return self._add_layers(LayerSelection.last_n(module, count))

    def add_layer_range(self, start: int, end: int, module):
        return self._add_layers(LayerSelection.by_range(module, start, end))

    def add_parameter(self, parameter, name: str):
        return self._add_named([(name, parameter)])

    def add_parameters(self, named: Dict[str, torch.Tensor]):
        return self._add_named(named.items())

    def with_learning_rate(self, lr: float):
        self._cur().learning_rate = lr
        return self

    def with_weight_decay(self, wd: float):
        self._cur().weight_decay = wd
        return self

    def with_momentum(self, m: float):
        self._cur().momentum = m
        return self

    def build(self) -> List[ParameterGroup]:
        return [g for g in self._groups if g.parameter_count]

    def build_dictionary(self) -> Dict[str, ParameterGroup]:
        return {g.name: g for g in self.build()}

    def reset(self):
        self._groups.clear()
        self._seen.clear()
        return self


# ------------------------------------------------------------------ layer-wise learning rates
class ScheduleType(enum.Enum):
    CONSTANT = "constant"
    LINEAR = "linear"
    COSINE = "cosine"
    STEP = "step"


@dataclass
class _LayerSchedule:
    pattern: str
    type: ScheduleType
    initial_multiplier: float
    final_multiplier: float
    total_steps: int


class LayerWiseLrScheduler:
    """Per-layer multipliers of one base rate, fixed or following a schedule over steps
    (LayerWiseLrScheduler.cs:11-520). A parameter takes the first schedule, else the first fixed
    multiplier, whose pattern occurs in its name; the empty pattern matches every name."""

    def __init__(self, base_learning_rate: float):
        if base_learning_rate <= 0:
            raise ValueError("the base learning rate must be positive")
        self.base_learning_rate = float(base_learning_rate)
        self._schedules: Dict[str, _LayerSchedule] = {}
        self._multipliers: Dict[str, float] = {}
        self.step_count = 0

    # ---- factories
    @classmethod
    def create_discriminative(cls, base_lr: float, multipliers: Sequence[float]):
        if not len(multipliers):
            raise ValueError("the multipliers must not be empty")
        s = cls(base_lr)
        for i, m in enumerate(multipliers):
            s.set_multiplier_by_layer_index(i, m)
        return s

    @classmethod
    def create_geometric_discriminative(cls, base_lr: float, num_layers: int, first_layer_multiplier: float = 0.1,
                                        last_layer_multiplier: float = 1.0):
        if num_layers <= 0:
            raise ValueError("the number of layers must be positive")
        ratio = (last_layer_multiplier / first_layer_multiplier) ** (1.0 / (num_layers - 1)) if num_layers > 1 else 1.0
        return cls.create_discriminative(base_lr, [first_layer_multiplier * ratio ** i for i in range(num_layers)])

    @classmethod
    def create_gradual_unfreezing(cls, base_lr: float, num_groups: int, frozen_lr: float, unfrozen_lr: float):
        if num_groups <= 0 or frozen_lr <= 0 or unfrozen_lr < frozen_lr:
            raise ValueError("need num_groups > 0 and 0 < frozen_lr <= unfrozen_lr")
        lrs = [frozen_lr + (unfrozen_lr - frozen_lr) * (i / (num_groups - 1) if num_groups > 1 else 0.0)
               for i in range(num_groups)]
        return cls.create_discriminative(base_lr, [lr / base_lr for lr in lrs])

    @classmethod
    def create_triangular(cls, base_lr: float, min_lr: float, max_lr: float, cycle_steps: int = 1000):
        if min_lr <= 0 or max_lr <= min_lr or cycle_steps <= 0:
            raise ValueError("need 0 < min_lr < max_lr and cycle_steps > 0")
        s = cls(base_lr)
        s.set_layer_schedule("", ScheduleType.COSINE, min_lr / base_lr, max_lr / base_lr, max(1, cycle_steps // 2))
        return s

    @classmethod
    def create_warmup_cosine(cls, base_lr: float, warmup_lr: float, warmup_steps: int, total_steps: int):
        """Layers named ``warmup*`` ramp linearly to ``warmup_lr``; layers named ``annealing*`` decay
        from it by a cosine to one hundredth of the base rate."""
        if warmup_lr <= 0 or warmup_steps < 0 or total_steps <= warmup_steps:
            raise ValueError("need warmup_lr > 0 and 0 <= warmup_steps < total_steps")
        s = cls(base_lr)
        s.set_layer_schedule("warmup", ScheduleType.LINEAR, 1.0, warmup_lr / base_lr, max(1, warmup_steps))
        s.set_layer_schedule("annealing", ScheduleType.COSINE, warmup_lr / base_lr, 0.01, total_steps - warmup_steps)
        return s

    # ---- configuration
    @property
    def scheduled_layer_count(self) -> int:
        return len(self._schedules) + len(self._multipliers)

    def set_multiplier(self, layer_pattern: str, multiplier: float):
        if multiplier < 0:
            raise ValueError("a multiplier cannot be negative")
        self._multipliers[layer_pattern] = float(multiplier)

    def set_multiplier_by_layer_index(self, layer_index: int, multiplier: float):
        if layer_index < 0:
            raise ValueError("the layer index cannot be negative")
        self.set_multiplier(f"layer_{layer_index}", multiplier)

    def set_layer_schedule(self, pattern: str, schedule_type: ScheduleType, initial_multiplier: float,
                           final_multiplier: float, total_steps: int):
        if total_steps <= 0:
            raise ValueError("total_steps must be positive")
        self._schedules[pattern] = _LayerSchedule(pattern, schedule_type, initial_multiplier, final_multiplier, total_steps)

    # ---- evaluation
    def step(self) -> int:
        self.step_count += 1
        return self.step_count

    @staticmethod
    def _multiplier_at(s: _LayerSchedule, step: int) -> float:
        t = min(1.0, step / s.total_steps)
        if s.type is ScheduleType.LINEAR:
            return s.initial_multiplier + (s.final_multiplier - s.initial_multiplier) * t
        if s.type is ScheduleType.COSINE:
            return s.final_multiplier + (s.initial_multiplier - s.final_multiplier) * (1.0 + math.cos(t * math.pi)) / 2.0
        if s.type is ScheduleType.STEP:
            return s.initial_multiplier if t < 0.5 else s.final_multiplier
        return s.initial_multiplier

    def get_learning_rate(self, step: int, base_learning_rate: float) -> float:
        """The base rate does not move; the layers do."""
        return base_learning_rate

    def get_current_lrs(self) -> Dict[str, float]:
        out = {k: self.base_learning_rate * m for k, m in self._multipliers.items()}
        out.update({k: self.base_learning_rate * self._multiplier_at(s, self.step_count)
                    for k, s in self._schedules.items()})
        return out

    def get_parameter_learning_rate(self, parameter_name: str) -> float:
        if not parameter_name:
            raise ValueError("the parameter name cannot be empty")
        for pat, s in self._schedules.items():
            if pat in parameter_name:
                return self.base_learning_rate * self._multiplier_at(s, self.step_count)
        for pat, m in self._multipliers.items():
            if pat in parameter_name:
                return self.base_learning_rate * m
        return self.base_learning_rate

    def get_group_learning_rate(self, group_index: int, layer_name: Optional[str] = None) -> float:
        return self.get_parameter_learning_rate(layer_name) if layer_name else self.base_learning_rate

    def apply(self, optimizer: torch.optim.Optimizer) -> List[float]:
        """Writes each named group's current rate (groups made by ``ParameterGroup.as_optimizer_group``
        carry ``name``; group ``i`` without a name is looked up as ``layer_i``)."""
        lrs = []
        for i, g in enumerate(optimizer.param_groups):
            g["lr"] = self.get_parameter_learning_rate(g.get("name") or f"layer_{i}")
            lrs.append(g["lr"])
        return lrs

    # ---- state
    def state_dict(self) -> Dict[str, object]:
        return {"base_learning_rate": self.base_learning_rate, "step_count": self.step_count,
                "multipliers": dict(self._multipliers),
                "schedules": {k: [s.type.value, s.initial_multiplier, s.final_multiplier, s.total_steps]
                              for k, s in self._schedules.items()}}

    def load_state_dict(self, state: Dict[str, object]):
        self.base_learning_rate = float(state["base_learning_rate"])
        self.step_count = int(state["step_count"])
        self._multipliers = {k: float(v) for k, v in state["multipliers"].items()}
        self._schedules = {k: _LayerSchedule(k, ScheduleType(v[0]), float(v[1]), float(v[2]), int(v[3]))
                           for k, v in state["schedules"].items()}


# ---- optimiser helpers (LayerWiseLrExtensions.cs:13-339)
def apply_parameter_groups(optimizer: torch.optim.Optimizer, groups) -> None:
    """Replaces the optimiser's groups by ``groups`` (a list or a builder); state of parameters that
    stay is kept, since torch keys it by tensor."""
    if isinstance(groups, ParameterGroupBuilder):
        groups = groups.build()
    if not groups:
        raise ValueError("no parameter groups to apply")
    defaults = optimizer.defaults
    optimizer.param_groups.clear()
    for g in groups:
        og = g.as_optimizer_group()
        if "momentum" in og and "momentum" not in defaults:
            og.pop("momentum")
        optimizer.add_param_group(og)


def parameter_groups_of(optimizer: torch.optim.Optimizer, model: nn.Module) -> List[ParameterGroup]:
    names = {id(p): n for n, p in model.named_parameters()}
    out = []
    for i, g in enumerate(optimizer.param_groups):
        pg = ParameterGroup(g.get("name") or f"group_{i}", g["lr"], g.get("weight_decay", 0.0), g.get("momentum"))
        for j, p in enumerate(g["params"]):
            pg.add_parameter(p, names.get(id(p), f"group_{i}.param_{j}"))
        out.append(pg)
    return out


def set_layer_wise_lrs(optimizer: torch.optim.Optimizer, model: nn.Module, layer_lrs: Dict[str, float],
                       default_lr: Optional[float] = None) -> None:
    """One group per entry of ``layer_lrs`` (a pattern that occurs in the parameter name; first match
    wins) plus a ``default`` group for the rest."""
    base = default_lr if default_lr is not None else optimizer.param_groups[0]["lr"]
    wd = optimizer.param_groups[0].get("weight_decay", 0.0)
    b = ParameterGroupBuilder()
    for pat, lr in layer_lrs.items():
        b.new_group(pat or "all", lr, wd)
        b.add_parameters({n: p for n, p in model.named_parameters() if pat in n})
    b.new_group("default", base, wd).add_parameters(dict(model.named_parameters()))
    apply_parameter_groups(optimizer, b)


def clear_layer_wise_lrs(optimizer: torch.optim.Optimizer, lr: Optional[float] = None) -> None:
    """Merges all groups back into one at ``lr`` (default: the optimiser's default rate)."""
    params = [p for g in optimizer.param_groups for p in g["params"]]
    first = {k: v for k, v in optimizer.param_groups[0].items() if k not in ("params", "name")}
    first["lr"] = lr if lr is not None else optimizer.defaults.get("lr", first["lr"])
    optimizer.param_groups.clear()
    optimizer.add_param_group({"params": params, **first})


def create_discriminative_groups(model: nn.Module, base_lr: float, multipliers: Optional[Sequence[float]] = None,
                                 decay: float = 0.9, weight_decay: float = 0.0) -> ParameterGroupBuilder:
    """One group per layer with parameters; layer ``i`` of ``L`` trains at ``base_lr * decay^(L-1-i)``
    unless ``multipliers`` gives the factors."""
    ls = [(n, m) for n, m in layers(model) if _has_params(m)]
    if multipliers is not None and len(multipliers) != len(ls):
        raise ValueError(f"{len(multipliers)} multipliers for {len(ls)} layers")
    b = ParameterGroupBuilder()
    for i, (n, m) in enumerate(ls):
        mult = multipliers[i] if multipliers is not None else decay ** (len(ls) - 1 - i)
        b.new_group(f"layer_{i}:{n}", base_lr * mult, weight_decay)
        b._add_layers([(n, m)])
    return b


# ------------------------------------------------------------------ gradual unfreezing
class GradualUnfreezingScheduler:
    """Starts frozen; stage ``s`` thaws the last ``s + 1`` layers that have parameters, reached when
    training progress passes ``thresholds[s]`` (GradualUnfreezingScheduler.cs:12-242)."""

    def __init__(self, module: nn.Module, unfreeze_thresholds: Sequence[float]):
        th = [float(t) for t in unfreeze_thresholds]
        if not th:
            raise ValueError("at least one threshold is needed")
        if any(t < 0.0 or t > 1.0 for t in th):
            raise ValueError("thresholds lie in [0, 1]")
        if any(b < a for a, b in zip(th, th[1:])):
            raise ValueError("thresholds must ascend")
        self.module, self.unfreeze_thresholds = module, th
        self.current_stage = -1
        self._initialized = False
        self.on_unfreeze_stage: List[Callable[[int, int], None]] = []

    @classmethod
    def create_evenly_distributed(cls, module: nn.Module, num_stages: int):
        if num_stages <= 0:
            raise ValueError("the number of stages must be positive")
        return cls(module, [(i + 1) / num_stages for i in range(num_stages)])

    @property
    def total_stages(self) -> int:
        return len(self.unfreeze_thresholds)

    def initialize(self):
        freeze(self.module)
        self.current_stage = -1
        self._initialized = True

    def _thaw(self, stage: int):
        with_params = [(n, m) for n, m in layers(self.module) if _has_params(m)]
        for _, m in with_params[len(with_params) - min(stage + 1, len(with_params)):]:
            unfreeze(m)

    def _enter(self, stage: int):
        self.current_stage = stage
        self._thaw(stage)
        for cb in self.on_unfreeze_stage:
            cb(stage, self.total_stages)

    def update_unfreezing(self, progress: float) -> bool:
        if not self._initialized:
            self.initialize()
        if progress < 0.0 or progress > 1.0:
            raise ValueError("progress lies in [0, 1]")
        target = -1
        for i, t in enumerate(self.unfreeze_thresholds):
            if progress >= t:
                target = i
            else:
                break
        if target > self.current_stage:
            self._enter(target)
            return True
        return False

    def advance_to_next_stage(self) -> bool:
        if not self._initialized:
            self.initialize()
        if self.current_stage >= self.total_stages - 1:
            return False
        self._enter(self.current_stage + 1)
        return True

    def set_stage(self, stage: int):
        if stage < -1 or stage >= self.total_stages:
            raise ValueError(f"stage must lie in [-1, {self.total_stages - 1}]")
        if stage < self.current_stage or not self._initialized:
            freeze(self.module)
            self._initialized = True
        self.current_stage = stage
        if stage >= 0:
            self._thaw(stage)

    def reset(self):
        self.initialize()

    def unfrozen_layer_count(self, stage: int) -> int:
        if stage < -1 or stage >= self.total_stages:
            raise ValueError("stage out of range")
        return max(0, stage + 1)

    def state_summary(self) -> str:
        return (f"stage {self.current_stage + 1}/{self.total_stages}, "
                f"{self.unfrozen_layer_count(self.current_stage)} layers thawed; {frozen_state_summary(self.module)}")
