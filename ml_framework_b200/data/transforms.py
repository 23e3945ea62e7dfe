"""Sample transforms (reference: src/MLFramework/Data/Transforms/*: Compose, Lambda, Normalize, ToTensor,
GpuNormalize, GpuResize). The "Gpu" variants run on whatever device the tensor is on."""
from __future__ import annotations

from typing import Callable, Sequence

import numpy as np
import torch
import torch.nn.functional as F


class Compose:
    def __init__(self, transforms: Sequence[Callable]):
        self.transforms = list(transforms)

    def __call__(self, x):
        for t in self.transforms:
            x = t(x)
        return x


class Lambda:
    def __init__(self, fn: Callable):
        self.fn = fn

    def __call__(self, x):
        return self.fn(x)


class ToTensor:
    """HWC uint8 / array-like -> CHW float in [0, 1] (2-D and other ranks pass through as float)."""

    def __call__(self, x):
        t = torch.as_tensor(np.asarray(x)) if not isinstance(x, torch.Tensor) else x
        if t.dtype == torch.uint8:
            t = t.float() / 255.0
        else:
            t = t.float()
        return t.permute(2, 0, 1).contiguous() if t.dim() == 3 else t


class Normalize:
    def __init__(self, mean: Sequence[float], std: Sequence[float]):
        if any(s == 0 for s in std):
            raise ValueError("std must be non-zero")
        self.mean, self.std = torch.tensor(mean), torch.tensor(std)

    def __call__(self, x: torch.Tensor):
        shape = (-1,) + (1,) * (x.dim() - 1 - (1 if x.dim() == 4 else 0))
        m, s = self.mean.to(x.device, x.dtype), self.std.to(x.device, x.dtype)
        if x.dim() == 4:
            return (x - m.view(1, -1, 1, 1)) / s.view(1, -1, 1, 1)
        return (x - m.view(shape)) / s.view(shape)


GpuNormalize = Normalize


class Resize:
    def __init__(self, size, mode: str = "bilinear"):
        self.size, self.mode = (size, size) if isinstance(size, int) else tuple(size), mode

    def __call__(self, x: torch.Tensor):
        batched = x.dim() == 4
        y = F.interpolate(x if batched else x[None], size=self.size, mode=self.mode,
                          align_corners=False if self.mode in ("bilinear", "bicubic") else None)
        return y if batched else y[0]


GpuResize = Resize


class RandomCrop:
    def __init__(self, size: int, seed: int = 0):
        self.size, self.gen = size, torch.Generator().manual_seed(seed)

    def __call__(self, x: torch.Tensor):
        H, W = x.shape[-2:]
        i = int(torch.randint(0, H - self.size + 1, (1,), generator=self.gen))
        j = int(torch.randint(0, W - self.size + 1, (1,), generator=self.gen))
        return x[..., i:i + self.size, j:j + self.size]
