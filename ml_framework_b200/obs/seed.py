"""Seeds and determinism (reference: src/MLFramework.Utilities/SeedManager.cs:36-448: global / device /
worker seeds, RNG snapshots, deterministic-mode flags, scoped determinism, registry of non-deterministic
operations)."""
from __future__ import annotations

import contextlib
import enum
import hashlib
import os
import random
from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch


class DeterministicModeFlags(enum.IntFlag):
    NONE = 0
    ALGORITHMS = 1          # torch.use_deterministic_algorithms
    CUDNN = 2               # cudnn.deterministic, benchmark off
    NO_TF32 = 4
    NO_ATOMIC_REDUCTIONS = 8   # this package: kernels whose fp32 atomics reorder sums are swapped for ordered variants
    ALL = 15


#: Kernels of this package whose floating-point result depends on scheduling order.
KNOWN_NON_DETERMINISTIC_OPERATIONS = {
    "flash_bwd (dQ accumulated with fp32 atomics across key tiles)": "bitwise run-to-run differences in dQ at the 1e-6 level",
    "embedding_bwd (fp32 atomics on repeated token ids)": "order of accumulation for repeated ids",
    "norm_bwd parameter gradients (fp32 atomics across row slabs)": "order of slab accumulation",
    "index_add / scatter_add (PyTorch)": "atomics",
}


@dataclass
class RNGSnapshot:
    python: object
    numpy: object
    torch_cpu: torch.Tensor
    torch_cuda: Optional[List[torch.Tensor]]


class SeedManager:
    def __init__(self):
        self.global_seed: Optional[int] = None
        self.flags = DeterministicModeFlags.NONE

    def set_global_seed(self, seed: int):
        self.global_seed = seed
        random.seed(seed)
        np.random.seed(seed % (1 << 32))
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)

    @staticmethod
    def deterministic_seed(base: int, *salt) -> int:
        """Stable derived seed (hash of base + salts), e.g. per device / worker / epoch."""
        h = hashlib.sha256(repr((base,) + salt).encode()).digest()
        return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)

    def seed_all_devices(self, base: Optional[int] = None):
        base = self.global_seed if base is None else base
        for d in range(torch.cuda.device_count()):
            with torch.cuda.device(d):
                torch.cuda.manual_seed(self.deterministic_seed(base, "device", d))

    def seed_workers(self, n: int, base: Optional[int] = None) -> List[int]:
        base = self.global_seed if base is None else base
        return [self.deterministic_seed(base, "worker", w) for w in range(n)]

    def capture_rng_state(self) -> RNGSnapshot:
        return RNGSnapshot(random.getstate(), np.random.get_state(), torch.get_rng_state(),
                           torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None)

    def restore_rng_state(self, s: RNGSnapshot):
        random.setstate(s.python)
        np.random.set_state(s.numpy)
        torch.set_rng_state(s.torch_cpu)
        if s.torch_cuda is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state_all(s.torch_cuda)

    def set_deterministic_mode(self, flags: DeterministicModeFlags):
        self.flags = flags
        torch.use_deterministic_algorithms(bool(flags & DeterministicModeFlags.ALGORITHMS), warn_only=True)
        torch.backends.cudnn.deterministic = bool(flags & DeterministicModeFlags.CUDNN)
        if flags & DeterministicModeFlags.CUDNN:
            torch.backends.cudnn.benchmark = False
        if flags & DeterministicModeFlags.NO_TF32:
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
        if flags & DeterministicModeFlags.ALGORITHMS:
            os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")

    @contextlib.contextmanager
    def with_determinism(self, seed: int, flags: DeterministicModeFlags = DeterministicModeFlags.ALL):
        snap, old = self.capture_rng_state(), self.flags
        try:
            self.set_global_seed(seed)
            self.set_deterministic_mode(flags)
            yield
        finally:
            self.set_deterministic_mode(old)
            self.restore_rng_state(snap)
