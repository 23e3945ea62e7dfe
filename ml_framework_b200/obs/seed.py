"""Seeds and determinism (reference: src/MLFramework.Utilities/SeedManager.cs:36-686: global / device /
worker seeds, RNG snapshots in memory and on disk, deterministic-mode flags with enable / disable /
query, scoped seed and determinism, registry of non-deterministic operations with the two categories
of src/MLFramework.Utilities/KnownNonDeterministicOperations.cs, configuration validation and
diagnostics)."""
from __future__ import annotations

import contextlib
import enum
import hashlib
import os
import random
import sys
import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch


class DeterministicModeFlags(enum.IntFlag):
    NONE = 0
    ALGORITHMS = 1          # torch.use_deterministic_algorithms
    CUDNN = 2               # cudnn.deterministic, benchmark off
    NO_TF32 = 4
    NO_ATOMIC_REDUCTIONS = 8   # a request that callers can query; this package's atomic-sum kernels (listed below) have
                               # no ordered variant, so validate_configuration names them when the flag is set
    ALL = 15


#: Kernels of this package whose floating-point result depends on scheduling order.
KNOWN_NON_DETERMINISTIC_OPERATIONS = {
    "flash_bwd (dQ accumulated with fp32 atomics across key tiles)": "bitwise run-to-run differences in dQ at the 1e-6 level",
    "embedding_bwd (fp32 atomics on repeated token ids)": "order of accumulation for repeated ids",
    "norm_bwd parameter gradients (fp32 atomics across row slabs)": "order of slab accumulation",
    "index_add / scatter_add (PyTorch)": "atomics",
}


#: Operation kinds whose result depends on scheduling order whatever the settings (atomics, hashing).
NON_DETERMINIZABLE = frozenset({"atomic_add", "atomic_sub", "scatter_add", "scatter_sub", "parallel_sort",
                                "hashmap_lookup", "index_add", "embedding_bwd_atomic", "flash_bwd_dq_atomic"})
#: Operation kinds that have an ordered variant, at a cost.
DETERMINIZABLE = frozenset({"convolution", "matmul", "dropout", "batch_norm", "shuffle", "random_sample",
                            "split_k_gemm", "norm_bwd_param_grads"})

_IMPACT = {
    DeterministicModeFlags.ALGORITHMS: "ordered algorithms: scatter / index kernels fall back to sorted variants",
    DeterministicModeFlags.CUDNN: "cuDNN: fixed algorithm, no autotuning (convolutions 20-30 % slower)",
    DeterministicModeFlags.NO_TF32: "fp32 products leave the tensor cores' TF32 path (several times slower)",
    DeterministicModeFlags.NO_ATOMIC_REDUCTIONS: "atomic-sum kernels are reported, not replaced: use the fp32 reference operators for bitwise repeats",
}


@dataclass
class ValidationResult:
    """Outcome of ``SeedManager.validate_configuration`` (SeedManager.cs:524-575)."""
    is_valid: bool = True
    messages: List[str] = field(default_factory=list)
    warnings: List[str] = field(default_factory=list)
    errors: List[str] = field(default_factory=list)


@dataclass
class DiagnosticInfo:
    deterministic_mode: "DeterministicModeFlags" = DeterministicModeFlags.NONE
    current_seed: Optional[int] = None
    device_count: int = 0
    worker_count: int = 0
    performance_impact: str = ""
    non_deterministic_operations: List[str] = field(default_factory=list)


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
        self._device_seeds: Dict[int, int] = {}
        self._worker_seeds: Dict[int, int] = {}
        self._ops: List[str] = []
        self._lock = threading.RLock()

    @property
    def current_seed(self) -> Optional[int]:
        return self.global_seed

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

    def seed_all_devices(self, base: Optional[int] = None, device_count: Optional[int] = None):
        """Derives one seed per device; ``device_count`` defaults to the visible GPUs (the seeds of
        devices that do not exist here are still recorded, for a plan made on another host)."""
        base = self._base(base)
        n = torch.cuda.device_count() if device_count is None else device_count
        for d in range(n):
            self.seed_device(d, self.deterministic_seed(base, "device", d))

    def seed_device(self, device_id: int, seed: int):
        if device_id < 0:
            raise ValueError("device id must be non-negative")
        with self._lock:
            self._device_seeds[device_id] = seed
        if torch.cuda.is_available() and device_id < torch.cuda.device_count():
            with torch.cuda.device(device_id):
                torch.cuda.manual_seed(seed)

    def device_seed(self, device_id: int) -> int:
        with self._lock:
            if device_id not in self._device_seeds:
                raise KeyError(f"device {device_id} has not been seeded")
            return self._device_seeds[device_id]

    def seed_workers(self, n: int, base: Optional[int] = None) -> List[int]:
        base = self._base(base)
        seeds = [self.deterministic_seed(base, "worker", w) for w in range(n)]
        for w, sd in enumerate(seeds):
            self.seed_worker(w, sd)
        return seeds

    def seed_worker(self, worker_id: int, seed: int):
        if worker_id < 0:
            raise ValueError("worker id must be non-negative")
        with self._lock:
            self._worker_seeds[worker_id] = seed

    def worker_seed(self, worker_id: int) -> int:
        with self._lock:
            if worker_id not in self._worker_seeds:
                raise KeyError(f"worker {worker_id} has not been seeded")
            return self._worker_seeds[worker_id]

    def _base(self, base: Optional[int]) -> int:
        base = self.global_seed if base is None else base
        if base is None:
            raise ValueError("no base seed: pass one or call set_global_seed first")
        return base

    # ---- snapshots on disk (SeedManager.cs:162-205)
    def save_rng_snapshot(self, snapshot: RNGSnapshot, path: str):
        torch.save({"python": snapshot.python, "numpy": snapshot.numpy, "torch_cpu": snapshot.torch_cpu,
                    "torch_cuda": snapshot.torch_cuda}, path)

    def load_rng_snapshot(self, path: str) -> RNGSnapshot:
        d = torch.load(path, weights_only=False)
        return RNGSnapshot(d["python"], d["numpy"], d["torch_cpu"], d["torch_cuda"])

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

    def enable_deterministic_mode(self, flag: DeterministicModeFlags):
        with self._lock:
            self.set_deterministic_mode(self.flags | flag)

    def disable_deterministic_mode(self, flag: DeterministicModeFlags):
        with self._lock:
            self.set_deterministic_mode(self.flags & ~flag)

    def is_deterministic_mode_enabled(self, flag: DeterministicModeFlags) -> bool:
        return bool(self.flags & flag)

    def performance_impact(self) -> str:
        """What the enabled flags cost, one clause per flag (SeedManager.cs:394-430)."""
        parts = [text for flag, text in _IMPACT.items() if self.flags & flag]
        return "; ".join(parts) if parts else "no deterministic mode enabled: no performance impact"

    def check_performance_impact(self) -> Optional[str]:
        """``None`` when nothing is enabled, else the warning text."""
        return None if self.flags == DeterministicModeFlags.NONE else self.performance_impact()

    @contextlib.contextmanager
    def with_global_seed(self, seed: int):
        """Seeds every generator inside the block; afterwards the generators continue where they
        were and the previous seed value is recorded again."""
        snap, old = self.capture_rng_state(), self.global_seed
        try:
            self.set_global_seed(seed)
            yield self
        finally:
            self.restore_rng_state(snap)
            self.global_seed = old

    @contextlib.contextmanager
    def with_deterministic_mode(self, flags: DeterministicModeFlags):
        old = self.flags
        try:
            self.set_deterministic_mode(flags)
            yield self
        finally:
            self.set_deterministic_mode(old)

    # ---- registry of operations seen (SeedManager.cs:494-520, 639-646)
    def register_non_deterministic_operation(self, name: str):
        if not name or not name.strip():
            raise ValueError("operation name cannot be empty")
        with self._lock:
            if name not in self._ops:
                self._ops.append(name)

    def non_deterministic_operations(self) -> List[str]:
        with self._lock:
            return list(self._ops)

    @staticmethod
    def can_be_deterministic(name: str) -> bool:
        return bool(name and name.strip()) and name not in NON_DETERMINIZABLE

    def validate_configuration(self) -> ValidationResult:
        r = ValidationResult()
        with self._lock:
            if self.flags == DeterministicModeFlags.NONE:
                r.messages.append("deterministic mode is not enabled")
                return r
            r.messages.append("deterministic mode is enabled")
            if self._device_seeds:
                r.messages.append(f"{len(self._device_seeds)} devices seeded")
            if self._worker_seeds:
                r.messages.append(f"{len(self._worker_seeds)} workers seeded")
            if self.flags & DeterministicModeFlags.NO_ATOMIC_REDUCTIONS:
                for op in KNOWN_NON_DETERMINISTIC_OPERATIONS:
                    r.warnings.append(f"no ordered variant of {op}")
            if self.global_seed is None:
                r.warnings.append("deterministic mode without a global seed: runs repeat only within one process")
            for op in self._ops:
                if not self.can_be_deterministic(op):
                    r.errors.append(f"operation '{op}' cannot be made deterministic and is used in deterministic mode")
                elif op in DETERMINIZABLE:
                    r.warnings.append(f"operation '{op}' is deterministic only under the matching mode flag")
            r.is_valid = not r.errors
        return r

    def diagnostic_info(self) -> DiagnosticInfo:
        with self._lock:
            return DiagnosticInfo(self.flags, self.global_seed, len(self._device_seeds), len(self._worker_seeds),
                                  self.performance_impact(), list(self._ops))

    def print_diagnostics(self, file=None):
        info = self.diagnostic_info()
        out = file or sys.stdout
        print("=== SeedManager diagnostics ===", file=out)
        print(f"deterministic mode: {info.deterministic_mode!r}", file=out)
        print(f"current seed: {info.current_seed}", file=out)
        print(f"devices seeded: {info.device_count}; workers seeded: {info.worker_count}", file=out)
        print(f"performance impact: {info.performance_impact}", file=out)
        for op in info.non_deterministic_operations:
            kind = "determinizable" if self.can_be_deterministic(op) else "non-determinizable"
            print(f"  - {op} ({kind})", file=out)
        if not info.non_deterministic_operations:
            print("non-deterministic operations: none registered", file=out)

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
