"""Validated collective wrappers, operation handles, completion events, tensor-level helpers, peer-access probe.

Reference (src/MLFramework/Communication/): Operations/{AllReduce.cs:21-67 (AllReduceTensor, AverageGradients,
AllReduceTensors), AllGather.cs, Broadcast.cs, Reduce.cs (ValidateReduceOperation), ReduceScatter.cs, Barrier.cs},
Operations/Async/*, CompletedOperationHandle.cs, PendingOperationHandle.cs, Async/AsyncCommunicationEventHandler.cs,
TensorCommunicationExtensions.cs (BroadcastToAll, AllReduceInPlace, Scatter), Optimizations/GPUDirectManager.cs
(``IsSupported`` is a constant false there; here it asks the driver whether two devices can map each other's memory).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch

from .process_group import CommunicationError, RankMismatchError, ReduceOp


# ------------------------------------------------------------------ validation
def validate_tensor(t, what: str = "tensor"):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{what} must be a tensor, got {type(t).__name__}")
    if t.numel() == 0:
        raise ValueError(f"{what} is empty")


def validate_rank(pg, rank: int, what: str = "rank"):
    if not (0 <= rank < pg.world_size):
        raise RankMismatchError(f"{what} {rank} is outside the group of {pg.world_size} ranks")


def validate_reduce_operation(op: ReduceOp, dtype: torch.dtype):
    if not isinstance(op, ReduceOp):
        raise TypeError(f"not a reduce operation: {op!r}")
    if op == ReduceOp.AVG and not dtype.is_floating_point:
        raise ValueError(f"averaging needs a floating-point tensor, got {dtype}")
    if dtype == torch.bool and op not in (ReduceOp.MAX, ReduceOp.MIN):
        raise ValueError("boolean tensors reduce with MAX (or) / MIN (and) only")


# ------------------------------------------------------------------ wrappers
def all_reduce_tensor(pg, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
    validate_tensor(t)
    validate_reduce_operation(op, t.dtype)
    pg.all_reduce(t, op)
    return t


def average_gradients(pg, params: Iterable[torch.Tensor]) -> int:
    """Sums every present ``.grad`` over the group and divides by the world size; returns how many were reduced."""
    n = 0
    for p in params:
        if p.grad is not None:
            pg.all_reduce(p.grad, ReduceOp.SUM)
            p.grad.div_(pg.world_size)
            n += 1
    return n


def all_reduce_tensors(pg, tensors: Sequence[torch.Tensor], op: ReduceOp = ReduceOp.SUM) -> List[torch.Tensor]:
    """Several tensors of one dtype as ONE collective over a flat buffer."""
    if not tensors:
        return []
    for t in tensors:
        validate_tensor(t)
    if len({t.dtype for t in tensors}) != 1:
        raise TypeError("tensors of one call share a dtype")
    validate_reduce_operation(op, tensors[0].dtype)
    flat = torch.cat([t.reshape(-1) for t in tensors])
    pg.all_reduce(flat, op)
    off = 0
    for t in tensors:
        t.copy_(flat[off:off + t.numel()].view_as(t))
        off += t.numel()
    return list(tensors)


def all_gather_tensor(pg, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
    validate_tensor(t)
    if not (-t.dim() <= dim < max(t.dim(), 1)):
        raise IndexError(f"dimension {dim} out of range for a {t.dim()}-d tensor")
    return pg.all_gather(t, dim)


def broadcast_tensor(pg, t: torch.Tensor, root: int = 0) -> torch.Tensor:
    validate_tensor(t)
    validate_rank(pg, root, "root")
    pg.broadcast(t, root)
    return t


def reduce_tensor(pg, t: torch.Tensor, root: int = 0, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
    validate_tensor(t)
    validate_rank(pg, root, "root")
    validate_reduce_operation(op, t.dtype)
    pg.reduce(t, root, op)
    return t


def reduce_scatter_tensor(pg, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM, dim: int = 0) -> torch.Tensor:
    validate_tensor(t)
    validate_reduce_operation(op, t.dtype)
    if t.shape[dim] % pg.world_size:
        raise ValueError(f"dimension {dim} of size {t.shape[dim]} does not split over {pg.world_size} ranks")
    return pg.reduce_scatter(t, op, dim)


def barrier(pg, timeout_s: Optional[float] = None):
    w = pg.barrier(async_op=timeout_s is not None)
    if timeout_s is not None and w is not None:
        w.wait(timeout_s)


# ------------------------------------------------------------------ handles and events
class CompletedOperationHandle:
    """A handle for work that was done by the time it was created (synchronous back-ends, world of one)."""

    def __init__(self, result=None):
        self._result = result

    @property
    def is_completed(self) -> bool:
        return True

    def wait(self, timeout: Optional[float] = None):
        return self._result

    def try_wait(self) -> bool:
        return True

    def get_result(self):
        return self._result


class PendingOperationHandle:
    """Wraps a ``Work``; ``on_complete`` / ``on_error`` callbacks fire once, from whichever call observes the end."""

    def __init__(self, work, result=None, name: str = "op"):
        self._w, self._result, self.name = work, result, name
        self._done = False
        self._error: Optional[BaseException] = None
        self._lock = threading.Lock()
        self.on_complete: List[Callable[["PendingOperationHandle"], None]] = []
        self.on_error: List[Callable[["PendingOperationHandle", BaseException], None]] = []
        self.started = time.perf_counter()
        self.elapsed_s: Optional[float] = None

    def _finish(self, err: Optional[BaseException]):
        with self._lock:
            if self._done:
                return
            self._done, self._error = True, err
            self.elapsed_s = time.perf_counter() - self.started
        for cb in (self.on_error if err is not None else self.on_complete):
            cb(self, err) if err is not None else cb(self)

    @property
    def is_completed(self) -> bool:
        if not self._done and self._w.is_completed():
            self._finish(None)
        return self._done

    def wait(self, timeout: Optional[float] = None):
        if not self._done:
            try:
                r = self._w.wait(timeout)
            except Exception as e:       # noqa: BLE001 - delivered to the error callbacks, then re-raised
                self._finish(e)
                raise
            if self._result is None:
                self._result = r
            self._finish(None)
        if self._error is not None:
            raise self._error
        return self._result

    def try_wait(self) -> bool:
        return self.is_completed

    def get_result(self):
        if not self._done:
            raise CommunicationError(f"operation {self.name!r} has not completed")
        if self._error is not None:
            raise self._error
        return self._result


class AsyncCommunicationEventHandler:
    """Collects completion and failure events of tracked handles (counts, durations, last error) and forwards them."""

    def __init__(self):
        self.completed = 0
        self.failed = 0
        self.total_seconds = 0.0
        self.last_error: Optional[BaseException] = None
        self.on_completed: List[Callable[[str, float], None]] = []
        self.on_failed: List[Callable[[str, BaseException], None]] = []
        self._lock = threading.Lock()

    def track(self, h: PendingOperationHandle) -> PendingOperationHandle:
        def ok(handle):
            with self._lock:
                self.completed += 1
                self.total_seconds += handle.elapsed_s or 0.0
            for cb in self.on_completed:
                cb(handle.name, handle.elapsed_s or 0.0)

        def bad(handle, err):
            with self._lock:
                self.failed += 1
                self.last_error = err
            for cb in self.on_failed:
                cb(handle.name, err)
        h.on_complete.append(ok)
        h.on_error.append(bad)
        return h

    def statistics(self) -> Dict[str, float]:
        with self._lock:
            return {"completed": self.completed, "failed": self.failed,
                    "mean_seconds": self.total_seconds / self.completed if self.completed else 0.0}


def all_reduce_async(pg, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM, events: Optional[AsyncCommunicationEventHandler] = None):
    validate_tensor(t)
    validate_reduce_operation(op, t.dtype)
    if pg.world_size == 1:
        return CompletedOperationHandle(t)
    h = PendingOperationHandle(pg.all_reduce(t, op, async_op=True), t, "all_reduce")
    return events.track(h) if events is not None else h


# ------------------------------------------------------------------ tensor-level helpers
def broadcast_to_all(pg, t: torch.Tensor, root: int = 0) -> torch.Tensor:
    """The root's values on every rank (in place; the argument is returned)."""
    return broadcast_tensor(pg, t, root)


def all_reduce_in_place(pg, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
    return all_reduce_tensor(pg, t, op)


def scatter_rows(pg, full: Optional[torch.Tensor], root: int = 0, like: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rank ``i`` receives the ``i``-th of ``world_size`` equal row blocks of the root's tensor. Non-root ranks pass
    ``like`` (a tensor with the block's shape and dtype)."""
    from .communicator import scatter
    validate_rank(pg, root, "root")
    if pg.rank == root:
        validate_tensor(full, "full tensor")
        if full.shape[0] % pg.world_size:
            raise ValueError(f"{full.shape[0]} rows do not split over {pg.world_size} ranks")
        chunks = list(full.chunk(pg.world_size, 0))
        return scatter(pg, chunks, chunks[0], root)
    if like is None:
        raise ValueError("non-root ranks pass `like`")
    return scatter(pg, None, like, root)


class GPUDirectManager:
    """Can two devices of this process read each other's memory directly (NVLink / PCIe peer access)? This is what the
    symmetric-memory collectives need; without it they fall back to the process group."""

    @staticmethod
    def is_supported(device_a: int = 0, device_b: Optional[int] = None) -> bool:
        if not torch.cuda.is_available():
            return False
        n = torch.cuda.device_count()
        if device_b is None:
            return n > 1 and all(torch.cuda.can_device_access_peer(device_a, j) for j in range(n) if j != device_a)
        if not (0 <= device_a < n and 0 <= device_b < n):
            return False
        return device_a == device_b or torch.cuda.can_device_access_peer(device_a, device_b)

    @staticmethod
    def peer_matrix() -> List[List[bool]]:
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
        return [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]
