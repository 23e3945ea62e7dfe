"""Process-group façade: one API over ``torch.distributed`` (NCCL on GPUs, gloo on CPU) and an
in-process simulated world for tests.

It exposes the union of the reference's three communication stacks:

* ``IProcessGroup`` (src/MLFramework/Distributed/IProcessGroup.cs:10-81): rank, world size,
  all_reduce / broadcast / barrier, send / recv and their async forms, ``ReduceOp``
  (``:122-148``), ``ProcessGroup.Init(backend, "env")`` reading ``RANK`` / ``WORLD_SIZE``
  (src/MLFramework/Distributed/ProcessGroup.cs:64-120).
* ``ICommunicator`` (src/MLFramework/Distributed/Communication/ICommunicator.cs:10-49):
  tensor-returning ``all_gather(t, dim)`` / ``reduce_scatter``.
* ``ICommunicationBackend`` (src/MLFramework/Communication/ICommunicationBackend.cs:8-58):
  reduce, all_gather, reduce_scatter, with handles exposing ``is_completed / wait``
  (src/MLFramework/Communication/ICommunicationHandle.cs:8-28).
"""
from __future__ import annotations

import enum
import os
import threading
from datetime import timedelta
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


class BackendType(enum.Enum):
    """src/MLFramework/Distributed/BackendType.cs:6-28. MPI and RCCL are accepted names only."""
    NCCL = "nccl"
    GLOO = "gloo"
    MPI = "mpi"
    RCCL = "rccl"
    FAKE = "fake"


class ReduceOp(enum.Enum):
    SUM = "sum"
    AVG = "avg"
    MAX = "max"
    MIN = "min"
    PRODUCT = "product"


class CommunicationError(RuntimeError):
    """src/MLFramework/Distributed/IProcessGroup.cs:153."""


class CommunicationTimeout(CommunicationError):
    pass


class RankMismatchError(CommunicationError):
    pass


_TORCH_OPS = {
    ReduceOp.SUM: dist.ReduceOp.SUM, ReduceOp.MAX: dist.ReduceOp.MAX, ReduceOp.MIN: dist.ReduceOp.MIN,
    ReduceOp.PRODUCT: dist.ReduceOp.PRODUCT, ReduceOp.AVG: dist.ReduceOp.SUM,
}


class Work:
    """Completion handle (``ICommunicationHandle``): ``is_completed``, ``wait``, ``result``."""

    def __init__(self, inner=None, result=None, post: Optional[Callable[[], None]] = None):
        self._inner, self._result, self._post, self._done = inner, result, post, inner is None

    def is_completed(self) -> bool:
        if self._done:
            return True
        return bool(self._inner.is_completed())

    def wait(self, timeout: Optional[float] = None):
        if not self._done:
            if timeout is not None:
                ok = self._inner.wait(timedelta(seconds=timeout))
                if ok is False:
                    raise CommunicationTimeout("collective did not complete in time")
            else:
                self._inner.wait()
            self._done = True
        if self._post is not None:
            post, self._post = self._post, None
            post()
        return self._result

    def try_wait(self) -> bool:
        if self.is_completed():
            self.wait()
            return True
        return False

    def result(self):
        return self.wait()


class ProcessGroup:
    """A communicator over a set of ranks."""

    def __init__(self, pg, ranks: Sequence[int], backend: BackendType):
        self._pg = pg
        self.ranks = list(ranks)
        self.backend = backend
        self._global_rank = dist.get_rank()
        if self._global_rank not in self.ranks:
            raise RankMismatchError(f"rank {self._global_rank} is not part of group {self.ranks}")

    # ---- identity
    @property
    def rank(self) -> int:
        return self.ranks.index(self._global_rank)

    @property
    def world_size(self) -> int:
        return len(self.ranks)

    def global_rank(self, group_rank: int) -> int:
        return self.ranks[group_rank]

    @property
    def torch_group(self):
        return self._pg

    # ---- collectives
    def all_reduce(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM, async_op: bool = False):
        w = dist.all_reduce(t, op=_TORCH_OPS[op], group=self._pg, async_op=async_op)
        post = (lambda: t.div_(self.world_size)) if op == ReduceOp.AVG else None
        if async_op:
            return Work(w, t, post)
        if post:
            post()
        return t

    def reduce(self, t: torch.Tensor, dst: int = 0, op: ReduceOp = ReduceOp.SUM, async_op: bool = False):
        w = dist.reduce(t, dst=self.ranks[dst], op=_TORCH_OPS[op], group=self._pg, async_op=async_op)
        post = (lambda: t.div_(self.world_size)) if (op == ReduceOp.AVG and self.rank == dst) else None
        if async_op:
            return Work(w, t, post)
        if post:
            post()
        return t

    def broadcast(self, t: torch.Tensor, src: int = 0, async_op: bool = False):
        w = dist.broadcast(t, src=self.ranks[src], group=self._pg, async_op=async_op)
        return Work(w, t) if async_op else t

    def all_gather(self, t: torch.Tensor, dim: int = 0, async_op: bool = False):
        """Returns the concatenation of every rank's ``t`` along ``dim``."""
        t = t.contiguous()
        parts = [torch.empty_like(t) for _ in range(self.world_size)]
        w = dist.all_gather(parts, t, group=self._pg, async_op=async_op)
        if async_op:
            holder: Dict[str, torch.Tensor] = {}
            wk = Work(w, None, None)
            wk._post = lambda: holder.setdefault("r", torch.cat(parts, dim=dim))
            orig_wait = wk.wait

            def wait(timeout=None):
                orig_wait(timeout)
                return holder.setdefault("r", torch.cat(parts, dim=dim))
            wk.wait = wait  # type: ignore
            return wk
        return torch.cat(parts, dim=dim)

    def all_gather_into(self, out: torch.Tensor, t: torch.Tensor, async_op: bool = False):
        w = dist.all_gather_into_tensor(out, t.contiguous(), group=self._pg, async_op=async_op)
        return Work(w, out) if async_op else out

    def reduce_scatter(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM, dim: int = 0, async_op: bool = False):
        """Reduces ``t`` over ranks and returns this rank's 1/W slice along ``dim``."""
        W = self.world_size
        if t.shape[dim] % W != 0:
            raise ValueError(f"reduce_scatter: dim {dim} of size {t.shape[dim]} not divisible by {W}")
        chunks = [c.contiguous() for c in t.chunk(W, dim=dim)]
        out = torch.empty_like(chunks[0])
        if self.backend == BackendType.GLOO:
            # gloo has no reduce_scatter: all_reduce then slice (CPU plumbing only)
            full = t.clone()
            w = dist.all_reduce(full, op=_TORCH_OPS[op], group=self._pg, async_op=async_op)

            def post():
                out.copy_(full.chunk(W, dim=dim)[self.rank])
                if op == ReduceOp.AVG:
                    out.div_(W)
            if async_op:
                return Work(w, out, post)
            post()
            return out
        w = dist.reduce_scatter(out, chunks, op=_TORCH_OPS[op], group=self._pg, async_op=async_op)
        post = (lambda: out.div_(W)) if op == ReduceOp.AVG else None
        if async_op:
            return Work(w, out, post)
        if post:
            post()
        return out

    def all_to_all(self, t: torch.Tensor, async_op: bool = False):
        """Equal-split exchange along dim 0: chunk ``j`` of ``t`` goes to rank ``j``; chunk ``j`` of
        the result came from rank ``j``."""
        W = self.world_size
        if t.shape[0] % W != 0:
            raise ValueError(f"all_to_all: dim 0 of size {t.shape[0]} not divisible by {W}")
        src = t.contiguous()
        out = torch.empty_like(src)
        w = dist.all_to_all_single(out, src, group=self._pg, async_op=async_op)
        return Work(w, out) if async_op else out

    def barrier(self, async_op: bool = False):
        if self.backend == BackendType.NCCL and torch.cuda.is_available():
            w = dist.barrier(group=self._pg, async_op=async_op, device_ids=[torch.cuda.current_device()])
        else:
            w = dist.barrier(group=self._pg, async_op=async_op)
        return Work(w) if async_op else None

    # ---- point to point
    def send(self, t: torch.Tensor, dst: int, tag: int = 0):
        dist.send(t, dst=self.ranks[dst], group=self._pg, tag=tag)

    def recv(self, t: torch.Tensor, src: int, tag: int = 0):
        dist.recv(t, src=self.ranks[src], group=self._pg, tag=tag)
        return t

    def isend(self, t: torch.Tensor, dst: int, tag: int = 0) -> Work:
        return Work(dist.isend(t, dst=self.ranks[dst], group=self._pg, tag=tag), t)

    def irecv(self, t: torch.Tensor, src: int, tag: int = 0) -> Work:
        return Work(dist.irecv(t, src=self.ranks[src], group=self._pg, tag=tag), t)

    def batch_isend_irecv(self, ops: List[tuple]) -> List[Work]:
        """ops: list of ("send"|"recv", tensor, peer_group_rank)."""
        p2p = [dist.P2POp(dist.isend if kind == "send" else dist.irecv, t, self.ranks[peer], group=self._pg)
               for kind, t, peer in ops]
        return [Work(w) for w in dist.batch_isend_irecv(p2p)]

    def all_gather_object(self, obj):
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self._pg)
        return out

    def broadcast_object(self, obj, src: int = 0):
        box = [obj]
        dist.broadcast_object_list(box, src=self.ranks[src], group=self._pg)
        return box[0]

    def new_subgroup(self, group_ranks: Sequence[int]) -> "ProcessGroup":
        return new_group([self.ranks[r] for r in group_ranks])

    def destroy(self):
        pass


_default: Optional[ProcessGroup] = None
_lock = threading.Lock()


def is_initialized() -> bool:
    return _default is not None


def init_process_group(backend: BackendType | str | None = None, init_method: str = "env",
                       timeout_s: float = 300.0, rank: Optional[int] = None,
                       world_size: Optional[int] = None) -> ProcessGroup:
    """Create the default group from the ``torchrun``-style environment.

    ``RANK`` / ``WORLD_SIZE`` / ``LOCAL_RANK`` / ``MASTER_ADDR`` / ``MASTER_PORT`` as in
    src/MLFramework/Distributed/ProcessLauncher.cs:74-80. The default timeout is the reference's
    ``CommunicationConfig.TimeoutMs`` = 300 s.
    """
    global _default
    with _lock:
        if _default is not None:
            return _default
        if backend is None:
            backend = BackendType.NCCL if torch.cuda.is_available() else BackendType.GLOO
        backend = BackendType(backend) if not isinstance(backend, BackendType) else backend
        if backend in (BackendType.MPI, BackendType.RCCL):
            raise CommunicationError(f"backend {backend.value} is not supported on this platform")
        rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        world_size = int(os.environ.get("WORLD_SIZE", "1")) if world_size is None else world_size
        if not (0 <= rank < world_size):
            raise RankMismatchError(f"invalid rank {rank} for world size {world_size}")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend == BackendType.NCCL:
            local = int(os.environ.get("LOCAL_RANK", str(rank % max(torch.cuda.device_count(), 1))))
            torch.cuda.set_device(local)
        if not dist.is_initialized():
            kwargs = dict(backend=backend.value, rank=rank, world_size=world_size, timeout=timedelta(seconds=timeout_s))
            if init_method not in ("env", "env://"):
                kwargs["init_method"] = init_method
            if backend == BackendType.NCCL:
                kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
            dist.init_process_group(**kwargs)
        _default = ProcessGroup(dist.group.WORLD, list(range(world_size)), backend)
        return _default


def default_group() -> ProcessGroup:
    if _default is None:
        raise CommunicationError("process group is not initialised; call init_process_group() first")
    return _default


def new_group(ranks: Sequence[int]) -> Optional[ProcessGroup]:
    """Collective over the default group: every rank must call it with the same list."""
    base = default_group()
    pg = dist.new_group(ranks=list(ranks))
    if dist.get_rank() not in ranks:
        return None
    return ProcessGroup(pg, list(ranks), base.backend)


def destroy_process_group():
    global _default
    with _lock:
        _default = None
        if dist.is_initialized():
            dist.destroy_process_group()


# --------------------------------------------------------------------------------------------
# in-process simulated world (tests, scheduler-level logic)
# --------------------------------------------------------------------------------------------
class _FakeWorld:
    def __init__(self, world_size: int):
        self.world_size = world_size
        self.lock = threading.Condition()
        self.slots: Dict[tuple, dict] = {}
        self.mail: Dict[tuple, list] = {}
        self.seq = [0] * world_size


class FakeProcessGroup:
    """W ranks simulated by W threads in one process; collectives rendezvous in memory.

    Plays the role of the reference's ``MockCommunicator``
    (src/MLFramework/Distributed/Communication/MockCommunicator.cs:13-232) and of the tests'
    mock process group (tests/MLFramework.Tests/Distributed/MockProcessGroup.cs:14-238).
    """

    backend = BackendType.FAKE

    def __init__(self, world: _FakeWorld, rank: int, timeout_s: float = 30.0):
        self._w, self.rank, self.world_size = world, rank, world.world_size
        self.ranks = list(range(world.world_size))
        self.timeout_s = timeout_s
        self.drop_next = False  # fault injection: skip participating once

    @staticmethod
    def create_world(world_size: int, timeout_s: float = 30.0) -> List["FakeProcessGroup"]:
        w = _FakeWorld(world_size)
        return [FakeProcessGroup(w, r, timeout_s) for r in range(world_size)]

    def _rendezvous(self, kind: str, payload, combine: Callable[[List], List]):
        w = self._w
        if self.drop_next:
            self.drop_next = False
            raise CommunicationError(f"rank {self.rank}: injected failure before {kind}")
        with w.lock:
            key = (kind, w.seq[self.rank])
            w.seq[self.rank] += 1
            slot = w.slots.setdefault(key, {"in": {}, "out": None, "taken": 0})
            slot["in"][self.rank] = payload
            if len(slot["in"]) == self.world_size:
                slot["out"] = combine([slot["in"][r] for r in range(self.world_size)])
                w.lock.notify_all()
            else:
                ok = w.lock.wait_for(lambda: slot["out"] is not None, timeout=self.timeout_s)
                if not ok:
                    raise CommunicationTimeout(f"rank {self.rank}: {kind} timed out after {self.timeout_s}s")
            out = slot["out"][self.rank]
            slot["taken"] += 1
            if slot["taken"] == self.world_size:
                del w.slots[key]
            return out

    def all_reduce(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM, async_op: bool = False):
        def comb(xs):
            st = torch.stack([x.clone() for x in xs])
            r = {ReduceOp.SUM: st.sum(0), ReduceOp.AVG: st.sum(0) / len(xs), ReduceOp.MAX: st.max(0).values,
                 ReduceOp.MIN: st.min(0).values, ReduceOp.PRODUCT: st.prod(0)}[op]
            return [r.clone() for _ in xs]
        t.copy_(self._rendezvous("all_reduce", t, comb))
        return Work(None, t) if async_op else t

    def broadcast(self, t, src: int = 0, async_op: bool = False):
        t.copy_(self._rendezvous("broadcast", t, lambda xs: [xs[src].clone() for _ in xs]))
        return Work(None, t) if async_op else t

    def reduce(self, t, dst: int = 0, op: ReduceOp = ReduceOp.SUM, async_op: bool = False):
        full = self._rendezvous("reduce", t, lambda xs: [torch.stack(xs).sum(0) for _ in xs])
        if self.rank == dst:
            t.copy_(full / self.world_size if op == ReduceOp.AVG else full)
        return Work(None, t) if async_op else t

    def all_gather(self, t, dim: int = 0, async_op: bool = False):
        r = self._rendezvous("all_gather", t, lambda xs: [torch.cat([x.clone() for x in xs], dim=dim) for _ in xs])
        return Work(None, r) if async_op else r

    def all_gather_into(self, out, t, async_op: bool = False):
        out.copy_(self.all_gather(t.reshape(-1), 0).view_as(out))
        return Work(None, out) if async_op else out

    def reduce_scatter(self, t, op: ReduceOp = ReduceOp.SUM, dim: int = 0, async_op: bool = False):
        def comb(xs):
            s = torch.stack(xs).sum(0)
            if op == ReduceOp.AVG:
                s = s / len(xs)
            return [c.clone() for c in s.chunk(len(xs), dim=dim)]
        r = self._rendezvous("reduce_scatter", t, comb)
        return Work(None, r) if async_op else r

    def all_to_all(self, t, async_op: bool = False):
        def comb(xs):
            W = len(xs)
            parts = [x.chunk(W, dim=0) for x in xs]
            return [torch.cat([parts[src][dst].clone() for src in range(W)], dim=0) for dst in range(W)]
        if t.shape[0] % self.world_size != 0:
            raise ValueError(f"all_to_all: dim 0 of size {t.shape[0]} not divisible by {self.world_size}")
        r = self._rendezvous("all_to_all", t, comb)
        return Work(None, r) if async_op else r

    def barrier(self, async_op: bool = False):
        self._rendezvous("barrier", None, lambda xs: [True for _ in xs])
        return Work(None) if async_op else None

    def all_gather_object(self, obj):
        return self._rendezvous("ago", obj, lambda xs: [list(xs) for _ in xs])

    def broadcast_object(self, obj, src: int = 0):
        return self._rendezvous("bo", obj, lambda xs: [xs[src] for _ in xs])

    def send(self, t, dst: int, tag: int = 0):
        w = self._w
        with w.lock:
            w.mail.setdefault((self.rank, dst, tag), []).append(t.clone())
            w.lock.notify_all()

    def recv(self, t, src: int, tag: int = 0):
        w = self._w
        key = (src, self.rank, tag)
        with w.lock:
            ok = w.lock.wait_for(lambda: w.mail.get(key), timeout=self.timeout_s)
            if not ok:
                raise CommunicationTimeout(f"rank {self.rank}: recv from {src} timed out")
            t.copy_(w.mail[key].pop(0))
        return t

    def isend(self, t, dst, tag: int = 0):
        self.send(t, dst, tag)
        return Work(None, t)

    def irecv(self, t, src, tag: int = 0):
        pg = self

        class _Lazy(Work):
            def __init__(self):
                super().__init__(None, t)
                self._got = False

            def is_completed(self):
                return self._got

            def wait(self, timeout=None):
                if not self._got:
                    pg.recv(t, src, tag)
                    self._got = True
                return t
        return _Lazy()

    def batch_isend_irecv(self, ops):
        out = []
        for kind, t, peer in ops:
            if kind == "send":
                out.append(self.isend(t, peer))
        for kind, t, peer in ops:
            if kind == "recv":
                out.append(self.irecv(t, peer))
        return out

    def global_rank(self, r):
        return r

    def destroy(self):
        pass


def run_fake_world(world_size: int, fn: Callable[[FakeProcessGroup], object], timeout_s: float = 30.0) -> List[object]:
    """Run ``fn(pg)`` on ``world_size`` threads, one simulated rank each; re-raises the first error."""
    pgs = FakeProcessGroup.create_world(world_size, timeout_s)
    results: List[object] = [None] * world_size
    errors: List[Optional[BaseException]] = [None] * world_size

    def runner(r):
        try:
            results[r] = fn(pgs[r])
        except BaseException as e:  # noqa: BLE001
            errors[r] = e
    threads = [threading.Thread(target=runner, args=(r,), daemon=True) for r in range(world_size)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout_s * 4)
    for e in errors:
        if e is not None:
            raise e
    return results
