"""Tensor-returning communicator API, point-to-point helpers and named sub-group helpers.

Reference: ``ICommunicator`` with ``AllReduceAsync / AllGatherAsync(t, dim) / ReduceScatterAsync / BroadcastAsync /
BarrierAsync`` (src/MLFramework/Distributed/Communication/ICommunicator.cs:10-49), ``CommunicatorFactory.Create("mock" |
"nccl")`` (:17-30), ``MockCommunicator`` (in-process simulation, MockCommunicator.cs:37-180); point-to-point helpers
``SendReceive / RingSendReceive / Probe / MessageInfo`` (src/MLFramework/Communication/PointToPoint/*.cs);
``ScatterGatherHelpers`` (Communication/Operations/ScatterGatherHelpers.cs:15-34); group helpers
``CreateSplitGroups / CreatePipelineGroups / CreateDataParallelGroups`` (Communication/ProcessGroupHelpers.cs:15-74).
Everything here is a thin layer over a ``ProcessGroup`` (NCCL / gloo) or a ``FakeProcessGroup`` (threads in one process).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .process_group import FakeProcessGroup, ProcessGroup, ReduceOp, Work


class Communicator:
    """Out-of-place collectives that return ``Work`` handles whose ``result()`` is the output tensor."""

    def __init__(self, pg):
        self.pg = pg

    @property
    def rank(self) -> int:
        return self.pg.rank

    @property
    def world_size(self) -> int:
        return self.pg.world_size

    def all_reduce_async(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> Work:
        out = t.clone()
        w = self.pg.all_reduce(out, op, async_op=True)
        return Work(w, out) if isinstance(w, Work) or w is not None else Work(None, out)

    def all_gather_async(self, t: torch.Tensor, dim: int = 0) -> Work:
        r = self.pg.all_gather(t, dim=dim)
        return Work(None, r)

    def reduce_scatter_async(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM, dim: int = 0) -> Work:
        r = self.pg.reduce_scatter(t, op, dim=dim)
        return Work(None, r)

    def broadcast_async(self, t: torch.Tensor, root: int = 0) -> Work:
        out = t.clone()
        self.pg.broadcast(out, root)
        return Work(None, out)

    def barrier_async(self) -> Work:
        self.pg.barrier()
        return Work(None, None)

    # blocking forms
    def all_reduce(self, t, op: ReduceOp = ReduceOp.SUM):
        w = self.all_reduce_async(t, op)
        w.wait()
        return w.result()

    def all_gather(self, t, dim: int = 0):
        return self.all_gather_async(t, dim).result()

    def reduce_scatter(self, t, op: ReduceOp = ReduceOp.SUM, dim: int = 0):
        return self.reduce_scatter_async(t, op, dim).result()

    def broadcast(self, t, root: int = 0):
        return self.broadcast_async(t, root).result()


class MockCommunicator(Communicator):
    """World of ``world_size`` communicators inside one process (threads): ``MockCommunicator.create_world(4)``."""

    @staticmethod
    def create_world(world_size: int) -> List["MockCommunicator"]:
        return [MockCommunicator(pg) for pg in FakeProcessGroup.create_world(world_size)]


class CommunicatorFactory:
    @staticmethod
    def create(backend: str = "nccl", pg=None, world_size: int = 1):
        backend = backend.lower()
        if backend == "mock":
            return MockCommunicator.create_world(world_size)
        if backend in ("nccl", "gloo"):
            if pg is None:
                from .process_group import default_group
                pg = default_group()
            return Communicator(pg)
        raise ValueError(f"unknown communicator backend {backend!r} (mock, nccl, gloo)")


# ------------------------------------------------------------------ point to point
@dataclass
class MessageInfo:
    source: int
    tag: int
    shape: Tuple[int, ...]
    dtype: torch.dtype

    @property
    def count(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


_DT = [torch.float32, torch.bfloat16, torch.float16, torch.int64, torch.int32, torch.uint8, torch.int8, torch.float64, torch.bool]


def send_with_header(pg, t: torch.Tensor, dst: int, tag: int = 0):
    """Sends an 8-int64 header (rank, dtype code, shape) and then the payload, so that the receiver can
    ``probe`` before it allocates."""
    if t.dim() > 6:
        raise ValueError("send_with_header supports at most 6 dimensions")
    h = torch.full((8,), -1, dtype=torch.int64)
    h[0], h[1] = t.dim(), _DT.index(t.dtype)
    for i, s in enumerate(t.shape):
        h[2 + i] = s
    dev = t.device if t.is_cuda else "cpu"
    pg.send(h.to(dev), dst, tag)
    pg.send(t.contiguous(), dst, tag)


def probe(pg, src: int, tag: int = 0, device="cpu") -> MessageInfo:
    """Blocks until the header of the next message from ``src`` has arrived; the payload follows with ``recv_probed``."""
    h = torch.empty(8, dtype=torch.int64, device=device)
    pg.recv(h, src, tag)
    h = h.cpu()
    nd = int(h[0])
    return MessageInfo(src, tag, tuple(int(x) for x in h[2:2 + nd]), _DT[int(h[1])])


def recv_probed(pg, info: MessageInfo, device="cpu") -> torch.Tensor:
    t = torch.empty(info.shape, dtype=info.dtype, device=device)
    pg.recv(t, info.source, info.tag)
    return t


def send_recv(pg, send: torch.Tensor, dst: int, recv: torch.Tensor, src: int, tag: int = 0) -> torch.Tensor:
    """Simultaneous send to ``dst`` and receive from ``src`` (deadlock-free: both are posted before either is waited for)."""
    works = pg.batch_isend_irecv([("send", send, dst), ("recv", recv, src)]) if hasattr(pg, "batch_isend_irecv") else None
    if works is None:
        a, b = pg.isend(send, dst, tag), pg.irecv(recv, src, tag)
        works = [a, b]
    for w in works:
        w.wait()
    return recv


def ring_send_recv(pg, t: torch.Tensor, shift: int = 1) -> torch.Tensor:
    """Every rank sends ``t`` to ``rank + shift`` and returns what it received from ``rank - shift``."""
    W, r = pg.world_size, pg.rank
    out = torch.empty_like(t)
    if W == 1:
        out.copy_(t)
        return out
    return send_recv(pg, t, (r + shift) % W, out, (r - shift) % W)


def scatter(pg, chunks: Optional[Sequence[torch.Tensor]], like: torch.Tensor, src: int = 0) -> torch.Tensor:
    """Rank ``src`` hands chunk ``i`` to rank ``i``; every rank returns its own chunk (shaped like ``like``)."""
    W, r = pg.world_size, pg.rank
    out = torch.empty_like(like)
    if r == src:
        if len(chunks) != W:
            raise ValueError(f"scatter needs {W} chunks, got {len(chunks)}")
        for d in range(W):
            if d == src:
                out.copy_(chunks[d])
            else:
                pg.send(chunks[d].contiguous(), d)
    else:
        pg.recv(out, src)
    return out


def gather(pg, t: torch.Tensor, dst: int = 0) -> Optional[List[torch.Tensor]]:
    """Rank ``dst`` returns the list of every rank's tensor; the others return None."""
    W, r = pg.world_size, pg.rank
    if r == dst:
        out = [torch.empty_like(t) for _ in range(W)]
        out[dst].copy_(t)
        for s in range(W):
            if s != dst:
                pg.recv(out[s], s)
        return out
    pg.send(t.contiguous(), dst)
    return None


# ------------------------------------------------------------------ group helpers
def split_groups(world_size: int, group_size: int) -> List[List[int]]:
    """Consecutive groups of ``group_size`` ranks: [[0..g-1], [g..2g-1], ...]."""
    if world_size % group_size:
        raise ValueError(f"world size {world_size} is not divisible by group size {group_size}")
    return [list(range(i, i + group_size)) for i in range(0, world_size, group_size)]


def pipeline_groups(world_size: int, num_stages: int) -> List[List[int]]:
    """One group per pipeline: ranks that differ only in their stage (stride world / stages)."""
    if world_size % num_stages:
        raise ValueError("world size must be divisible by the number of stages")
    per = world_size // num_stages
    return [[s * per + i for s in range(num_stages)] for i in range(per)]


def data_parallel_groups(world_size: int, model_parallel_size: int) -> List[List[int]]:
    """Ranks holding the same model shard: stride ``model_parallel_size``."""
    if world_size % model_parallel_size:
        raise ValueError("world size must be divisible by the model-parallel size")
    return [list(range(i, world_size, model_parallel_size)) for i in range(model_parallel_size)]


class ProcessGroupManager:
    """Named sub-groups of a parent group."""

    def __init__(self, pg):
        self.pg = pg
        self._groups: Dict[str, object] = {}

    def create_group(self, name: str, ranks: Sequence[int]):
        if name in self._groups:
            raise ValueError(f"group {name!r} already exists")
        g = self.pg.new_subgroup(list(ranks)) if hasattr(self.pg, "new_subgroup") else None
        self._groups[name] = g
        return g

    def get(self, name: str):
        return self._groups[name]

    def names(self) -> List[str]:
        return sorted(self._groups)


# ------------------------------------------------------------------ MPI-style facade
@dataclass
class MPIConfig:
    """src/MLFramework/Communication/Backends/MPIConfig.cs: CUDA-aware transfers, thread level, eager buffer size."""
    use_cuda_aware: bool = True          # device tensors are sent as they are (NCCL p2p); False stages them through the host
    thread_level: str = "multiple"       # single | funneled | serialized | multiple
    buffer_size: int = 64 * 1024

    def validate(self):
        if self.thread_level not in ("single", "funneled", "serialized", "multiple"):
            raise ValueError(f"unknown thread level {self.thread_level!r}")
        if self.buffer_size <= 0:
            raise ValueError("buffer_size must be positive")


class MPIStyleBackend:
    """The reference's MPI back-end surface (collectives plus ``send`` / ``receive`` / ``probe`` / async variants:
    Communication/Backends/MPIBackend.cs:54-218) on this package's process groups. No MPI library is involved: the
    point-to-point calls are the group's (NCCL or gloo), messages carry a small header so that ``receive`` can size its
    buffer and ``probe`` can look before it takes."""
    name = "mpi"

    def __init__(self, pg, config: Optional[MPIConfig] = None):
        self.pg, self.cfg = pg, config or MPIConfig()
        self.cfg.validate()

    @property
    def rank(self) -> int:
        return self.pg.rank

    @property
    def world_size(self) -> int:
        return self.pg.world_size

    def _stage(self, t: torch.Tensor) -> torch.Tensor:
        return t if self.cfg.use_cuda_aware or not t.is_cuda else t.cpu()

    # ---- collectives
    def broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        self.pg.broadcast(t, root)
        return t

    def reduce(self, t: torch.Tensor, root: int = 0, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        self.pg.reduce(t, root, op)
        return t

    def all_reduce(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM) -> torch.Tensor:
        self.pg.all_reduce(t, op)
        return t

    def all_gather(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        return self.pg.all_gather(t, dim)

    def reduce_scatter(self, t: torch.Tensor, op: ReduceOp = ReduceOp.SUM, dim: int = 0) -> torch.Tensor:
        return self.pg.reduce_scatter(t, op, dim)

    def barrier(self):
        self.pg.barrier()

    # ---- point to point
    def send(self, t: torch.Tensor, dst: int, tag: int = 0):
        send_with_header(self.pg, self._stage(t), dst, tag)

    def probe(self, src: int, tag: int = 0, device="cpu") -> MessageInfo:
        return probe(self.pg, src, tag, device)

    def receive(self, src: int, tag: int = 0, device="cpu", info: Optional[MessageInfo] = None) -> torch.Tensor:
        """The next message from ``src`` (its shape and dtype come from the header, or from an earlier ``probe``)."""
        info = info or self.probe(src, tag, "cpu" if not self.cfg.use_cuda_aware else device)
        t = recv_probed(self.pg, info, "cpu" if not self.cfg.use_cuda_aware else device)
        return t.to(device)

    def send_async(self, t: torch.Tensor, dst: int, tag: int = 0):
        import concurrent.futures as cf
        ex = cf.ThreadPoolExecutor(max_workers=1)
        f = ex.submit(self.send, t, dst, tag)
        ex.shutdown(wait=False)
        return f

    def receive_async(self, src: int, tag: int = 0, device="cpu"):
        import concurrent.futures as cf
        ex = cf.ThreadPoolExecutor(max_workers=1)
        f = ex.submit(self.receive, src, tag, device)
        ex.shutdown(wait=False)
        return f

    def send_receive(self, t: torch.Tensor, dst: int, src: int) -> torch.Tensor:
        """Exchange of equal-shaped tensors (both directions in flight at once)."""
        return send_recv(self.pg, self._stage(t), dst, torch.empty_like(self._stage(t)), src).to(t.device)
