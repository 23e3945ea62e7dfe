"""Symmetric memory: buffers of equal size on every rank, each mapped into every peer.

``SymmetricMemory(pg)`` is created once per process group. ``alloc(nbytes)`` is collective: each
rank allocates with the native layer, the CUDA IPC handles are exchanged through the process
group, and every rank maps every peer's buffer. The result is a :class:`SymmBuffer` with a
local tensor view and the table of peer pointers the fused kernels take. With a single rank
(or in ``emulate`` mode on one GPU, used by tests) all "peer" buffers are local allocations.

Collectives over these buffers (device barrier, reduce-scatter with fused unscale/overflow
check, two-shot / one-shot all-reduce, peer copy) are thin wrappers over
``csrc/symm/symm_mem.cu``. The reference's counterparts are its NCCL / ring backends
(src/MLFramework/Communication/Backends/NCCLBackend.cs:157-309,
src/MLFramework/Distributed/RingAllReduce.cs:30-163) and its placeholder GPUDirect probe
(src/MLFramework/Communication/Optimizations/GPUDirectManager.cs:22-28).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from .. import _lib


class _RawCuda:
    """Adapter exposing a raw device pointer through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def tensor_from_ptr(ptr: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=device)


class SymmBuffer:
    def __init__(self, local_ptr: int, peer_ptrs: List[int], nbytes: int, device, rank: int):
        self.nbytes, self.rank, self.world = nbytes, rank, len(peer_ptrs)
        self.ptrs = peer_ptrs                     # ptrs[r] = address of rank r's buffer in this process
        self.local = tensor_from_ptr(local_ptr, nbytes, device)
        self._arr = (C.c_void_p * 8)(*[C.c_void_p(p) for p in peer_ptrs] + [None] * (8 - len(peer_ptrs)))

    def view(self, dtype: torch.dtype, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        t = self.local[offset_bytes:]
        t = t.view(dtype)
        return t if numel is None else t[:numel]

    def peer_table(self, offset_bytes: int = 0):
        if offset_bytes == 0:
            return self._arr
        return (C.c_void_p * 8)(*[C.c_void_p(p + offset_bytes) for p in self.ptrs] + [None] * (8 - self.world))

    def peer_view(self, r: int, dtype: torch.dtype, device) -> torch.Tensor:
        """Tensor over rank r's buffer as mapped here (debug / tests; loads cross NVLink)."""
        return tensor_from_ptr(self.ptrs[r], self.nbytes, device).view(dtype)


class SymmetricMemory:
    def __init__(self, pg=None, device=None, emulate_world: int = 0):
        self.pg = pg
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.emulate = emulate_world > 0
        self.world = emulate_world if self.emulate else (pg.world_size if pg is not None else 1)
        self.rank = 0 if (self.emulate or pg is None) else pg.rank
        self._lib = _lib.get()
        self._owned: List[int] = []
        self._opened: List[int] = []
        self._epoch = 0
        self._pad: Optional[SymmBuffer] = None

    # ---- allocation
    def alloc(self, nbytes: int) -> SymmBuffer:
        nbytes = (nbytes + 255) // 256 * 256
        if self.emulate:
            raise RuntimeError("use alloc_emulated() in emulate mode")
        if self.world > 1 and self.device.type == "cuda":
            # Allocation, handle export and the handle exchange block the host. Every rank reaches this call at the
            # same point of its program, so each one first lets its own queued kernels finish (their counterparts on
            # the peers are queued before the peers' own call): no GPU is left spinning on a peer while hosts wait.
            torch.cuda.synchronize(self.device)
        ptr = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        _lib.check(self._lib.mlf_symm_alloc(C.c_longlong(nbytes), C.byref(ptr), handle), "mlf_symm_alloc")
        self._owned.append(ptr.value)
        if self.world == 1:
            return SymmBuffer(ptr.value, [ptr.value], nbytes, self.device, 0)
        handles = self.pg.all_gather_object(bytes(handle))
        peers = []
        for r, h in enumerate(handles):
            if r == self.rank:
                peers.append(ptr.value)
                continue
            hb = (C.c_ubyte * 64).from_buffer_copy(h)
            pp = C.c_void_p()
            _lib.check(self._lib.mlf_symm_open(hb, C.byref(pp)), "mlf_symm_open")
            self._opened.append(pp.value)
            peers.append(pp.value)
        return SymmBuffer(ptr.value, peers, nbytes, self.device, self.rank)

    def alloc_emulated(self, nbytes: int) -> List[SymmBuffer]:
        """One GPU, ``emulate_world`` local buffers: returns the per-"rank" views of the same table."""
        nbytes = (nbytes + 255) // 256 * 256
        ptrs = []
        for _ in range(self.world):
            ptr = C.c_void_p()
            handle = (C.c_ubyte * 64)()
            _lib.check(self._lib.mlf_symm_alloc(C.c_longlong(nbytes), C.byref(ptr), handle), "mlf_symm_alloc")
            self._owned.append(ptr.value)
            ptrs.append(ptr.value)
        return [SymmBuffer(ptrs[r], ptrs, nbytes, self.device, r) for r in range(self.world)]

    # ---- synchronisation
    def barrier(self, stream=None):
        """Device-side barrier on the current stream: returns immediately on the host; kernels
        queued after it run only once every rank has reached the same point."""
        if self.world == 1 or self.emulate:
            return
        if self._pad is None:
            self._pad = self.alloc(8 * 32 * 4)
            self.pg.barrier()
        self._epoch += 1
        rc = self._lib.mlf_symm_barrier(self._pad.peer_table(), self.rank, self.world, C.c_uint(self._epoch),
                                        C.c_uint64(_lib.stream_handle(stream)))
        _lib.check(rc, "mlf_symm_barrier")

    # ---- collectives
    def rs_reduce(self, buf: SymmBuffer, segs_dev: torch.Tensor, n_segs: int, out: torch.Tensor, total_numel: int, *,
                  rank: Optional[int] = None, scale: float = 1.0, scale_ptr: Optional[torch.Tensor] = None,
                  found_inf: Optional[torch.Tensor] = None, sumsq: Optional[torch.Tensor] = None, offset_bytes: int = 0):
        r = self.rank if rank is None else rank
        p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
        rc = self._lib.mlf_rs_reduce(buf.peer_table(offset_bytes), self.world, r, p(segs_dev), n_segs, p(out),
                                     int(out.dtype == torch.float32), C.c_float(scale), p(scale_ptr), p(found_inf), p(sumsq),
                                     C.c_longlong(total_numel), C.c_uint64(_lib.stream_handle()))
        _lib.check(rc, "mlf_rs_reduce")

    def all_reduce_two_shot(self, buf: SymmBuffer, numel: int, scale: float = 1.0, rank: Optional[int] = None,
                            offset_bytes: int = 0):
        r = self.rank if rank is None else rank
        rc = self._lib.mlf_ar_two_shot(buf.peer_table(offset_bytes), self.world, r, C.c_longlong(numel), C.c_float(scale),
                                       C.c_uint64(_lib.stream_handle()))
        _lib.check(rc, "mlf_ar_two_shot")

    def all_reduce_one_shot(self, buf: SymmBuffer, out: torch.Tensor, numel: int, residual: Optional[torch.Tensor] = None,
                            rank: Optional[int] = None, offset_bytes: int = 0):
        r = self.rank if rank is None else rank
        rc = self._lib.mlf_ar_one_shot(buf.peer_table(offset_bytes), self.world, r, C.c_void_p(out.data_ptr()),
                                       C.c_longlong(numel), C.c_void_p(residual.data_ptr()) if residual is not None else None,
                                       C.c_uint64(_lib.stream_handle()))
        _lib.check(rc, "mlf_ar_one_shot")

    # ---- graph-replayable variants: the epoch is kept on the device (see mlf_ar_one_shot_sync)
    def _sync_pad(self, key: str = "main") -> SymmBuffer:
        """Signal pad + device epoch for one ordered sequence of in-kernel-synchronised launches. Launches
        that share a pad must be issued in the same order on every rank and on one stream per rank, so a
        side stream gets a pad of its own (``key``). Collective on first use."""
        pads = self.__dict__.setdefault("_gpads", {})
        if key not in pads:
            pads[key] = self.alloc(2048)           # [0, 1024): signal slots written by peers; [1024, 1032): local {epoch, count}
            if self.pg is not None and self.world > 1:
                self.pg.barrier()
        return pads[key]

    def alloc_flag(self) -> SymmBuffer:
        """An int32 flag in symmetric memory (the overflow flag every rank can raise on every rank)."""
        b = self.alloc(256)
        if self.pg is not None and self.world > 1:
            self.pg.barrier()
        return b

    def rs_reduce_sync(self, buf: SymmBuffer, segs_dev: torch.Tensor, n_segs: int, out: torch.Tensor, total_numel: int, *,
                       scale: float = 1.0, scale_ptr: Optional[torch.Tensor] = None, flag: Optional[SymmBuffer] = None,
                       sumsq: Optional[torch.Tensor] = None, offset_bytes: int = 0, key: str = "main", max_ctas: int = 0,
                       stream=None):
        """Reduce-scatter by peer reads whose arrival and departure synchronisation run inside the kernel
        (no barrier launch, no flag all-reduce): see ``rs_reduce_sync_kernel``."""
        pad = self._sync_pad(key)
        p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
        rc = self._lib.mlf_rs_reduce_sync(buf.peer_table(offset_bytes), pad.peer_table(), C.c_void_p(pad.ptrs[self.rank] + 1024),
                                          flag.peer_table() if flag is not None else None, self.world, self.rank, p(segs_dev), n_segs,
                                          p(out), int(out.dtype == torch.float32), C.c_float(scale), p(scale_ptr), p(sumsq),
                                          C.c_longlong(total_numel), max_ctas, C.c_uint64(_lib.stream_handle(stream)))
        _lib.check(rc, "mlf_rs_reduce_sync")

    def all_reduce_two_shot_sync(self, buf: SymmBuffer, numel: int, *, scale: float = 1.0, scale_ptr: Optional[torch.Tensor] = None,
                                 flag: Optional[SymmBuffer] = None, offset_bytes: int = 0, key: str = "main", max_ctas: int = 0,
                                 stream=None):
        """In-place all-reduce of ``numel`` bf16 elements at ``offset_bytes`` of every rank's ``buf``; the whole
        buffer holds the (scaled) sum when the launch completes on a rank."""
        pad = self._sync_pad(key)
        rc = self._lib.mlf_ar_two_shot_sync(buf.peer_table(offset_bytes), pad.peer_table(), C.c_void_p(pad.ptrs[self.rank] + 1024),
                                            flag.peer_table() if flag is not None else None, self.world, self.rank,
                                            C.c_longlong(numel), C.c_float(scale),
                                            C.c_void_p(scale_ptr.data_ptr()) if scale_ptr is not None else None, max_ctas,
                                            C.c_uint64(_lib.stream_handle(stream)))
        _lib.check(rc, "mlf_ar_two_shot_sync")

    def check_status(self):
        """Reads (and clears) the device status word; a wait on a peer that ran out of its budget raises
        ``CommunicationTimeout`` (the reference's TimeoutManager -> CommunicationTimeoutException path,
        src/MLFramework/Communication/FaultTolerance/TimeoutManager.cs:33-90). Synchronises the device."""
        raise_for_status(_lib.read_status(True))

    def all_reduce_one_shot_sync(self, buf: SymmBuffer, out: torch.Tensor, numel: int, residual: Optional[torch.Tensor] = None,
                                 offset_bytes: int = 0):
        """Sum of every rank's ``buf`` (at ``offset_bytes``) into ``out`` (+ residual); waits inside the kernel for
        all ranks to reach the call, so the producers of the buffers are complete. Alternate between two
        staging offsets from one call to the next: nothing waits at the end."""
        pad = self._sync_pad()
        rc = self._lib.mlf_ar_one_shot_sync(buf.peer_table(offset_bytes), pad.peer_table(), C.c_void_p(pad.ptrs[self.rank] + 1024),
                                            self.world, self.rank, C.c_void_p(out.data_ptr()), C.c_longlong(numel),
                                            C.c_void_p(residual.data_ptr()) if residual is not None else None,
                                            C.c_uint64(_lib.stream_handle()))
        _lib.check(rc, "mlf_ar_one_shot_sync")

    def sum_partials_sync(self, part: SymmBuffer, rows: int, cols: int, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                          residual: Optional[torch.Tensor] = None, offset_bytes: int = 0):
        """``out[rows, cols]`` = sum over the W planes the peers stored into this rank's ``part`` (+ bias, + residual),
        after waiting inside the kernel for every rank to reach the call (their stores, earlier on their streams, have
        then landed). Nothing waits at the end: alternate between two partial buffers from one call to the next."""
        pad = self._sync_pad()
        p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
        rc = self._lib.mlf_sum_partials_sync(C.c_void_p(part.ptrs[self.rank] + offset_bytes), pad.peer_table(),
                                             C.c_void_p(pad.ptrs[self.rank] + 1024), self.world, self.rank, C.c_longlong(rows), cols,
                                             p(out), C.c_longlong(out.stride(0)), p(bias), p(residual),
                                             C.c_longlong(residual.stride(0) if residual is not None else 0),
                                             C.c_uint64(_lib.stream_handle()))
        _lib.check(rc, "mlf_sum_partials_sync")

    def tp_argmax(self, logits: torch.Tensor, index_base: int, vocab: int, cand: SymmBuffer) -> torch.Tensor:
        """Arg-max over a vocabulary split across ranks (``logits`` = this rank's columns starting at ``index_base``)."""
        pad = self._sync_pad()
        rows, cols = logits.shape
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
        rc = self._lib.mlf_tp_argmax(C.c_void_p(logits.data_ptr()), C.c_longlong(rows), C.c_longlong(logits.stride(0)), cols, index_base,
                                     vocab, cand.peer_table(), pad.peer_table(), C.c_void_p(pad.ptrs[self.rank] + 1024), self.world,
                                     self.rank, C.c_void_p(out.data_ptr()), C.c_uint64(_lib.stream_handle()))
        _lib.check(rc, "mlf_tp_argmax")
        return out

    def peer_copy(self, segs_dev: torch.Tensor, n_segs: int, ctas: int = 0):
        rc = self._lib.mlf_peer_copy(C.c_void_p(segs_dev.data_ptr()), n_segs, ctas, C.c_uint64(_lib.stream_handle()))
        _lib.check(rc, "mlf_peer_copy")

    def close(self):
        torch.cuda.synchronize()
        for p in self._opened:
            self._lib.mlf_symm_close(C.c_void_p(p))
        for p in self._owned:
            self._lib.mlf_symm_free(C.c_void_p(p))
        self._opened, self._owned = [], []


ERR_WAIT_PEER_FLAG, ERR_WAIT_CHUNK_FLAG = 5, 6


def raise_for_status(status: int):
    """Maps a non-zero kernel status to an exception: waits on a peer become ``CommunicationTimeout``."""
    if status == 0:
        return
    from .process_group import CommunicationError, CommunicationTimeout
    if status in (ERR_WAIT_PEER_FLAG, ERR_WAIT_CHUNK_FLAG):
        raise CommunicationTimeout(f"a device-side wait on a peer ran out of its cycle budget (kernel status {status})")
    raise CommunicationError(f"a kernel reported status {status}")


def set_wait_budget_cycles(cycles: int):
    """Cycle budget of every bounded device-side wait on the current device (0 = the default of about 1.5 s)."""
    _lib.check(_lib.get().mlf_set_wait_budget_cycles(C.c_longlong(int(cycles))), "mlf_set_wait_budget_cycles")


def make_reduce_segs(segs: Sequence[tuple], device) -> torch.Tensor:
    """Device table of (src_off, dst_off, numel) int64 triples for :meth:`SymmetricMemory.rs_reduce`."""
    return torch.tensor([list(s) for s in segs], dtype=torch.int64, device=device).contiguous()


def make_copy_segs(segs: Sequence[tuple], device) -> torch.Tensor:
    """Device table of (src_ptr, dst_ptr, bytes) int64 triples for :meth:`SymmetricMemory.peer_copy`."""
    return torch.tensor([list(s) for s in segs], dtype=torch.int64, device=device).contiguous()
