"""Python face of the native CUDA runtime binding (``csrc/hal/cuda_rt.cpp``): devices, raw memory, streams, events
and graphs, as thin classes over a C ABI reached with ``ctypes``.

The reference declares the same surface as P/Invoke signatures (src/MLFramework/HAL/CUDA/CudaApi.cs:19-184) with
safe-handle wrappers (CudaSafeHandles.cs, CudaStream.cs, CudaEvent.cs, CudaDevice.cs) and an error type
(CudaError.cs). Here every handle class owns its native object and releases it in ``close`` / on garbage
collection; failures raise :class:`CudaRuntimeError` with the runtime's message.

``Graph.node_kinds()`` returns the node types of a real captured ``cudaGraph_t``; the graph validator
(:mod:`ml_framework_b200.hal.cuda_graphs`) validates captures against that list.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional

from .. import _lib


class CudaRuntimeError(RuntimeError):
    """A CUDA runtime call failed (the reference's ``CudaException`` over ``CudaError``)."""


def _check(rc: int, what: str):
    if rc != 0:
        msg = _lib.get().mlf_last_error()
        raise CudaRuntimeError(f"{what} failed (rc={rc}): {msg.decode() if msg else ''}")


def _L():
    return _lib.get()


# cudaGraphNodeType values of the runtime
NODE_KINDS = {0: "kernel", 1: "memcpy", 2: "memset", 3: "host", 4: "graph", 5: "empty", 6: "wait_event", 7: "event_record",
              8: "ext_semaphore_signal", 9: "ext_semaphore_wait", 10: "mem_alloc", 11: "mem_free", 12: "batch_mem_op", 13: "conditional"}

MEMCPY_KINDS = {"h2h": 0, "h2d": 1, "d2h": 2, "d2d": 3, "default": 4}


def device_count() -> int:
    n = C.c_int(0)
    _check(_L().mlf_rt_device_count(C.byref(n)), "device_count")
    return n.value


def set_device(index: int):
    _check(_L().mlf_rt_set_device(int(index)), "set_device")


def current_device() -> int:
    d = C.c_int(0)
    _check(_L().mlf_rt_get_device(C.byref(d)), "get_device")
    return d.value


def device_properties(index: int = 0) -> Dict[str, object]:
    props = (C.c_longlong * 8)()
    name = C.create_string_buffer(256)
    _check(_L().mlf_rt_device_properties(int(index), props, name, 256), "device_properties")
    return {"name": name.value.decode(), "multiprocessors": props[0], "compute_capability": (props[1], props[2]),
            "total_memory_mib": props[3], "max_shared_memory_per_block": props[4], "l2_bytes": props[5],
            "sm_clock_khz": props[6], "memory_bus_bits": props[7]}


def synchronize():
    _check(_L().mlf_rt_device_synchronize(), "device_synchronize")


def mem_info():
    f, t = C.c_longlong(0), C.c_longlong(0)
    _check(_L().mlf_rt_mem_info(C.byref(f), C.byref(t)), "mem_info")
    return f.value, t.value


class DeviceBuffer:
    """Raw device (or pinned host) allocation with explicit lifetime."""

    def __init__(self, nbytes: int, pinned_host: bool = False):
        self.nbytes, self.pinned_host = int(nbytes), pinned_host
        p = C.c_uint64(0)
        fn = _L().mlf_rt_malloc_host if pinned_host else _L().mlf_rt_malloc
        _check(fn(C.c_longlong(self.nbytes), C.byref(p)), "malloc_host" if pinned_host else "malloc")
        self.ptr: Optional[int] = p.value

    def close(self):
        if self.ptr:
            fn = _L().mlf_rt_free_host if self.pinned_host else _L().mlf_rt_free
            _check(fn(C.c_uint64(self.ptr)), "free")
            self.ptr = None

    def memset(self, value: int, stream: Optional["Stream"] = None):
        _check(_L().mlf_rt_memset(C.c_uint64(self.ptr), int(value), C.c_longlong(self.nbytes),
                                  C.c_uint64(stream.handle if stream else 0), 1 if stream else 0), "memset")

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def memcpy(dst: int, src: int, nbytes: int, kind: str = "default", stream: Optional["Stream"] = None):
    _check(_L().mlf_rt_memcpy(C.c_uint64(dst), C.c_uint64(src), C.c_longlong(nbytes), MEMCPY_KINDS[kind],
                              C.c_uint64(stream.handle if stream else 0), 1 if stream else 0), "memcpy")


class Event:
    def __init__(self, timing: bool = True):
        h = C.c_uint64(0)
        _check(_L().mlf_rt_event_create(1 if timing else 0, C.byref(h)), "event_create")
        self.handle: Optional[int] = h.value

    def record(self, stream: Optional["Stream"] = None):
        _check(_L().mlf_rt_event_record(C.c_uint64(self.handle), C.c_uint64(stream.handle if stream else 0)), "event_record")

    def synchronize(self):
        _check(_L().mlf_rt_event_synchronize(C.c_uint64(self.handle)), "event_synchronize")

    def query(self) -> bool:
        d = C.c_int(0)
        _check(_L().mlf_rt_event_query(C.c_uint64(self.handle), C.byref(d)), "event_query")
        return bool(d.value)

    def elapsed_ms(self, later: "Event") -> float:
        ms = C.c_float(0)
        _check(_L().mlf_rt_event_elapsed_ms(C.c_uint64(self.handle), C.c_uint64(later.handle), C.byref(ms)), "event_elapsed")
        return ms.value

    def close(self):
        if self.handle:
            _check(_L().mlf_rt_event_destroy(C.c_uint64(self.handle)), "event_destroy")
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Stream:
    def __init__(self, non_blocking: bool = True, priority: int = 0, handle: Optional[int] = None):
        """``handle`` wraps an existing stream (e.g. ``torch.cuda.Stream.cuda_stream``) without owning it."""
        self._owned = handle is None
        if handle is None:
            h = C.c_uint64(0)
            _check(_L().mlf_rt_stream_create(1 if non_blocking else 0, int(priority), C.byref(h)), "stream_create")
            handle = h.value
        self.handle: Optional[int] = handle

    def synchronize(self):
        _check(_L().mlf_rt_stream_synchronize(C.c_uint64(self.handle)), "stream_synchronize")

    def query(self) -> bool:
        d = C.c_int(0)
        _check(_L().mlf_rt_stream_query(C.c_uint64(self.handle), C.byref(d)), "stream_query")
        return bool(d.value)

    def wait_event(self, ev: Event):
        _check(_L().mlf_rt_stream_wait_event(C.c_uint64(self.handle), C.c_uint64(ev.handle)), "stream_wait_event")

    def record_event(self, timing: bool = True) -> Event:
        e = Event(timing)
        e.record(self)
        return e

    # ---- capture
    def begin_capture(self, mode: str = "thread_local"):
        m = {"global": 0, "thread_local": 1, "relaxed": 2}[mode]
        _check(_L().mlf_rt_stream_begin_capture(C.c_uint64(self.handle), m), "stream_begin_capture")

    def end_capture(self) -> "Graph":
        g = C.c_uint64(0)
        _check(_L().mlf_rt_stream_end_capture(C.c_uint64(self.handle), C.byref(g)), "stream_end_capture")
        return Graph(g.value)

    def is_capturing(self) -> bool:
        c = C.c_int(0)
        _check(_L().mlf_rt_stream_is_capturing(C.c_uint64(self.handle), C.byref(c)), "stream_is_capturing")
        return bool(c.value)

    def close(self):
        if self.handle and self._owned:
            _check(_L().mlf_rt_stream_destroy(C.c_uint64(self.handle)), "stream_destroy")
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Graph:
    """A ``cudaGraph_t``. ``owned=False`` wraps a graph that somebody else destroys (a torch capture kept alive)."""

    def __init__(self, handle: int, owned: bool = True):
        self.handle: Optional[int] = handle
        self._owned = owned

    def node_types(self) -> List[int]:
        n = C.c_int(0)
        _check(_L().mlf_rt_graph_get_nodes(C.c_uint64(self.handle), None, 0, C.byref(n)), "graph_get_nodes")
        if n.value == 0:
            return []
        arr = (C.c_int * n.value)()
        _check(_L().mlf_rt_graph_get_nodes(C.c_uint64(self.handle), arr, n.value, C.byref(n)), "graph_get_nodes")
        return list(arr)

    def node_kinds(self) -> List[str]:
        return [NODE_KINDS.get(t, f"type{t}") for t in self.node_types()]

    def instantiate(self) -> "GraphExec":
        x = C.c_uint64(0)
        _check(_L().mlf_rt_graph_instantiate(C.c_uint64(self.handle), C.byref(x)), "graph_instantiate")
        return GraphExec(x.value)

    def close(self):
        if self.handle and self._owned:
            _check(_L().mlf_rt_graph_destroy(C.c_uint64(self.handle)), "graph_destroy")
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GraphExec:
    def __init__(self, handle: int):
        self.handle: Optional[int] = handle

    def launch(self, stream: Optional[Stream] = None):
        _check(_L().mlf_rt_graph_launch(C.c_uint64(self.handle), C.c_uint64(stream.handle if stream else 0)), "graph_launch")

    def close(self):
        if self.handle:
            _check(_L().mlf_rt_graph_exec_destroy(C.c_uint64(self.handle)), "graph_exec_destroy")
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
