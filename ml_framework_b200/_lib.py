"""ctypes loader for ``libmlfb200.so`` and mirrors of the structs in ``csrc/mlf_api.h``.

The library is built in-tree by :mod:`ml_framework_b200._build`. On a machine with a GPU the
kernels are mandatory: if the shared object is missing it is built on the spot, and if that
fails the import error is raised (there is no silent PyTorch fallback for GPU tensors).
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "libmlfb200.so"
_lock = threading.Lock()
_lib = None


class MlfError(RuntimeError):
    """Raised when a native call reports a host-side failure."""


class KernelStatusError(RuntimeError):
    """Raised when a kernel reported an expired bounded wait or a rejected index."""


class GemmComm(C.Structure):
    _fields_ = [
        ("gather_operand", C.c_int), ("world", C.c_int), ("rank", C.c_int), ("n_copy_ctas", C.c_int),
        ("rows_per_rank", C.c_int), ("flag_rows", C.c_int), ("row_bytes", C.c_int), ("_pad0", C.c_int),
        ("src", C.c_void_p * 8),
        ("gathered", C.c_void_p), ("flags", C.c_void_p), ("counters", C.c_void_p),
        ("scatter_out", C.c_int), ("rows_per_owner", C.c_int),
        ("out_peer", C.c_void_p * 8),
        ("extra_segs", C.c_void_p), ("n_extra", C.c_int), ("_pad1", C.c_int),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("b", C.c_void_p), ("out", C.c_void_p), ("bias", C.c_void_p),
        ("aux_in", C.c_void_p), ("aux_out", C.c_void_p),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("lda", C.c_int), ("ldb", C.c_int), ("ldo", C.c_int), ("ld_aux_in", C.c_int), ("ld_aux_out", C.c_int),
        ("a_mn", C.c_int), ("b_mn", C.c_int), ("flags", C.c_int), ("alpha", C.c_float),
        ("tile_n", C.c_int), ("max_ctas", C.c_int),
        ("comm", C.POINTER(GemmComm)),
    ]


EPI_BIAS, EPI_GELU, EPI_STORE_PRE, EPI_RESIDUAL, EPI_DGELU_MUL = 1, 2, 4, 8, 16
EPI_ACCUM, EPI_OUT_FP32, EPI_SWIGLU, EPI_DSWIGLU = 32, 64, 128, 256

STATUS_NAMES = {
    1: "wait for a free shared-memory stage expired",
    2: "wait for a filled shared-memory stage expired",
    3: "wait for a free TMEM accumulator expired",
    4: "wait for a finished TMEM accumulator expired",
    5: "wait for a peer flag expired",
    6: "wait for a gathered chunk expired",
    7: "an index was rejected by a bounds check",
    8: "attention pipeline wait expired",
}


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    """True when the native library can be loaded (built or buildable)."""
    try:
        get()
        return True
    except Exception:
        return False


def get() -> C.CDLL:
    """Load (building first if necessary) and return the native library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from . import _build
        if not _LIB_PATH.exists() or os.environ.get("MLF_REBUILD") == "1":
            _build.build(force=os.environ.get("MLF_REBUILD") == "1")
        elif _build.stale():
            # a source or header is newer than the library: a stale library would be called with the
            # new argument lists, so rebuild when a compiler is at hand and refuse to load otherwise
            _build.build()
        lib = C.CDLL(str(_LIB_PATH))
        lib.mlf_last_error.restype = C.c_char_p
        if os.environ.get("MLF_FLASH_BWD_WS") is not None:
            lib.mlf_set_flash_bwd_ws(int(os.environ["MLF_FLASH_BWD_WS"]))
        if os.environ.get("MLF_FLASH_WS") is not None:
            lib.mlf_set_flash_ws(int(os.environ["MLF_FLASH_WS"]))
        if os.environ.get("MLF_GEMM_2CTA") is not None:
            lib.mlf_set_gemm_2cta(int(os.environ["MLF_GEMM_2CTA"]))
        if os.environ.get("MLF_GEMM_SMALL_M_SPLIT") is not None:
            lib.mlf_set_gemm_small_m_split(int(os.environ["MLF_GEMM_SMALL_M_SPLIT"]))
        _lib = lib
        return lib


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = get().mlf_last_error()
        raise MlfError(f"{what or 'native call'} failed (rc={rc}): {msg.decode() if msg else ''}")


def read_status(clear: bool = True) -> int:
    """Synchronise and return the per-device kernel status word (0 = clean)."""
    return int(get().mlf_read_status(1 if clear else 0))


def raise_on_status() -> None:
    s = read_status(True)
    if s != 0:
        raise KernelStatusError(f"kernel status {s}: {STATUS_NAMES.get(s, 'unknown')}")


def stream_handle(stream=None) -> int:
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return int(s.cuda_stream)
