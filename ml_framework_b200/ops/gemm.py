"""bf16 GEMM on the tcgen05 kernel, plus the plain-PyTorch oracle used on CPU and in tests.

``gemm(a, b)`` computes ``alpha * A @ B^T`` where each operand is given either K-major
(``[rows, K]``, the contraction index contiguous) or MN-major (``[K, rows]``). The three
training products of a linear layer ``y = x W^T`` (W ``[out, in]``) are therefore

* forward  ``y  = gemm(x,  W)``                       (both K-major)
* dgrad    ``dx = gemm(dy, W, b_mn=True)``            (W read as ``[K=out, N=in]``)
* wgrad    ``dW = gemm(dy, x, a_mn=True, b_mn=True)`` (dy read as ``[K=tokens, M=out]``)

Reference semantics: ``Tensor.Matmul`` (src/MLFramework/Tensor/TensorExtensions.cs:429-504),
``TensorMathExtensions.MatMul(transposeA, transposeB)``
(src/MLFramework/Layers/TensorParallel/TensorMathExtensions.cs:21).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _lib
from .._lib import (EPI_ACCUM, EPI_BIAS, EPI_DGELU_MUL, EPI_DSWIGLU, EPI_GELU, EPI_OUT_FP32,
                    EPI_RESIDUAL, EPI_STORE_PRE, EPI_SWIGLU, GemmArgs, GemmComm)

__all__ = ["gemm", "gemm_reference", "gelu_tanh_ref", "dgelu_tanh_ref"]


_piggyback = None

# bytes per second one copy CTA moves over NVLink (bulk async copies, eight 16 KB pieces in flight) and the GEMM rate
# used to estimate how long a product keeps its grid busy: together they decide how many parts of a queued copy
# table one GEMM carries
_COPY_CTA_BPS = 20e9
_GEMM_FLOPS = 1.2e15


def set_piggyback(segs: torch.Tensor, n_segs: int, n_copy_ctas: int = 16, on_attached=None, min_flops: float = 2e10,
                  part_rows: Optional[list] = None, part_bytes: Optional[list] = None, tag=None):
    """Queue a table of {src, dst, bytes} peer copies to ride on the next large plain GEMMs: such a launch gives
    ``n_copy_ctas`` of its CTAs to the copies (bulk async copies over NVLink) while the rest compute. Used to
    prefetch the next FSDP unit's parameters.

    With ``part_rows`` (row offsets ``[0, r1, ..., n_segs]`` of consecutive parts of the table) and ``part_bytes``
    (bytes per part) every qualifying GEMM takes only as many parts as its copy CTAs can move in the time the product
    takes, so the copies spread over the unit's GEMMs instead of stretching the first one; ``on_attached`` runs when
    the last part has been handed out. Without them the whole table rides on one GEMM."""
    global _piggyback
    if part_rows is None:
        part_rows, part_bytes = [0, n_segs], [0]
    _piggyback = {"segs": segs, "rows": list(part_rows), "bytes": list(part_bytes), "next": 0, "ctas": n_copy_ctas,
                  "cb": on_attached, "min_flops": min_flops, "tag": tag}


def clear_piggyback():
    """Drop a queued piggyback that no GEMM picked up (the caller then copies by itself)."""
    global _piggyback
    _piggyback = None


def pending_piggyback(tag=None):
    """(table, first_row, n_rows) of the queued copies that no GEMM has taken yet (for ``tag`` when given), or None.
    The queue is cleared: the caller copies the rest itself."""
    global _piggyback
    pb = _piggyback
    if pb is None or (tag is not None and pb["tag"] != tag):
        return None
    _piggyback = None
    first = pb["rows"][pb["next"]]
    n = pb["rows"][-1] - first
    return (pb["segs"], first, n) if n > 0 else None


def _take_piggyback(M, N, K, comm):
    global _piggyback
    pb = _piggyback
    flops = 2.0 * M * N * K
    if pb is None or comm is not None or flops < pb["min_flops"]:
        return None
    n_parts = len(pb["rows"]) - 1
    i = pb["next"]
    # as many parts as the copy CTAs move while the product runs (at least one)
    budget = flops / _GEMM_FLOPS * pb["ctas"] * _COPY_CTA_BPS
    j, moved = i + 1, pb["bytes"][i]
    while j < n_parts and moved + pb["bytes"][j] <= budget:
        moved += pb["bytes"][j]
        j += 1
    first, n = pb["rows"][i], pb["rows"][j] - pb["rows"][i]
    pb["next"] = j
    if j >= n_parts:
        _piggyback = None
        if pb["cb"] is not None:
            pb["cb"]()
    if n <= 0:
        return None
    cm = GemmComm()
    cm.n_copy_ctas, cm.extra_segs, cm.n_extra = pb["ctas"], pb["segs"].data_ptr() + first * 24, n
    return cm


def gelu_tanh_ref(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(x, approximate="tanh")


def dgelu_tanh_ref(x: torch.Tensor) -> torch.Tensor:
    k0, k1 = 0.7978845608028654, 0.044715
    u = k0 * (x + k1 * x ** 3)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * k0 * (1 + 3 * k1 * x * x)


def gemm_reference(a, b, *, a_mn=False, b_mn=False, bias=None, aux_in=None, flags=0, alpha=1.0,
                   prev_out=None):
    """fp32 PyTorch statement of what the kernel computes. Returns (out_fp32, pre_fp32)."""
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    v = alpha * (A @ B.t())
    if flags & EPI_BIAS:
        v = v + bias.float()
    pre = v.clone()
    if flags & EPI_GELU:
        v = gelu_tanh_ref(v)
    if flags & EPI_RESIDUAL:
        v = v + aux_in.float()
    if flags & EPI_DGELU_MUL:
        v = v * dgelu_tanh_ref(aux_in.float())
    if flags & EPI_SWIGLU:
        g, u = v[:, 0::2], v[:, 1::2]
        v = torch.nn.functional.silu(g) * u
    if flags & EPI_DSWIGLU:
        gu = aux_in.float()
        g, u = gu[:, 0::2], gu[:, 1::2]
        sg = torch.sigmoid(g)
        out = torch.empty(v.shape[0], v.shape[1] * 2, dtype=torch.float32, device=v.device)
        out[:, 0::2] = v * u * sg * (1 + g * (1 - sg))
        out[:, 1::2] = v * g * sg
        v = out
    if flags & EPI_ACCUM:
        v = v + prev_out.float()
    return v, pre


def _rows_k(t: torch.Tensor, mn: bool):
    if t.dim() != 2:
        raise ValueError("gemm operands must be 2-D")
    if t.stride(1) != 1:
        raise ValueError("gemm operands must have a contiguous last dimension")
    return (t.shape[1], t.shape[0]) if mn else (t.shape[0], t.shape[1])


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
         aux_in: Optional[torch.Tensor] = None, aux_out: Optional[torch.Tensor] = None,
         flags: int = 0, alpha: float = 1.0, out_dtype: torch.dtype = torch.bfloat16,
         tile_n: int = 0, max_ctas: int = 0, comm: Optional[GemmComm] = None,
         m_override: Optional[int] = None, n_override: Optional[int] = None) -> torch.Tensor:
    """``out = epilogue(alpha * A @ B^T)``; see the module docstring for operand layouts.

    ``m_override`` / ``n_override`` give the logical row count of an operand that is gathered
    inside the kernel (``comm.gather_operand``), where ``a`` / ``b`` only hold the local shard.
    """
    M, K = _rows_k(a, a_mn)
    N, Kb = _rows_k(b, b_mn)
    if m_override is not None:
        M = m_override
    if n_override is not None:
        N = n_override
    if K != Kb:
        raise ValueError(f"contraction mismatch: {K} vs {Kb}")
    if bias is not None:
        flags |= EPI_BIAS
    if out_dtype == torch.float32:
        flags |= EPI_OUT_FP32
    out_cols = N // 2 if flags & EPI_SWIGLU else (2 * N if flags & EPI_DSWIGLU else N)
    if not a.is_cuda:
        v, pre = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, aux_in=aux_in, flags=flags,
                                alpha=alpha, prev_out=out)
        if aux_out is not None and flags & EPI_STORE_PRE:
            aux_out.copy_(pre.to(aux_out.dtype))
        res = v.to(out_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm expects bf16 operands on the GPU")
    if out is None:
        out = torch.empty((M, out_cols), dtype=out_dtype, device=a.device)
    else:
        # The epilogue's stores are sized from M, N and the pitch: anything else would be written past its end.
        scatter = comm is not None and bool(comm.scatter_out)
        want = (int(comm.rows_per_owner) if scatter else M, out_cols)      # routed rows land in the owners' partial buffers
        if out.dim() != 2 or out.shape[1] != want[1] or (out.shape[0] < want[0] if scatter else out.shape[0] != want[0]):
            raise ValueError(f"out has shape {tuple(out.shape)}, the product needs {want}")
        if out.dtype != out_dtype:
            raise ValueError(f"out is {out.dtype}, the epilogue writes {out_dtype}")
        if out.device != a.device:
            raise ValueError("out is on another device than the operands")
        if out.stride(-1) != 1 or out.data_ptr() % 16 or (out.stride(0) * out.element_size()) % 16:
            raise ValueError("out needs a contiguous last dimension, a 16-byte aligned base and a 16-byte multiple row pitch")
    for name, t, cols in (("aux_in", aux_in, 2 * N if flags & EPI_DSWIGLU else N), ("aux_out", aux_out, N)):
        if t is None:
            continue
        if t.dim() != 2 or t.shape[0] != M or t.shape[1] != cols or t.dtype != torch.bfloat16 or t.device != a.device \
                or t.stride(-1) != 1:
            raise ValueError(f"{name} must be a bf16 [{M}, {cols}] tensor on the operands' device with a contiguous last "
                             f"dimension, got {tuple(t.shape)} {t.dtype}")
    args = GemmArgs()
    args.a, args.b, args.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.bias = bias.data_ptr() if bias is not None else None
    args.aux_in = aux_in.data_ptr() if aux_in is not None else None
    args.aux_out = aux_out.data_ptr() if aux_out is not None else None
    args.M, args.N, args.K = M, N, K
    args.lda, args.ldb, args.ldo = a.stride(0), b.stride(0), out.stride(0)
    args.ld_aux_in = aux_in.stride(0) if aux_in is not None else 0
    args.ld_aux_out = aux_out.stride(0) if aux_out is not None else 0
    args.a_mn, args.b_mn = int(a_mn), int(b_mn)
    args.flags, args.alpha = flags, alpha
    args.tile_n, args.max_ctas = tile_n, max_ctas
    if comm is None and _piggyback is not None:
        comm = _take_piggyback(M, N, K, comm)
    args.comm = C.pointer(comm) if comm is not None else None
    rc = _lib.get().mlf_gemm_bf16(C.byref(args), C.c_uint64(_lib.stream_handle()))
    _lib.check(rc, "mlf_gemm_bf16")
    return out
