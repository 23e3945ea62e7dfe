"""Tensor parallelism (Megatron style) with optional sequence parallelism.

Layer semantics follow the reference (src/MLFramework/Layers/TensorParallel/ColumnParallelLinear.cs:54-143,
RowParallelLinear.cs:55-167, *WithInputGather.cs): a column-parallel linear holds the weight
shard ``[out/W, in]`` and bias shard ``[out/W]`` (``out % W == 0``), computes
``Y_local = X W_shard^T + b_shard`` and optionally all-gathers the output on the last dimension;
a row-parallel linear holds ``[out, in/W]`` (``in % W == 0``), takes an input that is already split
on the last dimension (or slices it), sums the partial products over ranks and adds the unsharded
bias once, after the reduction. Init: N(0, sqrt(2 / (in + out))).

Backward is complete here, unlike the reference whose column backward omits the all-reduce of
dX (Layers/TensorParallel/ColumnParallelLinearGrad.cs:120-166): the f / g operators of Megatron
are autograd functions (identity forward + all-reduce backward, and vice versa).

With ``sequence_parallel`` activations between blocks are sharded over tokens ``[T/W, d]``; the
column layer then computes all-gather(X) -> GEMM and the row layer GEMM -> reduce-scatter. On
GPUs with peer-mapped memory these run as ONE kernel each (copy CTAs pulling the peers' token
chunks while tensor-core CTAs consume them; epilogue stores routed to the owning rank), see
``csrc/gemm/gemm_tcgen05.cu``. Otherwise they are process-group collectives around the GEMM.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _lib
from ..dist.process_group import ReduceOp
from ..ops import functional as Fm
from ..ops.gemm import gemm


import os as _os

_DEBUG_ALLOC = _os.environ.get("MLF_DEBUG_ALLOC") == "1"     # log every collective buffer allocation with its time


# ------------------------------------------------------------------ context
class TPContext:
    """Tensor-parallel group state: communicator, rank, and the fused-kernel resources."""

    def __init__(self, pg, symm=None, fused: bool = True, n_copy_ctas: int = 16):
        self.pg = pg
        self.world = pg.world_size if pg is not None else 1
        self.rank = pg.rank if pg is not None else 0
        self.symm = symm
        self.fused = bool(fused and symm is not None and self.world > 1)
        self.n_copy_ctas = n_copy_ctas
        self._bufs: Dict[tuple, object] = {}
        self._flags: Dict[int, torch.Tensor] = {}

    def symm_buffer(self, key: str, nbytes: int):
        k = (key, nbytes)
        if k not in self._bufs:
            if _DEBUG_ALLOC:
                import sys, time
                print(f"[tp alloc] rank {self.rank} t={time.time() % 1000:.3f} {key} {nbytes}", file=sys.stderr, flush=True)
            self._bufs[k] = self.symm.alloc(nbytes)
        return self._bufs[k]

    def flags(self, n: int, device) -> torch.Tensor:
        if n not in self._flags:
            self._flags[n] = torch.zeros(2 * n, dtype=torch.int32, device=device)
        return self._flags[n]


_GLOBAL: Optional[TPContext] = None


def initialize(pg, symm=None, fused: bool = True) -> TPContext:
    """``TensorParallel.Initialize`` (src/MLFramework/Layers/TensorParallel/TensorParallel.cs:53)."""
    global _GLOBAL
    _GLOBAL = TPContext(pg, symm, fused)
    return _GLOBAL


def get_context() -> TPContext:
    if _GLOBAL is None:
        raise RuntimeError("tensor parallelism is not initialised")
    return _GLOBAL


def get_world_size() -> int:
    return get_context().world


def get_rank() -> int:
    return get_context().rank


# ------------------------------------------------------------------ f / g and SP operators
class _CopyToTP(torch.autograd.Function):      # f: identity forward, all-reduce backward
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        if ctx.tp.world > 1:
            ctx.tp.pg.all_reduce(g, ReduceOp.SUM)
        return g, None


class _ReduceFromTP(torch.autograd.Function):  # g: all-reduce forward, identity backward
    @staticmethod
    def forward(ctx, x, tp):
        x = x.contiguous()
        if tp.world > 1:
            tp.pg.all_reduce(x, ReduceOp.SUM)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherLastDim(torch.autograd.Function):  # all-gather on last dim fwd, slice bwd
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return tp.pg.all_gather(x, dim=-1) if tp.world > 1 else x

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        return (g.chunk(tp.world, dim=-1)[tp.rank].contiguous() if tp.world > 1 else g), None


class _GatherTokens(torch.autograd.Function):   # SP: all-gather tokens fwd, reduce-scatter bwd
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return tp.pg.all_gather(x, dim=0) if tp.world > 1 else x

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        return (tp.pg.reduce_scatter(g.contiguous(), ReduceOp.SUM, dim=0) if tp.world > 1 else g), None


class _ScatterTokens(torch.autograd.Function):  # SP: reduce-scatter tokens fwd, all-gather bwd
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return tp.pg.reduce_scatter(x.contiguous(), ReduceOp.SUM, dim=0) if tp.world > 1 else x

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        return (tp.pg.all_gather(g.contiguous(), dim=0) if tp.world > 1 else g), None


def copy_to_tp_region(x, tp): return _CopyToTP.apply(x, tp)
def reduce_from_tp_region(x, tp): return _ReduceFromTP.apply(x, tp)
def gather_last_dim(x, tp): return _GatherLastDim.apply(x, tp)
def gather_tokens(x, tp): return _GatherTokens.apply(x, tp)
def scatter_tokens(x, tp): return _ScatterTokens.apply(x, tp)


# ------------------------------------------------------------------ fused kernels (GPU, peer memory)
def _copy_ctas_for(tp: TPContext, flops: float, link_bytes: float) -> int:
    """Copy CTAs of a gather GEMM: enough of them (about 25 GB/s each over NVLink) to move the remote rows in the
    time the product takes, or in the time the links need when those are the bound; a multiple of 8 between 8 and 40
    (the kernel forms groups of up to 8 copy CTAs per row chunk, and the group size has to divide the count)."""
    t = max(flops / 1.4e15, link_bytes / 700e9, 1e-6)
    n = int(min(40, max(8, -(-link_bytes // (25e9 * t)))))
    return (n + 7) // 8 * 8


def _fused_ag_gemm(tp: TPContext, x_shard: torch.Tensor, w: torch.Tensor, key: str, bias=None, flags=0, aux_out=None,
                   b_mn: bool = False, persistent: bool = True):
    """out[T, N] = all_gather_tokens(x_shard)[T, K] @ B in one kernel, B = w[N, K]^T or, with ``b_mn``, w[K, N].
    Returns (out, x_full).

    The gathered operand lives in a symmetric buffer ``[T, K]`` per ``key``: this rank's shard is written into its own
    row range there, the peers pull exactly that range, and the copy CTAs of the GEMM fetch only the W - 1 remote
    ranges (the local rows need no copy). ``persistent`` buffers are one per key (the forward operand is kept for the
    weight gradient); otherwise two buffers per shape alternate between calls (backward operands are consumed at once)."""
    rows, K = x_shard.shape
    W, T = tp.world, x_shard.shape[0] * tp.world
    live = tp.__dict__.setdefault("_ag_live", {})
    if persistent and live.get(key, 0) > 0:
        # the buffer of this key still holds an operand whose backward has not run (several micro-batches in flight
        # without recomputation): this call gathers into memory of its own from a staged copy of the shard
        stage = tp.symm_buffer(key + ".ag_stage", rows * K * 2)
        stage.view(torch.bfloat16, rows * K).view(rows, K).copy_(x_shard)
        x_full = torch.empty(T, K, dtype=torch.bfloat16, device=x_shard.device)
        src = [stage.ptrs[r] for r in range(W)]
    else:
        if persistent:
            buf = tp.symm_buffer(key + ".ag_full", T * K * 2)
        else:
            n = tp._ag_calls = getattr(tp, "_ag_calls", 0) + 1
            buf = tp.symm_buffer(f"ag_tmp{n % 2}.{T}x{K}", T * K * 2)
        x_full = buf.view(torch.bfloat16, T * K).view(T, K)
        x_full[tp.rank * rows:(tp.rank + 1) * rows].copy_(x_shard)
        src = [buf.ptrs[r] + r * rows * K * 2 for r in range(W)]     # rank r's own rows inside rank r's buffer
    tp.symm.barrier()                                   # every peer's rows are written
    flag_rows = 128
    while rows % flag_rows:
        flag_rows //= 2
    nfl = T // max(flag_rows, 1)
    fl = tp.flags(nfl, x_shard.device)
    fl.zero_()
    N = w.shape[1] if b_mn else w.shape[0]
    cm = _lib.GemmComm()
    cm.gather_operand, cm.world, cm.rank = 1, W, tp.rank
    cm.n_copy_ctas = _copy_ctas_for(tp, 2.0 * T * K * N, (W - 1) * rows * K * 2.0)
    cm.rows_per_rank, cm.flag_rows, cm.row_bytes = rows, flag_rows, K * 2
    for r in range(W):
        cm.src[r] = src[r]
    cm.gathered, cm.flags, cm.counters = x_full.data_ptr(), fl.data_ptr(), fl[nfl:].data_ptr()
    out = gemm(x_shard, w, comm=cm, m_override=T, bias=bias, flags=flags, aux_out=aux_out, b_mn=b_mn)
    return out, x_full


def _fused_gemm_rs(tp: TPContext, a: torch.Tensor, b: torch.Tensor, key: str, *, b_mn=False, bias=None, residual=None):
    """out[T/W, N] = reduce_scatter_tokens(a[T, K] @ B^T): epilogue stores routed to the owners, then a local sum."""
    T = a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    W = tp.world
    rows = T // W
    # two partial buffers per shape, shared by every layer and used alternately: the arrival wait inside the sum of
    # call n - 1 tells this rank that every peer has finished the sum of call n - 2, i.e. is done reading the buffer
    # that this call's epilogue is about to store into -- no barrier launch before or after the product
    n = tp.__dict__.setdefault("_rs_calls", {})
    n[(rows, N)] = n.get((rows, N), 0) + 1
    part = tp.symm_buffer(f"rs_part{n[(rows, N)] % 2}.{rows}x{N}", W * rows * N * 2)
    cm = _lib.GemmComm()
    cm.scatter_out, cm.rows_per_owner, cm.world, cm.rank = 1, rows, W, tp.rank
    for r in range(W):
        cm.out_peer[r] = part.ptrs[r]
    dummy = part.view(torch.bfloat16, rows * N).view(rows, N)
    gemm(a, b, b_mn=b_mn, out=dummy, comm=cm, m_override=T)
    out = torch.empty(rows, N, dtype=torch.bfloat16, device=a.device)
    tp.symm.sum_partials_sync(part, rows, N, out, bias, residual)
    return out


class _ColumnSPFused(torch.autograd.Function):
    """Sequence-parallel column linear on the fused kernels: AG->GEMM forward, GEMM->RS backward."""

    @staticmethod
    def forward(ctx, x_shard, w, b, tp, key):
        out, x_full = _fused_ag_gemm(tp, x_shard, w, key, bias=b)
        ctx.save_for_backward(x_full, w)
        ctx.tp, ctx.key, ctx.b = tp, key, b
        ctx.counted = torch.is_grad_enabled() or any(ctx.needs_input_grad[:3])
        if ctx.counted:
            live = tp.__dict__.setdefault("_ag_live", {})
            live[key] = live.get(key, 0) + 1          # the key's gathered buffer is spoken for until backward has read it
        return out

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx_shard = _fused_gemm_rs(ctx.tp, dy, w, ctx.key + ".bwd", b_mn=True)
        dw = Fm._wgrad(dy, x_full, w)
        db = Fm._bgrad(dy, ctx.b)
        if ctx.counted:
            live = ctx.tp.__dict__.setdefault("_ag_live", {})
            live[ctx.key] = max(0, live.get(ctx.key, 0) - 1)
        return dx_shard, dw, db, None, None


class _RowSPFused(torch.autograd.Function):
    """Sequence-parallel row linear: GEMM->RS forward (bias / residual added after the sum), AG->GEMM backward."""

    @staticmethod
    def forward(ctx, x, w, b, residual, tp, key):
        out = _fused_gemm_rs(tp, x, w, key, bias=b, residual=residual)
        ctx.save_for_backward(x, w)
        ctx.tp, ctx.key, ctx.b, ctx.has_res = tp, key, b, residual is not None
        return out

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        dy_shard = dy_shard.contiguous()
        # dX[T, in/W] = all_gather(dY)[T, out] @ W[out, in/W]  (W read as [K=out, N=in/W])
        tp = ctx.tp
        if tp.fused:
            # the gathered operand (dY rows) is K-major; W is read as [K = out, N = in/W] (MN-major B)
            dx, dy_full = _fused_ag_gemm(tp, dy_shard, w, ctx.key + ".bwd", b_mn=True, persistent=False)
        else:
            dy_full = tp.pg.all_gather(dy_shard, dim=0)
            dx = gemm(dy_full, w, b_mn=True)
        dw = Fm._wgrad(dy_full, x, w)
        db = None
        if ctx.b is not None:
            db = Fm._bgrad(dy_full, ctx.b)      # identical on every rank (bias is replicated)
        return dx, dw, db, (dy_shard if ctx.has_res else None), None, None


def _fused_ag_gemm_only(tp: TPContext, x_shard: torch.Tensor, key: str):
    """All-gather of token shards through peer memory (no GEMM attached)."""
    rows, K = x_shard.shape
    W = tp.world
    stage = tp.symm_buffer(key + ".ag_stage", rows * K * 2)
    stage.view(torch.bfloat16, rows * K).view(rows, K).copy_(x_shard)
    tp.symm.barrier()
    full = torch.empty(W * rows, K, dtype=torch.bfloat16, device=x_shard.device)
    from ..dist.symm import make_copy_segs
    segs = make_copy_segs([(stage.ptrs[(tp.rank + i) % W], full.data_ptr() + ((tp.rank + i) % W) * rows * K * 2, rows * K * 2)
                           for i in range(W)], x_shard.device)
    tp.symm.peer_copy(segs, W)
    return None, full


# ------------------------------------------------------------------ layers
def _init_weight(out_f: int, in_f: int, rows: int, cols: int, dtype, device, seed: int = 42):
    std = math.sqrt(2.0 / (in_f + out_f))
    return torch.empty(rows, cols, dtype=dtype, device=device).normal_(0.0, std)


class ColumnParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, gather_output: bool = False,
                 sequence_parallel: bool = False, tp: Optional[TPContext] = None, dtype=None, device=None, name: str = ""):
        super().__init__()
        self.tp = tp or get_context()
        W = self.tp.world
        if out_features % W != 0:
            raise ValueError(f"out_features {out_features} must be divisible by the tensor-parallel size {W}")
        self.in_features, self.out_features, self.local_out = in_features, out_features, out_features // W
        self.gather_output, self.sequence_parallel = gather_output, sequence_parallel
        self.weight = nn.Parameter(_init_weight(out_features, in_features, self.local_out, in_features, dtype, device))
        self.bias = nn.Parameter(torch.zeros(self.local_out, dtype=dtype, device=device)) if bias else None
        self.key = name or f"col{id(self)}"

    def local_weight_shape(self):
        return (self.local_out, self.in_features)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        tp = self.tp
        if self.sequence_parallel:
            x2 = x.reshape(-1, x.shape[-1])
            if tp.fused and Fm._native(x2, self.weight):
                y = _ColumnSPFused.apply(x2, self.weight, self.bias, tp, self.key)
            else:
                y = Fm.linear(gather_tokens(x2, tp), self.weight, self.bias)
        else:
            y = Fm.linear(copy_to_tp_region(x, tp), self.weight, self.bias)
        if self.gather_output:
            y = gather_last_dim(y, tp)
        return y


class RowParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, input_is_parallel: bool = True,
                 sequence_parallel: bool = False, tp: Optional[TPContext] = None, dtype=None, device=None, name: str = ""):
        super().__init__()
        self.tp = tp or get_context()
        W = self.tp.world
        if in_features % W != 0:
            raise ValueError(f"in_features {in_features} must be divisible by the tensor-parallel size {W}")
        self.in_features, self.out_features, self.local_in = in_features, out_features, in_features // W
        self.input_is_parallel, self.sequence_parallel = input_is_parallel, sequence_parallel
        self.weight = nn.Parameter(_init_weight(out_features, in_features, out_features, self.local_in, dtype, device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        self.key = name or f"row{id(self)}"

    def local_weight_shape(self):
        return (self.out_features, self.local_in)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        tp = self.tp
        if not self.input_is_parallel:
            x = x.chunk(tp.world, dim=-1)[tp.rank].contiguous()
        if self.sequence_parallel:
            x2 = x.reshape(-1, x.shape[-1])
            if tp.fused and Fm._native(x2, self.weight):
                return _RowSPFused.apply(x2, self.weight, self.bias, residual, tp, self.key)
            y = scatter_tokens(Fm.linear(x2, self.weight), tp)
        else:
            y = reduce_from_tp_region(Fm.linear(x, self.weight), tp)
        if self.bias is not None:
            y = y + self.bias          # once, after the reduction
        if residual is not None:
            y = y + residual
        return y


class ColumnParallelLinearWithInputGather(ColumnParallelLinear):
    """Input arrives split on the last dimension and is all-gathered first."""

    def forward(self, x):
        return super().forward(gather_last_dim(x, self.tp))


class RowParallelLinearWithInputGather(RowParallelLinear):
    """Input arrives split on the last dimension across ranks *and* is gathered then re-sliced
    (used when the producer's split does not match this layer's)."""

    def forward(self, x, residual=None):
        full = gather_last_dim(x, self.tp)
        return super().forward(full.chunk(self.tp.world, dim=-1)[self.tp.rank].contiguous(), residual)


class Conv2dOutputParallel(nn.Module):
    """Output channels split over ranks; optional gather on the channel dim
    (src/MLFramework/Layers/TensorParallel/Conv2dOutputParallel.cs:45-128)."""

    def __init__(self, in_ch, out_ch, kernel_size, stride=1, padding=0, bias=True, gather_output=True, tp=None):
        super().__init__()
        self.tp = tp or get_context()
        if out_ch % self.tp.world:
            raise ValueError("out_channels must be divisible by the tensor-parallel size")
        self.conv = nn.Conv2d(in_ch, out_ch // self.tp.world, kernel_size, stride, padding, bias=bias)
        self.gather_output = gather_output

    def forward(self, x):
        y = self.conv(copy_to_tp_region(x, self.tp))
        if self.gather_output and self.tp.world > 1:
            y = _GatherLastDim.apply(y.movedim(1, -1).contiguous(), self.tp).movedim(-1, 1)
        return y


class Conv2dInputParallel(nn.Module):
    """Input channels split over ranks; partial outputs all-reduced, bias added once
    (Conv2dInputParallel.cs:44-118)."""

    def __init__(self, in_ch, out_ch, kernel_size, stride=1, padding=0, bias=True, input_is_parallel=True, tp=None):
        super().__init__()
        self.tp = tp or get_context()
        if in_ch % self.tp.world:
            raise ValueError("in_channels must be divisible by the tensor-parallel size")
        self.conv = nn.Conv2d(in_ch // self.tp.world, out_ch, kernel_size, stride, padding, bias=False)
        self.bias = nn.Parameter(torch.zeros(out_ch)) if bias else None
        self.input_is_parallel = input_is_parallel

    def forward(self, x):
        if not self.input_is_parallel:
            x = x.chunk(self.tp.world, dim=1)[self.tp.rank]
        y = reduce_from_tp_region(self.conv(x), self.tp)
        return y + self.bias.view(1, -1, 1, 1) if self.bias is not None else y


class TPMLP(nn.Module):
    """Column -> activation -> Row block (``TPMLPFactory.CreateMLPBlock``, TPMLPFactory.cs:20-140)."""

    def __init__(self, dim, hidden, activation="gelu", bias=True, tp=None, dtype=None, device=None):
        super().__init__()
        self.fc1 = ColumnParallelLinear(dim, hidden, bias, tp=tp, dtype=dtype, device=device)
        self.fc2 = RowParallelLinear(hidden, dim, bias, tp=tp, dtype=dtype, device=device)
        self.activation = activation

    def forward(self, x):
        h = self.fc1(x)
        h = torch.relu(h) if self.activation == "relu" else F.gelu(h, approximate="tanh")
        return self.fc2(h)


# ------------------------------------------------------------------ vocabulary-parallel head
def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def local_vocab(vocab: int, world: int, multiple: int = 1) -> int:
    """Vocabulary rows held by one rank: ceil(vocab / W), rounded up to ``multiple`` (128 gives whole GEMM tiles)."""
    return _round_up((vocab + world - 1) // world, multiple)


class _VocabParallelCE(torch.autograd.Function):
    """Mean token cross-entropy from this rank's columns of the logits. Only three numbers per row cross
    the ranks (row maximum, sum of exponentials, the target's logit); full logits never do. On the GPU
    two kernels do the work (``mlf_vp_cross_entropy``): per-row statistics into a buffer the peers can
    read, then - after waiting inside the kernel for every rank's statistics - the loss and, in place
    of the logits, d loss / d logits times the loss scale. The upstream gradient is taken to be 1."""

    @staticmethod
    def forward(ctx, logits, targets, tp, vocab, loss_scale):
        T, Vl = logits.shape
        lo = tp.rank * Vl
        t = targets.reshape(-1)
        if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.stride(1) == 1 and logits.stride(0) % 8 == 0:
            import ctypes as C
            W = tp.world
            loss_sum = torch.zeros((), dtype=torch.float32, device=logits.device)
            pads = state = None
            if tp.fused and W > 1:
                buf = tp.symm_buffer("vpce.stats", T * 16)
                table = buf.peer_table()
                pad = tp.symm._sync_pad("main")
                pads, state, sync = pad.peer_table(), C.c_void_p(pad.ptrs[tp.rank] + 1024), 1
                keep = buf
            elif W > 1:
                mine = torch.empty(T, 4, dtype=torch.float32, device=logits.device)
                table = (C.c_void_p * 8)(*([C.c_void_p(mine.data_ptr())] * W + [None] * (8 - W)))
                keep, sync = mine, -1          # statistics first, exchange through the process group, then the gradient
            else:
                mine = torch.empty(T, 4, dtype=torch.float32, device=logits.device)
                table = (C.c_void_p * 8)(C.c_void_p(mine.data_ptr()), *([None] * 7))
                keep, sync = mine, 0
            lib = _lib.get()
            args = lambda tb, mode: (C.c_void_p(logits.data_ptr()), C.c_longlong(logits.stride(0)), Vl, C.c_void_p(t.data_ptr()), T,  # noqa: E731
                                     C.c_longlong(lo), C.c_longlong(vocab), tb, pads, state, W, tp.rank, mode, None,
                                     C.c_void_p(loss_sum.data_ptr()), C.c_float(1.0 / T),
                                     C.c_void_p(loss_scale.data_ptr()) if loss_scale is not None else None, C.c_float(1.0 / T),
                                     C.c_uint64(_lib.stream_handle()))
            if sync == -1:
                _lib.check(lib.mlf_vp_ce_stats(C.c_void_p(logits.data_ptr()), C.c_longlong(logits.stride(0)), Vl, C.c_void_p(t.data_ptr()), T,
                                               C.c_longlong(lo), C.c_longlong(vocab), C.c_void_p(mine.data_ptr()),
                                               C.c_uint64(_lib.stream_handle())), "mlf_vp_ce_stats")
                allst = tp.pg.all_gather(mine, dim=0).contiguous()           # [W * T, 4]
                table = (C.c_void_p * 8)(*[C.c_void_p(allst.data_ptr() + r * T * 16) for r in range(W)] + [None] * (8 - W))
                keep = allst
                _lib.check(lib.mlf_vp_ce_grad(*args(table, 0)), "mlf_vp_ce_grad")
            else:
                _lib.check(lib.mlf_vp_cross_entropy(*args(table, sync)), "mlf_vp_cross_entropy")
            ctx.keep = keep
            ctx.save_for_backward(logits)
            return loss_sum
        lg = logits.float()
        valid_cols = max(0, min(Vl, vocab - lo))
        if valid_cols < Vl:
            lg = lg.clone()
            lg[:, valid_cols:] = float("-inf")
        mx = lg.max(dim=-1).values if valid_cols > 0 else torch.full((T,), -3.0e38)
        if tp.world > 1:
            tp.pg.all_reduce(mx, ReduceOp.MAX)
        ex = torch.exp(lg - mx[:, None])
        se = ex.sum(-1)
        mine = (t >= lo) & (t < lo + valid_cols)
        tl = torch.zeros_like(mx)
        idx = (t - lo).clamp(0, Vl - 1)
        rows = torch.arange(len(t), device=t.device)
        tl[mine] = lg[rows[mine], idx[mine]]
        if tp.world > 1:
            tp.pg.all_reduce(se, ReduceOp.SUM)
            tp.pg.all_reduce(tl, ReduceOp.SUM)
        keep_row = (t >= 0).to(lg.dtype)
        loss = ((torch.log(se) + mx - tl) * keep_row).sum() / t.numel()
        p = ex / se[:, None]
        p[rows[mine], idx[mine]] -= 1.0
        dlogits = (p * keep_row[:, None] * (1.0 / t.numel())).to(logits.dtype)
        if loss_scale is not None:
            dlogits = dlogits * loss_scale.to(dlogits.dtype)
        ctx.save_for_backward(dlogits)
        return loss

    @staticmethod
    def backward(ctx, g):
        (dl,) = ctx.saved_tensors
        return dl, None, None, None, None


def vocab_parallel_cross_entropy(logits, targets, tp: TPContext, vocab: int, loss_scale=None):
    """Loss from vocabulary-parallel logits ``[T, Vl]`` (this rank's global columns ``rank * Vl ...``). On the GPU
    the logits' storage is overwritten with their gradient."""
    return _VocabParallelCE.apply(logits, targets, tp, vocab, loss_scale)


def vocab_parallel_lm_loss(h, w_shard, targets, tp: TPContext, vocab: int, loss_scale=None, sequence_parallel: bool = False,
                           key: str = "lm_head"):
    """Cross-entropy with the LM head split over the vocabulary. ``h`` is ``[T, d]`` replicated over the ranks, or with
    ``sequence_parallel`` this rank's token shard ``[T/W, d]``: the head is then a sequence-parallel column linear
    (all-gather -> GEMM forward, GEMM -> reduce-scatter backward; one kernel each on the fused path), which is what
    sums the W partial gradients of ``h`` - no further all-reduce."""
    h2 = h.reshape(-1, h.shape[-1])
    if sequence_parallel and tp.world > 1:
        if tp.fused and Fm._native(h2, w_shard):
            logits = _ColumnSPFused.apply(h2, w_shard, None, tp, key)
        else:
            logits = Fm.linear(gather_tokens(h2, tp), w_shard)
    else:
        logits = Fm.linear(copy_to_tp_region(h2, tp), w_shard)
    return vocab_parallel_cross_entropy(logits, targets, tp, vocab, loss_scale)


class VocabParallelEmbedding(nn.Module):
    """Embedding table split over the vocabulary: every rank looks up the ids it owns (zeros for the others) and the
    partial results are summed over the ranks - an all-reduce, or with ``sequence_parallel`` a reduce-scatter over
    tokens (its backward all-gathers the token-shard gradients, so every rank's rows see every token)."""

    def __init__(self, vocab: int, dim: int, tp: Optional[TPContext] = None, dtype=None, device=None, init_std=0.02,
                 local_multiple: int = 1):
        super().__init__()
        self.tp = tp or get_context()
        W = self.tp.world
        self.vocab = vocab
        self.local_v = local_vocab(vocab, W, local_multiple)
        self.lo = self.tp.rank * self.local_v
        self.weight = nn.Parameter(torch.empty(self.local_v, dim, dtype=dtype, device=device).normal_(0, init_std))

    def forward(self, ids, sequence_parallel: bool = False):
        mask = (ids >= self.lo) & (ids < self.lo + self.local_v)
        local = (ids - self.lo).clamp(0, self.local_v - 1)
        out = F.embedding(local, self.weight) * mask[..., None].to(self.weight.dtype)
        if sequence_parallel and self.tp.world > 1:
            return scatter_tokens(out.reshape(-1, out.shape[-1]), self.tp)
        return reduce_from_tp_region(out, self.tp)


# ------------------------------------------------------------------ gradient utilities
class TPGradientManager:
    """DP-group gradient sync, global-norm clipping reduced over the TP group, consistency checks
    (src/MLFramework/Layers/TensorParallel/TPGradientManager.cs:24-135)."""

    def __init__(self, tp: TPContext, dp_group=None):
        self.tp, self.dp = tp, dp_group
        self.reducer = None
        self.dp_symm = None

    def attach_flat(self, params: Sequence[nn.Parameter], bucket_size_mb: float = 25.0, fused: bool = True,
                    grad_dtype: Optional[torch.dtype] = None):
        """Re-homes ``params`` (this rank's tensor-parallel shards and replicated parameters) into one flat buffer
        whose gradients are averaged over the DATA-parallel group bucket by bucket while backward runs: the same
        hook-driven reducer as DDP (:class:`ml_framework_b200.parallel.ddp.FlatGradReducer`). With ``fused`` and a
        data-parallel group whose ranks can map each other's memory, the flat gradient buffer lives in symmetric memory
        of that group and every bucket is one launch of the in-kernel two-shot all-reduce (1/W scaling and overflow
        check included); otherwise buckets are process-group all-reduces. Returns the ``FlatParams``; call
        ``finish_gradient_sync()`` after backward."""
        from .ddp import FlatGradReducer, fused_comm_possible
        from .flat import FlatParams
        params = list(params)
        dev = params[0].device
        gdt = grad_dtype or params[0].dtype
        grad_alloc, holder, flag = None, {}, None
        multi = self.dp is not None and self.dp.world_size > 1
        if multi and fused and fused_comm_possible(self.dp, dev, True, gdt):
            from ..dist.symm import SymmetricMemory
            self.dp_symm = SymmetricMemory(self.dp, dev)

            def grad_alloc(n, dt, holder=holder):
                holder["buf"] = self.dp_symm.alloc(n * torch.empty(0, dtype=dt).element_size())
                return holder["buf"].view(dt, n)
        flat = FlatParams(params, grad_dtype=grad_dtype, grad_alloc=grad_alloc)
        if multi:
            self.dp.broadcast(flat.flat, src=0)            # data-parallel replicas start from the same values
            if self.dp_symm is not None:
                flag = self.dp_symm.alloc_flag()
            self.reducer = FlatGradReducer(flat, self.dp, bucket_size_mb, symm=self.dp_symm, symm_buf=holder.get("buf"), flag=flag)
        self.flat, self.overflow_flag = flat, flag
        return flat

    def finish_gradient_sync(self):
        """Reduces what the gradient-ready hooks could not and waits for the communication stream (after backward)."""
        if getattr(self, "flat", None) is not None:
            self.flat.gather_missing_grads()
        if self.reducer is not None:
            self.reducer.finish()

    def close(self):
        if self.dp_symm is not None:
            self.dp_symm.close()
            self.dp_symm = None

    def synchronize_gradients(self, params: Iterable[nn.Parameter]):
        if self.dp is None or self.dp.world_size == 1:
            return
        if self.reducer is not None:                       # flat path: the buckets are (being) reduced already
            self.finish_gradient_sync()
            return
        grads = [p.grad for p in params if p.grad is not None]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1) for g in grads])
        self.dp.all_reduce(flat, ReduceOp.AVG)
        off = 0
        for g in grads:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()

    def clip_gradients_by_norm(self, params: Iterable[nn.Parameter], max_norm: float, replicated: Optional[set] = None):
        """Sharded parameters contribute their local squares, replicated ones only on TP rank 0,
        and the sum is all-reduced over the TP group before scaling."""
        params = [p for p in params if p.grad is not None]
        ss = torch.zeros((), device=params[0].device) if params else torch.zeros(())
        for p in params:
            if replicated is not None and id(p) in replicated and self.tp.rank != 0:
                continue
            ss = ss + p.grad.float().pow(2).sum()
        if self.tp.world > 1:
            ss = ss.reshape(1)
            self.tp.pg.all_reduce(ss, ReduceOp.SUM)
            ss = ss.squeeze(0)
        norm = ss.sqrt()
        coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
        for p in params:
            p.grad.mul_(coef.to(p.grad.dtype))
        return norm

    def verify_gradients(self, params: Iterable[nn.Parameter]) -> bool:
        return all(p.grad is None or bool(torch.isfinite(p.grad).all()) for p in params)


# ------------------------------------------------------------------ model analysis / conversion
@dataclass
class LayerAnalysisResult:
    name: str
    parallelism: str           # column | row | replicate
    params: int
    local_params: int


class TPModelAnalyzer:
    """Decides which linear layers become column- or row-parallel: projections that expand
    (qkv, fc1, gate/up) are column, projections that contract back (proj, fc2, down) are row
    (src/MLFramework/Conversion/TPModelAnalyzer.cs)."""

    COLUMN = ("qkv", "q_proj", "k_proj", "v_proj", "fc1", "gate", "up", "gate_up", "c_attn", "c_fc")
    ROW = ("proj", "o_proj", "fc2", "down", "c_proj")

    def analyze(self, model: nn.Module, world: int) -> List[LayerAnalysisResult]:
        out = []
        for name, m in model.named_modules():
            if not hasattr(m, "weight") or not isinstance(getattr(m, "weight"), torch.Tensor) or m.weight.dim() != 2:
                continue
            leaf = name.rsplit(".", 1)[-1]
            n = m.weight.numel() + (m.bias.numel() if getattr(m, "bias", None) is not None else 0)
            if leaf in self.COLUMN and m.weight.shape[0] % world == 0:
                out.append(LayerAnalysisResult(name, "column", n, n // world))
            elif leaf in self.ROW and m.weight.shape[1] % world == 0:
                out.append(LayerAnalysisResult(name, "row", n, m.weight.numel() // world + (m.bias.numel() if getattr(m, "bias", None) is not None else 0)))
            else:
                out.append(LayerAnalysisResult(name, "replicate", n, n))
        return out


class TPMemoryEstimator:
    @staticmethod
    def estimate(analysis: List[LayerAnalysisResult], bytes_per_param: int = 2, optimizer_bytes_per_param: int = 12):
        local = sum(a.local_params for a in analysis)
        total = sum(a.params for a in analysis)
        return {"total_params": total, "local_params": local, "param_bytes": local * bytes_per_param,
                "optimizer_bytes": local * optimizer_bytes_per_param, "savings": 1.0 - local / max(total, 1)}


class TPModelConverter:
    """Rewrites the linear layers of a dense model in place into their parallel forms, slicing the
    existing weights so the parallel model computes the same function."""

    def __init__(self, tp: TPContext, sequence_parallel: bool = False):
        self.tp, self.sp = tp, sequence_parallel

    def convert(self, model: nn.Module) -> nn.Module:
        plan = {a.name: a.parallelism for a in TPModelAnalyzer().analyze(model, self.tp.world)}
        W, r = self.tp.world, self.tp.rank
        for name, module in list(model.named_modules()):
            for cn, child in list(module.named_children()):
                full = f"{name}.{cn}" if name else cn
                kind = plan.get(full)
                if kind not in ("column", "row") or isinstance(child, (ColumnParallelLinear, RowParallelLinear)):
                    continue
                w, b = child.weight.data, (child.bias.data if getattr(child, "bias", None) is not None else None)
                if kind == "column":
                    new = ColumnParallelLinear(w.shape[1], w.shape[0], b is not None, False, self.sp, self.tp, w.dtype, w.device, full)
                    new.weight.data.copy_(w.chunk(W, 0)[r])
                    if b is not None:
                        new.bias.data.copy_(b.chunk(W, 0)[r])
                else:
                    new = RowParallelLinear(w.shape[1], w.shape[0], b is not None, True, self.sp, self.tp, w.dtype, w.device, full)
                    new.weight.data.copy_(w.chunk(W, 1)[r])
                    if b is not None:
                        new.bias.data.copy_(b)
                setattr(module, cn, new)
        return model
