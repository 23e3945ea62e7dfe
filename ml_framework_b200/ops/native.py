"""Thin, typed wrappers over the C ABI of ``libmlfb200.so`` (one Python function per kernel).

Every wrapper takes CUDA tensors, launches on the current stream and returns its outputs.
They fail loudly (``MlfError``) on a host-side problem; nothing here falls back to PyTorch.
The PyTorch statements of the same math, used on CPU tensors and as test oracles, live in
:mod:`ml_framework_b200.ops.reference`.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _lib

_BIN_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4, "min": 5}
_UN_OPS = {"relu": 0, "sigmoid": 1, "tanh": 2, "gelu": 3, "silu": 4, "exp": 5, "neg": 6, "sqrt": 7, "log": 8, "abs": 9}
_RED = {"sum": 0, "max": 1, "min": 2, "mean": 3}


def _L():
    return _lib.get()


def _st():
    return C.c_uint64(_lib.stream_handle())


def _p(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError(f"unsupported dtype {t.dtype}; kernels take float32 or bfloat16")


_scratch: dict = {}


def scratch(name: str, nbytes: int, device) -> torch.Tensor:
    """Per-device, per-purpose scratch buffer that only ever grows (uint8)."""
    key = (name, torch.device(device).index)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


# ------------------------------------------------------------------ element-wise / reductions
def ew_binary(op: str, a: torch.Tensor, b, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    a = a.contiguous()
    out = torch.empty_like(a) if out is None else out
    if isinstance(b, torch.Tensor):
        b = b.contiguous()
        assert b.shape == a.shape and b.dtype == a.dtype
        rc = _L().mlf_ew_binary(_p(out), _p(a), _p(b), C.c_float(0.0), C.c_longlong(a.numel()), _BIN_OPS[op], _dt(a), _st())
    else:
        rc = _L().mlf_ew_binary(_p(out), _p(a), None, C.c_float(float(b)), C.c_longlong(a.numel()), _BIN_OPS[op], _dt(a), _st())
    _lib.check(rc, "mlf_ew_binary")
    return out


def ew_unary(op: str, a: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    a = a.contiguous()
    out = torch.empty_like(a) if out is None else out
    _lib.check(_L().mlf_ew_unary(_p(out), _p(a), C.c_longlong(a.numel()), _UN_OPS[op], _dt(a), _st()), "mlf_ew_unary")
    return out


def fill_(t: torch.Tensor, value: float) -> torch.Tensor:
    assert t.is_contiguous()
    _lib.check(_L().mlf_fill(_p(t), C.c_float(value), C.c_longlong(t.numel()), _dt(t), _st()), "mlf_fill")
    return t


def reduce_all(op: str, a: torch.Tensor) -> torch.Tensor:
    a = a.contiguous()
    out = torch.empty((), dtype=torch.float32, device=a.device)
    sc = scratch("reduce", 4096, a.device)
    _lib.check(_L().mlf_reduce_all(_p(out), _p(a), C.c_longlong(a.numel()), _RED[op], _dt(a), _p(sc), _st()), "mlf_reduce_all")
    return out


# ------------------------------------------------------------------ norms
def norm_fwd(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float, rms: bool,
             want_stats: bool = True):
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    assert x2.is_contiguous() and x2.dtype == torch.bfloat16
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device) if want_stats and not rms else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device) if want_stats else None
    rc = _L().mlf_norm_fwd(_p(x2), _p(gamma), _p(beta), _p(y), _p(mean), _p(rstd), rows, D, C.c_float(eps), int(rms), _st())
    _lib.check(rc, "mlf_norm_fwd")
    return y.view(x.shape), mean, rstd


def norm_bwd(x: torch.Tensor, dy: torch.Tensor, gamma: torch.Tensor, mean, rstd, rms: bool,
             dgamma_out: Optional[torch.Tensor] = None, dbeta_out: Optional[torch.Tensor] = None,
             accumulate: bool = False, dx_add: Optional[torch.Tensor] = None):
    """``dx_add`` (same shape as x) is added to the returned dx inside the kernel: the gradient of a skip
    connection that branched off x."""
    D = x.shape[-1]
    x2, dy2 = x.reshape(-1, D), dy.reshape(-1, D)
    assert x2.is_contiguous() and dy2.is_contiguous()
    add2 = None
    if dx_add is not None:
        add2 = dx_add.reshape(-1, D)
        assert add2.is_contiguous() and add2.dtype == x2.dtype and add2.shape == x2.shape
    rows = x2.shape[0]
    dx = torch.empty_like(x2)
    dgamma = dgamma_out if dgamma_out is not None else torch.empty(D, dtype=gamma.dtype, device=x.device)
    dbeta = None
    if not rms:
        dbeta = dbeta_out if dbeta_out is not None else torch.empty(D, dtype=gamma.dtype, device=x.device)
    L = _L()
    L.mlf_norm_bwd_scratch_elems.restype = C.c_longlong
    n = L.mlf_norm_bwd_scratch_elems(rows, D)
    part = scratch("norm_bwd", n * 4, x.device)
    rc = L.mlf_norm_bwd_add(_p(x2), _p(dy2), _p(gamma), _p(mean), _p(rstd), _p(dx), _p(dgamma), _p(dbeta), _p(part),
                            rows, D, int(rms), int(dgamma.dtype == torch.float32), int(accumulate), _p(add2), _st())
    _lib.check(rc, "mlf_norm_bwd_add")
    return dx.view(x.shape), dgamma, dbeta


# ------------------------------------------------------------------ activations
def gelu_bwd(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    dx = torch.empty_like(x)
    _lib.check(_L().mlf_gelu_bwd(_p(dx), _p(dy.contiguous()), _p(x.contiguous()), C.c_longlong(x.numel()), _st()), "mlf_gelu_bwd")
    return dx


def swiglu_fwd(gu: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    F = gu.shape[-1] // 2
    g2 = gu.reshape(-1, 2 * F)
    out = torch.empty(g2.shape[0], F, dtype=gu.dtype, device=gu.device)
    _lib.check(_L().mlf_swiglu_fwd(_p(out), _p(g2), C.c_longlong(g2.shape[0]), F, int(interleaved), _st()), "mlf_swiglu_fwd")
    return out.view(*gu.shape[:-1], F)


def swiglu_bwd(dout: torch.Tensor, gu: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    F = gu.shape[-1] // 2
    g2 = gu.reshape(-1, 2 * F)
    dgu = torch.empty_like(g2)
    _lib.check(_L().mlf_swiglu_bwd(_p(dgu), _p(dout.reshape(-1, F).contiguous()), _p(g2), C.c_longlong(g2.shape[0]), F,
                                   int(interleaved), _st()), "mlf_swiglu_bwd")
    return dgu.view(gu.shape)


def colsum(dy: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """bf16 column sums of a 2-D bf16 matrix (bias gradient)."""
    assert dy.dim() == 2 and dy.stride(1) == 1
    M, N = dy.shape
    out = torch.empty(N, dtype=torch.bfloat16, device=dy.device) if out is None else out
    L = _L()
    L.mlf_colsum_scratch_bytes.restype = C.c_longlong
    need = int(L.mlf_colsum_scratch_bytes(M, N))
    key = ("colsum0", dy.device.index)
    sc = _scratch.get(key)
    if sc is None or sc.numel() < need:                  # zero-filled once: the kernel keeps its counters at zero
        sc = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=dy.device)
        _scratch[key] = sc
    _lib.check(L.mlf_colsum(_p(out), _p(dy), M, N, C.c_longlong(dy.stride(0)), _p(sc), int(accumulate), _st()), "mlf_colsum")
    return out


def embedding_fwd(ids: torch.Tensor, wte: torch.Tensor, pos: Optional[torch.Tensor] = None,
                  wpe: Optional[torch.Tensor] = None) -> torch.Tensor:
    T = ids.numel()
    D = wte.shape[1]
    out = torch.empty(T, D, dtype=wte.dtype, device=wte.device)
    rc = _L().mlf_embedding_fwd(_p(out), _p(ids.reshape(-1).contiguous()), _p(pos.reshape(-1).contiguous()) if pos is not None else None,
                                _p(wte), _p(wpe), C.c_longlong(T), D, wte.shape[0], wpe.shape[0] if wpe is not None else 0, _st())
    _lib.check(rc, "mlf_embedding_fwd")
    return out.view(*ids.shape, D)


def embedding_bwd(dout: torch.Tensor, ids: torch.Tensor, vocab: int, dw_fp32: Optional[torch.Tensor] = None) -> torch.Tensor:
    D = dout.shape[-1]
    T = ids.numel()
    if dw_fp32 is None:
        dw_fp32 = torch.zeros(vocab, D, dtype=torch.float32, device=dout.device)
    rc = _L().mlf_embedding_bwd(_p(dw_fp32), _p(dout.reshape(T, D).contiguous()), _p(ids.reshape(-1).contiguous()),
                                C.c_longlong(T), D, vocab, _st())
    _lib.check(rc, "mlf_embedding_bwd")
    return dw_fp32


def cast_f32_to_bf16(src: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    _lib.check(_L().mlf_cast_f32_to_bf16(_p(out), _p(src), C.c_longlong(src.numel()), int(accumulate), _st()), "mlf_cast")
    return out


def rope_(x: torch.Tensor, pos: torch.Tensor, theta: float, inverse: bool = False) -> torch.Tensor:
    """In-place rotary embedding on ``x`` [T, H, Dh] (may be a strided view over a packed row)."""
    T, H, Dh = x.shape
    assert x.stride(2) == 1 and x.stride(1) == Dh
    rc = _L().mlf_rope(_p(x), _p(pos.contiguous()), C.c_longlong(T), H, Dh, C.c_longlong(x.stride(0)), C.c_float(theta),
                       int(inverse), _st())
    _lib.check(rc, "mlf_rope")
    return x


# ------------------------------------------------------------------ optimizer / AMP / loss
def adamw_(master, m, v, grad, param_out, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
           inv_scale: Optional[torch.Tensor] = None, found_inf: Optional[torch.Tensor] = None, vmax=None):
    n = master.numel()
    rc = _L().mlf_adamw(_p(master), _p(m), _p(v), _p(vmax), _p(grad), _dt(grad), _p(param_out), C.c_longlong(n),
                        C.c_float(lr), C.c_float(beta1), C.c_float(beta2), C.c_float(eps), C.c_float(weight_decay),
                        int(step), C.c_float(grad_scale), _p(inv_scale), _p(found_inf), _st())
    _lib.check(rc, "mlf_adamw")


def sgd_(master, mom, grad, param_out, *, lr, momentum=0.0, weight_decay=0.0, grad_scale=1.0, inv_scale=None, found_inf=None):
    rc = _L().mlf_sgd(_p(master), _p(mom), _p(grad), _dt(grad), _p(param_out), C.c_longlong(master.numel()), C.c_float(lr),
                      C.c_float(momentum), C.c_float(weight_decay), C.c_float(grad_scale), _p(inv_scale), _p(found_inf), _st())
    _lib.check(rc, "mlf_sgd")


def amp_unscale_check_(grad, found_inf: torch.Tensor, *, inv_scale: Optional[torch.Tensor] = None, inv_scale_host: float = 1.0,
                       sumsq: Optional[torch.Tensor] = None, write_back: bool = True):
    rc = _L().mlf_amp_unscale_check(_p(grad), _dt(grad), C.c_longlong(grad.numel()), _p(inv_scale), C.c_float(inv_scale_host),
                                    _p(found_inf), _p(sumsq), int(write_back), _st())
    _lib.check(rc, "mlf_amp_unscale_check")


def scaler_update_(scale: torch.Tensor, tracker: torch.Tensor, found_inf: torch.Tensor, *, growth, backoff, interval,
                   min_scale, max_scale, skipped: Optional[torch.Tensor] = None):
    rc = _L().mlf_scaler_update(_p(scale), _p(tracker), _p(found_inf), C.c_float(growth), C.c_float(backoff), int(interval),
                                C.c_float(min_scale), C.c_float(max_scale), _p(skipped), _st())
    _lib.check(rc, "mlf_scaler_update")


def clip_scale_(grad, sumsq: torch.Tensor, max_norm: float, eps: float = 1e-6):
    rc = _L().mlf_clip_scale(_p(grad), _dt(grad), C.c_longlong(grad.numel()), _p(sumsq), C.c_float(max_norm), C.c_float(eps), _st())
    _lib.check(rc, "mlf_clip_scale")


def cross_entropy_(logits: torch.Tensor, targets: torch.Tensor, vocab: int, *, grad_scale: float = 1.0,
                   grad_scale_dev: Optional[torch.Tensor] = None, loss_weight: float = 1.0):
    """Overwrites ``logits`` [T, ld] with d(loss)/d(logits) * grad_scale; returns (loss_rows, loss_sum)."""
    assert logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype == torch.bfloat16
    T = logits.shape[0]
    loss_rows = torch.empty(T, dtype=torch.float32, device=logits.device)
    loss_sum = torch.zeros((), dtype=torch.float32, device=logits.device)
    rc = _L().mlf_cross_entropy(_p(logits), _p(targets.contiguous()), _p(loss_rows), _p(loss_sum), T, vocab,
                                C.c_longlong(logits.stride(0)), C.c_float(grad_scale), _p(grad_scale_dev),
                                C.c_float(loss_weight), _st())
    _lib.check(rc, "mlf_cross_entropy")
    return loss_rows, loss_sum


# ------------------------------------------------------------------ attention
def flash_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, B: int, S: int, *, causal: bool = True,
              scale: Optional[float] = None, want_lse: bool = True):
    """q [B*S, Hq, 128], k/v [B*S, Hkv, 128] (views with unit stride over heads*128)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    assert D == 128 and T == B * S
    for t in (q, k, v):
        assert t.stride(2) == 1 and t.stride(1) == D and t.dtype == torch.bfloat16
    out = torch.empty(T, Hq, D, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device) if want_lse else None
    scale = scale if scale is not None else D ** -0.5
    rc = _L().mlf_flash_fwd(_p(q), _p(k), _p(v), _p(out), _p(lse), B, S, Hq, Hkv, C.c_longlong(q.stride(0)),
                            C.c_longlong(k.stride(0)), C.c_longlong(v.stride(0)), C.c_longlong(Hq * D), C.c_float(scale),
                            int(causal), _st())
    _lib.check(rc, "mlf_flash_fwd")
    return out, lse


def flash_fwd_prefix(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, B: int, Sq: int, Skv: int, *, causal: bool = True,
                     scale: Optional[float] = None) -> torch.Tensor:
    """Attention of the LAST ``Sq`` positions of each sequence over all ``Skv`` keys / values (a prompt chunk over
    its cached prefix plus itself). q [B*Sq, Hq, 128]; k, v [B*Skv, Hkv, 128]; token stride arbitrary."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    assert D == 128 and T == B * Sq and k.shape[0] == B * Skv and v.shape[0] == B * Skv and Skv >= Sq
    for t in (q, k, v):
        assert t.stride(2) == 1 and t.stride(1) == D and t.dtype == torch.bfloat16
    out = torch.empty(T, Hq, D, dtype=torch.bfloat16, device=q.device)
    scale = scale if scale is not None else D ** -0.5
    rc = _L().mlf_flash_fwd_prefix(_p(q), _p(k), _p(v), _p(out), None, B, Sq, Skv, Hq, Hkv, C.c_longlong(q.stride(0)),
                                   C.c_longlong(k.stride(0)), C.c_longlong(v.stride(0)), C.c_longlong(Hq * D), C.c_float(scale),
                                   int(causal), _st())
    _lib.check(rc, "mlf_flash_fwd_prefix")
    return out


def flash_fwd_paged(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, B: int, Sq: int, Skv: int, *,
                    causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    """Attention of the LAST ``Sq`` positions of each of ``B`` sequences over their ``Skv`` cached tokens, keys and
    values read page by page through ``block_table`` inside the kernel (the chunk's own K / V must already be in the
    cache). q [B*Sq, Hq, 128]; kv_cache [num_blocks, 2, 16, Hkv, 128] bf16; block_table int32 [B, max_blocks]."""
    T, Hq, D = q.shape
    nb, two, bs, Hkv, Dc = kv_cache.shape
    assert D == 128 and Dc == 128 and two == 2 and T == B * Sq and Skv >= Sq
    assert q.stride(2) == 1 and q.stride(1) == D and q.dtype == torch.bfloat16 and kv_cache.dtype == torch.bfloat16
    assert kv_cache.is_contiguous() and block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.shape[0] == B
    table = block_table.contiguous()
    out = torch.empty(T, Hq, D, dtype=torch.bfloat16, device=q.device)
    scale = scale if scale is not None else D ** -0.5
    rc = _L().mlf_flash_fwd_paged(_p(q), _p(kv_cache), _p(table), _p(out), None, B, Sq, Skv, Hq, Hkv, C.c_longlong(q.stride(0)),
                                  C.c_longlong(Hq * D), int(nb), int(bs), int(table.shape[1]), C.c_float(scale), int(causal), _st())
    _lib.check(rc, "mlf_flash_fwd_paged")
    return out


def flash_bwd(q, k, v, o, dout, lse, B: int, S: int, *, causal: bool = True, scale: Optional[float] = None,
              dq: Optional[torch.Tensor] = None, dk: Optional[torch.Tensor] = None, dv: Optional[torch.Tensor] = None):
    """Gradients of :func:`flash_fwd`. ``dq/dk/dv`` may be views into a packed dQKV buffer."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    assert D == 128 and T == B * S
    dout = dout if (dout.stride(2) == 1 and dout.stride(1) == D) else dout.contiguous()
    for t in (q, k, v, o, dout):
        assert t.stride(2) == 1 and t.stride(1) == D and t.dtype == torch.bfloat16
    dq = torch.empty(T, Hq, D, dtype=torch.bfloat16, device=q.device) if dq is None else dq
    dk = torch.empty(T, Hkv, D, dtype=torch.bfloat16, device=q.device) if dk is None else dk
    dv = torch.empty(T, Hkv, D, dtype=torch.bfloat16, device=q.device) if dv is None else dv
    scale = scale if scale is not None else D ** -0.5
    L = _L()
    L.mlf_flash_bwd_scratch_bytes.restype = C.c_longlong
    sc = scratch("flash_bwd", L.mlf_flash_bwd_scratch_bytes(B, S, Hq), q.device)
    ll = C.c_longlong
    rc = L.mlf_flash_bwd(_p(q), _p(k), _p(v), _p(o), _p(dout), _p(lse), _p(dq), _p(dk), _p(dv), _p(sc), B, S, Hq, Hkv,
                         ll(q.stride(0)), ll(k.stride(0)), ll(v.stride(0)), ll(o.stride(0)), ll(dout.stride(0)),
                         ll(dq.stride(0)), ll(dk.stride(0)), ll(dv.stride(0)), C.c_float(scale), int(causal), _st())
    _lib.check(rc, "mlf_flash_bwd")
    return dq, dk, dv


# ------------------------------------------------------------------ paged attention / KV cache
def paged_decode(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                 max_seq_len: int, *, scale: Optional[float] = None, split_tokens: int = 512, fused_merge: bool = False) -> torch.Tensor:
    """One query token per sequence against its paged KV cache.

    q [B, Hq, 128]; kv_cache [num_blocks, 2, block_size, Hkv, 128]; block_table int32 [B, max_blocks];
    seq_lens int32 [B] (cached tokens including the current one). ``max_seq_len`` (host int, an upper
    bound of seq_lens) fixes the number of splits so the launch shape does not depend on device data;
    ``split_tokens`` <= 0 picks the split count from the batch size (enough CTAs to fill the GPU).
    ``fused_merge`` lets the last split of each (sequence, kv head) merge the splits inside the same launch instead of
    a second small kernel; it measured slower (57 us against 48 us at batch 64, 576 cached tokens), hence off.
    """
    B, Hq, D = q.shape
    nb, two, bs, Hkv, D2 = kv_cache.shape
    assert D == 128 and D2 == 128 and two == 2 and kv_cache.is_contiguous()
    assert q.stride(2) == 1 and q.stride(1) == D and q.dtype == torch.bfloat16      # sequence pitch (stride 0) is free
    out = torch.empty(B, Hq, D, dtype=q.dtype, device=q.device)
    L = _L()
    L.mlf_paged_decode_ws_elems.restype = C.c_longlong
    if split_tokens <= 0:
        # automatic: about two waves of CTAs (three resident per SM on 148 SMs), at least 128 tokens per split
        want = max(1, -(-888 // (B * Hkv)))
        want = min(want, max(1, (max_seq_len + 127) // 128))
        split_tokens = -(-max_seq_len // want)
    st = (max(split_tokens, 128) + 127) // 128 * 128
    splits = max(1, (max_seq_len + st - 1) // st)
    ws = scratch("paged_decode", L.mlf_paged_decode_ws_elems(B, Hq, splits) * 4, q.device) if splits > 1 else None
    scale = scale if scale is not None else D ** -0.5
    ctr = None
    if splits > 1 and fused_merge:        # finished-split counters: zero at creation, left zero by every launch
        key = ("paged_decode_ctr", q.device.index)
        ctr = _scratch.get(key)
        if ctr is None or ctr.numel() < B * Hkv:
            ctr = torch.zeros(max(B * Hkv, 4096), dtype=torch.int32, device=q.device)
            _scratch[key] = ctr
    rc = L.mlf_paged_decode_ld(_p(q), C.c_longlong(q.stride(0)), _p(kv_cache), _p(block_table), _p(seq_lens), _p(out), _p(ws), _p(ctr), B, Hq, Hkv,
                               bs, block_table.shape[1], nb, int(max_seq_len), st, C.c_float(scale), _st())
    _lib.check(rc, "mlf_paged_decode_ld")
    return out


def kv_cache_write(kv_cache: torch.Tensor, k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor):
    """Scatter k, v [T, Hkv, 128] into cache slots (slot = block * block_size + offset; < 0 skips)."""
    nb, _, bs, Hkv, D = kv_cache.shape
    T = k.shape[0]
    assert k.stride(2) == 1 and k.stride(1) == D and v.stride(2) == 1 and v.stride(1) == D
    rc = _L().mlf_kv_cache_write(_p(kv_cache), _p(k), _p(v), _p(slots.contiguous()), C.c_longlong(T), Hkv, bs, nb,
                                 C.c_longlong(k.stride(0)), C.c_longlong(v.stride(0)), _st())
    _lib.check(rc, "mlf_kv_cache_write")


def rope_kv_write_(qkv: torch.Tensor, pos: torch.Tensor, slots: torch.Tensor, kv_cache: torch.Tensor, Hq: int, Hkv: int, theta: float):
    """In place on packed ``qkv`` [T, (Hq + 2 Hkv) * 128]: rotary embedding of the query and key heads; the rotated
    keys and the values are also written to their cache slots (one launch)."""
    nb, _, bs, Hc, D = kv_cache.shape
    assert D == 128 and Hc == Hkv and qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] == (Hq + 2 * Hkv) * 128
    assert qkv.dtype == torch.bfloat16 and pos.dtype == torch.int64 and slots.dtype == torch.int64
    rc = _L().mlf_rope_kv_write(_p(qkv), C.c_longlong(qkv.stride(0)), _p(pos.contiguous()), _p(slots.contiguous()), _p(kv_cache),
                                C.c_longlong(qkv.shape[0]), Hq, Hkv, bs, nb, C.c_float(theta), _st())
    _lib.check(rc, "mlf_rope_kv_write")
    return qkv


def kv_gather(kv_cache: torch.Tensor, block_table_row: torch.Tensor, length: int):
    """Contiguous (k, v) [length, Hkv, 128] of one sequence from its pages."""
    nb, _, bs, Hkv, D = kv_cache.shape
    k = torch.empty(length, Hkv, D, dtype=kv_cache.dtype, device=kv_cache.device)
    v = torch.empty_like(k)
    row = block_table_row.contiguous()
    rc = _L().mlf_kv_gather(_p(kv_cache), _p(row), int(row.numel()), int(length), Hkv, bs, nb, _p(k), _p(v), _st())
    _lib.check(rc, "mlf_kv_gather")
    return k, v


def argmax_rows(logits: torch.Tensor, vocab: int) -> torch.Tensor:
    """Greedy sampling: int64 argmax over the first ``vocab`` columns of bf16 ``logits`` [rows, ld]."""
    assert logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype == torch.bfloat16
    out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    rc = _L().mlf_argmax_rows(_p(logits), C.c_longlong(logits.shape[0]), C.c_longlong(logits.stride(0)), int(vocab), _p(out), _st())
    _lib.check(rc, "mlf_argmax_rows")
    return out
