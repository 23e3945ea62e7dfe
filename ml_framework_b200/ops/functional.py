"""Differentiable operators built on the native kernels.

Each function takes ordinary tensors. For bf16 CUDA tensors it runs the hand-written kernels
through a ``torch.autograd.Function`` whose backward launches the matching gradient kernels;
for anything else (CPU, fp32) it evaluates the same math with plain PyTorch ops so that models
and parallel wrappers can be exercised without a GPU.

Gradient placement: a parameter may carry a ``main_grad`` attribute (a view into a flat
gradient bucket owned by DDP/FSDP). Weight-gradient kernels then write (first micro-batch) or
accumulate (later ones) straight into that view, nothing is returned to autograd for the
parameter, and the parameter's ``grad_ready`` callback, if any, is invoked right after the
kernel is queued, which is what lets bucket reduction overlap the rest of backward.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from .. import _lib
from . import native, reference
from .gemm import gemm

EPI = _lib


def _native(*ts: torch.Tensor) -> bool:
    return all(t is None or (t.is_cuda and t.dtype == torch.bfloat16) for t in ts)


# ------------------------------------------------------------------------------------------
# gradient sinks
# ------------------------------------------------------------------------------------------
def _sink(param: Optional[torch.Tensor]):
    """(target tensor or None, accumulate flag). Target is the bucket view when present."""
    if param is None:
        return None, False
    mg = getattr(param, "main_grad", None)
    if mg is None:
        return None, False
    return mg, bool(getattr(param, "_main_grad_started", False))


def _done(param: Optional[torch.Tensor]):
    if param is None or getattr(param, "main_grad", None) is None:
        return
    param._main_grad_started = True
    cb = getattr(param, "grad_ready", None)
    if cb is not None:
        cb(param)


def _wgrad(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor):
    """dW[out, in] = dy^T x, into the parameter's bucket view when it has one."""
    tgt, acc = _sink(w)
    if tgt is not None:
        gemm(dy2, x2, a_mn=True, b_mn=True, out=tgt.view(w.shape), flags=EPI.EPI_ACCUM if acc else 0,
             out_dtype=tgt.dtype)
        _done(w)
        return None
    return gemm(dy2, x2, a_mn=True, b_mn=True)


def _bgrad(dy2: torch.Tensor, b: Optional[torch.Tensor]):
    if b is None:
        return None
    tgt, acc = _sink(b)
    if tgt is not None:
        if tgt.dtype == torch.bfloat16:
            native.colsum(dy2, out=tgt, accumulate=acc)
        else:
            s = native.colsum(dy2).float()
            tgt.copy_(tgt + s if acc else s)
        _done(b)
        return None
    return native.colsum(dy2)


# ------------------------------------------------------------------------------------------
# linear
# ------------------------------------------------------------------------------------------
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, residual):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        res2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        out = gemm(x2, w, bias=b, aux_in=res2, flags=EPI.EPI_RESIDUAL if residual is not None else 0)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = b is not None
        ctx.bias_ref = b
        ctx.has_res = residual is not None
        ctx.x_shape = x.shape
        return out.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, w.shape[0])
        if dy2.stride(-1) != 1 or (dy2.stride(0) % 8) != 0:
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dw = _wgrad(dy2, x2, w)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _bgrad(dy2, ctx.bias_ref)
        dres = dy if ctx.has_res else None
        return dx, dw, db, dres


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T + b (+ residual)``; ``w`` is ``[out, in]`` (src/MLFramework/Modules/Linear.cs:81-111)."""
    if _native(x, w, b, residual):
        return _LinearFn.apply(x, w, b, residual)
    y = F.linear(x, w, b)
    return y + residual if residual is not None else y


# ------------------------------------------------------------------------------------------
# fused MLPs
# ------------------------------------------------------------------------------------------
class _MlpGeluFn(torch.autograd.Function):
    """y = gelu_tanh(x W1^T + b1) W2^T + b2 (+ residual) with activation and its derivative fused
    into the GEMM epilogues."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        M = x2.shape[0]
        pre = torch.empty(M, w1.shape[0], dtype=torch.bfloat16, device=x.device)
        act = gemm(x2, w1, bias=b1, aux_out=pre, flags=EPI.EPI_GELU | EPI.EPI_STORE_PRE)
        res2 = residual.reshape(M, -1) if residual is not None else None
        y = gemm(act, w2, bias=b2, aux_in=res2, flags=EPI.EPI_RESIDUAL if residual is not None else 0)
        ctx.save_for_backward(x2, w1, w2, pre, act)
        ctx.b1, ctx.b2 = b1, b2
        ctx.has_res = residual is not None
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, pre, act = ctx.saved_tensors
        dy2 = dy.reshape(-1, w2.shape[0])
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        dpre = gemm(dy2, w2, b_mn=True, aux_in=pre, flags=EPI.EPI_DGELU_MUL)
        dw2 = _wgrad(dy2, act, w2)
        db2 = _bgrad(dy2, ctx.b2)
        dw1 = _wgrad(dpre, x2, w1)
        db1 = _bgrad(dpre, ctx.b1)
        dx = gemm(dpre, w1, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        return dx, dw1, db1, dw2, db2, (dy if ctx.has_res else None)


def mlp_gelu(x, w1, b1, w2, b2, residual=None):
    if _native(x, w1, b1, w2, b2, residual):
        return _MlpGeluFn.apply(x, w1, b1, w2, b2, residual)
    y = F.linear(F.gelu(F.linear(x, w1, b1), approximate="tanh"), w2, b2)
    return y + residual if residual is not None else y


class _MlpSwigluFn(torch.autograd.Function):
    """y = (silu(x Wg^T) * (x Wu^T)) Wd^T (+ residual). ``w_gu`` holds gate and up rows
    interleaved (row 2i = gate_i, row 2i+1 = up_i) so one GEMM feeds the SwiGLU epilogue."""

    @staticmethod
    def forward(ctx, x, w_gu, w_down, residual):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        M = x2.shape[0]
        gu = torch.empty(M, w_gu.shape[0], dtype=torch.bfloat16, device=x.device)
        h = gemm(x2, w_gu, aux_out=gu, flags=EPI.EPI_SWIGLU | EPI.EPI_STORE_PRE)
        res2 = residual.reshape(M, -1) if residual is not None else None
        y = gemm(h, w_down, aux_in=res2, flags=EPI.EPI_RESIDUAL if residual is not None else 0)
        ctx.save_for_backward(x2, w_gu, w_down, gu, h)
        ctx.has_res = residual is not None
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w_down.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w_gu, w_down, gu, h = ctx.saved_tensors
        dy2 = dy.reshape(-1, w_down.shape[0])
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        dgu = gemm(dy2, w_down, b_mn=True, aux_in=gu, flags=EPI.EPI_DSWIGLU)
        dwd = _wgrad(dy2, h, w_down)
        dwgu = _wgrad(dgu, x2, w_gu)
        dx = gemm(dgu, w_gu, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        return dx, dwgu, dwd, (dy if ctx.has_res else None)


def mlp_swiglu(x, w_gu, w_down, residual=None):
    if _native(x, w_gu, w_down, residual):
        return _MlpSwigluFn.apply(x, w_gu, w_down, residual)
    gu = F.linear(x, w_gu)
    h = (F.silu(gu[..., 0::2].float()) * gu[..., 1::2].float()).to(x.dtype)
    y = F.linear(h, w_down)
    return y + residual if residual is not None else y


# ------------------------------------------------------------------------------------------
# norms
# ------------------------------------------------------------------------------------------
class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, rms):
        xc = x.contiguous()
        y, mean, rstd = native.norm_fwd(xc, gamma, beta, eps, rms)
        ctx.save_for_backward(xc, gamma, mean if mean is not None else rstd, rstd)
        ctx.rms = rms
        ctx.gamma_ref, ctx.beta_ref = gamma, beta
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma, mean, rstd = ctx.saved_tensors
        gt, gacc = _sink(ctx.gamma_ref)
        bt, _ = _sink(ctx.beta_ref)
        dx, dg, db = native.norm_bwd(x, dy.contiguous(), gamma, None if ctx.rms else mean, rstd, ctx.rms,
                                     dgamma_out=gt, dbeta_out=bt if not ctx.rms else None, accumulate=gacc)
        if gt is not None:
            _done(ctx.gamma_ref)
            dg = None
        if bt is not None and not ctx.rms:
            _done(ctx.beta_ref)
            db = None
        return dx, dg, (db if not ctx.rms else None), None, None


class _NormSkipFn(torch.autograd.Function):
    """Normalisation that also hands its input on as the skip connection: ``(norm(x), x)``. The backward
    receives both gradients at once and the kernel adds the skip gradient to the normalisation's input
    gradient, so the sum at the branch point needs no pass of its own."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps, rms):
        xc = x.contiguous()
        y, mean, rstd = native.norm_fwd(xc, gamma, beta, eps, rms)
        ctx.save_for_backward(xc, gamma, mean if mean is not None else rstd, rstd)
        ctx.rms = rms
        ctx.gamma_ref, ctx.beta_ref = gamma, beta
        return y, xc.view_as(xc)

    @staticmethod
    def backward(ctx, dy, dskip):
        x, gamma, mean, rstd = ctx.saved_tensors
        gt, gacc = _sink(ctx.gamma_ref)
        bt, _ = _sink(ctx.beta_ref)
        if dy is None:
            return dskip, None, None, None, None
        add = None
        if dskip is not None:
            add = dskip.contiguous()
            if add.dtype != x.dtype:
                add = add.to(x.dtype)
        dx, dg, db = native.norm_bwd(x, dy.contiguous(), gamma, None if ctx.rms else mean, rstd, ctx.rms,
                                     dgamma_out=gt, dbeta_out=bt if not ctx.rms else None, accumulate=gacc, dx_add=add)
        if gt is not None:
            _done(ctx.gamma_ref)
            dg = None
        if bt is not None and not ctx.rms:
            _done(ctx.beta_ref)
            db = None
        return dx, dg, (db if not ctx.rms else None), None, None


def layer_norm_skip(x, gamma, beta, eps: float = 1e-5):
    """``(layer_norm(x), x)`` with the two gradients summed inside the backward kernel."""
    if _native(x, gamma, beta) and x.shape[-1] % 256 == 0:
        return _NormSkipFn.apply(x, gamma, beta, eps, False)
    return F.layer_norm(x, (x.shape[-1],), gamma, beta, eps), x


def rms_norm_skip(x, gamma, eps: float = 1e-5):
    if _native(x, gamma) and x.shape[-1] % 256 == 0:
        return _NormSkipFn.apply(x, gamma, None, eps, True)
    return rms_norm(x, gamma, eps), x


def layer_norm(x, gamma, beta, eps: float = 1e-5):
    if _native(x, gamma, beta) and x.shape[-1] % 256 == 0:
        return _NormFn.apply(x, gamma, beta, eps, False)
    return F.layer_norm(x, (x.shape[-1],), gamma, beta, eps)


def rms_norm(x, gamma, eps: float = 1e-5):
    if _native(x, gamma) and x.shape[-1] % 256 == 0:
        return _NormFn.apply(x, gamma, None, eps, True)
    xf = x.float()
    return (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * gamma.float()).to(x.dtype)


# ------------------------------------------------------------------------------------------
# attention (packed QKV, head_dim 128 on the native path)
# ------------------------------------------------------------------------------------------
class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, B, S, Hq, Hkv, causal, rope_theta, positions):
        D = 128
        T = B * S
        qkv2 = qkv.reshape(T, (Hq + 2 * Hkv) * D)
        q = qkv2[:, :Hq * D].view(T, Hq, D)
        k = qkv2[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        v = qkv2[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        if rope_theta is not None:
            qkv2 = qkv2.clone()  # rotate a private copy; the GEMM output stays untouched for autograd
            q = qkv2[:, :Hq * D].view(T, Hq, D)
            k = qkv2[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
            v = qkv2[:, (Hq + Hkv) * D:].view(T, Hkv, D)
            native.rope_(q, positions, rope_theta)
            native.rope_(k, positions, rope_theta)
        out, lse = native.flash_fwd(q, k, v, B, S, causal=causal)
        ctx.save_for_backward(qkv2, out, lse, positions if rope_theta is not None else None)
        ctx.dims = (B, S, Hq, Hkv, causal, rope_theta)
        ctx.in_shape = qkv.shape
        return out.view(*qkv.shape[:-1], Hq * D)

    @staticmethod
    def backward(ctx, dout):
        qkv2, out, lse, positions = ctx.saved_tensors
        B, S, Hq, Hkv, causal, rope_theta = ctx.dims
        D, T = 128, B * S
        q = qkv2[:, :Hq * D].view(T, Hq, D)
        k = qkv2[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        v = qkv2[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        dqkv = torch.empty_like(qkv2)
        dq = dqkv[:, :Hq * D].view(T, Hq, D)
        dk = dqkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        dv = dqkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        do = dout.reshape(T, Hq, D)
        native.flash_bwd(q, k, v, out, do, lse, B, S, causal=causal, dq=dq, dk=dk, dv=dv)
        if rope_theta is not None:
            native.rope_(dq, positions, rope_theta, inverse=True)
            native.rope_(dk, positions, rope_theta, inverse=True)
        return dqkv.view(ctx.in_shape), None, None, None, None, None, None, None


def attention_packed(qkv: torch.Tensor, B: int, S: int, Hq: int, Hkv: int, head_dim: int, causal: bool = True,
                     rope_theta: Optional[float] = None, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Self-attention over a packed ``[B*S, (Hq + 2*Hkv) * head_dim]`` projection.

    Layout per token: Hq query heads, then Hkv key heads, then Hkv value heads. With
    ``rope_theta`` the rotary embedding (rotate-half) is applied to queries and keys first.
    """
    if _native(qkv) and head_dim == 128:
        if rope_theta is not None and positions is None:
            positions = torch.arange(S, device=qkv.device).repeat(B)
        return _AttentionFn.apply(qkv, B, S, Hq, Hkv, causal, rope_theta, positions)
    D = head_dim
    T = B * S
    x = qkv.reshape(T, (Hq + 2 * Hkv) * D)
    q = x[:, :Hq * D].reshape(T, Hq, D)
    k = x[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D)
    v = x[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    if rope_theta is not None:
        if positions is None:
            positions = torch.arange(S, device=qkv.device).repeat(B)
        q = reference.rope_ref(q, positions, rope_theta).to(qkv.dtype)
        k = reference.rope_ref(k, positions, rope_theta).to(qkv.dtype)
    o, _ = reference.attention_ref(q.reshape(B, S, Hq, D), k.reshape(B, S, Hkv, D), v.reshape(B, S, Hkv, D),
                                   causal=causal)
    return o.to(qkv.dtype).reshape(*qkv.shape[:-1], Hq * D)


# ------------------------------------------------------------------------------------------
# embedding
# ------------------------------------------------------------------------------------------
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, wte, pos, wpe):
        out = native.embedding_fwd(ids, wte, pos, wpe)
        ctx.save_for_backward(ids, pos)
        ctx.wte, ctx.wpe = wte, wpe
        return out

    @staticmethod
    def backward(ctx, dout):
        ids, pos = ctx.saved_tensors
        wte, wpe = ctx.wte, ctx.wpe

        def one(w, idx):
            if w is None or not w.requires_grad:
                return None
            acc = native.embedding_bwd(dout, idx, w.shape[0])
            tgt, accum = _sink(w)
            if tgt is not None:
                if tgt.dtype == torch.bfloat16:
                    native.cast_f32_to_bf16(acc, tgt.view(w.shape), accumulate=accum)
                else:
                    tgt.view(w.shape).copy_(tgt.view(w.shape) + acc if accum else acc)
                _done(w)
                return None
            return acc.to(w.dtype)
        dwte = one(wte, ids)
        dwpe = one(wpe, pos) if wpe is not None else None
        return None, dwte, None, dwpe


def embedding(ids: torch.Tensor, wte: torch.Tensor, pos: Optional[torch.Tensor] = None,
              wpe: Optional[torch.Tensor] = None) -> torch.Tensor:
    if _native(wte, wpe) and wte.shape[1] % 8 == 0:
        return _EmbeddingFn.apply(ids, wte, pos, wpe)
    out = F.embedding(ids, wte)
    if wpe is not None:
        out = out + F.embedding(pos, wpe)
    return out


# ------------------------------------------------------------------------------------------
# language-model head + cross-entropy, fused
# ------------------------------------------------------------------------------------------
class _LmLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, targets, vocab, loss_scale):
        K = h.shape[-1]
        h2 = h.reshape(-1, K)
        T = h2.shape[0]
        logits = gemm(h2, w)  # [T, Vpad] bf16
        n_valid = T  # targets < 0 are rare (padding); normalise by all rows like mean over tokens
        loss_rows, loss_sum = native.cross_entropy_(logits, targets.reshape(-1), vocab, grad_scale=1.0 / n_valid,
                                                    grad_scale_dev=loss_scale, loss_weight=1.0 / n_valid)
        ctx.save_for_backward(h2, w, logits)
        ctx.w_ref = w
        ctx.h_shape = h.shape
        return loss_sum

    @staticmethod
    def backward(ctx, g):
        # The upstream gradient is taken to be 1: loss scaling is already folded into dlogits.
        h2, w, dlogits = ctx.saved_tensors
        dh = gemm(dlogits, w, b_mn=True).view(ctx.h_shape) if ctx.needs_input_grad[0] else None
        dw = _wgrad(dlogits, h2, ctx.w_ref) if ctx.needs_input_grad[1] else None
        return dh, dw, None, None, None


def lm_head_loss(h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, vocab: int,
                 loss_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Mean token cross-entropy of ``h @ w.T`` against ``targets``.

    ``w`` may have more rows than ``vocab`` (padding to a multiple of 128); padded logits are
    ignored. On the native path the gradient w.r.t. the logits is produced by the same kernel
    that computes the loss, multiplied by the device-resident ``loss_scale`` (dynamic loss
    scaling), so callers run ``loss.backward()`` on the returned *unscaled* loss.
    """
    if _native(h, w):
        return _LmLossFn.apply(h, w, targets, vocab, loss_scale)
    logits = F.linear(h, w)[..., :vocab].float()
    loss = F.cross_entropy(logits.reshape(-1, vocab), targets.reshape(-1), ignore_index=-100, reduction="sum")
    loss = loss / targets.numel()
    if loss_scale is not None:
        # keep the value unscaled but scale the gradient, like the native path
        s = loss_scale.detach().to(loss.dtype)
        loss = loss * s + (loss - loss * s).detach()
    return loss
