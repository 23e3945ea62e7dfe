"""Plain-PyTorch (fp32) statements of every native kernel.

They serve three purposes: the CPU execution path of the framework (so models, parallel
wrappers and the serving stack run and are tested without a GPU), the oracle that GPU tests
compare the CUDA kernels against, and executable documentation of the math.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def layer_norm_ref(x, gamma, beta, eps=1e-5):
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = ((xf - mean) ** 2).mean(-1, keepdim=True)
    rstd = torch.rsqrt(var + eps)
    y = (xf - mean) * rstd * gamma.float() + (beta.float() if beta is not None else 0.0)
    return y, mean.squeeze(-1), rstd.squeeze(-1)


def rms_norm_ref(x, gamma, eps=1e-5):
    xf = x.float()
    rstd = torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
    return xf * rstd * gamma.float(), rstd.squeeze(-1)


def rope_ref(x: torch.Tensor, pos: torch.Tensor, theta: float, inverse: bool = False) -> torch.Tensor:
    """x [T, H, Dh], rotate-half convention: pairs (d, d + Dh/2)."""
    T, H, Dh = x.shape
    half = Dh // 2
    inv_freq = torch.exp(-math.log(theta) * (2.0 * torch.arange(half, device=x.device, dtype=torch.float32) / Dh))
    ang = pos.float()[:, None] * inv_freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    if inverse:
        s = -s
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def swiglu_ref(gu: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    f = gu.float()
    if interleaved:
        g, u = f[..., 0::2], f[..., 1::2]
    else:
        Fh = f.shape[-1] // 2
        g, u = f[..., :Fh], f[..., Fh:]
    return F.silu(g) * u


def attention_ref(q, k, v, *, causal=True, scale=None, start_pos: int = 0):
    """q [B, Sq, Hq, D], k/v [B, Sk, Hkv, D] -> (out [B, Sq, Hq, D], lse [B, Hq, Sq]).

    With ``causal`` query i sees keys ``<= start_pos + i`` (start_pos = Sk - Sq for decode),
    the rule of StandardPagedAttentionKernel.ApplyCausalMask
    (src/MLFramework/Inference/PagedAttention/Kernels/StandardPagedAttentionKernel.cs:219-255).
    """
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else D ** -0.5
    rep = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        qi = torch.arange(Sq, device=q.device)[:, None] + start_pos
        kj = torch.arange(Sk, device=q.device)[None, :]
        s = s.masked_fill(kj > qi, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return o, lse


def paged_attention_ref(q, kv_cache, block_table, seq_lens, *, scale=None):
    """Decode attention through a block table.

    q [B, Hq, D]; kv_cache [num_blocks, 2, block_size, Hkv, D]; block_table [B, max_blocks]
    (int32); seq_lens [B] = number of cached tokens including the current one. Returns [B, Hq, D].
    """
    B, Hq, D = q.shape
    bs = kv_cache.shape[2]
    outs = []
    for b in range(B):
        n = int(seq_lens[b])
        nb = (n + bs - 1) // bs
        blocks = block_table[b, :nb].long()
        k = kv_cache[blocks, 0].reshape(nb * bs, -1, D)[:n]
        v = kv_cache[blocks, 1].reshape(nb * bs, -1, D)[:n]
        o, _ = attention_ref(q[b][None, None], k[None], v[None], causal=False, scale=scale)
        outs.append(o[0, 0])
    return torch.stack(outs)


def adamw_ref(p, m, v, g, *, lr, beta1, beta2, eps, weight_decay, step, vmax=None):
    """One AdamW step in fp32, decay first then the Adam update
    (src/MLFramework/Optimizers/Adam.cs:167-213). Returns new (p, m, v[, vmax])."""
    m = beta1 * m + (1 - beta1) * g
    v = beta2 * v + (1 - beta2) * g * g
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    vh = v
    if vmax is not None:
        vmax = torch.maximum(vmax, v)
        vh = vmax
    p = p - lr * weight_decay * p
    p = p - lr * (m / bc1) / (torch.sqrt(vh / bc2) + eps)
    return (p, m, v) if vmax is None else (p, m, v, vmax)


def cross_entropy_ref(logits: torch.Tensor, targets: torch.Tensor, vocab: int, grad_scale: float = 1.0):
    """Returns (loss_rows fp32, dlogits fp32 * grad_scale); target < 0 rows are ignored."""
    lf = logits.float()[:, :vocab]
    lse = torch.logsumexp(lf, dim=-1)
    valid = targets >= 0
    tg = targets.clamp(min=0)
    loss = (lse - lf.gather(1, tg[:, None]).squeeze(1)) * valid
    p = torch.softmax(lf, dim=-1)
    p[torch.arange(lf.shape[0]), tg] -= 1.0
    p = p * valid[:, None] * grad_scale
    d = torch.zeros(logits.shape, dtype=torch.float32, device=logits.device)
    d[:, :vocab] = p
    return loss, d
