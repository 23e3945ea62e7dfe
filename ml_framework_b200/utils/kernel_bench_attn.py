"""Attention and bandwidth-kernel micro-benchmarks (see kernel_bench.py for the timing rules)."""
from __future__ import annotations

import torch

from .kernel_bench import peaks, time_cuda


def bench_attn(args):
    from ..ops import native
    pk = peaks()
    rows = []
    for name, B, S, Hq, Hkv in [("gpt1.3b", 4, 2048, 16, 16), ("llama8b tp8", 8, 4096, 4, 1), ("llama13b tp2", 1, 4096, 20, 20)]:
        D = 128
        T = B * S
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
        q = qkv[:, :Hq * D].view(T, Hq, D)
        k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        do = torch.randn(T, Hq, D, device="cuda").to(torch.bfloat16)
        out, lse = native.flash_fwd(q, k, v, B, S)
        ms_f = time_cuda(lambda: native.flash_fwd(q, k, v, B, S))
        dqkv = torch.empty_like(qkv)
        dq = dqkv[:, :Hq * D].view(T, Hq, D)
        dk = dqkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
        dv = dqkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        ms_b = time_cuda(lambda: native.flash_bwd(q, k, v, out, do, lse, B, S, dq=dq, dk=dk, dv=dv))
        fl_f = 4.0 * B * Hq * S * S * D / 2
        qt = q.view(B, S, Hq, D).transpose(1, 2)
        kt = k.view(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
        vt = v.view(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
        ms_ref = time_cuda(lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True))
        rows.append({"shape": name, "fwd_ms": round(ms_f, 4), "fwd_tflops": round(fl_f / ms_f / 1e9, 1),
                     "bwd_ms": round(ms_b, 4), "bwd_tflops": round(2.5 * fl_f / ms_b / 1e9, 1),
                     "sdpa_fwd_ms": round(ms_ref, 4), "fwd_frac_of_" + pk["source"]: round(fl_f / ms_f / 1e9 / pk["bf16_tflops"], 3)})
        print(rows[-1], flush=True)
    return rows


def bench_elementwise(args):
    from ..ops import native
    pk = peaks()
    rows = []
    R, D = 8192, 2048
    x = torch.randn(R, D, device="cuda").to(torch.bfloat16)
    g = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(D, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(R, D, device="cuda").to(torch.bfloat16)
    y, mean, rstd = native.norm_fwd(x, g, b, 1e-5, False)

    def add(name, ms, nbytes):
        rows.append({"kernel": name, "ms": round(ms, 4), "GBps": round(nbytes / ms / 1e6, 1),
                     "frac_of_" + pk["source"]: round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3)})
        print(rows[-1], flush=True)
    add("layernorm_fwd 8192x2048", time_cuda(lambda: native.norm_fwd(x, g, b, 1e-5, False)), 2 * R * D * 2)
    add("layernorm_bwd 8192x2048", time_cuda(lambda: native.norm_bwd(x, dy, g, mean, rstd, False)), 3 * R * D * 2)
    n = 1_315_819_520 // 8 * 8
    p = torch.zeros(n, device="cuda"); m = torch.zeros_like(p); v = torch.zeros_like(p)
    gr = torch.randn(n, device="cuda").to(torch.bfloat16); pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    add("adamw 1.3B", time_cuda(lambda: native.adamw_(p, m, v, gr, pb, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                                                       weight_decay=0.1, step=1), iters=5), n * (24 + 2 + 2))
    del p, m, v, gr, pb
    T, V = 8192, 50304
    lg = torch.randn(T, V, device="cuda").to(torch.bfloat16)
    tg = torch.randint(0, 50257, (T,), device="cuda")
    add("cross_entropy 8192x50304", time_cuda(lambda: native.cross_entropy_(lg, tg, 50257), iters=5), 2 * T * V * 2)
    dyb = torch.randn(8192, 8192, device="cuda").to(torch.bfloat16)
    add("colsum 8192x8192", time_cuda(lambda: native.colsum(dyb)), 8192 * 8192 * 2)
    return rows


def run_attn_small():
    """Two forward + backward launches on B=2, S=2048, 16 heads (Q/K/V/dO 134 MB > L2): the case
    profiled with ncu."""
    from ..ops import native
    B, S, H, D = 2, 2048, 16, 128
    T = B * S
    qkv = torch.randn(T, 3 * H * D, device="cuda").to(torch.bfloat16)
    q, k, v = (qkv[:, i * H * D:(i + 1) * H * D].view(T, H, D) for i in range(3))
    do = torch.randn(T, H, D, device="cuda").to(torch.bfloat16)
    for _ in range(2):
        out, lse = native.flash_fwd(q, k, v, B, S)
        native.flash_bwd(q, k, v, out, do, lse, B, S)
    torch.cuda.synchronize()
    return [{"ran": "attn fwd+bwd x2"}]
