"""Micro-benchmarks of the native kernels against the measured roofline.

Usage: ``python -m ml_framework_b200.utils.kernel_bench gemm|attn|elementwise [--json out]``

Timing: CUDA events on the launching stream, 3 warm-up launches, a write of a 256 MB buffer
between timed launches to flush L2, median of the timed launches. Peaks come from
``MEASURED_PEAKS.json`` at the repository root when present (else 6650 GB/s, 1590 TFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
from pathlib import Path

import torch


def peaks() -> dict:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


_flush_buf = None


def flush_l2():
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_cuda(fn, iters: int = 10, warmup: int = 3, flush: bool = True) -> float:
    """Median milliseconds per call of ``fn``."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    return statistics.median(ts)


GEMM_SHAPES = [
    # (name, M, N, K, a_mn, b_mn)
    ("gpt1.3b qkv fwd", 8192, 6144, 2048, False, False),
    ("gpt1.3b proj fwd", 8192, 2048, 2048, False, False),
    ("gpt1.3b fc1 fwd", 8192, 8192, 2048, False, False),
    ("gpt1.3b fc2 fwd", 8192, 2048, 8192, False, False),
    ("gpt1.3b fc1 dgrad", 8192, 2048, 8192, False, True),
    ("gpt1.3b fc1 wgrad", 8192, 2048, 8192, True, True),
    ("gpt1.3b lm head", 8192, 50304, 2048, False, False),
    ("llama8b tp8 gate_up", 32768, 3584, 4096, False, False),
    ("llama8b tp8 down", 32768, 4096, 1792, False, False),
    ("llama8b tp8 qkv", 32768, 768, 4096, False, False),
    ("llama8b tp8 o", 32768, 4096, 512, False, False),
    ("llama8b tp8 o wgrad", 4096, 512, 32768, True, True),
    ("llama8b tp8 qkv wgrad", 768, 4096, 32768, True, True),
    ("llama8b tp8 gate_up dgrad", 32768, 4096, 3584, False, True),
    ("llama8b tp8 lm head", 32768, 16032, 4096, False, False),
    ("square 8192", 8192, 8192, 8192, False, False),
    ("decode m=256 qkv", 256, 768, 4096, False, False),
]


def bench_gemm(args) -> list[dict]:
    from ..ops.gemm import gemm
    pk = peaks()
    rows = []
    for name, M, N, K, a_mn, b_mn in GEMM_SHAPES:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = time_cuda(lambda: gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out))
        A = a.t() if a_mn else a
        Bt = b if b_mn else b.t()
        ms_ref = time_cuda(lambda: torch.matmul(A, Bt, out=out))
        tf = 2.0 * M * N * K / ms / 1e9
        tf_ref = 2.0 * M * N * K / ms_ref / 1e9
        rows.append({"shape": name, "M": M, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(tf, 1),
                     "frac_of_" + pk["source"]: round(tf / pk["bf16_tflops"], 3),
                     "cublas_ms": round(ms_ref, 4), "cublas_tflops": round(tf_ref, 1),
                     "vs_cublas": round(ms_ref / ms, 3)})
        print(rows[-1], flush=True)
        del a, b, out
    return rows


def bench_gemm_epilogues(args) -> list[dict]:
    """The GPT-1.3B forward / backward GEMMs with the epilogues the model runs them with, against the plain product."""
    from .. import _lib
    from ..ops.gemm import gemm
    rows = []
    M = 8192
    cases = [("proj", 2048, 2048, [("plain", 0), ("bias", _lib.EPI_BIAS), ("residual", _lib.EPI_RESIDUAL), ("bias+residual", _lib.EPI_BIAS | _lib.EPI_RESIDUAL)]),
             ("qkv", 6144, 2048, [("plain", 0), ("bias", _lib.EPI_BIAS)]),
             ("fc1", 8192, 2048, [("plain", 0), ("bias+gelu", _lib.EPI_BIAS | _lib.EPI_GELU),
                                  ("bias+gelu+store_pre", _lib.EPI_BIAS | _lib.EPI_GELU | _lib.EPI_STORE_PRE), ("dgelu_mul", _lib.EPI_DGELU_MUL)])]
    for name, N, K, variants in cases:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        bias = torch.randn(N, device="cuda").to(torch.bfloat16)
        aux = torch.randn(M, N, device="cuda").to(torch.bfloat16)
        pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for vname, fl in variants:
            kw = {}
            if fl & _lib.EPI_BIAS:
                kw["bias"] = bias
            if fl & (_lib.EPI_RESIDUAL | _lib.EPI_DGELU_MUL):
                kw["aux_in"] = aux
            if fl & _lib.EPI_STORE_PRE:
                kw["aux_out"] = pre
            ms = time_cuda(lambda: gemm(a, b, out=out, flags=fl, **kw))
            rows.append({"gemm": name, "epilogue": vname, "M": M, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(2.0 * M * N * K / ms / 1e9, 1)})
            print(rows[-1], flush=True)
    return rows


def run_fused_small() -> list[dict]:
    """The fused communication + GEMM kernel on ONE GPU with emulated ranks (every "peer" buffer lives on this
    GPU): all-gather of A fused into the GEMM (copy CTAs + compute CTAs in one grid), then a GEMM whose
    epilogue routes row blocks to four owners' partial buffers. M = 8192, N = 4096, K = 4096, world 4.
    This is the case profiled with ncu (a multi-rank run is never profiled)."""
    from .. import _lib
    from ..ops.gemm import gemm
    W, M, N, K = 4, 8192, 4096, 4096
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
    shards = [a[r * M // W:(r + 1) * M // W].clone() for r in range(W)]
    out = None
    for _ in range(2):
        gathered = torch.zeros_like(a)
        flag_rows = 256
        flags = torch.zeros(M // flag_rows, dtype=torch.int32, device="cuda")
        counters = torch.zeros_like(flags)
        cm = _lib.GemmComm()
        cm.gather_operand, cm.world, cm.rank, cm.n_copy_ctas = 1, W, 1, 16
        cm.rows_per_rank, cm.flag_rows, cm.row_bytes = M // W, flag_rows, K * 2
        for r in range(W):
            cm.src[r] = shards[r].data_ptr()
        cm.gathered, cm.flags, cm.counters = gathered.data_ptr(), flags.data_ptr(), counters.data_ptr()
        out = gemm(shards[1], b, comm=cm, m_override=M)
        parts = [torch.zeros(W, M // W, N, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
        cs = _lib.GemmComm()
        cs.scatter_out, cs.rows_per_owner, cs.world, cs.rank = 1, M // W, W, 2
        for r in range(W):
            cs.out_peer[r] = parts[r].data_ptr()
        gemm(a, b, out=torch.empty(M, N, device="cuda", dtype=torch.bfloat16), comm=cs)
    torch.cuda.synchronize()
    ok = bool(torch.equal(gathered, a))
    return [{"ran": "fused gather-GEMM + scatter-GEMM x2 (emulated world 4)", "gather_exact": ok}]


DECODE_SHAPES = [
    # Llama-8B weights against one decode step of 64 sequences (M = 64): (name, N, K)
    ("llama8b decode qkv", 6144, 4096),
    ("llama8b decode o", 4096, 4096),
    ("llama8b decode gate_up", 28672, 4096),
    ("llama8b decode down", 4096, 14336),
    ("llama8b tp8 decode gate_up", 3584, 4096),
    ("llama8b tp8 decode down", 4096, 1792),
]


def bench_gemm_decode(args) -> list[dict]:
    """Few-row GEMMs of a decode step: the weight is read once, so the bound is weight bytes / HBM bandwidth.
    Columns: the weight-as-M stream-K route (the default up to 128 rows), the split-K CTA-pair route, the single-CTA
    route, and torch.matmul (cuBLAS)."""
    from .. import _lib
    from ..ops.gemm import gemm
    pk = peaks()
    rows = []
    lib = _lib.get()
    for M in (16, 64, 128, 256):
        for name, N, K in DECODE_SHAPES:
            a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            lib.mlf_set_gemm_fewrow(1)
            ms_fr = time_cuda(lambda: gemm(a, b, out=out), iters=20)           # weight-as-M stream-K route (M <= 128)
            lib.mlf_set_gemm_fewrow(0)
            lib.mlf_set_gemm_small_m_split(1)
            ms = time_cuda(lambda: gemm(a, b, out=out), iters=20)
            lib.mlf_set_gemm_small_m_split(0)
            ms_1 = time_cuda(lambda: gemm(a, b, out=out), iters=20)
            lib.mlf_set_gemm_small_m_split(1)
            lib.mlf_set_gemm_fewrow(1)
            ms_ref = time_cuda(lambda: torch.matmul(a, b.t(), out=out), iters=20)
            bound_ms = (N * K + M * K + M * N) * 2 / (pk["hbm_gbs"] * 1e9) * 1e3
            rows.append({"shape": name, "M": M, "N": N, "K": K, "fewrow_ms": round(ms_fr, 4) if M <= 128 else None,
                         "split_k_ms": round(ms, 4), "single_cta_ms": round(ms_1, 4),
                         "cublas_ms": round(ms_ref, 4), "hbm_bound_ms": round(bound_ms, 4),
                         "frac_of_" + pk["source"] + "_hbm": round(bound_ms / min(ms_fr, ms), 3)})
            print(rows[-1], flush=True)
    return rows


def bench_paged_decode(args) -> list[dict]:
    """Paged-attention decode (block 16) on Llama-8B head shapes; bound = K and V bytes of the cached tokens / HBM bandwidth."""
    from ..ops import native
    pk = peaks()
    rows = []
    bs, D = 16, 128
    for name, B, Hq, Hkv, ln in [("llama8b B64 ctx576", 64, 32, 8, 576), ("llama8b B256 ctx1024", 256, 32, 8, 1024),
                                 ("llama8b tp8 B64 ctx576", 64, 4, 1, 576), ("llama8b B8 ctx4096", 8, 32, 8, 4096)]:
        nblk = (ln + bs - 1) // bs
        cache = torch.randn(B * nblk, 2, bs, Hkv, D, device="cuda").to(torch.bfloat16)
        table = torch.randperm(B * nblk, device="cuda").to(torch.int32).view(B, nblk)
        sl = torch.full((B,), ln, dtype=torch.int32, device="cuda")
        q = torch.randn(B, Hq, D, device="cuda").to(torch.bfloat16)
        max_len = (ln + 511) // 512 * 512
        ms = time_cuda(lambda: native.paged_decode(q, cache, table, sl, max_len, split_tokens=0), iters=20)
        ms512 = time_cuda(lambda: native.paged_decode(q, cache, table, sl, max_len, split_tokens=512), iters=20)
        bound = B * ln * 2 * Hkv * D * 2 / (pk["hbm_gbs"] * 1e9) * 1e3
        rows.append({"shape": name, "auto_split_ms": round(ms, 4), "split512_ms": round(ms512, 4), "hbm_bound_ms": round(bound, 4),
                     "frac_of_" + pk["source"] + "_hbm": round(bound / ms, 3)})
        print(rows[-1], flush=True)
    return rows


def run_paged_small() -> list[dict]:
    """Two launches of the paged decode kernel at B = 256, ctx 1024 (K / V of the cached tokens: 1.07 GB > L2):
    the case profiled with ncu."""
    from ..ops import native
    bs, D, B, Hq, Hkv, ln = 16, 128, 256, 32, 8, 1024
    nblk = ln // bs
    cache = torch.randn(B * nblk, 2, bs, Hkv, D, device="cuda").to(torch.bfloat16)
    table = torch.randperm(B * nblk, device="cuda").to(torch.int32).view(B, nblk)
    sl = torch.full((B,), ln, dtype=torch.int32, device="cuda")
    q = torch.randn(B, Hq, D, device="cuda").to(torch.bfloat16)
    for _ in range(2):
        native.paged_decode(q, cache, table, sl, ln, split_tokens=0)
    torch.cuda.synchronize()
    return [{"ran": "paged decode B256 ctx1024 x2"}]


def bench_jit_chain(args) -> list[dict]:
    """A fused element-wise chain compiled at run time (``compiler.jit_cuda``): relu(a * b + c) on 64 Mi bf16 elements
    per tensor (three reads and one write of 128 MB each), default configuration and the autotuner's pick, against the
    same chain as three PyTorch kernels. Bound = bytes moved / copy bandwidth."""
    from ..compiler.jit_cuda import FusedElementwise
    pk = peaks()
    n = 64 * 1024 * 1024
    a, b, c = (torch.randn(n, device="cuda").to(torch.bfloat16) for _ in range(3))
    out = torch.empty_like(a)
    rows = []
    bound = 4 * n * 2 / (pk["hbm_gbs"] * 1e9) * 1e3
    f = FusedElementwise(["mul", "add", "relu"])
    ms = time_cuda(lambda: f(a, b, c, out=out), iters=10)
    ft = FusedElementwise(["mul", "add", "relu"], autotune=True)
    ft(a, b, c, out=out)
    ms_t = time_cuda(lambda: ft(a, b, c, out=out), iters=10)
    ms_torch = time_cuda(lambda: torch.relu(a * b + c), iters=10)
    ref = torch.relu(a.float() * b.float() + c.float())
    err = (out.float() - ref).abs().max().item()
    rows.append({"chain": "relu(a * b + c)", "elements": n, "generated_ms": round(ms, 4), "autotuned_ms": round(ms_t, 4),
                 "autotuned_config": next(iter(ft.chosen.values())).key(), "torch_three_kernels_ms": round(ms_torch, 4),
                 "hbm_bound_ms": round(bound, 4), "frac_of_" + pk["source"] + "_hbm": round(bound / min(ms, ms_t), 3), "max_abs_err": err})
    print(rows[-1], flush=True)
    return rows


def run_fewrow_small() -> list[dict]:
    """Three launches of the few-row GEMM at the Llama-8B gate_up shape (64 rows against a 28672 x 4096 weight, 235 MB
    > L2), accumulating into the output so that no zeroing launch sits in between: the case profiled with ncu."""
    from .. import _lib
    from ..ops.gemm import gemm
    M, N, K = 64, 28672, 4096
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        gemm(a, b, out=out, flags=_lib.EPI_ACCUM)
    torch.cuda.synchronize()
    ref = 3.0 * (a.float() @ b.float().t())
    err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
    return [{"ran": "few-row GEMM 64 x 28672 x 4096, three accumulating launches", "max_rel_err": round(err, 5)}]


def run_decode_step_small() -> list[dict]:
    """Llama-8B layer shapes, 4 layers, 64 sequences with 576 cached tokens: a batched prefill, then three decode steps
    launched eagerly (no graph replay), so that a launch list shows every kernel of a decode step."""
    from ..modelzoo.zoo import ModelInfo, build_model, default_registry
    from ..serving.executor import ExecutorConfig, PagedLlamaExecutor
    from ..serving.kv_cache import KVCacheBlockManager
    from ..serving.scheduler import Batch, Request
    info = default_registry().get("llama-3-8b")
    cfg = dict(info.config)
    cfg["n_layers"] = 4
    model = build_model(ModelInfo("llama-8b-4l", "llama", cfg), "cuda", torch.bfloat16).eval()
    mc = model.cfg
    B, ctx = 64, 576
    kv = KVCacheBlockManager(B * (ctx // 16 + 2), 16, mc.head_dim, mc.n_layers, mc.n_kv_heads, device="cuda", dtype=torch.bfloat16)
    ex = PagedLlamaExecutor(model, kv, ExecutorConfig(max_batch=B, max_seq_len=1024, prefill_chunk=1024, use_cuda_graphs=False,
                                                      max_prefill_tokens=16384))
    reqs = [Request([(7 * i + 3 * j) % 1000 + 1 for j in range(ctx)], max_tokens=8) for i in range(B)]
    out = ex.execute_batch(Batch(requests=reqs, prefill=reqs, decode=[]))
    for r in reqs:
        r.generated.append(out.generated_tokens[r.id])
    for _ in range(3):
        out = ex.execute_batch(Batch(requests=reqs, prefill=[], decode=reqs))
        for r in reqs:
            r.generated.append(out.generated_tokens[r.id])
    torch.cuda.synchronize()
    return [{"ran": "llama-8b (4 layers) prefill 64 x 576 + 3 decode steps"}]


def run_elementwise_small() -> list[dict]:
    """LayerNorm forward / backward on 8192 x 2048 and the bias-gradient column sum on 8192 x 8192, two launches each
    (a few hundred MB on the device): the case profiled with ncu."""
    from ..ops import native
    R, D = 8192, 2048
    x = torch.randn(R, D, device="cuda").to(torch.bfloat16)
    g = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(D, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(R, D, device="cuda").to(torch.bfloat16)
    dyb = torch.randn(8192, 8192, device="cuda").to(torch.bfloat16)
    for _ in range(2):
        y, mean, rstd = native.norm_fwd(x, g, b, 1e-5, False)
        native.norm_bwd(x, dy, g, mean, rstd, False, dx_add=dy)
        native.colsum(dyb)
    torch.cuda.synchronize()
    return [{"ran": "layernorm fwd/bwd 8192x2048 + colsum 8192x8192, x2"}]


def run_gemm_small() -> list[dict]:
    """Two launches of one 8192 x 8192 x 2048 GEMM (operands 160 MB > L2): the case profiled with ncu."""
    from ..ops.gemm import gemm
    a = torch.randn(8192, 2048, device="cuda").to(torch.bfloat16)
    b = torch.randn(8192, 2048, device="cuda").to(torch.bfloat16)
    out = torch.empty(8192, 8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):
        gemm(a, b, out=out)
    torch.cuda.synchronize()
    return [{"ran": "gemm 8192x8192x2048 x2"}]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "gemm_epi", "attn", "elementwise", "attn_small", "gemm_small", "fused_small", "gemm_decode", "paged", "paged_small", "decode_step_small", "elementwise_small", "fewrow_small", "jit_chain"])
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    if args.what == "gemm":
        rows = bench_gemm(args)
    elif args.what == "gemm_epi":
        rows = bench_gemm_epilogues(args)
    elif args.what == "attn_small":
        from .kernel_bench_attn import run_attn_small
        rows = run_attn_small()
    elif args.what == "fused_small":
        rows = run_fused_small()
        print(rows)
    elif args.what == "gemm_small":
        rows = run_gemm_small()
    elif args.what == "gemm_decode":
        rows = bench_gemm_decode(args)
    elif args.what == "paged":
        rows = bench_paged_decode(args)
    elif args.what == "paged_small":
        rows = run_paged_small()
    elif args.what == "decode_step_small":
        rows = run_decode_step_small()
    elif args.what == "fewrow_small":
        rows = run_fewrow_small()
    elif args.what == "jit_chain":
        rows = bench_jit_chain(args)
    elif args.what == "elementwise_small":
        rows = run_elementwise_small()
    elif args.what == "attn":
        from .kernel_bench_attn import bench_attn
        rows = bench_attn(args)
    else:
        from .kernel_bench_attn import bench_elementwise
        rows = bench_elementwise(args)
    from .. import _lib
    rows.append({"kernel_status": _lib.read_status(True)})
    if args.json:
        os.makedirs(os.path.dirname(args.json) or ".", exist_ok=True)
        Path(args.json).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
