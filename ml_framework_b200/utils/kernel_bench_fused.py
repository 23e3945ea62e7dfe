"""Per-kernel timings of the fused compute + collective paths on real links, against their roofline.

Run one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 --master-port 29561 \
        -m ml_framework_b200.utils.kernel_bench_fused [--json out.json] [--md out.md]

For every path the table gives the CUDA-event time (median over the timed launches of the maximum over ranks,
each launch preceded by a process-group barrier so that the ranks start together), the FLOPs of the GEMM part,
the bytes that cross NVLink into and out of each GPU, the roofline time
``max(FLOPs / bf16 peak, max(bytes in, bytes out) / link bandwidth)`` and achieved = roofline / measured.
The peak is the sustained cuBLAS bf16 rate of ``MEASURED_PEAKS.json`` (1387.6 TFLOP/s when absent); the link
bandwidth is the measured peer-copy rate of this pool, 770 GB/s per direction per GPU (nominal 900).

Paths: the tensor-parallel all-gather -> GEMM and GEMM -> reduce-scatter at the Llama-8B shapes of a TP group of
this world size (32768 tokens), the FSDP parameter gather riding on a GEMM of the GPT-1.3B block, the in-kernel
synchronised reduce-scatter of one block's gradients, and the two-shot all-reduce of a 25 MB DDP bucket.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

LINK_GBS = 770.0


def _peak_tflops() -> float:
    from .kernel_bench import peaks
    return float(peaks()["bf16_tflops_sustained"])


def _time(fn, pg, iters=8, warmup=3):
    """Median over launches of the max over ranks, in ms."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        pg.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e)], device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ts.append(float(t))
    return statistics.median(ts)


def _row(name, ms, flops, bytes_in, bytes_out, peak):
    t_c = flops / (peak * 1e12) * 1e3
    t_l = max(bytes_in, bytes_out) / (LINK_GBS * 1e9) * 1e3
    roof = max(t_c, t_l)
    return {"path": name, "ms": round(ms, 4), "tflop": round(flops / 1e12, 4), "nvlink_in_mb": round(bytes_in / 1e6, 1),
            "nvlink_out_mb": round(bytes_out / 1e6, 1), "t_compute_ms": round(t_c, 4), "t_link_ms": round(t_l, 4),
            "roofline_ms": round(roof, 4), "achieved": round(roof / ms, 3) if ms > 0 else None,
            "bound": "compute" if t_c >= t_l else "link"}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    ap.add_argument("--md", default="")
    ap.add_argument("--tokens", type=int, default=32768)
    a = ap.parse_args(argv)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    from .. import _lib
    from ..dist.process_group import destroy_process_group, init_process_group
    from ..dist.symm import SymmetricMemory, make_copy_segs, make_reduce_segs
    from ..ops import gemm as gemm_mod
    from ..ops.gemm import gemm
    from ..parallel import tensor_parallel as tpm
    pg = init_process_group("nccl")
    W, r = pg.world_size, pg.rank
    dev = torch.device("cuda", torch.cuda.current_device())
    peak = _peak_tflops()
    symm = SymmetricMemory(pg, dev)
    tp = tpm.TPContext(pg, symm, True)
    rows_out = []
    T, d, bf = a.tokens, 4096, torch.bfloat16
    frac = (W - 1) / W

    def rnd(*shape):
        return (torch.randn(*shape, device=dev) * 0.05).to(bf)

    # ---- K8a: all-gather -> GEMM (column-parallel linears of Llama-8B split W ways)
    x_shard = rnd(T // W, d)
    for name, n_total in (("K8a AG->GEMM qkv", 6144), ("K8a AG->GEMM gate+up", 2 * 14336)):
        n = n_total // W
        w = rnd(n, d)
        ms = _time(lambda: tpm._fused_ag_gemm(tp, x_shard, w, name), pg)
        rows_out.append(_row(f"{name} [{T}x{d}]x[{d}x{n}]", ms, 2.0 * T * d * n, frac * T * d * 2, frac * T * d * 2, peak))
        del w
    # ---- K8b: GEMM -> reduce-scatter (row-parallel linears)
    for name, k_total in (("K8b GEMM->RS o_proj", 4096), ("K8b GEMM->RS down", 14336)):
        k = k_total // W
        xa, w = rnd(T, k), rnd(d, k)
        ms = _time(lambda: tpm._fused_gemm_rs(tp, xa, w, name), pg)
        rows_out.append(_row(f"{name} [{T}x{k}]x[{k}x{d}]", ms, 2.0 * T * k * d, frac * T * d * 2, frac * T * d * 2, peak))
        del xa, w
    del x_shard
    torch.cuda.empty_cache()

    # ---- K6: FSDP parameter gather of one GPT-1.3B block (50.36 M parameters) riding on the qkv GEMM
    unit = 50_360_320 // (8 * W) * (8 * W)
    shard = unit // W
    pbuf = symm.alloc(shard * 2)
    pbuf.view(bf, shard).normal_(0, 0.02)
    full = torch.empty(unit, dtype=bf, device=dev)
    segs = make_copy_segs([(pbuf.ptrs[(r + i) % W], full.data_ptr() + ((r + i) % W) * shard * 2, shard * 2) for i in range(W)], dev)
    xa, wq = rnd(8192, 2048), rnd(6144, 2048)
    pg.barrier()
    ms_plain = _time(lambda: gemm(xa, wq), pg)

    def gemm_with_gather():
        gemm_mod.set_piggyback(segs, segs.shape[0], n_copy_ctas=16)
        gemm(xa, wq)
    ms = _time(gemm_with_gather, pg)
    fl = 2.0 * 8192 * 2048 * 6144
    rows_out.append(_row("K6 FSDP gather (100 MB unit) inside qkv GEMM [8192x2048]x[2048x6144]", ms, fl, frac * unit * 2, frac * unit * 2, peak))
    rows_out[-1]["gemm_alone_ms"] = round(ms_plain, 4)
    ms_copy = _time(lambda: symm.peer_copy(segs, segs.shape[0], ctas=32), pg)
    rows_out.append(_row("K6 first-unit gather, copy kernel alone (32 CTAs)", ms_copy, 0.0, frac * unit * 2, frac * unit * 2, peak))

    # ---- K7: reduce-scatter of one block's gradients with both synchronisations inside, and the DDP bucket all-reduce
    gbuf = symm.alloc(unit * 2)
    gbuf.view(bf, unit).normal_(0, 0.01)
    flag = symm.alloc_flag()
    out = torch.empty(shard, dtype=bf, device=dev)
    rsegs = make_reduce_segs([(r * shard, 0, shard)], dev)
    for ctas in (32, 0):
        ms = _time(lambda: symm.rs_reduce_sync(gbuf, rsegs, 1, out, shard, flag=flag, key="bench", max_ctas=ctas), pg)
        by = (W - 1) * shard * 2          # this rank's slice read out of every peer's buffer
        rows_out.append(_row(f"K7 reduce-scatter + overflow check, 100 MB of gradients ({'32 CTAs' if ctas else '74 CTAs'})", ms, 0.0, by, by,
                             peak))
    bucket = 25 * 1024 * 1024 // 2 // (8 * W) * (8 * W)
    for ctas in (32, 0):
        ms = _time(lambda: symm.all_reduce_two_shot_sync(gbuf, bucket, scale=1.0 / W, flag=flag, key="bench", max_ctas=ctas), pg)
        by = (W - 1) * (bucket // W) * 2
        rows_out.append(_row(f"K7 DDP bucket all-reduce (two-shot, in-kernel sync), 25 MB ({'32 CTAs' if ctas else '74 CTAs'})", ms, 0.0, by, by, peak))
    torch.cuda.synchronize()
    status = _lib.read_status(True)
    if r == 0:
        res = {"world": W, "bf16_peak_tflops": peak, "link_gbs": LINK_GBS, "kernel_status": status, "rows": rows_out}
        print(json.dumps(res))
        if a.json:
            with open(a.json, "w") as f:
                json.dump(res, f, indent=1)
        if a.md:
            with open(a.md, "w") as f:
                f.write(f"| path (W = {W}) | ms | TFLOP | NVLink in / out MB | t_compute ms | t_link ms | roofline ms | achieved |\n|---|---|---|---|---|---|---|---|\n")
                for x in rows_out:
                    f.write(f"| {x['path']} | {x['ms']} | {x['tflop']} | {x['nvlink_in_mb']} / {x['nvlink_out_mb']} | {x['t_compute_ms']} | "
                            f"{x['t_link_ms']} | {x['roofline_ms']} ({x['bound']}) | {x['achieved']} |\n")
    pg.barrier()
    symm.close()
    destroy_process_group()


if __name__ == "__main__":
    main()
