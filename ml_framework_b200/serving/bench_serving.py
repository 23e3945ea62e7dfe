"""Serving benchmark: continuous batching over the paged KV cache under Poisson arrivals.

Reports time to first token (p50 / p99), end-to-end latency, decode tokens/s and scheduler iteration
statistics for a Llama-architecture model with random-init weights and synthetic prompts.

    python -m ml_framework_b200.serving.bench_serving --model llama-3-8b --requests 256 --rate 64 \
        --prompt-len 512 --max-tokens 128 --max-batch 256

Under torchrun (one process per GPU) the model is tensor parallel over all ranks: rank 0 runs the scheduler and
the load generator, the other ranks follow its plan (``serving/tp_driver.py``). ``--prompt-len A:B`` and
``--max-tokens A:B`` draw lengths uniformly from [A, B].
"""
from __future__ import annotations

import argparse
import json
import random
import time

import torch


def _rng_len(spec, rng) -> int:
    if isinstance(spec, (tuple, list)):
        return rng.randint(int(spec[0]), int(spec[1]))
    return int(spec)


def _max_len(spec) -> int:
    return int(spec[1]) if isinstance(spec, (tuple, list)) else int(spec)


def run(model_name: str = "llama-tiny", n_requests: int = 32, rate: float = 0.0, prompt_len=64, max_tokens=16,
        max_batch: int = 32, block_size: int = 16, device: str = "cpu", seed: int = 0, kv_fraction: float = 0.5, pg=None, fused: bool = True,
        torch_ops: bool = False):
    """``torch_ops``: the comparison arm -- the same scheduler, block manager and request stream, with every operator of
    the model step taken from torch (cuBLAS linears, ``F.rms_norm``, SDPA over pages gathered by indexing the block
    table, NCCL reductions), launched eagerly."""
    fused = fused and not torch_ops
    from ..modelzoo.zoo import build_model, default_registry
    from .executor import ExecutorConfig, PagedLlamaExecutor
    from .kv_cache import KVCacheBlockManager
    from .scheduler import (BatchConstraints, CapacityConstraints, CompletionConfiguration, ContinuousBatchScheduler, Request,
                            SchedulerConfiguration)
    info = default_registry().get(model_name)
    dev = torch.device(device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    W = pg.world_size if pg is not None else 1
    rank = pg.rank if pg is not None else 0
    tp = None
    if W > 1:
        from ..dist.symm import SymmetricMemory
        from ..models.llama import LlamaConfig
        from ..models.llama_tp import LlamaTP
        from ..parallel.tensor_parallel import TPContext
        torch.manual_seed(seed + 1 + rank)
        tp = TPContext(pg, SymmetricMemory(pg) if fused else None, fused)
        model = LlamaTP(LlamaConfig(**info.config), tp, sequence_parallel=False, dtype=dtype, device=dev).eval()
        for prm in model.replicated_parameters():
            pg.broadcast(prm.data, src=0)
    else:
        torch.manual_seed(seed)
        model = build_model(info, dev, dtype).eval()
    mc = model.cfg
    p_max, t_max = _max_len(prompt_len), _max_len(max_tokens)
    kv_heads = mc.n_kv_heads // W
    per_block = 2 * block_size * kv_heads * mc.head_dim * mc.n_layers * (2 if dtype == torch.bfloat16 else 4)
    need = (p_max + t_max + block_size) // block_size * max(max_batch, 1) + 8
    if dev.type == "cuda":
        free, _ = torch.cuda.mem_get_info(dev)
        need = min(max(need, 64), int(free * kv_fraction) // per_block)
    if pg is not None and W > 1:                       # every rank must size its cache alike
        t = torch.tensor([need], device=dev, dtype=torch.int64)
        from ..dist.process_group import ReduceOp
        pg.all_reduce(t, ReduceOp.MIN)
        need = int(t.item())
    kv = KVCacheBlockManager(need, block_size, mc.head_dim, mc.n_layers, kv_heads, device=dev, dtype=dtype)
    ex = PagedLlamaExecutor(model, kv, ExecutorConfig(max_batch=max_batch, max_seq_len=p_max + t_max + block_size,
                                                      prefill_chunk=max(p_max, 16), torch_ops=torch_ops), tp=tp)
    leader = None
    if W > 1:
        from .tp_driver import TPLeaderExecutor, follower_loop
        if rank != 0:
            n_it = follower_loop(ex, pg)
            return {"rank": rank, "iterations": n_it}
        leader = TPLeaderExecutor(ex, pg)
    sched = ContinuousBatchScheduler(leader or ex, kv, SchedulerConfiguration(max_batch_size=max_batch, warmup_iterations=0),
                                     BatchConstraints(max_batch_size=max_batch), CapacityConstraints(max_batch_size=max_batch,
                                                                                                     max_concurrent_requests=max(64, max_batch)),
                                     CompletionConfiguration(eos_token_id=-1, default_max_tokens=t_max))
    if leader is not None:
        leader.live_ids_fn = lambda: [q.id for q in sched.batch_manager.running]
    rng = random.Random(seed)
    reqs = [Request([rng.randrange(1, mc.vocab_size) for _ in range(_rng_len(prompt_len, rng))], max_tokens=_rng_len(max_tokens, rng))
            for _ in range(n_requests)]
    n_prompt_tokens = sum(len(q.prompt_tokens) for q in reqs)
    # warm-up: one short request end to end (loads kernels, fills caches of tensor maps)
    w = Request([1] * min(p_max, 16), max_tokens=2)
    sched.enqueue(w)
    sched.run_until_idle()
    if dev.type == "cuda":
        torch.cuda.synchronize()
    sched.start()
    t0 = time.time()
    futures = []
    for r in reqs:
        if rate > 0:
            time.sleep(rng.expovariate(rate))
        futures.append(sched.enqueue(r))
    results = [f.result(timeout=3600) for f in futures]
    if dev.type == "cuda":
        torch.cuda.synchronize()
    wall = time.time() - t0
    sched.stop()
    if leader is not None:
        leader.shutdown()
    ttft = sorted(r.ttft_s for r in results if r.ttft_s is not None)
    lat = sorted(r.latency_s for r in results if r.latency_s is not None)
    gen = sum(len(r.tokens) for r in results)
    pct = lambda v, q: v[min(len(v) - 1, int(q * len(v)))] if v else float("nan")
    snap = sched.metrics.snapshot()
    return {"impl": "torch" if torch_ops else "ours", "model": model_name, "tensor_parallel": W, "fused_reduce": bool(tp is not None and tp.fused), "requests": n_requests, "arrival_rate": rate,
            "prompt_len": prompt_len, "max_tokens": max_tokens,
            "max_batch": max_batch, "wall_s": wall, "generated_tokens": gen, "decode_tokens_per_s": gen / wall,
            "total_tokens_per_s": (gen + n_prompt_tokens) / wall, "ttft_p50_ms": pct(ttft, 0.5) * 1e3, "ttft_p99_ms": pct(ttft, 0.99) * 1e3,
            "latency_p50_ms": pct(lat, 0.5) * 1e3, "latency_p99_ms": pct(lat, 0.99) * 1e3, "iterations": sched.iterations,
            "kv_blocks": need, "scheduler": {k: v for k, v in snap.items() if isinstance(v, (int, float))}}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"],
                    help="torch: same scheduler and block tables, model step from torch operators only (the comparison arm)")
    ap.add_argument("--model", default="llama-tiny")
    ap.add_argument("--requests", type=int, default=32)
    ap.add_argument("--rate", type=float, default=0.0, help="Poisson arrival rate in requests/s (0 = all at once)")
    ap.add_argument("--prompt-len", default="64", help="N or A:B (uniform)")
    ap.add_argument("--max-tokens", default="16", help="N or A:B (uniform)")
    ap.add_argument("--no-fused", action="store_true", help="tensor parallel: reduce partial sums with NCCL instead of the peer-memory kernel")
    ap.add_argument("--max-batch", type=int, default=32)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    spec = lambda v: tuple(int(x) for x in v.split(":")) if ":" in str(v) else int(v)
    pg = None
    import os
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        from ..dist.process_group import init_process_group
        pg = init_process_group("nccl")
        a.device = f"cuda:{torch.cuda.current_device()}"
    out = run(a.model, a.requests, a.rate, spec(a.prompt_len), spec(a.max_tokens), a.max_batch, device=a.device, pg=pg, fused=not a.no_fused,
              torch_ops=a.impl == "torch")
    if pg is None or pg.rank == 0:
        print(json.dumps(out))
    if pg is not None:
        pg.barrier()
        from ..dist.process_group import destroy_process_group
        destroy_process_group()


if __name__ == "__main__":
    main()
