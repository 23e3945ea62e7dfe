"""Serving benchmark: continuous batching over the paged KV cache under Poisson arrivals.

Reports time to first token (p50 / p99), end-to-end latency, decode tokens/s and scheduler iteration
statistics for a Llama-architecture model with random-init weights and synthetic prompts.

    python -m ml_framework_b200.serving.bench_serving --model llama-3-8b --requests 256 --rate 64 \
        --prompt-len 512 --max-tokens 128 --max-batch 256
"""
from __future__ import annotations

import argparse
import json
import random
import threading
import time
from typing import Dict, List

import torch


def run(model_name: str = "llama-tiny", n_requests: int = 32, rate: float = 0.0, prompt_len: int = 64, max_tokens: int = 16,
        max_batch: int = 32, block_size: int = 16, device: str = "cpu", seed: int = 0, kv_fraction: float = 0.5) -> Dict[str, float]:
    from ..modelzoo.zoo import build_model, default_registry
    from .executor import ExecutorConfig, PagedLlamaExecutor
    from .kv_cache import KVCacheBlockManager
    from .scheduler import (BatchConstraints, CapacityConstraints, CompletionConfiguration, ContinuousBatchScheduler, Request,
                            SchedulerConfiguration)
    info = default_registry().get(model_name)
    dev = torch.device(device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    torch.manual_seed(seed)
    model = build_model(info, dev, dtype).eval()
    mc = model.cfg
    per_block = 2 * block_size * mc.n_kv_heads * mc.head_dim * mc.n_layers * (2 if dtype == torch.bfloat16 else 4)
    need = (prompt_len + max_tokens + block_size) // block_size * max(max_batch, 1) + 8
    if dev.type == "cuda":
        free, _ = torch.cuda.mem_get_info(dev)
        need = min(max(need, 64), int(free * kv_fraction) // per_block)
    kv = KVCacheBlockManager(need, block_size, mc.head_dim, mc.n_layers, mc.n_kv_heads, device=dev, dtype=dtype)
    ex = PagedLlamaExecutor(model, kv, ExecutorConfig(max_batch=max_batch, max_seq_len=prompt_len + max_tokens + block_size,
                                                      prefill_chunk=max(prompt_len, 16)))
    sched = ContinuousBatchScheduler(ex, kv, SchedulerConfiguration(max_batch_size=max_batch, warmup_iterations=0),
                                     BatchConstraints(max_batch_size=max_batch), CapacityConstraints(max_batch_size=max_batch,
                                                                                                     max_concurrent_requests=max(64, max_batch)),
                                     CompletionConfiguration(eos_token_id=-1, default_max_tokens=max_tokens))
    rng = random.Random(seed)
    reqs = [Request([rng.randrange(1, mc.vocab_size) for _ in range(prompt_len)], max_tokens=max_tokens) for _ in range(n_requests)]
    # warm-up: one short request end to end (loads kernels, fills caches of tensor maps)
    w = Request([1] * min(prompt_len, 16), max_tokens=2)
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
    ttft = sorted(r.ttft_s for r in results if r.ttft_s is not None)
    lat = sorted(r.latency_s for r in results if r.latency_s is not None)
    gen = sum(len(r.tokens) for r in results)
    pct = lambda v, q: v[min(len(v) - 1, int(q * len(v)))] if v else float("nan")
    snap = sched.metrics.snapshot()
    return {"model": model_name, "requests": n_requests, "arrival_rate": rate, "prompt_len": prompt_len, "max_tokens": max_tokens,
            "max_batch": max_batch, "wall_s": wall, "generated_tokens": gen, "decode_tokens_per_s": gen / wall,
            "total_tokens_per_s": (gen + n_requests * prompt_len) / wall, "ttft_p50_ms": pct(ttft, 0.5) * 1e3, "ttft_p99_ms": pct(ttft, 0.99) * 1e3,
            "latency_p50_ms": pct(lat, 0.5) * 1e3, "latency_p99_ms": pct(lat, 0.99) * 1e3, "iterations": sched.iterations,
            "kv_blocks": need, "scheduler": {k: v for k, v in snap.items() if isinstance(v, (int, float))}}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-tiny")
    ap.add_argument("--requests", type=int, default=32)
    ap.add_argument("--rate", type=float, default=0.0, help="Poisson arrival rate in requests/s (0 = all at once)")
    ap.add_argument("--prompt-len", type=int, default=64)
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--max-batch", type=int, default=32)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    print(json.dumps(run(a.model, a.requests, a.rate, a.prompt_len, a.max_tokens, a.max_batch, device=a.device)))


if __name__ == "__main__":
    main()
