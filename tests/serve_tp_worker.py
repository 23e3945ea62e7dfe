"""Worker for the multi-GPU serving test (one process per GPU, launched by torchrun): a tensor-parallel Llama served
with continuous batching over the paged KV cache. Rank 0 runs the scheduler and broadcasts each iteration's plan;
the partial sums of the row-parallel projections are reduced with the one-shot peer-memory kernel (eagerly, and
with decode steps replayed from CUDA graphs) and with a process-group all-reduce; all runs must generate the same
tokens."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from ml_framework_b200 import _lib
    from ml_framework_b200.dist.process_group import destroy_process_group, init_process_group
    from ml_framework_b200.dist.symm import SymmetricMemory
    from ml_framework_b200.models.llama import LlamaConfig
    from ml_framework_b200.models.llama_tp import LlamaTP
    from ml_framework_b200.parallel.tensor_parallel import TPContext
    from ml_framework_b200.serving.executor import ExecutorConfig, PagedLlamaExecutor
    from ml_framework_b200.serving.kv_cache import KVCacheBlockManager
    from ml_framework_b200.serving.scheduler import (BatchConstraints, CompletionConfiguration, ContinuousBatchScheduler, Request,
                                                     SchedulerConfiguration)
    from ml_framework_b200.serving.tp_driver import TPLeaderExecutor, follower_loop
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    pg = init_process_group("nccl")
    W, r = pg.world_size, pg.rank
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = LlamaConfig(n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, d_ff=1024, vocab_size=2048, max_seq=256)
    prompts = [[(11 * i + 5 * j) % (cfg.vocab_size - 1) + 1 for j in range(18 + 7 * i)] for i in range(5)]
    symm = SymmetricMemory(pg)
    outs = {}
    for mode, fused, graphs in (("fused", True, False), ("fused+graphs", True, True), ("nccl", False, False)):
        torch.manual_seed(100 + r)
        tp = TPContext(pg, symm if fused else None, fused)
        model = LlamaTP(cfg, tp, sequence_parallel=False, dtype=torch.bfloat16, device=dev).eval()
        for p in model.replicated_parameters():
            pg.broadcast(p.data, src=0)
        kv = KVCacheBlockManager(128, 16, cfg.head_dim, cfg.n_layers, cfg.n_kv_heads // W, device=dev, dtype=torch.bfloat16)
        ex = PagedLlamaExecutor(model, kv, ExecutorConfig(max_batch=8, max_seq_len=256, prefill_chunk=64, use_cuda_graphs=graphs,
                                                          graph_warmup_steps=1), tp=tp)
        if r == 0:
            leader = TPLeaderExecutor(ex, pg)
            sched = ContinuousBatchScheduler(leader, kv, SchedulerConfiguration(max_batch_size=8, warmup_iterations=0), BatchConstraints(max_batch_size=8),
                                             completion=CompletionConfiguration(eos_token_id=-1, default_max_tokens=10))
            leader.live_ids_fn = lambda: [q.id for q in sched.batch_manager.running]
            futs = [sched.enqueue(Request(list(p), max_tokens=10)) for p in prompts]
            sched.run_until_idle()
            leader.shutdown()
            outs[mode] = [f.result(1).tokens for f in futs]
        else:
            n = follower_loop(ex, pg)
            assert n > 0
        torch.cuda.synchronize()
        assert _lib.read_status(True) == 0, f"kernel status after {mode}"
        pg.barrier()
    if r == 0:
        total = sum(len(x) for x in outs["nccl"])
        for mode in ("fused", "fused+graphs"):
            assert all(len(t) == 10 for t in outs[mode]), outs
            same = sum(a == b for x, y in zip(outs[mode], outs["nccl"]) for a, b in zip(x, y))
            assert same >= 0.9 * total, (mode, same, total, outs)
        print("SERVE_TP_WORKER_OK", same, total)
    destroy_process_group()


if __name__ == "__main__":
    main()
