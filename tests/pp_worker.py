"""Worker for the multi-GPU pipeline test (one process per GPU, launched by torchrun): a stack of GPT blocks
split into one stage per rank, 1F1B and GPipe schedules over NCCL point-to-point, bf16 with this package's
kernels. Rank 0 also runs the whole stack on its GPU; the pipeline's loss and the first stage's gradients must
match it."""
import copy
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from ml_framework_b200 import _lib
    from ml_framework_b200.dist.process_group import destroy_process_group, init_process_group
    from ml_framework_b200.models.gpt import GPTBlock, GPTConfig
    from ml_framework_b200.parallel.pipeline import (LayerPartitioner, PartitionMode, PipelineConfig, ProcessGroupPipelineCommunicator,
                                                     SchedulingStrategy, build_stage, make_scheduler)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    pg = init_process_group("nccl")
    W, r = pg.world_size, pg.rank
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = GPTConfig(n_layers=2 * W, d_model=256, n_heads=2, d_ff=512, vocab_size=128, max_seq=128)
    torch.manual_seed(5)
    layers = [GPTBlock(cfg, dtype=torch.bfloat16, device=dev) for _ in range(cfg.n_layers)]     # same seed on every rank: identical stacks
    N, mb_seqs, S = 4, 2, 128                                  # 4 micro-batches of 2 sequences of 128 tokens
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(N * mb_seqs, S, cfg.d_model, generator=g) * 0.5).to(dev).to(torch.bfloat16)
    y = (torch.randn(N * mb_seqs, S, cfg.d_model, generator=g) * 0.5).to(dev).to(torch.bfloat16)
    loss_fn = lambda out, tgt: F.mse_loss(out.float(), tgt.float())
    ref = None
    if r == 0:
        net = nn.Sequential(*copy.deepcopy(layers))
        tot = 0.0
        for i in range(N):                                     # the same micro-batching: attention sees 2 sequences at a time
            xi, yi = x[i * mb_seqs:(i + 1) * mb_seqs], y[i * mb_seqs:(i + 1) * mb_seqs]
            l = loss_fn(net(xi), yi) / N
            l.backward()
            tot += float(l.detach())
        ref = (tot, [p.grad.float().clone() for p in net[0].parameters()])
    results = {}
    for sched in (SchedulingStrategy.ONE_F_ONE_B, SchedulingStrategy.GPIPE):
        stage = build_stage(copy.deepcopy(layers), r, W, LayerPartitioner(PartitionMode.UNIFORM), device=dev)
        comm = ProcessGroupPipelineCommunicator(pg)
        pc = PipelineConfig(num_stages=W, micro_batches=N, schedule=sched)
        s = make_scheduler(stage, comm, pc, loss_fn=loss_fn, act_shape_fn=lambda _x: (mb_seqs, S, cfg.d_model), act_dtype=torch.bfloat16)
        loss = s.train_iteration(x if r == 0 else x, y if r == W - 1 else None)
        torch.cuda.synchronize()
        assert _lib.read_status(True) == 0
        lt = torch.zeros(1, device=dev)
        if r == W - 1:
            lt[0] = loss.float()
        pg.broadcast(lt, src=W - 1)
        results[sched] = (float(lt), [p.grad.float().clone() for p in stage.parameters()] if r == 0 else None)
    if r == 0:
        for sched, (l, grads) in results.items():
            assert abs(l - ref[0]) < 2e-2 * abs(ref[0]) + 1e-3, (sched, l, ref[0])
            for a, b in zip(grads, ref[1]):
                assert (a - b).abs().max() <= 5e-2 * b.abs().max() + 1e-4, (sched, (a - b).abs().max().item(), b.abs().max().item())
    pg.barrier()
    if r == 0:
        print("PP_WORKER_OK", {k.value: v[0] for k, v in results.items()}, ref[0])
    destroy_process_group()


if __name__ == "__main__":
    main()
