"""Worker for the multi-GPU data-parallel test (one process per GPU, launched by torchrun): trains a
small GPT through the engine's ``ddp`` strategy with the in-kernel all-reduce of gradient buckets and
with NCCL, from the same weights, and checks that they agree with each other; then checks the module
wrapper: bucket buffers in symmetric memory, ``no_sync`` keeps gradients local, a synchronised
micro-step after an unsynchronised one gives the big-batch gradient."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from ml_framework_b200 import _lib
    from ml_framework_b200.dist.process_group import init_process_group, destroy_process_group
    from ml_framework_b200.engine import EngineConfig, TrainEngine
    from ml_framework_b200.models import GPT, GPTConfig
    from ml_framework_b200.parallel.ddp import DistributedDataParallel
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    pg = init_process_group("nccl")
    W, r = pg.world_size, pg.rank
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = GPTConfig(n_layers=3, d_model=512, n_heads=4, d_ff=2048, vocab_size=2000, max_seq=256)
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, cfg.vocab_size, (W, 2, 256), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (W, 2, 256), generator=g)
    results = {}
    for mode, fused in (("fused", True), ("nccl", False)):
        torch.manual_seed(0)
        model = GPT(cfg, dtype=torch.bfloat16, device=dev)
        eng = TrainEngine(model, EngineConfig(strategy="ddp", lr=1e-3, fused_comm=fused, bucket_size_mb=2.0), pg)
        assert (eng.symm is not None) == fused and len(eng.reducer.ranges) > 1
        losses = [float(eng.step(ids[r].to(dev), tgt[r].to(dev))) for _ in range(4)]
        torch.cuda.synchronize()
        results[mode] = (losses, eng.flat.flat.float().cpu().clone())
        assert _lib.read_status(True) == 0, f"kernel status after {mode}"
        assert eng.scaler.get_stats().skipped_steps == 0
        # every rank holds the same parameters
        mine = eng.flat.flat.float()
        ref = mine.clone()
        pg.broadcast(ref, src=0)
        assert torch.equal(mine, ref), mode
    lf, pf = results["fused"]
    ln, pn = results["nccl"]
    for a, b in zip(lf, ln):
        assert abs(a - b) < 2e-2 * abs(b), (lf, ln)
    assert ((pf - pn).abs().max() / pn.abs().max()).item() < 5e-2
    assert ln[-1] < ln[0], ln

    # ---- module wrapper, bf16 buckets in symmetric memory
    torch.manual_seed(1)
    lin = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 16)).to(dev).to(torch.bfloat16)
    ddp = DistributedDataParallel(lin, pg, bucket_size_mb=0.01)
    assert ddp.symm is not None and len(ddp.bucket_manager.buckets) > 1
    x = torch.randn(W, 2, 8, 64, generator=torch.Generator().manual_seed(3)).to(dev).to(torch.bfloat16)
    with ddp.no_sync():
        ddp(x[r, 0]).float().pow(2).mean().backward()
        ddp.finish_backward()
    local = [p.grad.clone() for p in lin.parameters()]
    for p in lin.parameters():     # reference of the unsynchronised step: plain autograd
        assert p.grad is not None
    ddp(x[r, 1]).float().pow(2).mean().backward()
    ddp.finish_backward()
    torch.cuda.synchronize()
    got = [p.grad.float().clone() for p in lin.parameters()]
    # reference: same two micro-steps without DDP, gradients averaged over ranks with NCCL
    torch.manual_seed(1)
    ref = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 16)).to(dev).to(torch.bfloat16)
    ref(x[r, 0]).float().pow(2).mean().backward()
    for a, p in zip(local, ref.parameters()):
        assert torch.allclose(a.float(), p.grad.float(), atol=1e-3, rtol=2e-2)
    ref(x[r, 1]).float().pow(2).mean().backward()
    for gt, p in zip(got, ref.parameters()):
        want = p.grad.float().clone()
        torch.distributed.all_reduce(want)
        want /= W
        assert torch.allclose(gt, want, atol=2e-3, rtol=3e-2), (gt - want).abs().max()
    assert _lib.read_status(True) == 0
    pg.barrier()
    if r == 0:
        print("DDP_WORKER_OK", lf, ln)
    destroy_process_group()


if __name__ == "__main__":
    main()
