"""Worker for the multi-GPU tensor-parallel test (one process per GPU, launched by torchrun): trains a
small sequence-parallel Llama for a few steps with the in-kernel NVLink paths (all-gather fused into
the column-parallel GEMM, reduce-scatter fused into the row-parallel GEMM's epilogue) and again over
NCCL collectives from the same initial weights, and checks that losses and weights agree."""
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
    from ml_framework_b200.optim.optimizers import AdamW
    from ml_framework_b200.parallel.flat import FlatParams
    from ml_framework_b200.parallel.tensor_parallel import TPContext
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    pg = init_process_group("nccl")
    W, r = pg.world_size, pg.rank
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = LlamaConfig(n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, d_ff=1024, vocab_size=2048, max_seq=256)
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=g).to(dev)       # TP ranks see the same batch
    tgt = torch.randint(0, cfg.vocab_size, (2, 256), generator=g).to(dev)
    symm = SymmetricMemory(pg)
    results = {}
    for mode, fused in (("fused", True), ("nccl", False)):
        torch.manual_seed(100 + r)                      # weight shards differ per rank, identically in both modes
        tp = TPContext(pg, symm if fused else None, fused)
        assert tp.fused == fused
        model = LlamaTP(cfg, tp, sequence_parallel=True, dtype=torch.bfloat16, device=dev)
        for p in model.replicated_parameters():         # replicated parameters start equal on every rank
            pg.broadcast(p.data, src=0)
        flat = FlatParams([p for p in model.parameters()])
        opt = AdamW(flat, lr=1e-3, betas=(0.9, 0.95), eps=1e-6, weight_decay=0.0)
        losses = []
        for _ in range(4):
            flat.zero_grad()
            loss = model(ids, tgt)
            loss.backward()
            model.sync_replicated_grads()
            flat.gather_missing_grads()
            opt.step()
            losses.append(float(loss.detach()))
        torch.cuda.synchronize()
        assert _lib.read_status(True) == 0, f"kernel status after {mode}"
        results[mode] = (losses, flat.flat.float().cpu().clone())
    lf, pf = results["fused"]
    ln, pn = results["nccl"]
    for a, b in zip(lf, ln):
        assert abs(a - b) < 2e-2 * abs(b), (lf, ln)
    worst = ((pf - pn).abs().max() / (pn.abs().max() + 1e-6)).item()
    assert worst < 5e-2, worst
    assert ln[-1] < ln[0], ln
    pg.barrier()
    if r == 0:
        print("TP_WORKER_OK", lf, ln, worst)
    destroy_process_group()


if __name__ == "__main__":
    main()
