"""Tensor-parallel training benchmark: Llama-architecture model, TP = world size (sequence parallel), bf16,
AdamW, synthetic token ids, random-init weights. Run under torchrun, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29533 \
        -m ml_framework_b200.utils.bench_tp --model llama-3-8b --batch 8 --seq 4096 --steps 5 --warmup 3

``--impl torch`` runs the plain torch.distributed + cuBLAS + SDPA statement of the same model
(``baseline/llama_tp.py``); ``--no-fused`` keeps this package's kernels but moves the collectives to NCCL.
Rank 0 prints one JSON line; timing is CUDA events around the timed steps, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = the model's own)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"])
    ap.add_argument("--no-fused", action="store_true")
    a = ap.parse_args(argv)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if os.environ.get("MLF_HANG_DUMP_S"):
        # a rank that is still running after this many seconds prints every thread's Python stack and exits
        import faulthandler
        faulthandler.dump_traceback_later(int(os.environ["MLF_HANG_DUMP_S"]), exit=True)
    from ..dist.process_group import destroy_process_group, init_process_group
    from ..modelzoo.zoo import default_registry
    pg = init_process_group("nccl", timeout_s=float(os.environ.get("MLF_PG_TIMEOUT_S", "120")))
    W, r = pg.world_size, pg.rank
    dev = torch.device("cuda", torch.cuda.current_device())
    info = default_registry().get(a.model)
    cfgd = dict(info.config)
    if a.layers:
        cfgd["n_layers"] = a.layers
    cfgd["max_seq"] = max(cfgd.get("max_seq", a.seq), a.seq)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfgd["vocab_size"], (a.batch, a.seq), generator=g).to(dev)
    tgt = torch.randint(0, cfgd["vocab_size"], (a.batch, a.seq), generator=g).to(dev)
    torch.manual_seed(1 + r)
    if a.impl == "torch":
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "baseline"))
        import llama_tp as base
        step, n_params = base.build(cfgd, dev, ids, tgt)
    else:
        from ..dist.symm import SymmetricMemory
        from ..models.llama import LlamaConfig
        from ..models.llama_tp import LlamaTP
        from ..optim.optimizers import AdamW
        from ..parallel.flat import FlatParams
        from ..parallel.tensor_parallel import TPContext
        fused = not a.no_fused and W > 1
        tp = TPContext(pg, SymmetricMemory(pg) if fused else None, fused)
        cfg = LlamaConfig(**cfgd)
        model = LlamaTP(cfg, tp, sequence_parallel=True, dtype=torch.bfloat16, device=dev)
        flat = FlatParams([p for p in model.parameters()])
        opt = AdamW(flat, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
        n_params = cfg.num_params()

        def step():
            flat.zero_grad()
            loss = model(ids, tgt)
            loss.backward()
            model.sync_replicated_grads()
            flat.gather_missing_grads()
            opt.step()
            return loss
    trace = [] if os.environ.get("MLF_LOSS_TRACE") else None      # per-step losses of the warm-up steps (reads the device)
    for _ in range(a.warmup):
        loss = step()
        if trace is not None:
            trace.append(round(float(loss.detach()), 4))
    torch.cuda.synchronize()
    pg.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    from ..dist.process_group import ReduceOp
    pg.all_reduce(ms, ReduceOp.MAX)
    pg.barrier()
    if r == 0:
        tok = a.batch * a.seq
        print(json.dumps({"metric": "train tokens/s (tensor parallel, sequence parallel, bf16)", "impl": a.impl, "fused_comm": a.impl == "ours" and not a.no_fused,
                          "value": tok / (ms.item() / 1e3), "unit": "tokens/s", "n_gpus": W, "ms_per_step": ms.item(), "steps": a.steps, "warmup": a.warmup,
                          "final_loss": float(loss.detach()), **({"warmup_losses": trace} if trace is not None else {}), "config": {"model": a.model, "layers": cfgd["n_layers"], "params": n_params, "global_batch": a.batch,
                                                                          "seq_len": a.seq, "parallelism": f"tp{W}"}}))
    destroy_process_group()


if __name__ == "__main__":
    main()
