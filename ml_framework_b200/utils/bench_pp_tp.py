"""Pipeline x tensor-parallel training benchmark: a Llama-architecture model cut into ``--pp`` stages, each
stage tensor-parallel (sequence-parallel) over ``--tp`` GPUs, 1F1B (or GPipe) over micro-batches of one
sequence, bf16, activation recomputation, AdamW per stage. Stage activations travel over NCCL point-to-point
on a side stream; the tensor-parallel collectives use the fused peer-memory kernels unless ``--no-fused``.
Run under torchrun with pp * tp processes, one per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29544 \
        -m ml_framework_b200.utils.bench_pp_tp --model llama-2-13b --pp 4 --tp 2 --micro-batches 16 --seq 4096

(the configuration of the reference's pipeline example, src/MLFramework/Pipeline/PipelineConfig.cs:10-79 and
GPipeScheduler.cs:80-202, with the layer partitioning of LayerPartitioner.cs:43-231 in uniform mode).
Rank 0 prints one JSON line; timing is CUDA events around the timed iterations, max over ranks.
``--device cpu --backend gloo`` runs the same composition on CPU for tests.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.nn as nn


class _Stage(nn.Module):
    """One pipeline stage of the tensor-parallel Llama: the embedding in front of the first stage's blocks, the
    final norm (and the vocabulary-parallel head used by the loss) behind the last stage's."""

    def __init__(self, cfg, tp, blocks, first: bool, last: bool, seqs: int, seq_len: int, dtype, device):
        super().__init__()
        from ..nn.layers import RMSNorm
        from ..parallel.tensor_parallel import VocabParallelEmbedding
        self.cfg, self.tp, self.first, self.last, self.B, self.S = cfg, tp, first, last, seqs, seq_len
        self.embed = VocabParallelEmbedding(cfg.padded_vocab, cfg.d_model, tp, dtype, device, cfg.init_std) if first else None
        self.blocks = nn.ModuleList(blocks)
        self.norm_f = RMSNorm(cfg.d_model, cfg.norm_eps, dtype, device) if last else None
        if last:
            vl = (cfg.padded_vocab + tp.world - 1) // tp.world
            self.lm_head = nn.Parameter(torch.empty(vl, cfg.d_model, dtype=dtype, device=device).normal_(0, cfg.init_std))

    def forward(self, x):
        from ..parallel.tensor_parallel import gather_tokens
        if self.first:
            x = self.embed(x).reshape(self.B * self.S, -1)
            if self.tp.world > 1:
                x = x.chunk(self.tp.world, dim=0)[self.tp.rank].contiguous()
        for blk in self.blocks:
            x = blk(x, self.B, self.S)
        if self.last:
            x = self.norm_f(x)
            if self.tp.world > 1:
                x = gather_tokens(x, self.tp)
        return x

    def loss(self, hidden, targets):
        from ..parallel.tensor_parallel import vocab_parallel_lm_loss
        return vocab_parallel_lm_loss(hidden, self.lm_head, targets, self.tp, self.cfg.vocab_size, None)


def _torch_arm(a):
    """The comparison arm: same model, layout, micro-batches and timing, built from torch ops and NCCL only."""
    import sys
    import torch.distributed as dist
    from ..modelzoo.zoo import default_registry
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "baseline"))
    import llama_pp_tp as base
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    W, r = dist.get_world_size(), dist.get_rank()
    cfgd = dict(default_registry().get(a.model).config)
    if a.layers:
        cfgd["n_layers"] = a.layers
    for kv in a.override:
        k, v = kv.split("=")
        cfgd[k] = int(v)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfgd["vocab_size"], (a.micro_batches, a.seq), generator=g).to(dev)
    tgt = torch.randint(0, cfgd["vocab_size"], (a.micro_batches, a.seq), generator=g).to(dev)
    torch.manual_seed(1 + r)
    step, n_local = base.build(cfgd, dev, ids, tgt, a.pp, a.tp, a.micro_batches)
    loss = None
    for _ in range(a.warmup):
        loss = step()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    lt = loss.float().reshape(1).clone()
    dist.all_reduce(lt, op=dist.ReduceOp.MAX)
    npar = torch.tensor([float(n_local)], device=dev)
    dist.all_reduce(npar)
    if r == 0:
        tok = a.micro_batches * a.seq
        print(json.dumps({"metric": "train tokens/s (pipeline x tensor parallel, bf16)", "impl": "torch", "fused_comm": False,
                          "value": tok / (ms.item() / 1e3), "unit": "tokens/s", "n_gpus": W, "ms_per_step": ms.item(), "steps": a.steps,
                          "warmup": a.warmup, "final_loss": lt.item(),
                          "config": {"model": a.model, "layers": cfgd["n_layers"], "params": int(npar.item()), "micro_batches": a.micro_batches,
                                     "seq_len": a.seq, "schedule": "1f1b", "recompute": True, "parallelism": f"pp{a.pp} x tp{a.tp}"}}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-2-13b")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = the model's own)")
    ap.add_argument("--pp", type=int, default=4)
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--micro-batches", type=int, default=16)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--schedule", default="1f1b", choices=["1f1b", "gpipe"])
    ap.add_argument("--no-recompute", action="store_true")
    ap.add_argument("--no-fused", action="store_true")
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"],
                    help="torch: the plain torch.distributed 1F1B x Megatron tensor-parallel arm under baseline/ (none of this package's kernels)")
    ap.add_argument("--override", action="append", default=[], help="model config override key=int (repeatable), e.g. n_kv_heads=2")
    ap.add_argument("--backend", default=None)
    ap.add_argument("--device", default="cuda")
    a = ap.parse_args(argv)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if a.impl == "torch":
        return _torch_arm(a)
    from ..dist.mesh import ParallelismDimension, init_device_mesh
    from ..dist.process_group import ReduceOp, destroy_process_group, init_process_group
    from ..models.llama import LlamaConfig
    from ..models.llama_tp import LlamaBlockTP
    from ..modelzoo.zoo import default_registry
    from ..optim.optimizers import AdamW
    from ..parallel.flat import FlatParams
    from ..parallel.pipeline import (CheckpointStrategy, LayerPartitioner, PartitionMode, PipelineConfig, PipelineStage,
                                     ProcessGroupPipelineCommunicator, SchedulingStrategy, make_scheduler)
    from ..parallel.tensor_parallel import TPContext
    pg = init_process_group(a.backend)
    W, r = pg.world_size, pg.rank
    if a.pp * a.tp != W:
        raise SystemExit(f"pp {a.pp} x tp {a.tp} needs {a.pp * a.tp} ranks, world has {W}")
    cuda = a.device == "cuda"
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    mesh = init_device_mesh((1, a.tp, a.pp))
    tp_pg = mesh.process_group(ParallelismDimension.TENSOR)
    pp_pg = mesh.process_group(ParallelismDimension.PIPELINE)
    stage_i = mesh.local_rank(ParallelismDimension.PIPELINE)
    fused = cuda and not a.no_fused and a.tp > 1
    symm = None
    if fused:
        from ..dist.symm import SymmetricMemory
        symm = SymmetricMemory(tp_pg)
    tp = TPContext(tp_pg, symm, fused)
    cfgd = dict(default_registry().get(a.model).config)
    if a.layers:
        cfgd["n_layers"] = a.layers
    for kv in a.override:
        k, v = kv.split("=")
        cfgd[k] = int(v)
    cfgd["max_seq"] = max(cfgd.get("max_seq", a.seq), a.seq)
    cfg = LlamaConfig(**cfgd)
    bounds = LayerPartitioner(PartitionMode.UNIFORM).partition([nn.Identity() for _ in range(cfg.n_layers)], a.pp).boundaries
    lo, hi = bounds[stage_i]
    torch.manual_seed(1 + r)
    blocks = [LlamaBlockTP(cfg, tp, True, dtype, dev, i) for i in range(lo, hi)]
    mod = _Stage(cfg, tp, blocks, stage_i == 0, stage_i == a.pp - 1, 1, a.seq, dtype, dev)
    stage = PipelineStage(mod, stage_i, a.pp)
    flat = FlatParams([p for p in mod.parameters()])
    opt = AdamW(flat, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    comm = ProcessGroupPipelineCommunicator(pp_pg)
    pc = PipelineConfig(num_stages=a.pp, micro_batches=a.micro_batches,
                        schedule=SchedulingStrategy.GPIPE if a.schedule == "gpipe" else SchedulingStrategy.ONE_F_ONE_B,
                        checkpoint_strategy=CheckpointStrategy.STORE_ALL if a.no_recompute else CheckpointStrategy.RECOMPUTE_ALL)
    t_local = a.seq // a.tp
    sched = make_scheduler(stage, comm, pc, loss_fn=mod.loss, act_shape_fn=lambda _x: (t_local, cfg.d_model), act_dtype=dtype)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (a.micro_batches, a.seq), generator=g).to(dev)
    tgt = torch.randint(0, cfg.vocab_size, (a.micro_batches, a.seq), generator=g).to(dev)
    norms = [p for n, p in mod.named_parameters() if "norm" in n]

    def step():
        flat.zero_grad()
        loss = sched.train_iteration(ids if stage.is_first else None, tgt if stage.is_last else None)
        if a.tp > 1:                      # replicated parameters saw token shards: sum their gradients over the TP group
            for p in norms:
                gr = getattr(p, "main_grad", None) if getattr(p, "_main_grad_started", False) else p.grad
                if gr is not None:
                    tp_pg.all_reduce(gr, ReduceOp.SUM)
        flat.gather_missing_grads()
        opt.step()
        return loss

    loss = None
    for _ in range(a.warmup):
        loss = step()
    if cuda:
        torch.cuda.synchronize()
    pg.barrier()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        loss = step()
    if cuda:
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    else:
        ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / a.steps])
    pg.all_reduce(ms, ReduceOp.MAX)
    lt = torch.zeros(1, device=dev)
    if stage.is_last and loss is not None:
        lt[0] = loss.float()
    pg.all_reduce(lt, ReduceOp.MAX)
    status = 0
    if cuda:
        from .. import _lib
        status = _lib.read_status(True)
    st = torch.tensor([float(status)], device=dev)
    pg.all_reduce(st, ReduceOp.MAX)
    pg.barrier()
    if r == 0:
        tok = a.micro_batches * a.seq
        print(json.dumps({"metric": "train tokens/s (pipeline x tensor parallel, bf16)", "impl": "ours", "fused_comm": fused,
                          "value": tok / (ms.item() / 1e3), "unit": "tokens/s", "n_gpus": W, "ms_per_step": ms.item(), "steps": a.steps,
                          "warmup": a.warmup, "final_loss": lt.item(), "kernel_status": int(st.item()),
                          "config": {"model": a.model, "layers": cfg.n_layers, "params": cfg.num_params(), "micro_batches": a.micro_batches,
                                     "seq_len": a.seq, "schedule": a.schedule, "recompute": not a.no_recompute,
                                     "parallelism": f"pp{a.pp} x tp{a.tp}"}}), flush=True)
    destroy_process_group()


if __name__ == "__main__":
    main()
