"""Command line: ``python -m ml_framework_b200.cli <train|serve|bench|launch|convert|zoo> ...``.

The reference's only CLI is the mobile model converter (tools/MobileModelConverter/Options.cs:7-17:
``convert -i <in> -o <out> [-q int8|uint8|fp16] [-v]``); ``convert`` keeps those flags. The other
sub-commands front the training engine, the serving benchmark, the process launcher
(src/MLFramework/Distributed/Launcher/ProcessLauncher.cs) and the model zoo.
"""
from __future__ import annotations

import argparse
import json
import sys


def _train(a):
    import torch
    from .engine import EngineConfig, TrainEngine
    from .modelzoo.zoo import build_model, default_registry
    from .data.loader import DataLoader, DataLoaderConfig, SyntheticTokenDataset
    info = default_registry().get(a.model)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    pg = None
    import os
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        from .dist.process_group import ProcessGroup
        pg = ProcessGroup.init_from_env() if hasattr(ProcessGroup, "init_from_env") else None
        if dev == "cuda":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    model = build_model(info, dev, torch.bfloat16 if dev == "cuda" else torch.float32)
    eng = TrainEngine(model, EngineConfig(strategy=a.strategy, lr=a.lr, loss_scaling=dev == "cuda"), pg)
    ds = SyntheticTokenDataset(a.steps * a.batch, a.seq, info.config["vocab_size"], seed=a.seed)
    dl = DataLoader(ds, DataLoaderConfig(batch_size=a.batch, num_workers=2, device=dev if dev == "cuda" else None))
    for i, (x, y) in enumerate(dl):
        loss = eng.step(x.to(dev), y.to(dev))
        if i % a.log_every == 0:
            print(json.dumps({"step": i, "loss": float(loss.detach().float().cpu())}), flush=True)


def _serve(a):
    from .serving.bench_serving import run
    print(json.dumps(run(a.model, a.requests, a.rate, a.prompt_len, a.max_tokens, a.max_batch, device=a.device)))


def _bench(a):
    from .utils import kernel_bench
    sys.argv = ["kernel_bench", a.what] + (["--json", a.json] if a.json else [])
    kernel_bench.main()


def _launch(a):
    from .dist.launcher import launch_local, launch_multi_node
    if a.nnodes > 1:
        rc = launch_multi_node(a.script, a.nnodes, a.node_rank, a.nproc, a.master_addr, a.port, a.script_args)
        return
    rc = launch_local(a.script, a.nproc, a.script_args, master_port=a.port)
    sys.exit(rc if isinstance(rc, int) else 0)


def _convert(a):
    from .mobile.runtime import convert
    convert(a.input, a.output, a.quantize, a.verbose)


def _zoo(a):
    from .modelzoo.zoo import ModelZoo, default_registry
    reg = default_registry()
    for i in reg.search(a.query or ""):
        print(f"{i.name:16s} {i.architecture:6s} {i.num_params() / 1e6:10.1f} M  {i.description}")


def main(argv=None):
    ap = argparse.ArgumentParser(prog="ml_framework_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    t = sub.add_parser("train"); t.add_argument("--model", default="llama-tiny"); t.add_argument("--strategy", default="none")
    t.add_argument("--steps", type=int, default=10); t.add_argument("--batch", type=int, default=2); t.add_argument("--seq", type=int, default=128)
    t.add_argument("--lr", type=float, default=3e-4); t.add_argument("--seed", type=int, default=0); t.add_argument("--log-every", type=int, default=1)
    t.set_defaults(fn=_train)
    s = sub.add_parser("serve"); s.add_argument("--model", default="llama-tiny"); s.add_argument("--requests", type=int, default=16)
    s.add_argument("--rate", type=float, default=0.0); s.add_argument("--prompt-len", type=int, default=32); s.add_argument("--max-tokens", type=int, default=8)
    s.add_argument("--max-batch", type=int, default=16); s.add_argument("--device", default="cpu"); s.set_defaults(fn=_serve)
    b = sub.add_parser("bench"); b.add_argument("what", choices=["gemm", "gemm_epi", "gemm_decode", "attn", "paged", "elementwise"]); b.add_argument("--json", default=None); b.set_defaults(fn=_bench)
    l = sub.add_parser("launch"); l.add_argument("--nproc", type=int, required=True); l.add_argument("--port", type=int, default=29500)
    l.add_argument("--nnodes", type=int, default=1); l.add_argument("--node-rank", type=int, default=0); l.add_argument("--master-addr", default="127.0.0.1")
    l.add_argument("script"); l.add_argument("script_args", nargs=argparse.REMAINDER); l.set_defaults(fn=_launch)
    c = sub.add_parser("convert"); c.add_argument("-i", "--input", required=True); c.add_argument("-o", "--output", required=True)
    c.add_argument("-q", "--quantize", choices=["int8", "uint8", "fp16"], default=None); c.add_argument("-v", "--verbose", action="store_true"); c.set_defaults(fn=_convert)
    z = sub.add_parser("zoo"); z.add_argument("query", nargs="?"); z.set_defaults(fn=_zoo)
    a = ap.parse_args(argv)
    a.fn(a)


if __name__ == "__main__":
    main()
