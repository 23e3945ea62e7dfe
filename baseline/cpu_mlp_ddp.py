"""CPU plumbing run: 2-layer MLP 784 -> 256 (ReLU) -> 10 in fp32, DDP over gloo, per-rank batch 64
of x ~ N(0, 1), uniform labels, cross-entropy, SGD lr 0.01, seed 0. After every step the script
checks that the all-reduced gradients are bit-identical on all ranks and that parameters stay in
sync. Launch: ``python -m ml_framework_b200.cli launch -n 2 baseline/cpu_mlp_ddp.py`` or through
``ml_framework_b200.dist.launcher.launch_local``. Prints one JSON line on rank 0.
"""
import json
import os
import sys
import time

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ml_framework_b200.dist.process_group import ReduceOp, init_process_group, destroy_process_group  # noqa: E402
from ml_framework_b200.models.mlp import MLP  # noqa: E402
from ml_framework_b200.optim.optimizers import SGD  # noqa: E402
from ml_framework_b200.parallel.ddp import DistributedDataParallel  # noqa: E402


def main(steps: int = 100):
    pg = init_process_group("gloo")
    torch.manual_seed(0 + 17 * pg.rank)          # different initial weights: the broadcast must fix that
    model = MLP()
    ddp = DistributedDataParallel(model, pg, bucket_size_mb=25, reduce_op=ReduceOp.AVG)
    opt = SGD(list(model.parameters()), lr=0.01)
    g = torch.Generator().manual_seed(1000 + pg.rank)
    t0 = time.time()
    equal = True
    for step in range(steps):
        x = torch.randn(64, 784, generator=g)
        y = torch.randint(0, 10, (64,), generator=g)
        opt.zero_grad()
        loss = F.cross_entropy(ddp(x), y)
        loss.backward()
        ddp.finish_backward()
        flat = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
        lo, hi = flat.clone(), flat.clone()
        pg.all_reduce(lo, ReduceOp.MIN)
        pg.all_reduce(hi, ReduceOp.MAX)
        equal = equal and bool(torch.equal(lo, hi))
        opt.step()
    w = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    lo, hi = w.clone(), w.clone()
    pg.all_reduce(lo, ReduceOp.MIN)
    pg.all_reduce(hi, ReduceOp.MAX)
    in_sync = bool(torch.equal(lo, hi))
    if pg.rank == 0:
        print(json.dumps({"config": "cpu_mlp_ddp", "world_size": pg.world_size, "steps": steps,
                          "gradients_equal_across_ranks": equal, "parameters_in_sync": in_sync,
                          "buckets": len(ddp.bucket_manager.buckets), "final_loss": float(loss),
                          "steps_per_s": steps / (time.time() - t0)}))
    destroy_process_group()
    return 0 if (equal and in_sync) else 1


if __name__ == "__main__":
    sys.exit(main(int(sys.argv[1]) if len(sys.argv) > 1 else 100))
