"""Child process of test_collective_algorithms_cpu: the software all-reduce algorithms over gloo point-to-point."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ml_framework_b200.dist import algorithms as A  # noqa: E402
from ml_framework_b200.dist.fault_tolerance import CollectiveAlgorithm  # noqa: E402
from ml_framework_b200.dist.process_group import BackendType, ReduceOp, destroy_process_group, init_process_group  # noqa: E402


def main():
    pg = init_process_group(BackendType.GLOO)
    W, r = pg.world_size, pg.rank
    ok = {}
    for alg in (CollectiveAlgorithm.RECURSIVE_DOUBLING, CollectiveAlgorithm.RABENSEIFNER, CollectiveAlgorithm.TREE, CollectiveAlgorithm.RING):
        t = torch.arange(1001, dtype=torch.float64) * (r + 1)
        A.all_reduce_with(pg, t, alg)
        big = torch.full((1 << 18,), float(r + 1))                 # 1 MiB: both directions of an exchange must be in flight at once
        A.all_reduce_with(pg, big, alg, ReduceOp.AVG)
        ok[alg.value] = bool(torch.equal(t, torch.arange(1001, dtype=torch.float64) * (W * (W + 1) / 2))
                             and torch.allclose(big, torch.full_like(big, (W + 1) / 2)))
    pg.barrier()
    if r == 0:
        print(json.dumps({"world": W, "ok": ok}))
    destroy_process_group()


if __name__ == "__main__":
    main()
