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
    # equal-split all-to-all: chunk j of the result is what rank j addressed to this rank
    got = pg.all_to_all(torch.arange(W * 2, dtype=torch.float32) + 100 * r)
    want = torch.cat([torch.arange(2 * r, 2 * r + 2, dtype=torch.float32) + 100 * j for j in range(W)])
    ok["all_to_all"] = bool(torch.equal(got, want))
    # ring attention over real point-to-point transfers, forward and backward
    from ml_framework_b200.ops.reference import attention_ref
    from ml_framework_b200.parallel.context_parallel import ring_attention, shard_sequence
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, 12 * W, h, 8, generator=g) for h in (4, 2, 2))
    fq, fk, fv = (t.clone().requires_grad_(True) for t in (q, k, v))
    full = attention_ref(fq, fk, fv, causal=True)[0]
    full.square().sum().backward()
    lq, lk, lv = (shard_sequence(t, r, W, zigzag=True).requires_grad_(True) for t in (q, k, v))
    out = ring_attention(lq, lk, lv, pg, causal=True, zigzag=True)
    out.square().sum().backward()
    ok["ring_attention"] = bool(
        torch.allclose(out, shard_sequence(full.detach(), r, W, zigzag=True), atol=1e-5)
        and torch.allclose(lq.grad, shard_sequence(fq.grad, r, W, zigzag=True), atol=1e-4)
        and torch.allclose(lk.grad, shard_sequence(fk.grad, r, W, zigzag=True), atol=1e-4)
        and torch.allclose(lv.grad, shard_sequence(fv.grad, r, W, zigzag=True), atol=1e-4))
    flags = pg.all_gather_object(ok)
    ok = {key: all(f[key] for f in flags) for key in ok}
    pg.barrier()
    if r == 0:
        print(json.dumps({"world": W, "ok": ok}))
    destroy_process_group()


if __name__ == "__main__":
    main()
