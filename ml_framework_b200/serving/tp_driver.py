"""Tensor-parallel serving: rank 0 owns the request queue and the continuous-batching scheduler; every iteration it
broadcasts the batch plan, and all ranks run the same executor step on their shard of the model and of the KV
cache (KV heads are split over the ranks, so each rank's block manager makes the same allocations in the same
order and the block tables stay identical without being sent).

The reference has no multi-GPU serving path; its scheduler drives one ``IModelExecutor``
(src/MLFramework/Inference/ContinuousBatching/Scheduler/ContinuousBatchScheduler.cs:114-276). The plan broadcast is
the host-side half of the design; the device-side half is the all-reduce of the o- and down-projection partial
sums inside ``PagedLlamaExecutor._reduce`` (one-shot peer-memory kernel or a process-group all-reduce).
"""
from __future__ import annotations

from typing import Dict

from .executor import PagedLlamaExecutor
from .scheduler import Batch, BatchOutput, Request


class TPLeaderExecutor:
    """Wraps rank 0's executor: publishes the plan of each iteration before executing it."""

    def __init__(self, executor: PagedLlamaExecutor, pg):
        self.ex, self.pg = executor, pg
        self.kv = executor.kv
        self.live_ids_fn = None                   # callable returning the ids the scheduler still tracks (set by the owner)

    def execute_batch(self, batch: Batch) -> BatchOutput:
        live = {r.id for r in batch.requests} | {r.id for r in batch.prefill} | {r.id for r in batch.decode}
        if self.live_ids_fn is not None:
            live |= set(self.live_ids_fn())
        plan = {"prefill": [(r.id, list(r.prompt_tokens), r.prefilled) for r in batch.prefill],
                "decode": [(r.id, (r.generated[-1] if r.generated else r.prompt_tokens[-1])) for r in batch.decode],
                "live": sorted(live)}
        self.pg.broadcast_object(plan, src=0)
        return self.ex.execute_batch(batch)

    def shutdown(self):
        self.pg.broadcast_object(None, src=0)


def follower_loop(executor: PagedLlamaExecutor, pg) -> int:
    """Runs on every rank but 0 until the leader sends the stop message; returns the number of iterations executed."""
    shadow: Dict[int, Request] = {}
    iters = 0
    while True:
        plan = pg.broadcast_object(None, src=0)
        if plan is None:
            return iters
        live = set(plan["live"])
        for rid in [k for k in shadow if k not in live]:          # the leader's scheduler released these
            executor.kv.free_sequence_blocks(rid)
            del shadow[rid]
        prefill, decode = [], []
        for rid, prompt, prefilled in plan["prefill"]:
            r = shadow.get(rid)
            if r is None:
                r = Request(list(prompt))
                r.id = rid
                shadow[rid] = r
            r.prefilled = prefilled
            prefill.append(r)
        for rid, last in plan["decode"]:
            r = shadow[rid]
            r.generated = [last]                                   # the executor reads only the last token
            decode.append(r)
        executor.execute_batch(Batch(requests=list(shadow.values()), prefill=prefill, decode=decode))
        iters += 1
