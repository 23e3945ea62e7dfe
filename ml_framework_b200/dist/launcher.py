"""Local multi-process launcher.

Same contract as the reference's ``ProcessLauncher`` / ``DistributedLauncher.LaunchLocal``
(src/MLFramework/Distributed/ProcessLauncher.cs:48-186, DistributedLauncher.cs:18-60): spawn
N ranks with ``RANK, WORLD_SIZE, LOCAL_RANK, MASTER_ADDR=127.0.0.1, MASTER_PORT`` (default
29500) and, when GPUs are used, one visible device per rank; keep per-rank log files; wait
for all; report the first failure. Multi-node launch is delegated to ``torchrun`` (the
reference's ``LaunchMultiNode`` is not implemented, DistributedLauncher.cs:110-122).
"""
from __future__ import annotations

import os
import signal
import subprocess
import sys
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional, Sequence


class DistributedTrainingError(RuntimeError):
    def __init__(self, msg: str, rank: Optional[int] = None, exit_code: Optional[int] = None):
        super().__init__(msg)
        self.rank, self.exit_code = rank, exit_code


@dataclass
class RankProcess:
    rank: int
    proc: subprocess.Popen
    log_path: Optional[Path]
    exit_code: Optional[int] = None


class ProcessLauncher:
    def __init__(self, master_addr: str = "127.0.0.1", master_port: int = 29500, log_dir: Optional[str] = None,
                 assign_gpus: bool = False):
        self.master_addr, self.master_port = master_addr, master_port
        self.log_dir = Path(log_dir) if log_dir else None
        self.assign_gpus = assign_gpus
        self.ranks: List[RankProcess] = []
        self._failed_first: Optional[RankProcess] = None   # the rank whose non-zero exit was observed first

    def launch(self, argv: Sequence[str], num_processes: int, extra_env: Optional[Dict[str, str]] = None, rank_offset: int = 0,
               world_size: Optional[int] = None) -> List[RankProcess]:
        """Starts ``num_processes`` local ranks. On one node of a multi-node job ``rank_offset`` is the global rank of
        this node's first process and ``world_size`` the job's total; ``LOCAL_RANK`` always counts from zero."""
        if num_processes <= 0:
            raise ValueError("num_processes must be positive")
        world = num_processes if world_size is None else world_size
        if rank_offset < 0 or rank_offset + num_processes > world:
            raise ValueError(f"ranks {rank_offset}..{rank_offset + num_processes - 1} do not fit a world of {world}")
        if self.log_dir:
            self.log_dir.mkdir(parents=True, exist_ok=True)
        for local in range(num_processes):
            rank = rank_offset + local
            env = dict(os.environ)
            env.update({"RANK": str(rank), "LOCAL_RANK": str(local), "WORLD_SIZE": str(world), "LOCAL_WORLD_SIZE": str(num_processes),
                        "MASTER_ADDR": self.master_addr, "MASTER_PORT": str(self.master_port)})
            if self.assign_gpus:
                env["CUDA_VISIBLE_DEVICES"] = str(local)
                env["LOCAL_RANK"] = "0"
            if extra_env:
                env.update(extra_env)
            log_path = self.log_dir / f"rank_{rank}.log" if self.log_dir else None
            out = open(log_path, "w") if log_path else None
            proc = subprocess.Popen(list(argv), env=env, stdout=out or None, stderr=subprocess.STDOUT if out else None,
                                    start_new_session=True)
            if out:
                out.close()
            self.ranks.append(RankProcess(rank, proc, log_path))
        return self.ranks

    def wait_for_all(self, timeout_s: Optional[float] = None, kill_on_failure: bool = True) -> bool:
        """True when every rank exited 0. On the first failure the others are terminated."""
        deadline = None if timeout_s is None else time.time() + timeout_s
        pending = {r.rank for r in self.ranks}
        while pending:
            for r in self.ranks:
                if r.rank in pending:
                    code = r.proc.poll()
                    if code is not None:
                        r.exit_code = code
                        pending.discard(r.rank)
                        if code != 0 and self._failed_first is None:
                            self._failed_first = r      # before the others are terminated (they then exit with -SIGTERM)
                        if code != 0 and kill_on_failure:
                            self.terminate_all()
                            for o in self.ranks:
                                if o.exit_code is None:
                                    o.exit_code = o.proc.wait()
                            return False
            if deadline is not None and time.time() > deadline:
                self.terminate_all()
                raise DistributedTrainingError(f"ranks {sorted(pending)} did not finish within {timeout_s}s")
            time.sleep(0.02)
        return all(r.exit_code == 0 for r in self.ranks)

    def terminate_all(self):
        for r in self.ranks:
            if r.proc.poll() is None:
                try:
                    os.killpg(r.proc.pid, signal.SIGTERM)
                except (ProcessLookupError, PermissionError):
                    pass
        t0 = time.time()
        for r in self.ranks:
            while r.proc.poll() is None and time.time() - t0 < 5:
                time.sleep(0.02)
            if r.proc.poll() is None:
                try:
                    os.killpg(r.proc.pid, signal.SIGKILL)
                except (ProcessLookupError, PermissionError):
                    pass

    def has_failed_process(self) -> bool:
        return any(r.exit_code not in (None, 0) for r in self.ranks)

    def first_failed_process(self) -> Optional[RankProcess]:
        """The rank that failed first in time (ProcessLauncher.cs:128-186), not the lowest-numbered rank with a
        non-zero code: ranks terminated because of that failure also end with a non-zero code."""
        if self._failed_first is not None:
            return self._failed_first
        for r in self.ranks:
            if r.exit_code not in (None, 0):
                return r
        return None


def launch_local(script: str, num_processes: int, script_args: Sequence[str] = (), master_port: int = 29500,
                 log_dir: Optional[str] = None, assign_gpus: bool = False, timeout_s: Optional[float] = None,
                 extra_env: Optional[Dict[str, str]] = None) -> ProcessLauncher:
    """Run ``python script args...`` as ``num_processes`` local ranks and wait for them."""
    launcher = ProcessLauncher(master_port=master_port, log_dir=log_dir, assign_gpus=assign_gpus)
    launcher.launch([sys.executable, script, *script_args], num_processes, extra_env)
    ok = launcher.wait_for_all(timeout_s)
    if not ok:
        bad = launcher.first_failed_process()
        tail = ""
        if bad and bad.log_path and bad.log_path.exists():
            tail = "\n" + "\n".join(bad.log_path.read_text().splitlines()[-20:])
        raise DistributedTrainingError(f"rank {bad.rank if bad else '?'} failed with exit code "
                                       f"{bad.exit_code if bad else '?'}{tail}", bad.rank if bad else None,
                                       bad.exit_code if bad else None)
    return launcher


def launch_multi_node(script: str, nnodes: int, node_rank: int, nproc_per_node: int, master_addr: str, master_port: int = 29500,
                      script_args: Sequence[str] = (), log_dir: Optional[str] = None, assign_gpus: bool = False,
                      timeout_s: Optional[float] = None, extra_env: Optional[Dict[str, str]] = None) -> ProcessLauncher:
    """This node's share of a multi-node job: run the same call on every node with its own ``node_rank`` (0 .. nnodes-1)
    and the address of node 0. Local processes get global ranks ``node_rank * nproc_per_node + local``; rendezvous is
    the TCP store at ``master_addr:master_port`` that ``init_process_group`` opens. (The reference's
    ``LaunchMultiNode`` is a NotImplemented stub: src/MLFramework/Distributed/DistributedLauncher.cs:76-122.)"""
    if nnodes <= 0 or not (0 <= node_rank < nnodes) or nproc_per_node <= 0:
        raise ValueError(f"invalid layout: {nnodes} nodes, node rank {node_rank}, {nproc_per_node} processes per node")
    launcher = ProcessLauncher(master_addr=master_addr, master_port=master_port, log_dir=log_dir, assign_gpus=assign_gpus)
    env = {"GROUP_RANK": str(node_rank), "NNODES": str(nnodes)}
    env.update(extra_env or {})
    launcher.launch([sys.executable, script, *script_args], nproc_per_node, env, rank_offset=node_rank * nproc_per_node,
                    world_size=nnodes * nproc_per_node)
    if not launcher.wait_for_all(timeout_s):
        bad = launcher.first_failed_process()
        raise DistributedTrainingError(f"node {node_rank}: rank {bad.rank if bad else '?'} failed with exit code {bad.exit_code if bad else '?'}",
                                       bad.rank if bad else None, bad.exit_code if bad else None)
    return launcher
