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

    def launch(self, argv: Sequence[str], num_processes: int, extra_env: Optional[Dict[str, str]] = None) -> List[RankProcess]:
        if num_processes <= 0:
            raise ValueError("num_processes must be positive")
        if self.log_dir:
            self.log_dir.mkdir(parents=True, exist_ok=True)
        for rank in range(num_processes):
            env = dict(os.environ)
            env.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(num_processes),
                        "MASTER_ADDR": self.master_addr, "MASTER_PORT": str(self.master_port)})
            if self.assign_gpus:
                env["CUDA_VISIBLE_DEVICES"] = str(rank)
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


def launch_multi_node(*_a, **_k):
    raise NotImplementedError("use torchrun (--nnodes, --rdzv-endpoint) for multi-node jobs; every rank then calls "
                              "init_process_group() which reads the torchrun environment")
