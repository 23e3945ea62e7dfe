"""Pipeline parallelism: stages, layer partitioning, micro-batching, GPipe and 1F1B schedules.

Reference semantics (src/MLFramework/Pipeline/): ``PipelineStage`` wraps a sub-module with
(rank, total stages, device) (PipelineStage.cs:14-142); ``LayerPartitioner`` splits a layer list
Automatic (cost-balanced greedy) / Uniform / Manual (LayerPartitioner.cs:60-420);
``MicroBatchManager`` splits dim 0 into N micro-batches (the last takes the remainder),
accumulates gradients and averages by 1/N (MicroBatchManager.cs:106-262); ``GPipeScheduler`` runs
all forwards then all backwards in reverse order (GPipeScheduler.cs:73-189). The reference has
no 1F1B ("to be implemented later", SchedulingStrategy.cs:14-16); it is implemented here: rank r
of p runs ``p - r - 1`` warm-up forwards, then alternates one forward / one backward, then
drains, which bounds live activations to ``p - r`` micro-batches instead of N.

One process per stage. Activations / gradients cross stage boundaries through an
``IPipelineCommunicator`` (IPipelineCommunicator.cs:10-71): ``ProcessGroupPipelineCommunicator``
uses the process group's point-to-point ops (NCCL ``batch_isend_irecv`` on GPUs, issued on a side
stream so transfers overlap compute), ``LocalPipelineCommunicator`` uses in-process queues for
single-process tests (LocalPipelineCommunicator.cs:55-249).
"""
from __future__ import annotations

import enum
import queue
import threading
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn


class SchedulingStrategy(enum.Enum):
    GPIPE = "gpipe"
    ONE_F_ONE_B = "1f1b"


class PartitionMode(enum.Enum):
    AUTOMATIC = "automatic"
    UNIFORM = "uniform"
    MANUAL = "manual"


class CheckpointStrategy(enum.Enum):
    STORE_ALL = "store_all"
    RECOMPUTE_ALL = "recompute_all"
    SELECTIVE = "selective"
    MEMORY_BASED = "memory_based"


class GradientSyncMode(enum.Enum):
    AVERAGE = "average"
    SUM = "sum"
    NONE = "none"


@dataclass
class PipelineConfig:
    num_stages: int = 2
    micro_batches: int = 4
    schedule: SchedulingStrategy = SchedulingStrategy.ONE_F_ONE_B
    checkpoint_strategy: CheckpointStrategy = CheckpointStrategy.STORE_ALL
    checkpoint_interval: int = 2
    devices: Optional[List[int]] = None

    def validate(self):
        if self.num_stages <= 0:
            raise ValueError("num_stages must be positive")
        if self.micro_batches <= 0:
            raise ValueError("micro_batches must be positive")
        if self.devices is not None and len(self.devices) != self.num_stages:
            raise ValueError("devices must list one entry per stage")


@dataclass
class PipelineStats:
    forward_time_s: float = 0.0
    backward_time_s: float = 0.0
    comm_time_s: float = 0.0
    micro_batches: int = 0
    stages: int = 0

    @property
    def bubble_fraction(self) -> float:
        """(p - 1) / (m + p - 1) for both GPipe and 1F1B."""
        p, m = self.stages, self.micro_batches
        return (p - 1) / (m + p - 1) if m + p - 1 > 0 else 0.0


# ------------------------------------------------------------------ partitioning
@dataclass
class PartitionResult:
    boundaries: List[Tuple[int, int]]      # [start, end) layer indices per stage
    costs: List[float]


class LayerPartitioner:
    def __init__(self, mode: PartitionMode = PartitionMode.AUTOMATIC, manual: Optional[Sequence[int]] = None):
        self.mode, self.manual = mode, manual

    @staticmethod
    def layer_cost(layer: nn.Module) -> float:
        """Parameter count as the proxy for both memory and compute (LayerPartitioner.cs:337-420)."""
        return float(sum(p.numel() for p in layer.parameters())) + 1.0

    def partition(self, layers: Sequence[nn.Module], num_stages: int) -> PartitionResult:
        n = len(layers)
        if num_stages <= 0 or num_stages > n:
            raise ValueError(f"cannot split {n} layers into {num_stages} stages")
        costs = [self.layer_cost(l) for l in layers]
        if self.mode == PartitionMode.MANUAL:
            if not self.manual or len(self.manual) != num_stages or sum(self.manual) != n:
                raise ValueError("manual partition must list one positive size per stage summing to the layer count")
            sizes = list(self.manual)
        elif self.mode == PartitionMode.UNIFORM:
            sizes = [n // num_stages + (1 if i < n % num_stages else 0) for i in range(num_stages)]
        else:
            sizes = self._balanced(costs, num_stages)
        bounds, s = [], 0
        for k in sizes:
            bounds.append((s, s + k))
            s += k
        return PartitionResult(bounds, [sum(costs[a:b]) for a, b in bounds])

    @staticmethod
    def _balanced(costs: List[float], k: int) -> List[int]:
        """Contiguous split minimising the heaviest stage (binary search on the bottleneck)."""
        n = len(costs)
        lo, hi = max(costs), sum(costs)

        def fits(cap):
            parts, cur, sizes, cnt = 1, 0.0, [], 0
            for c in costs:
                if cur + c > cap and cnt > 0:
                    parts += 1
                    sizes.append(cnt)
                    cur, cnt = 0.0, 0
                cur += c
                cnt += 1
            sizes.append(cnt)
            return parts <= k, sizes
        for _ in range(60):
            mid = (lo + hi) / 2
            ok, _ = fits(mid)
            if ok:
                hi = mid
            else:
                lo = mid
        _, sizes = fits(hi)
        while len(sizes) < k:      # split the largest multi-layer stage until there are k stages
            i = max(range(len(sizes)), key=lambda j: sizes[j])
            if sizes[i] < 2:
                break
            sizes[i:i + 1] = [sizes[i] - sizes[i] // 2, sizes[i] // 2]
        return sizes


class PipelineStage(nn.Module):
    def __init__(self, module: nn.Module, rank: int, total_stages: int, device=None):
        super().__init__()
        if not (0 <= rank < total_stages):
            raise ValueError("stage rank out of range")
        self.module, self.rank, self.total_stages = module, rank, total_stages
        self.device = device
        if device is not None:
            self.module.to(device)

    @property
    def is_first(self):
        return self.rank == 0

    @property
    def is_last(self):
        return self.rank == self.total_stages - 1

    def forward(self, x):
        return self.module(x)


def build_stage(layers: Sequence[nn.Module], rank: int, num_stages: int, partitioner: Optional[LayerPartitioner] = None,
                device=None) -> PipelineStage:
    part = (partitioner or LayerPartitioner()).partition(layers, num_stages)
    a, b = part.boundaries[rank]
    return PipelineStage(nn.Sequential(*layers[a:b]), rank, num_stages, device)


# ------------------------------------------------------------------ micro-batches
class MicroBatchManager:
    def __init__(self, num_micro_batches: int):
        if num_micro_batches <= 0:
            raise ValueError("num_micro_batches must be positive")
        self.n = num_micro_batches
        self._acc: Dict[int, torch.Tensor] = {}
        self._count = 0

    def split_batch(self, batch: torch.Tensor) -> List[torch.Tensor]:
        B = batch.shape[0]
        if B < self.n:
            raise ValueError(f"batch of {B} cannot be split into {self.n} micro-batches")
        base = B // self.n
        sizes = [base] * self.n
        sizes[-1] += B - base * self.n          # the last micro-batch takes the remainder
        return list(batch.split(sizes, dim=0))

    def combine_outputs(self, outs: Sequence[torch.Tensor]) -> torch.Tensor:
        return torch.cat(list(outs), dim=0)

    def accumulate_gradients(self, params: Sequence[nn.Parameter]):
        for i, p in enumerate(params):
            if p.grad is None:
                continue
            if i in self._acc:
                self._acc[i].add_(p.grad)
            else:
                self._acc[i] = p.grad.detach().clone()
            p.grad = None
        self._count += 1

    def get_accumulated_gradients(self, average: bool = True) -> Dict[int, torch.Tensor]:
        out = {i: (g / self.n if average else g) for i, g in self._acc.items()}
        self._acc, self._count = {}, 0
        return out


class ActivationCheckpointManager:
    """Which micro-batch activations to keep and which to recompute (ActivationCheckpointManager.cs:49-175)."""

    def __init__(self, strategy: CheckpointStrategy = CheckpointStrategy.STORE_ALL, interval: int = 2,
                 memory_budget_bytes: Optional[int] = None):
        self.strategy, self.interval, self.budget = strategy, max(1, interval), memory_budget_bytes
        self.stored_bytes = 0

    def should_checkpoint(self, micro_batch: int, nbytes: int = 0) -> bool:
        """True = do not keep the autograd graph; recompute in backward."""
        if self.strategy == CheckpointStrategy.STORE_ALL:
            return False
        if self.strategy == CheckpointStrategy.RECOMPUTE_ALL:
            return True
        if self.strategy == CheckpointStrategy.SELECTIVE:
            return micro_batch % self.interval != 0
        if self.budget is None:
            return False
        if self.stored_bytes + nbytes > self.budget:
            return True
        self.stored_bytes += nbytes
        return False

    def release(self, nbytes: int):
        self.stored_bytes = max(0, self.stored_bytes - nbytes)


# ------------------------------------------------------------------ communicators
class LocalPipelineCommunicator:
    """In-process queues keyed by (src, dst, kind); one instance shared by all stage threads."""

    def __init__(self, num_stages: int, timeout_s: float = 30.0):
        self.num_stages, self.timeout_s = num_stages, timeout_s
        self._q: Dict[tuple, "queue.Queue"] = {}
        self._lock = threading.Lock()
        self._barrier = threading.Barrier(num_stages)

    def _queue(self, key):
        with self._lock:
            return self._q.setdefault(key, queue.Queue())

    def send(self, t: torch.Tensor, src: int, dst: int, kind: str = "fwd"):
        self._queue((src, dst, kind)).put(t.detach().clone())

    def recv(self, src: int, dst: int, kind: str = "fwd") -> torch.Tensor:
        try:
            return self._queue((src, dst, kind)).get(timeout=self.timeout_s)
        except queue.Empty:
            raise TimeoutError(f"pipeline recv {kind} {src}->{dst} timed out") from None

    def barrier(self):
        self._barrier.wait(self.timeout_s)

    def view(self, rank: int) -> "_LocalView":
        return _LocalView(self, rank)


class _LocalView:
    def __init__(self, comm: LocalPipelineCommunicator, rank: int):
        self.c, self.rank = comm, rank

    def send_forward(self, t): self.c.send(t, self.rank, self.rank + 1, "fwd")
    def recv_forward(self, shape=None, dtype=None, device=None): return self.c.recv(self.rank - 1, self.rank, "fwd")
    def send_backward(self, t): self.c.send(t, self.rank, self.rank - 1, "bwd")
    def recv_backward(self, shape=None, dtype=None, device=None): return self.c.recv(self.rank + 1, self.rank, "bwd")
    def barrier(self): self.c.barrier()

    def send_forward_recv_backward(self, t, shape=None, dtype=None, device=None):
        self.send_forward(t)
        return self.recv_backward()

    def send_backward_recv_forward(self, t, shape=None, dtype=None, device=None):
        self.send_backward(t)
        return self.recv_forward()


class ProcessGroupPipelineCommunicator:
    """Stage-to-stage transfers over a process group (stage s == group rank s).

    Over NCCL every transfer runs on a communication stream of its own and the compute stream is never made to wait
    for a transfer as a whole (the reference's per-micro-batch compute / communication streams joined by events,
    src/MLFramework/Pipeline/AsyncPipelineExecutor.cs:76-320, StreamManager.cs:51-141): the communication stream
    waits for an event recorded after the producing kernels, a sent tensor is only kept alive until its transfer's
    event has passed, and a received tensor carries an event that the compute stream waits for at the point where
    the schedule consumes it (``wait_ready``). The host therefore queues the next compute phase while the
    transfer is in flight, and sends overlap whatever compute follows them."""

    def __init__(self, pg, use_side_stream: bool = True):
        self.pg, self.rank = pg, pg.rank
        self.stream = None
        self._pending: list = []
        self._ready: Dict[int, object] = {}       # received buffer address -> event of its transfer
        self._inflight: list = []                 # (event, tensor) of sends not known to be complete
        if use_side_stream and torch.cuda.is_available() and str(getattr(pg, "backend", "")).lower().endswith("nccl"):
            self.stream = torch.cuda.Stream()

    def _run(self, ops):
        if self.stream is None:
            # Host-blocking backends: only receives are waited for here. A send completes when the peer posts
            # its receive, which in 1F1B can be after the peer's own send to this rank, so sends stay pending
            # (tensor kept alive) and are collected later.
            works = self.pg.batch_isend_irecv(ops)
            for (kind, t, _), w in zip(ops, works):
                if kind == "recv":
                    w.wait()
                else:
                    self._pending.append((w, t))
            while len(self._pending) > 64:
                self._pending.pop(0)[0].wait()
            return
        produced = torch.cuda.Event()
        produced.record()                          # after the kernels that wrote the tensors being sent
        self.stream.wait_event(produced)
        with torch.cuda.stream(self.stream):
            works = self.pg.batch_isend_irecv(ops)
            for w in works:
                w.wait()                           # orders the communication stream, not the host
            done = torch.cuda.Event()
            done.record(self.stream)
        for kind, t, _ in ops:
            t.record_stream(self.stream)           # the allocator must not hand the memory out before the transfer ran
            if kind == "recv":
                self._ready[t.data_ptr()] = done
            else:
                self._inflight.append((done, t))
        while self._inflight and (len(self._inflight) > 32 or self._inflight[0][0].query()):
            self._inflight.pop(0)

    def wait_ready(self, t: Optional[torch.Tensor]):
        """Called by the schedule where a received tensor is first used: the compute stream waits for that transfer only."""
        if t is None or self.stream is None:
            return
        ev = self._ready.pop(t.data_ptr(), None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def send_forward(self, t): self._run([("send", t.contiguous(), self.rank + 1)])
    def send_backward(self, t): self._run([("send", t.contiguous(), self.rank - 1)])

    def recv_forward(self, shape, dtype, device):
        buf = torch.empty(shape, dtype=dtype, device=device)
        self._run([("recv", buf, self.rank - 1)])
        return buf

    def recv_backward(self, shape, dtype, device):
        buf = torch.empty(shape, dtype=dtype, device=device)
        self._run([("recv", buf, self.rank + 1)])
        return buf

    def send_forward_recv_backward(self, t, shape, dtype, device):
        buf = torch.empty(shape, dtype=dtype, device=device)
        self._run([("send", t.contiguous(), self.rank + 1), ("recv", buf, self.rank + 1)])
        return buf

    def send_backward_recv_forward(self, t, shape, dtype, device):
        buf = torch.empty(shape, dtype=dtype, device=device)
        self._run([("send", t.contiguous(), self.rank - 1), ("recv", buf, self.rank - 1)])
        return buf

    def barrier(self):
        while self._pending:
            self._pending.pop(0)[0].wait()
        if self.stream is not None:
            torch.cuda.current_stream().wait_stream(self.stream)
            self._inflight.clear()
        self.pg.barrier()


# ------------------------------------------------------------------ schedules
class _ScheduleBase:
    def __init__(self, stage: PipelineStage, comm, config: PipelineConfig, loss_fn: Optional[Callable] = None,
                 act_shape_fn: Optional[Callable[[torch.Tensor], tuple]] = None, act_dtype=None):
        config.validate()
        self.stage, self.comm, self.cfg, self.loss_fn = stage, comm, config, loss_fn
        self.ckpt = ActivationCheckpointManager(config.checkpoint_strategy, config.checkpoint_interval)
        self.act_shape_fn, self.act_dtype = act_shape_fn, act_dtype
        self.stats = PipelineStats(stages=stage.total_stages, micro_batches=config.micro_batches)
        self._saved: Dict[int, tuple] = {}
        self._out_spec: Dict[int, tuple] = {}
        self.losses: List[torch.Tensor] = []

    def _consume(self, t):
        """A tensor that arrived from a neighbour is about to be read: wait for its transfer (asynchronous communicators)."""
        fn = getattr(self.comm, "wait_ready", None)
        if fn is not None and t is not None:
            fn(t)

    def _act_spec(self, x_local=None):
        st = self.stage
        shape = self.act_shape_fn(x_local) if self.act_shape_fn else None
        return shape, self.act_dtype or next(st.parameters()).dtype, next(st.parameters()).device

    # one micro-batch forward on this stage
    def _forward(self, mb: int, x_local: Optional[torch.Tensor], target: Optional[torch.Tensor]):
        st = self.stage
        if st.is_first:
            x = x_local
        else:
            x = self.comm.recv_forward(*self._act_spec(x_local))
        y = self._forward_compute(mb, x, target)
        if not st.is_last:
            self.comm.send_forward(y.detach())

    def _forward_compute(self, mb: int, x: torch.Tensor, target: Optional[torch.Tensor]):
        """Runs the stage on one micro-batch (input already here); returns the stage output."""
        st = self.stage
        t0 = time.perf_counter()
        self._consume(x)
        if not st.is_first:
            x = x.detach().requires_grad_(True)
        recompute = self.ckpt.should_checkpoint(mb, x.numel() * x.element_size())
        if recompute and st.is_last and self.loss_fn is not None:
            # nothing downstream needs this stage's output now, and the backward pass runs the forward again anyway:
            # the last stage only remembers its input (its loss is recorded when the micro-batch is recomputed)
            self._saved[mb] = (x, None, True, target)
            self.stats.forward_time_s += time.perf_counter() - t0
            return None
        if recompute:
            with torch.no_grad():
                y = st(x)
            self._saved[mb] = (x, None, True, target)
        else:
            y = st(x)
            self._saved[mb] = (x, y, False, target)
        if st.is_last:
            if self.loss_fn is not None:
                loss = self.loss_fn(y, target) if not recompute else None
                if loss is not None:
                    self._saved[mb] = (x, loss, False, target)
                    self.losses.append(loss.detach())
        self._out_spec[mb] = (tuple(y.shape), y.dtype, y.device)
        self.stats.forward_time_s += time.perf_counter() - t0
        return y

    def _backward(self, mb: int):
        st = self.stage
        g = None
        if not st.is_last:
            g = self.comm.recv_backward(*self._out_spec[mb])
        dx = self._backward_compute(mb, g)
        if not st.is_first:
            self.comm.send_backward(dx)

    def _backward_compute(self, mb: int, g: Optional[torch.Tensor]):
        """Backward of one micro-batch given the gradient of the stage output (None on the last stage);
        returns the gradient of the stage input (None on the first stage)."""
        st = self.stage
        t0 = time.perf_counter()
        self._consume(g)
        x, y, recompute, target = self._saved.pop(mb)
        if recompute:
            y = st(x)
            if st.is_last and self.loss_fn is not None:
                y = self.loss_fn(y, target)
                self.losses.append(y.detach())
        if st.is_last:
            (y / self.cfg.micro_batches).backward() if self.loss_fn is not None else y.backward(torch.ones_like(y) / self.cfg.micro_batches)
        else:
            y.backward(g.reshape(y.shape))
        self.stats.backward_time_s += time.perf_counter() - t0
        return None if st.is_first else x.grad

    def order(self) -> List[Tuple[str, int]]:
        raise NotImplementedError

    def train_iteration(self, inputs: Optional[torch.Tensor], targets: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Runs one pipeline iteration on this stage. ``inputs`` is needed on the first stage (and,
        for its batch shape, optionally elsewhere), ``targets`` on the last. Gradients of all
        micro-batches accumulate into ``param.grad`` scaled by 1/N. Returns the mean loss on the
        last stage, None elsewhere."""
        n = self.cfg.micro_batches
        mbm = MicroBatchManager(n)
        xs = mbm.split_batch(inputs) if inputs is not None else [None] * n
        ts = mbm.split_batch(targets) if targets is not None else [None] * n
        self.losses = []
        for kind, mb in self.order():
            if kind == "F":
                self._forward(mb, xs[mb], ts[mb])
            else:
                self._backward(mb)
        if self.stage.is_last and self.losses:
            return torch.stack(self.losses).mean()
        return None


class GPipeScheduler(_ScheduleBase):
    def order(self):
        n = self.cfg.micro_batches
        return [("F", i) for i in range(n)] + [("B", i) for i in reversed(range(n))]


class OneFOneBScheduler(_ScheduleBase):
    def order(self):
        n, p, r = self.cfg.micro_batches, self.stage.total_stages, self.stage.rank
        warm = min(p - r - 1, n)
        seq = [("F", i) for i in range(warm)]
        f, b = warm, 0
        while f < n:
            seq.append(("F", f)); f += 1
            seq.append(("B", b)); b += 1
        while b < n:
            seq.append(("B", b)); b += 1
        return seq

    def train_iteration(self, inputs: Optional[torch.Tensor], targets: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """1F1B with paired transfers in the steady state: a stage hands its output forward and takes the
        gradient of an earlier micro-batch back in ONE batched point-to-point group (and the mirror image
        after each backward). Separate blocking sends in opposite directions between two neighbours wait on
        each other once a message exceeds the transport's buffering; paired groups cannot."""
        n, p, r = self.cfg.micro_batches, self.stage.total_stages, self.stage.rank
        st, comm = self.stage, self.comm
        if not hasattr(comm, "send_forward_recv_backward"):
            return super().train_iteration(inputs, targets)
        mbm = MicroBatchManager(n)
        xs = mbm.split_batch(inputs) if inputs is not None else [None] * n
        ts = mbm.split_batch(targets) if targets is not None else [None] * n
        self.losses = []
        spec = self._act_spec(None) if (not st.is_first or not st.is_last) else None
        warm = min(p - r - 1, n)
        steady = n - warm
        for i in range(warm):
            x = xs[i] if st.is_first else comm.recv_forward(*spec)
            y = self._forward_compute(i, x, ts[i])
            if not st.is_last:
                comm.send_forward(y.detach())
        x = None
        if steady > 0:
            x = xs[warm] if st.is_first else comm.recv_forward(*spec)
        for i in range(steady):
            f = warm + i
            y = self._forward_compute(f, x, ts[f])
            g = None if st.is_last else comm.send_forward_recv_backward(y.detach(), *self._out_spec[i])
            dx = self._backward_compute(i, g)
            last_fwd = i == steady - 1
            if st.is_first:
                x = None if last_fwd else xs[f + 1]
            elif last_fwd:
                comm.send_backward(dx)
            else:
                x = comm.send_backward_recv_forward(dx, *spec)
        for b in range(steady, n):
            g = None if st.is_last else comm.recv_backward(*self._out_spec[b])
            dx = self._backward_compute(b, g)
            if not st.is_first:
                comm.send_backward(dx)
        if st.is_last and self.losses:
            return torch.stack(self.losses).mean()
        return None

    def max_live_activations(self) -> int:
        live = peak = 0
        for kind, _ in self.order():
            live += 1 if kind == "F" else -1
            peak = max(peak, live)
        return peak


def make_scheduler(stage, comm, config: PipelineConfig, **kw) -> _ScheduleBase:
    cls = GPipeScheduler if config.schedule == SchedulingStrategy.GPIPE else OneFOneBScheduler
    return cls(stage, comm, config, **kw)


# ------------------------------------------------------------------ optimizer / validator
@dataclass
class PipelineOptimizerConfig:
    sync_mode: GradientSyncMode = GradientSyncMode.AVERAGE
    timeout_s: float = 30.0


class PipelineOptimizer:
    """Per-stage optimizer step; gradients of parameters shared between stages (tied embeddings)
    are all-reduced over ``shared_group`` first (PipelineOptimizer.cs:63-118)."""

    def __init__(self, optimizer, shared_params: Sequence[nn.Parameter] = (), shared_group=None,
                 config: Optional[PipelineOptimizerConfig] = None, dp_group=None):
        self.opt, self.shared, self.group, self.cfg, self.dp = optimizer, list(shared_params), shared_group, config or PipelineOptimizerConfig(), dp_group

    def synchronize_gradients(self, params: Sequence[nn.Parameter] = ()):
        from ..dist.process_group import ReduceOp
        if self.group is not None:
            for p in self.shared:
                if p.grad is not None:
                    self.group.all_reduce(p.grad, ReduceOp.SUM)
        if self.dp is not None and self.cfg.sync_mode != GradientSyncMode.NONE:
            op = ReduceOp.AVG if self.cfg.sync_mode == GradientSyncMode.AVERAGE else ReduceOp.SUM
            for p in params:
                if p.grad is not None:
                    self.dp.all_reduce(p.grad, op)

    def step(self, params: Sequence[nn.Parameter] = ()):
        self.synchronize_gradients(params)
        self.opt.step()

    def broadcast_parameters(self, src: int = 0):
        if self.group is not None:
            for p in self.shared:
                self.group.broadcast(p.data, src=src)


class PipelineValidator:
    """Configuration, numerical-stability and gradient-equivalence checks (PipelineValidator.cs:53-483)."""

    @staticmethod
    def validate_configuration(cfg: PipelineConfig, num_layers: int, batch: int) -> List[str]:
        errs = []
        try:
            cfg.validate()
        except ValueError as e:
            errs.append(str(e))
        if cfg.num_stages > num_layers:
            errs.append("more stages than layers")
        if batch < cfg.micro_batches:
            errs.append("batch smaller than the number of micro-batches")
        return errs

    @staticmethod
    def validate_numerical_stability(tensors: Sequence[torch.Tensor]) -> bool:
        return all(bool(torch.isfinite(t).all()) for t in tensors if t is not None)

    @staticmethod
    def validate_gradients(pipeline_grads: Sequence[torch.Tensor], reference_grads: Sequence[torch.Tensor], atol=1e-5) -> bool:
        return len(pipeline_grads) == len(reference_grads) and all(
            torch.allclose(a, b, atol=atol) for a, b in zip(pipeline_grads, reference_grads))


# ------------------------------------------------------------------ streams for compute / communication overlap
class StreamManager:
    """Round-robin pools of compute and communication CUDA streams with named events
    (src/MLFramework/Pipeline/StreamManager.cs:51-141). On a CPU device every stream is ``None`` and
    events complete immediately."""

    def __init__(self, device=None, num_compute: int = 2, num_comm: int = 2):
        self.device = torch.device(device) if device is not None else (torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu"))
        cuda = self.device.type == "cuda"
        self.compute = [torch.cuda.Stream(self.device) if cuda else None for _ in range(max(1, num_compute))]
        self.comm = [torch.cuda.Stream(self.device, priority=-1) if cuda else None for _ in range(max(1, num_comm))]
        self._events = {}

    def compute_stream(self, micro_batch: int):
        return self.compute[micro_batch % len(self.compute)]

    def comm_stream(self, micro_batch: int):
        return self.comm[micro_batch % len(self.comm)]

    def record_event(self, name: str, stream):
        if stream is None:
            self._events[name] = None
            return
        ev = torch.cuda.Event()
        ev.record(stream)
        self._events[name] = ev

    def wait_for_event(self, name: str, stream):
        if name not in self._events:
            raise KeyError(f"event {name!r} was never recorded")
        ev = self._events[name]
        if ev is not None and stream is not None:
            stream.wait_event(ev)

    def synchronize(self):
        for s in self.compute + self.comm:
            if s is not None:
                s.synchronize()


class AsyncPipelineExecutor:
    """Runs a stage's forward / backward of micro-batch ``i`` on compute stream ``i mod n`` and its sends /
    receives on communication stream ``i mod n``, ordering the two with events, so that the transfer of one
    micro-batch overlaps the computation of the next (src/MLFramework/Pipeline/AsyncPipelineExecutor.cs:76-320)."""

    def __init__(self, stage: "PipelineStage", comm, streams: Optional[StreamManager] = None):
        self.stage, self.comm = stage, comm
        self.streams = streams or StreamManager(next(stage.parameters()).device)
        self._outs = {}

    def _on(self, stream):
        import contextlib
        return torch.cuda.stream(stream) if stream is not None else contextlib.nullcontext()

    def forward_async(self, x: torch.Tensor, micro_batch: int) -> torch.Tensor:
        cs = self.streams.compute_stream(micro_batch)
        if f"recv_f{micro_batch}" in self.streams._events:
            self.streams.wait_for_event(f"recv_f{micro_batch}", cs)
        with self._on(cs):
            y = self.stage(x)
        self.streams.record_event(f"fwd{micro_batch}", cs)
        self._outs[micro_batch] = (x, y)
        return y

    def send_async(self, t: torch.Tensor, micro_batch: int, direction: str = "forward"):
        ms = self.streams.comm_stream(micro_batch)
        self.streams.wait_for_event(f"{'fwd' if direction == 'forward' else 'bwd'}{micro_batch}", ms)
        with self._on(ms):
            (self.comm.send_forward if direction == "forward" else self.comm.send_backward)(t)
        self.streams.record_event(f"send_{direction[0]}{micro_batch}", ms)

    def receive_async(self, like: torch.Tensor, micro_batch: int, direction: str = "forward") -> torch.Tensor:
        ms = self.streams.comm_stream(micro_batch)
        with self._on(ms):
            t = (self.comm.recv_forward if direction == "forward" else self.comm.recv_backward)(tuple(like.shape), like.dtype, like.device)
        self.streams.record_event(f"recv_{direction[0]}{micro_batch}", ms)
        return t

    def backward_async(self, grad_out: torch.Tensor, micro_batch: int) -> Optional[torch.Tensor]:
        cs = self.streams.compute_stream(micro_batch)
        x, y = self._outs.pop(micro_batch)
        if f"recv_b{micro_batch}" in self.streams._events:
            self.streams.wait_for_event(f"recv_b{micro_batch}", cs)
        with self._on(cs):
            y.backward(grad_out)
        self.streams.record_event(f"bwd{micro_batch}", cs)
        return x.grad if x.requires_grad else None

    def sync_compute(self):
        for s in self.streams.compute:
            if s is not None:
                s.synchronize()

    def sync_comm(self):
        for s in self.streams.comm:
            if s is not None:
                s.synchronize()
