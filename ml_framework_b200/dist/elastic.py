"""Elastic training: membership coordinator, worker state machine, data redistribution planning,
learning-rate adaptation, rescaling checkpoints.

Semantics follow the reference: ``ElasticCoordinator`` (src/MLFramework/Distributed/Coordinator/
ElasticCoordinator.cs:45-278) keeps the worker table, ages heartbeats (stale after
``worker_heartbeat_timeout_ms`` -> non-graceful unregister), debounces topology changes through a
stability window before raising one ``RescalingEvent``, and aborts when more than
``failure_tolerance_percentage`` of the workers failed; ``ElasticWorker`` (Worker/ElasticWorker.cs:
72-190) walks Joining -> Active -> Rescaling -> Active and, on a rescale, updates its sampler,
synchronises state and resumes; ``AdaptiveLearningRateScheduler`` (Scheduling/
AdaptiveLearningRateScheduler.cs:47-118) rescales the learning rate linearly or by the square root
of the world-size ratio; ``DataRedistributor`` (Data/DataRedistributor.cs:23) plans which sample
ranges move. Defaults from ElasticTrainingConfig.cs:8-59.

Time is injected (``clock``) so tests drive the health timer and the stability window
deterministically; failures are injected on the host (a worker that stops sending heartbeats).
"""
from __future__ import annotations

import enum
import math
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple


class WorkerStatus(enum.Enum):
    JOINING = "joining"
    ACTIVE = "active"
    RESCALING = "rescaling"
    LEAVING = "leaving"
    FAILED = "failed"


class LRAdaptationStrategy(enum.Enum):
    LINEAR = "linear"
    SQUARE_ROOT = "sqrt"
    NONE = "none"


class RedistributionType(enum.Enum):
    FULL_RESHUFFLE = "full_reshuffle"
    INCREMENTAL = "incremental"


class RescaleType(enum.Enum):
    SCALE_UP = "scale_up"
    SCALE_DOWN = "scale_down"


@dataclass
class ElasticTrainingConfig:
    min_workers: int = 1
    max_workers: int = 64
    rescale_timeout_ms: int = 30_000
    max_consecutive_failures: int = 3
    lr_adaptation: LRAdaptationStrategy = LRAdaptationStrategy.LINEAR
    redistribution: RedistributionType = RedistributionType.FULL_RESHUFFLE
    use_synchronous_rescaling: bool = True
    stability_window_ms: int = 30_000
    worker_heartbeat_timeout_ms: int = 10_000
    failure_tolerance_percentage: float = 20.0

    def validate(self):
        if self.min_workers < 1 or self.max_workers < self.min_workers:
            raise ValueError("need 1 <= min_workers <= max_workers")
        if not (0 <= self.failure_tolerance_percentage <= 100):
            raise ValueError("failure_tolerance_percentage must be in [0, 100]")
        if self.stability_window_ms < 0 or self.worker_heartbeat_timeout_ms <= 0:
            raise ValueError("invalid time settings")


@dataclass
class WorkerInfo:
    worker_id: str
    status: WorkerStatus = WorkerStatus.JOINING
    last_heartbeat: float = 0.0
    rank: int = -1


@dataclass
class ClusterTopology:
    world_size: int
    workers: List[str]
    version: int


@dataclass
class RescalingEvent:
    kind: RescaleType
    old: ClusterTopology
    new: ClusterTopology
    added: List[str]
    removed: List[str]
    time: float


class ElasticError(RuntimeError):
    pass


class ElasticCoordinator:
    def __init__(self, config: Optional[ElasticTrainingConfig] = None, clock: Callable[[], float] = time.time):
        self.cfg = config or ElasticTrainingConfig()
        self.cfg.validate()
        self.clock = clock
        self.workers: Dict[str, WorkerInfo] = {}
        self.topology = ClusterTopology(0, [], 0)
        self._pending_since: Optional[float] = None
        self._listeners: List[Callable[[RescalingEvent], None]] = []
        self.failed_total = 0
        self.peak_workers = 0
        self.events: List[RescalingEvent] = []

    def on_rescaling(self, fn: Callable[[RescalingEvent], None]):
        self._listeners.append(fn)

    # ---- membership
    def register_worker(self, worker_id: str):
        if worker_id in self.workers and self.workers[worker_id].status not in (WorkerStatus.FAILED, WorkerStatus.LEAVING):
            raise ElasticError(f"worker {worker_id!r} already registered")
        if sum(1 for w in self.workers.values() if w.status in (WorkerStatus.ACTIVE, WorkerStatus.JOINING)) >= self.cfg.max_workers:
            raise ElasticError("cluster is at max_workers")
        self.workers[worker_id] = WorkerInfo(worker_id, WorkerStatus.JOINING, self.clock())
        self._mark_change()

    def unregister_worker(self, worker_id: str, graceful: bool = True):
        w = self.workers.get(worker_id)
        if w is None:
            return
        w.status = WorkerStatus.LEAVING if graceful else WorkerStatus.FAILED
        if not graceful:
            self.failed_total += 1
            self.check_failure_tolerance()
        self._mark_change()

    def update_heartbeat(self, worker_id: str):
        w = self.workers.get(worker_id)
        if w is None:
            raise ElasticError(f"unknown worker {worker_id!r}")
        w.last_heartbeat = self.clock()

    def _mark_change(self):
        self._pending_since = self.clock()

    def live_workers(self) -> List[str]:
        return sorted(i for i, w in self.workers.items() if w.status in (WorkerStatus.ACTIVE, WorkerStatus.JOINING, WorkerStatus.RESCALING))

    # ---- timers (called periodically; period = heartbeat timeout / 2 in the reference)
    def check_health(self) -> List[str]:
        now, dead = self.clock(), []
        for w in self.workers.values():
            if w.status in (WorkerStatus.ACTIVE, WorkerStatus.JOINING, WorkerStatus.RESCALING) and \
                    (now - w.last_heartbeat) * 1e3 > self.cfg.worker_heartbeat_timeout_ms:
                dead.append(w.worker_id)
        for wid in dead:
            self.unregister_worker(wid, graceful=False)
        return dead

    def check_failure_tolerance(self):
        self.peak_workers = max(self.peak_workers, len(self.workers))
        if self.peak_workers and 100.0 * self.failed_total / self.peak_workers > self.cfg.failure_tolerance_percentage:
            raise ElasticError(f"{self.failed_total} of {self.peak_workers} workers failed: above the "
                               f"{self.cfg.failure_tolerance_percentage}% tolerance")

    def start_health_timer(self, period_s: Optional[float] = None):
        """Polls on a background thread every ``period_s`` (default: half the heartbeat timeout, as the reference's
        timer does). Errors raised by a poll (tolerance exceeded, too few workers) are kept in ``timer_error`` and stop
        the timer; the training loop reads them with ``raise_timer_error()``."""
        import threading
        if getattr(self, "_timer", None) is not None:
            return
        period = period_s if period_s is not None else self.cfg.worker_heartbeat_timeout_ms / 2e3
        self._timer_stop = threading.Event()
        self.timer_error: Optional[BaseException] = None

        def loop():
            while not self._timer_stop.wait(period):
                try:
                    self.poll()
                except ElasticError as e:
                    self.timer_error = e
                    return
        self._timer = threading.Thread(target=loop, daemon=True, name="mlf-elastic-health")
        self._timer.start()

    def stop_health_timer(self):
        t = getattr(self, "_timer", None)
        if t is not None:
            self._timer_stop.set()
            t.join(timeout=2.0)
            self._timer = None

    def raise_timer_error(self):
        e = getattr(self, "timer_error", None)
        if e is not None:
            self.timer_error = None
            raise e

    def poll(self) -> Optional[RescalingEvent]:
        """Health check + debounce: raises at most one rescaling event once the membership has been
        stable for the stability window."""
        self.check_health()
        if self._pending_since is None:
            return None
        if (self.clock() - self._pending_since) * 1e3 < self.cfg.stability_window_ms:
            return None
        return self.trigger_rescaling()

    def trigger_rescaling(self) -> Optional[RescalingEvent]:
        self._pending_since = None
        live = self.live_workers()
        if len(live) < self.cfg.min_workers:
            raise ElasticError(f"only {len(live)} workers left, fewer than min_workers={self.cfg.min_workers}")
        old = self.topology
        if live == old.workers:
            return None
        new = ClusterTopology(len(live), live, old.version + 1)
        ev = RescalingEvent(RescaleType.SCALE_UP if new.world_size > old.world_size else RescaleType.SCALE_DOWN, old, new,
                            [w for w in live if w not in old.workers], [w for w in old.workers if w not in live], self.clock())
        self.topology = new
        for rank, wid in enumerate(live):
            self.workers[wid].rank = rank
            self.workers[wid].status = WorkerStatus.ACTIVE
        for wid in list(self.workers):
            if self.workers[wid].status in (WorkerStatus.LEAVING, WorkerStatus.FAILED):
                del self.workers[wid]
        self.events.append(ev)
        for fn in self._listeners:
            fn(ev)
        return ev


class AdaptiveLearningRateScheduler:
    def __init__(self, base_lr: float, base_world_size: int, strategy: LRAdaptationStrategy = LRAdaptationStrategy.LINEAR):
        self.base_lr, self.base_world, self.strategy = base_lr, base_world_size, strategy

    def adapt_learning_rate(self, new_world_size: int) -> float:
        ratio = new_world_size / self.base_world
        if self.strategy == LRAdaptationStrategy.LINEAR:
            return self.base_lr * ratio
        if self.strategy == LRAdaptationStrategy.SQUARE_ROOT:
            return self.base_lr * math.sqrt(ratio)
        return self.base_lr

    def transition_learning_rate(self, old_lr: float, new_lr: float, step: int, transition_steps: int) -> float:
        if transition_steps <= 0 or step >= transition_steps:
            return new_lr
        return old_lr + (new_lr - old_lr) * step / transition_steps


class LearningRateTransitionManager:
    """Moves an optimizer's learning rate from its current value to a target over ``transition_steps`` optimizer steps
    (linear or half-cosine) instead of jumping on a rescale; a new target mid-way restarts from the rate in force
    (reference: src/MLFramework/Distributed/Scheduling/LearningRateTransitionManager.cs)."""

    def __init__(self, optimizer=None, transition_steps: int = 100, mode: str = "linear"):
        if transition_steps < 0:
            raise ValueError("transition_steps must be non-negative")
        if mode not in ("linear", "cosine"):
            raise ValueError(f"unknown mode {mode!r}")
        self.optimizer, self.transition_steps, self.mode = optimizer, transition_steps, mode
        self._from = self._to = None
        self._k = 0
        self.history: List[Tuple[float, float]] = []        # (from, to) of every transition started

    @property
    def in_transition(self) -> bool:
        return self._to is not None

    def current_lr(self) -> Optional[float]:
        if self.optimizer is not None:
            g = self.optimizer.param_groups[0] if hasattr(self.optimizer, "param_groups") else None
            return g["lr"] if g is not None else getattr(self.optimizer, "lr", None)
        return self._value() if self.in_transition else None

    def _value(self) -> float:
        if self.transition_steps == 0 or self._k >= self.transition_steps:
            return self._to
        f = self._k / self.transition_steps
        if self.mode == "cosine":
            f = 0.5 * (1.0 - math.cos(math.pi * f))
        return self._from + (self._to - self._from) * f

    def _apply(self, lr: float):
        if self.optimizer is None:
            return
        if hasattr(self.optimizer, "param_groups"):
            for g in self.optimizer.param_groups:
                g["lr"] = lr
        else:
            self.optimizer.lr = lr

    def start_transition(self, target_lr: float, from_lr: Optional[float] = None):
        start = from_lr if from_lr is not None else (self._value() if self.in_transition else self.current_lr())
        if start is None:
            raise ElasticError("no starting learning rate: give from_lr or an optimizer")
        self._from, self._to, self._k = float(start), float(target_lr), 0
        self.history.append((self._from, self._to))
        self._apply(self._value())

    def step(self) -> Optional[float]:
        """Call once per optimizer step; returns the rate now in force (``None`` when no transition is running)."""
        if not self.in_transition:
            return None
        self._k += 1
        lr = self._value()
        self._apply(lr)
        if self._k >= self.transition_steps:
            self._from = self._to = None
        return lr


@dataclass
class DataTransfer:
    src_rank: int
    dst_rank: int
    start: int
    end: int


class DataRedistributor:
    """Plans which contiguous sample ranges move when the world goes from W_old to W_new."""

    @staticmethod
    def shard_range(n: int, world: int, rank: int) -> Tuple[int, int]:
        per = (n + world - 1) // world
        return min(rank * per, n), min((rank + 1) * per, n)

    def calculate_plan(self, dataset_size: int, old_world: int, new_world: int) -> List[DataTransfer]:
        plan = []
        for dst in range(new_world):
            lo, hi = self.shard_range(dataset_size, new_world, dst)
            for src in range(old_world):
                a, b = self.shard_range(dataset_size, old_world, src)
                s, e = max(lo, a), min(hi, b)
                if s < e and src != dst:
                    plan.append(DataTransfer(src, dst, s, e))
        return plan


class ElasticWorker:
    def __init__(self, worker_id: str, coordinator: ElasticCoordinator, sampler=None, lr_scheduler: Optional[AdaptiveLearningRateScheduler] = None,
                 optimizer=None, on_sync: Optional[Callable[[RescalingEvent], None]] = None):
        self.id, self.coord, self.sampler, self.lr_sched, self.opt, self.on_sync = worker_id, coordinator, sampler, lr_scheduler, optimizer, on_sync
        self.status = WorkerStatus.JOINING
        self.rank, self.world_size = -1, 0
        self.history: List[str] = []

    def connect_to_cluster(self):
        self.coord.register_worker(self.id)
        self.coord.on_rescaling(self.on_rescaling_event)
        self.history.append("connected")

    def heartbeat(self):
        self.coord.update_heartbeat(self.id)

    def on_rescaling_event(self, ev: RescalingEvent):
        if self.id not in ev.new.workers:
            self.status = WorkerStatus.LEAVING
            return
        self.status = WorkerStatus.RESCALING
        self.rank, self.world_size = ev.new.workers.index(self.id), ev.new.world_size
        self.history.append(f"rescaling->{self.world_size}")
        self.redistribute_data()
        self.synchronize_state(ev)
        self.resume_training()

    def redistribute_data(self):
        if self.sampler is not None and hasattr(self.sampler, "update_topology"):
            self.sampler.update_topology(self.world_size, self.rank)

    def synchronize_state(self, ev: RescalingEvent):
        if self.lr_sched is not None and self.opt is not None:
            self.opt.set_learning_rate(self.lr_sched.adapt_learning_rate(self.world_size))
        if self.on_sync is not None:
            self.on_sync(ev)

    def resume_training(self):
        self.status = WorkerStatus.ACTIVE
        self.history.append("active")

    def leave(self):
        self.coord.unregister_worker(self.id, graceful=True)
        self.status = WorkerStatus.LEAVING


class ElasticCheckpointManager:
    """Keeps the latest checkpoint and writes a "rescaling checkpoint" right before the topology
    changes (src/MLFramework/Distributed/Checkpointing/ElasticCheckpointManager.cs:40-111); loading
    at the new world size reshards through the multi-shard loader."""

    def __init__(self, checkpoint, state_fn: Callable[[], Tuple[dict, dict, dict]]):
        self.ckpt, self.state_fn, self.latest = checkpoint, state_fn, None

    def save_checkpoint(self, step: int):
        model, optim, slices = self.state_fn()
        tag = f"elastic_step{step}"
        self.ckpt.save(tag, model, optim, slice_info=slices, step=step, strategy="fsdp")
        self.latest = tag
        return tag

    def create_rescaling_checkpoint(self, ev: RescalingEvent, step: int):
        return self.save_checkpoint(step)

    def load_latest_checkpoint(self, device="cpu"):
        if self.latest is None:
            tags = self.ckpt.list_checkpoints()
            if not tags:
                return None
            self.latest = tags[-1]
        return self.ckpt.load(self.latest, device=device)


# ------------------------------------------------------------------ state records and plan execution
@dataclass
class DataShard:
    shard_id: int
    start_index: int
    end_index: int

    @property
    def size(self) -> int:
        return self.end_index - self.start_index

    @staticmethod
    def split(dataset_size: int, world: int) -> List["DataShard"]:
        return [DataShard(r, *DataRedistributor.shard_range(dataset_size, world, r)) for r in range(world)]


@dataclass
class WorkerMetadata:
    """What the cluster knows about a worker beyond its status (src/MLFramework/Distributed/Models/WorkerMetadata.cs)."""
    worker_id: str
    status: WorkerStatus
    join_time: float
    last_heartbeat: float
    rank: int = -1
    local_world_size: int = 1
    custom_attributes: Dict[str, str] = field(default_factory=dict)

    def is_healthy(self, timeout_s: float, now: Optional[float] = None) -> bool:
        return self.status not in (WorkerStatus.FAILED, WorkerStatus.LEAVING) and ((now if now is not None else time.time()) - self.last_heartbeat) <= timeout_s


@dataclass
class GlobalTrainingState:
    """The state every worker must agree on after a rescale (Models/GlobalTrainingState.cs)."""
    current_epoch: int = 0
    current_step: int = 0
    learning_rate: float = 0.0
    global_batch_size: int = 0
    active_worker_count: int = 0
    consumed_samples: int = 0
    state_timestamp: float = field(default_factory=time.time)
    optimizer_state: Optional[bytes] = None

    def to_json(self) -> str:
        import base64
        import json
        d = dict(self.__dict__)
        d["optimizer_state"] = base64.b64encode(self.optimizer_state).decode() if self.optimizer_state is not None else None
        return json.dumps(d)

    @staticmethod
    def from_json(text: str) -> "GlobalTrainingState":
        import base64
        import json
        d = json.loads(text)
        if d.get("optimizer_state") is not None:
            d["optimizer_state"] = base64.b64decode(d["optimizer_state"])
        return GlobalTrainingState(**d)

    def after_rescale(self, new_world: int, lr: Optional[float] = None, per_worker_batch: Optional[int] = None) -> "GlobalTrainingState":
        """The state the new topology starts from: same progress, new worker count (and batch / rate when given)."""
        pw = per_worker_batch if per_worker_batch is not None else (self.global_batch_size // self.active_worker_count if self.active_worker_count else 0)
        return GlobalTrainingState(self.current_epoch, self.current_step, lr if lr is not None else self.learning_rate, pw * new_world, new_world,
                                   self.consumed_samples, time.time(), self.optimizer_state)


@dataclass
class SamplerState:
    """Position of an elastic sampler, enough to rebuild it on any topology (Data/SamplerState.cs)."""
    dataset_size: int
    worker_count: int
    worker_rank: int
    epoch: int
    consumed: int
    seed: int
    shuffle: bool
    drop_last: bool

    @staticmethod
    def capture(sampler) -> "SamplerState":
        return SamplerState(sampler.dataset_size, sampler.num_replicas, sampler.rank, sampler.epoch, getattr(sampler, "consumed", 0), sampler.seed,
                            sampler.shuffle, sampler.drop_last)

    def restore(self, worker_count: Optional[int] = None, worker_rank: Optional[int] = None):
        """A sampler at the recorded position; with a new ``worker_count`` / ``worker_rank`` the remaining samples of the
        epoch are re-split over the new topology."""
        from ..data.samplers import ElasticDistributedSampler
        W = worker_count if worker_count is not None else self.worker_count
        r = worker_rank if worker_rank is not None else self.worker_rank
        s = ElasticDistributedSampler(self.dataset_size, W, r, self.shuffle, self.seed, self.drop_last)
        s.set_epoch(self.epoch)
        s.consumed = self.consumed
        if self.consumed or W != self.worker_count:
            s.update_topology(W, r)
        return s


class DataTransferManager:
    """Carries out a redistribution plan: every transfer is ``copy(transfer)`` (whatever moves samples between ranks:
    a file copy, a point-to-point send, nothing at all for a shared file system), at most ``max_concurrent`` at a time,
    each retried up to ``max_retries`` times; the outcome per transfer is kept (Data/DataTransferManager.cs:12-20)."""

    def __init__(self, max_concurrent_transfers: int = 4, max_retries: int = 2):
        if max_concurrent_transfers <= 0:
            raise ValueError("max_concurrent_transfers must be positive")
        self.max_concurrent, self.max_retries = max_concurrent_transfers, max_retries
        self.completed: List[DataTransfer] = []
        self.failed: List[Tuple[DataTransfer, str]] = []
        self.bytes_moved = 0

    def execute_plan(self, plan: Sequence[DataTransfer], copy: Callable[[DataTransfer], Optional[int]], only_rank: Optional[int] = None,
                     cancel: Optional[Callable[[], bool]] = None) -> bool:
        """``only_rank``: run just the transfers this rank takes part in. Returns True when every transfer succeeded."""
        from concurrent.futures import ThreadPoolExecutor
        todo = [t for t in plan if only_rank is None or only_rank in (t.src_rank, t.dst_rank)]

        def one(t: DataTransfer):
            err = ""
            for _ in range(self.max_retries + 1):
                if cancel is not None and cancel():
                    return t, None, "cancelled"
                try:
                    return t, copy(t), ""
                except Exception as e:       # noqa: BLE001 - retried, then reported
                    err = str(e)
            return t, None, err
        with ThreadPoolExecutor(max_workers=self.max_concurrent, thread_name_prefix="mlf-data-transfer") as ex:
            for t, moved, err in ex.map(one, todo):
                if err:
                    self.failed.append((t, err))
                else:
                    self.completed.append(t)
                    self.bytes_moved += int(moved or 0)
        return not self.failed

    def progress(self, plan_size: int) -> float:
        return (len(self.completed) + len(self.failed)) / plan_size if plan_size else 1.0
