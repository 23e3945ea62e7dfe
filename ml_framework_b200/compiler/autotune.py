"""Launch-configuration autotuning: search strategies, benchmark runner, device-keyed cache.

Reference: src/MLFramework/Autotuning — Autotuner.cs:8-101, IAutotuner.cs:10-92 (result, options,
strategy and device records), ISearchSpaceGenerator.cs:7-171, IBenchmarkRunner.cs:8-102,
IPerformanceProfiler.cs:8-71, ITuningCache.cs:7-90, IDeviceQuery.cs, IKernelExecutor.cs,
ITensorGenerator.cs.

A tunable is anything that can run under a ``KernelLaunchConfiguration``: the generated
element-wise kernels of ``compiler.jit_cuda`` (threads, vectors in flight, grid limit), a GEMM
tile choice, a Python callable in tests. The four strategies really differ here: the grid walks
the whole space; random samples it; the model-based one fits a quadratic in the log2 of each
knob to what it has measured and measures the predicted minimum next; the genetic one breeds
the fastest configurations. Times come from CUDA events on a GPU and from the wall clock
otherwise; bandwidth is the operation's bytes over the measured time.
"""
from __future__ import annotations

import enum
import itertools
import json
import math
import os
import random
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

__all__ = [
    "SearchStrategy", "DeviceInfo", "DeviceQuery", "ThreadBlockConfiguration", "KernelLaunchConfiguration",
    "TunableOperation", "AutotuningOptions", "TuningBenchmarkResult", "AutotuningResult", "TuningCacheEntry",
    "InMemoryTuningCache", "FileTuningCache", "SearchSpaceGenerator", "WallClockProfiler", "CudaPerformanceProfiler",
    "BenchmarkRunner", "TensorGenerator", "KernelAutotuner", "tune_fused_elementwise",
]


class SearchStrategy(enum.Enum):
    GRID_SEARCH = "grid"
    RANDOM_SEARCH = "random"
    BAYESIAN_OPTIMIZATION = "model"
    GENETIC_ALGORITHM = "genetic"


@dataclass(frozen=True)
class DeviceInfo:
    device_name: str
    compute_capability: int
    sm_count: int
    total_memory_bytes: int
    max_threads_per_block: int
    max_shared_memory_per_block: int
    architecture: str

    def key(self) -> str:
        return f"{self.device_name}|sm{self.compute_capability}|{self.sm_count}"


class DeviceQuery:
    """The current device, or the B200 figures when no GPU is visible (plans made off the machine)."""

    B200 = DeviceInfo("NVIDIA B200", 100, 148, 180 * 1024 ** 3, 1024, 227 * 1024, "blackwell")

    def get_current_device_info(self) -> DeviceInfo:
        if not torch.cuda.is_available():
            return self.B200
        p = torch.cuda.get_device_properties(torch.cuda.current_device())
        cc = p.major * 10 + p.minor
        arch = {10: "blackwell", 9: "hopper", 8: "ampere"}.get(p.major, f"sm_{cc}")
        smem = getattr(p, "shared_memory_per_block_optin", 48 * 1024)
        return DeviceInfo(p.name, cc, p.multi_processor_count, p.total_memory, 1024, smem, arch)


@dataclass(frozen=True)
class ThreadBlockConfiguration:
    x: int = 1
    y: int = 1
    z: int = 1

    def total(self) -> int:
        return self.x * self.y * self.z


@dataclass(frozen=True)
class KernelLaunchConfiguration:
    block_dim: ThreadBlockConfiguration = ThreadBlockConfiguration(256)
    grid_dim: ThreadBlockConfiguration = ThreadBlockConfiguration(1)
    shared_memory_bytes: int = 0
    parameters: Tuple[Tuple[str, Any], ...] = ()          # further knobs (unroll, tile, stages) as sorted pairs

    def parameter(self, name: str, default=None):
        return dict(self.parameters).get(name, default)

    def key(self) -> str:
        b, g = self.block_dim, self.grid_dim
        extra = ",".join(f"{k}={v}" for k, v in self.parameters)
        return f"b{b.x}x{b.y}x{b.z}|g{g.x}x{g.y}x{g.z}|s{self.shared_memory_bytes}|{extra}"

    def to_json(self) -> Dict[str, Any]:
        return {"block": [self.block_dim.x, self.block_dim.y, self.block_dim.z],
                "grid": [self.grid_dim.x, self.grid_dim.y, self.grid_dim.z],
                "smem": self.shared_memory_bytes, "params": [list(p) for p in self.parameters]}

    @classmethod
    def from_json(cls, d: Dict[str, Any]) -> "KernelLaunchConfiguration":
        return cls(ThreadBlockConfiguration(*d["block"]), ThreadBlockConfiguration(*d["grid"]), d["smem"],
                   tuple((k, v) for k, v in d["params"]))


@dataclass
class TunableOperation:
    """What is tuned: an identity for the cache, the output size that fixes the grid, the bytes it
    moves, the knobs beyond the block shape, and ``run(config, *inputs)``."""
    op_id: str
    output_elements: int
    bytes_moved: int = 0
    shared_memory_bytes: int = 0
    input_shapes: Tuple[Tuple[int, ...], ...] = ()
    dtype: torch.dtype = torch.float32
    knobs: Dict[str, Sequence[Any]] = field(default_factory=dict)
    block_x: Sequence[int] = (32, 64, 128, 256, 512)
    block_y: Sequence[int] = (1, 2, 4, 8)
    elements_per_thread: int = 1
    run: Optional[Callable[..., Any]] = None

    def signature(self) -> str:
        return f"{self.op_id}|{self.output_elements}|{self.dtype}|{self.input_shapes}"


@dataclass(frozen=True)
class AutotuningOptions:
    max_iterations: int = 10
    warmup_runs: int = 3
    measurement_runs: int = 5
    enable_memory_measurement: bool = True
    enable_sm_utilization: bool = True
    search_strategy: SearchStrategy = SearchStrategy.GRID_SEARCH
    seed: int = 0


@dataclass(frozen=True)
class TuningBenchmarkResult:
    configuration: KernelLaunchConfiguration
    execution_time_ms: float
    memory_bandwidth_gbps: float = 0.0
    sm_utilization_percent: int = 0


@dataclass(frozen=True)
class AutotuningResult:
    best_configuration: KernelLaunchConfiguration
    best_execution_time_ms: float
    benchmarks: Tuple[TuningBenchmarkResult, ...]
    cache_hit: bool
    timestamp: float


@dataclass
class TuningCacheEntry:
    result: AutotuningResult
    device_key: str
    signature: str


class InMemoryTuningCache:
    def __init__(self):
        self._d: Dict[Tuple[str, str], TuningCacheEntry] = {}

    def get(self, op: TunableOperation, device: DeviceInfo) -> Optional[TuningCacheEntry]:
        return self._d.get((op.signature(), device.key()))

    def put(self, op: TunableOperation, result: AutotuningResult, device: DeviceInfo) -> None:
        self._d[(op.signature(), device.key())] = TuningCacheEntry(result, device.key(), op.signature())

    def contains(self, op: TunableOperation, device: DeviceInfo) -> bool:
        return (op.signature(), device.key()) in self._d

    def remove(self, op: TunableOperation, device: DeviceInfo) -> bool:
        return self._d.pop((op.signature(), device.key()), None) is not None

    def clear(self) -> None:
        self._d.clear()

    @property
    def count(self) -> int:
        return len(self._d)


class FileTuningCache(InMemoryTuningCache):
    """The same, kept in a JSON file (best configuration and time; the trial list is not stored)."""

    def __init__(self, path: str):
        super().__init__()
        self.path = path
        if os.path.exists(path):
            with open(path) as f:
                for e in json.load(f):
                    cfg = KernelLaunchConfiguration.from_json(e["best"])
                    res = AutotuningResult(cfg, e["ms"], (), True, e["timestamp"])
                    self._d[(e["signature"], e["device"])] = TuningCacheEntry(res, e["device"], e["signature"])

    def _flush(self):
        rows = [{"signature": s, "device": d, "best": e.result.best_configuration.to_json(),
                 "ms": e.result.best_execution_time_ms, "timestamp": e.result.timestamp} for (s, d), e in self._d.items()]
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(rows, f, indent=1)
        os.replace(tmp, self.path)

    def put(self, op, result, device):
        super().put(op, result, device)
        self._flush()

    def remove(self, op, device):
        gone = super().remove(op, device)
        if gone:
            self._flush()
        return gone

    def clear(self):
        super().clear()
        self._flush()


# ------------------------------------------------------------------ search space
class SearchSpaceGenerator:
    """All legal configurations of an operation on a device, and samples of them."""

    def create_configuration(self, op: TunableOperation, tx: int, ty: int, tz: int, device: DeviceInfo,
                             params: Tuple[Tuple[str, Any], ...] = ()) -> KernelLaunchConfiguration:
        threads = tx * ty * tz
        per_block = threads * max(1, op.elements_per_thread)
        need = max(1, -(-op.output_elements // per_block))
        grid = min(need, device.sm_count * 32)                     # the kernels loop grid-stride beyond this
        smem = min(op.shared_memory_bytes, device.max_shared_memory_per_block)
        return KernelLaunchConfiguration(ThreadBlockConfiguration(tx, ty, tz), ThreadBlockConfiguration(grid), smem, params)

    def full_grid(self, op: TunableOperation, device: DeviceInfo) -> List[KernelLaunchConfiguration]:
        names = sorted(op.knobs)
        combos = list(itertools.product(*(op.knobs[n] for n in names))) or [()]
        out = []
        for tx in op.block_x:
            for ty in op.block_y:
                if tx * ty > device.max_threads_per_block:
                    continue
                for combo in combos:
                    out.append(self.create_configuration(op, tx, ty, 1, device, tuple(zip(names, combo))))
        return out

    def generate_search_space(self, op: TunableOperation, device: DeviceInfo, strategy: SearchStrategy,
                              max_iterations: int, seed: int = 0) -> List[KernelLaunchConfiguration]:
        """The configurations to measure first: everything for the grid, ``max_iterations`` distinct
        samples for random search, a spread of starting points for the two adaptive strategies."""
        space = self.full_grid(op, device)
        if strategy is SearchStrategy.GRID_SEARCH or len(space) <= max_iterations:
            return space
        rng = random.Random(seed)
        if strategy is SearchStrategy.RANDOM_SEARCH:
            return rng.sample(space, max_iterations)
        n0 = max(2, min(len(space), max_iterations // 2))
        step = len(space) / n0
        return [space[int(i * step)] for i in range(n0)]


# ------------------------------------------------------------------ measuring
class WallClockProfiler:
    def __init__(self, synchronize: Optional[Callable[[], None]] = None, clock: Callable[[], float] = time.perf_counter):
        self._sync, self._clock = synchronize or (lambda: None), clock

    def measure_execution(self, action: Callable[[], Any]) -> float:
        self._sync()
        t0 = self._clock()
        action()
        self._sync()
        return (self._clock() - t0) * 1e3

    @staticmethod
    def measure_memory_bandwidth(op: TunableOperation, ms: float) -> float:
        return op.bytes_moved / (ms * 1e-3) / 1e9 if ms > 0 and op.bytes_moved else 0.0

    @staticmethod
    def measure_sm_utilization(config: KernelLaunchConfiguration, device: DeviceInfo) -> int:
        """Resident-thread estimate: launched threads over what the SMs can hold (2048 each)."""
        threads = config.block_dim.total() * config.grid_dim.total()
        return int(min(100, 100 * threads / (device.sm_count * 2048)))


class CudaPerformanceProfiler(WallClockProfiler):
    """Times with CUDA events on the current stream."""

    def measure_execution(self, action: Callable[[], Any]) -> float:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        action()
        b.record()
        b.synchronize()
        return a.elapsed_time(b)


class TensorGenerator:
    def __init__(self, device="cpu", seed: int = 0):
        self.device, self._g = torch.device(device), torch.Generator().manual_seed(seed)

    def generate_random_tensor(self, shape: Sequence[int], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        if dtype.is_floating_point:
            return torch.randn(*shape, generator=self._g).to(device=self.device, dtype=dtype)
        return torch.randint(-8, 8, tuple(shape), generator=self._g).to(device=self.device, dtype=dtype)


class BenchmarkRunner:
    def __init__(self, profiler: Optional[WallClockProfiler] = None, device: Optional[DeviceInfo] = None):
        self.profiler = profiler or (CudaPerformanceProfiler() if torch.cuda.is_available() else WallClockProfiler())
        self.device = device or DeviceQuery().get_current_device_info()
        self.failures: List[Tuple[str, str]] = []

    def benchmark(self, op: TunableOperation, config: KernelLaunchConfiguration, inputs: Sequence[torch.Tensor],
                  options: AutotuningOptions) -> Optional[TuningBenchmarkResult]:
        """Median of the measured runs; ``None`` when the configuration cannot run (recorded in ``failures``)."""
        try:
            for _ in range(options.warmup_runs):
                op.run(config, *inputs)
            times = sorted(self.profiler.measure_execution(lambda: op.run(config, *inputs))
                           for _ in range(max(1, options.measurement_runs)))
        except Exception as e:                           # noqa: BLE001 - an illegal configuration is data, not an error
            self.failures.append((config.key(), str(e)))
            return None
        ms = times[len(times) // 2]
        bw = self.profiler.measure_memory_bandwidth(op, ms) if options.enable_memory_measurement else 0.0
        sm = self.profiler.measure_sm_utilization(config, self.device) if options.enable_sm_utilization else 0
        return TuningBenchmarkResult(config, ms, bw, sm)

    def benchmark_all(self, op, configs, inputs, options) -> List[TuningBenchmarkResult]:
        return [r for r in (self.benchmark(op, c, inputs, options) for c in configs) if r is not None]


# ------------------------------------------------------------------ the tuner
def _features(c: KernelLaunchConfiguration, names: Sequence[str]) -> List[float]:
    v = [math.log2(c.block_dim.x), math.log2(c.block_dim.y)]
    for n in names:
        p = c.parameter(n)
        v.append(math.log2(p) if isinstance(p, (int, float)) and p > 0 else float(hash(str(p)) % 7))
    return v


class KernelAutotuner:
    """Cache lookup, search, cache store (Autotuner.cs:32-90)."""

    def __init__(self, cache=None, search_space_generator: Optional[SearchSpaceGenerator] = None,
                 benchmark_runner: Optional[BenchmarkRunner] = None, tensor_generator: Optional[TensorGenerator] = None,
                 device_query: Optional[DeviceQuery] = None, log: Optional[Callable[[str], None]] = None):
        self.cache = cache if cache is not None else InMemoryTuningCache()
        self.space = search_space_generator or SearchSpaceGenerator()
        self.devices = device_query or DeviceQuery()
        self.runner = benchmark_runner or BenchmarkRunner(device=self.devices.get_current_device_info())
        self.tensors = tensor_generator or TensorGenerator()
        self._log = log or (lambda m: None)

    def get_cached_result(self, op: TunableOperation, device: DeviceInfo) -> Optional[TuningCacheEntry]:
        return self.cache.get(op, device)

    def cache_result(self, op: TunableOperation, result: AutotuningResult, device: DeviceInfo) -> None:
        self.cache.put(op, result, device)

    def tune(self, op: TunableOperation, options: Optional[AutotuningOptions] = None,
             benchmark_inputs: Optional[Sequence[torch.Tensor]] = None) -> AutotuningResult:
        options = options or AutotuningOptions()
        if op.run is None:
            raise ValueError(f"operation {op.op_id!r} has no run function")
        device = self.devices.get_current_device_info()
        hit = self.get_cached_result(op, device)
        if hit is not None:
            self._log(f"cache hit for {op.op_id}")
            r = hit.result
            return AutotuningResult(r.best_configuration, r.best_execution_time_ms, r.benchmarks, True, time.time())
        inputs = list(benchmark_inputs) if benchmark_inputs is not None else \
            [self.tensors.generate_random_tensor(s, op.dtype) for s in op.input_shapes]
        first = self.space.generate_search_space(op, device, options.search_strategy, options.max_iterations, options.seed)
        done: Dict[str, TuningBenchmarkResult] = {}
        tried: set = set()

        def measure(cfgs):
            for c in cfgs:
                if c.key() in tried:
                    continue
                tried.add(c.key())
                r = self.runner.benchmark(op, c, inputs, options)
                if r is not None:
                    done[c.key()] = r
        measure(first)
        if options.search_strategy in (SearchStrategy.BAYESIAN_OPTIMIZATION, SearchStrategy.GENETIC_ALGORITHM):
            space = self.space.full_grid(op, device)
            rng = random.Random(options.seed)
            while len(tried) < min(options.max_iterations, len(space)):
                rest = [c for c in space if c.key() not in tried]
                if options.search_strategy is SearchStrategy.BAYESIAN_OPTIMIZATION:
                    nxt = self._model_pick(op, list(done.values()), rest)
                else:
                    nxt = self._breed(op, device, list(done.values()), rest, rng)
                measure([nxt])
        if not done:
            raise RuntimeError(f"no configuration of {op.op_id!r} ran: {self.runner.failures[:3]}")
        benchmarks = tuple(sorted(done.values(), key=lambda r: r.execution_time_ms))
        result = AutotuningResult(benchmarks[0].configuration, benchmarks[0].execution_time_ms, benchmarks, False, time.time())
        self.cache_result(op, result, device)
        self._log(f"tuned {op.op_id}: {benchmarks[0].configuration.key()} at {benchmarks[0].execution_time_ms:.4f} ms "
                  f"after {len(tried)} trials")
        return result

    # quadratic surrogate in log2 space: cheap, and launch-shape costs are close to bowl-shaped there
    def _model_pick(self, op, measured: List[TuningBenchmarkResult], rest: List[KernelLaunchConfiguration]):
        names = sorted(op.knobs)
        if len(measured) < 3:
            return rest[len(rest) // 2]
        X = np.array([_features(r.configuration, names) for r in measured])
        y = np.log(np.array([max(r.execution_time_ms, 1e-9) for r in measured]))
        A = np.hstack([np.ones((len(X), 1)), X, X ** 2])
        coef, *_ = np.linalg.lstsq(A, y, rcond=None)
        R = np.array([_features(c, names) for c in rest])
        pred = np.hstack([np.ones((len(R), 1)), R, R ** 2]) @ coef
        return rest[int(np.argmin(pred))]

    def _breed(self, op, device, measured: List[TuningBenchmarkResult], rest: List[KernelLaunchConfiguration], rng):
        """Child of two of the fastest quarter (each gene from either parent), mutated now and then;
        falls to the unmeasured configuration nearest to the child."""
        names = sorted(op.knobs)
        elite = sorted(measured, key=lambda r: r.execution_time_ms)[:max(2, len(measured) // 4)]
        if len(elite) < 2:
            return rng.choice(rest)
        a, b = rng.sample(elite, 2)
        fa, fb = _features(a.configuration, names), _features(b.configuration, names)
        child = [rng.choice(pair) for pair in zip(fa, fb)]
        if rng.random() < 0.3:
            i = rng.randrange(len(child))
            child[i] += rng.choice((-1.0, 1.0))
        return min(rest, key=lambda c: sum((x - y) ** 2 for x, y in zip(_features(c, names), child)))


def tune_fused_elementwise(fused, example_inputs: Sequence[torch.Tensor], options: Optional[AutotuningOptions] = None,
                           tuner: Optional[KernelAutotuner] = None) -> AutotuningResult:
    """Tunes a ``jit_cuda.FusedElementwise`` on ``example_inputs`` (CUDA tensors) over threads per block,
    vectors in flight and CTAs per SM, and makes the winner its default configuration."""
    from .jit_cuda import KernelConfig
    a = example_inputs[0]
    if not a.is_cuda:
        raise ValueError("tuning a generated kernel needs CUDA tensors")
    out = torch.empty_like(a)
    sms = torch.cuda.get_device_properties(a.device).multi_processor_count

    def run(cfg: KernelLaunchConfiguration, *ins):
        kc = KernelConfig(cfg.block_dim.x, cfg.parameter("unroll", 2), cfg.parameter("ctas_per_sm", 8))
        fused.variant(a.dtype, kc).launch(out, list(ins), sms * kc.ctas_per_sm)

    n = a.numel()
    op = TunableOperation("fused:" + "|".join(fused.chain), n, bytes_moved=(len(example_inputs) + 1) * n * a.element_size(),
                          dtype=a.dtype, knobs={"unroll": (1, 2, 4), "ctas_per_sm": (4, 8)}, block_x=(256, 512), block_y=(1,),
                          elements_per_thread=16 // a.element_size(), run=run)
    result = (tuner or KernelAutotuner()).tune(op, options, [t.contiguous() for t in example_inputs])
    best = result.best_configuration
    fused.default_config = KernelConfig(best.block_dim.x, best.parameter("unroll", 2), best.parameter("ctas_per_sm", 8))
    return result
