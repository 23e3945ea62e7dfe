"""Model benchmarking: timed inference with percentiles, history with regression check, comparisons, reports.

Reference: src/ModelZoo/Benchmark/{ModelBenchmarkService.cs:53-254, BenchmarkOptions.cs, BenchmarkResult.cs,
BenchmarkHistory.cs:52-388, ComparisonOptions.cs, ComparisonResult.cs, BenchmarkReporter.cs:41-101}. Timing follows this
package's rules: warm-up iterations first, CUDA events on the launching stream for GPU models (host clock on CPU),
and an L2 flush between timed iterations on the GPU so that a small model is not measured out of cache.
"""
from __future__ import annotations

import csv
import io
import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch


@dataclass
class BenchmarkOptions:
    batch_size: int = 1
    seq_len: int = 128
    warmup_iterations: int = 3
    iterations: int = 10
    device: str = "cpu"
    dtype: Optional[str] = None             # default: bfloat16 on cuda, float32 on cpu
    flush_l2: bool = True
    include_memory: bool = True

    def validate(self):
        if self.batch_size <= 0 or self.seq_len <= 0 or self.iterations <= 0 or self.warmup_iterations < 0:
            raise ValueError("batch_size, seq_len and iterations must be positive, warmup non-negative")


@dataclass
class BenchmarkResult:
    model_name: str
    device: str
    batch_size: int
    seq_len: int
    iterations: int
    latencies_ms: List[float]
    peak_memory_bytes: int = 0
    timestamp: float = field(default_factory=time.time)
    extra: Dict[str, Any] = field(default_factory=dict)

    def _pct(self, q: float) -> float:
        s = sorted(self.latencies_ms)
        pos = q * (len(s) - 1)
        lo = int(pos)
        hi = min(lo + 1, len(s) - 1)
        return s[lo] + (s[hi] - s[lo]) * (pos - lo)

    @property
    def mean_ms(self) -> float: return sum(self.latencies_ms) / len(self.latencies_ms)
    @property
    def min_ms(self) -> float: return min(self.latencies_ms)
    @property
    def max_ms(self) -> float: return max(self.latencies_ms)
    @property
    def p50_ms(self) -> float: return self._pct(0.5)
    @property
    def p95_ms(self) -> float: return self._pct(0.95)
    @property
    def p99_ms(self) -> float: return self._pct(0.99)
    @property
    def std_ms(self) -> float:
        m = self.mean_ms
        return (sum((x - m) ** 2 for x in self.latencies_ms) / len(self.latencies_ms)) ** 0.5
    @property
    def throughput(self) -> float:
        """Tokens (batch x sequence) per second at the median latency."""
        return self.batch_size * self.seq_len / (self.p50_ms * 1e-3)

    def summary(self) -> Dict[str, Any]:
        return {"model": self.model_name, "device": self.device, "batch_size": self.batch_size, "seq_len": self.seq_len,
                "iterations": self.iterations, "mean_ms": self.mean_ms, "p50_ms": self.p50_ms, "p95_ms": self.p95_ms, "p99_ms": self.p99_ms,
                "min_ms": self.min_ms, "max_ms": self.max_ms, "std_ms": self.std_ms, "tokens_per_s": self.throughput,
                "peak_memory_bytes": self.peak_memory_bytes, "timestamp": self.timestamp}


@dataclass
class BenchmarkComparison:
    model_name: str
    previous_p50_ms: float
    current_p50_ms: float

    @property
    def change(self) -> float:
        """Relative change of the median latency (positive = slower)."""
        return self.current_p50_ms / self.previous_p50_ms - 1.0 if self.previous_p50_ms > 0 else 0.0

    def is_regression(self, tolerance: float = 0.05) -> bool:
        return self.change > tolerance


class BenchmarkHistory:
    """Results by model, newest last; kept in a JSON file when ``storage_path`` is given."""

    def __init__(self, storage_path: Optional[str] = None, max_per_model: int = 100):
        self.storage_path, self.max_per_model = storage_path, max_per_model
        self._h: Dict[str, List[BenchmarkResult]] = {}
        if storage_path and os.path.exists(storage_path):
            with open(storage_path) as f:
                for name, lst in json.load(f).items():
                    self._h[name] = [BenchmarkResult(**r) for r in lst]

    @property
    def total_count(self) -> int:
        return sum(len(v) for v in self._h.values())

    def _persist(self):
        if self.storage_path:
            d = os.path.dirname(self.storage_path)
            if d:
                os.makedirs(d, exist_ok=True)
            tmp = self.storage_path + ".tmp"
            with open(tmp, "w") as f:
                json.dump({k: [asdict(r) for r in v] for k, v in self._h.items()}, f)
            os.replace(tmp, self.storage_path)

    def save_result(self, r: BenchmarkResult):
        lst = self._h.setdefault(r.model_name, [])
        lst.append(r)
        del lst[:-self.max_per_model]
        self._persist()

    def get_history(self, model_name: str, limit: int = 10) -> List[BenchmarkResult]:
        return list(self._h.get(model_name, ()))[-limit:]

    def get_latest(self, model_name: str) -> Optional[BenchmarkResult]:
        lst = self._h.get(model_name)
        return lst[-1] if lst else None

    def compare_with_previous(self, r: BenchmarkResult) -> Optional[BenchmarkComparison]:
        """Against the newest stored result of the same model, device, batch and sequence length."""
        for old in reversed(self._h.get(r.model_name, ())):
            if old is not r and (old.device, old.batch_size, old.seq_len) == (r.device, r.batch_size, r.seq_len):
                return BenchmarkComparison(r.model_name, old.p50_ms, r.p50_ms)
        return None

    def get_history_in_range(self, model_name: str, start: float, end: float) -> List[BenchmarkResult]:
        return [r for r in self._h.get(model_name, ()) if start <= r.timestamp <= end]

    def clear_history(self, model_name: str):
        self._h.pop(model_name, None)
        self._persist()

    def clear_all(self):
        self._h.clear()
        self._persist()

    def export_json(self, path: str):
        with open(path, "w") as f:
            json.dump({k: [r.summary() for r in v] for k, v in self._h.items()}, f, indent=1)

    def summary(self) -> str:
        return "\n".join(f"{k}: {len(v)} runs, latest p50 {v[-1].p50_ms:.3f} ms, best p50 {min(r.p50_ms for r in v):.3f} ms"
                         for k, v in sorted(self._h.items()))


@dataclass
class ComparisonOptions:
    metric: str = "p50_ms"                 # any key of BenchmarkResult.summary()
    lower_is_better: bool = True
    benchmark: BenchmarkOptions = field(default_factory=BenchmarkOptions)


@dataclass
class ComparisonResult:
    metric: str
    results: Dict[str, BenchmarkResult]
    ranking: List[str]
    winner: str

    def relative_to_winner(self) -> Dict[str, float]:
        w = self.results[self.winner].summary()[self.metric]
        return {k: (r.summary()[self.metric] / w if w else 0.0) for k, r in self.results.items()}


class ModelBenchmarkService:
    def __init__(self, zoo=None, history: Optional[BenchmarkHistory] = None):
        self.zoo, self.history = zoo, history or BenchmarkHistory()

    def benchmark_model(self, name: str, forward: Callable[[], Any], options: BenchmarkOptions, device: Optional[torch.device] = None) -> BenchmarkResult:
        """Times ``forward()`` (which runs one inference on inputs it has closed over)."""
        options.validate()
        dev = torch.device(device if device is not None else options.device)
        cuda = dev.type == "cuda"
        flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev) if cuda and options.flush_l2 else None
        with torch.no_grad():
            for _ in range(options.warmup_iterations):
                forward()
            if cuda:
                torch.cuda.synchronize(dev)
                torch.cuda.reset_peak_memory_stats(dev)
            lat = []
            for _ in range(options.iterations):
                if flush is not None:
                    flush.zero_()
                if cuda:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    forward()
                    b.record()
                    b.synchronize()
                    lat.append(a.elapsed_time(b))
                else:
                    t0 = time.perf_counter()
                    forward()
                    lat.append((time.perf_counter() - t0) * 1e3)
        peak = torch.cuda.max_memory_allocated(dev) if cuda and options.include_memory else 0
        r = BenchmarkResult(name, str(dev), options.batch_size, options.seq_len, options.iterations, lat, int(peak))
        self.history.save_result(r)
        return r

    def benchmark(self, model_name: str, options: Optional[BenchmarkOptions] = None) -> BenchmarkResult:
        """Builds the registered architecture with random weights and times its forward pass on synthetic tokens."""
        if self.zoo is None:
            raise RuntimeError("benchmarking by name needs a model zoo")
        from .zoo import build_model
        o = options or BenchmarkOptions()
        info = self.zoo.registry.get(model_name)
        dt = getattr(torch, o.dtype) if o.dtype else (torch.bfloat16 if o.device.startswith("cuda") else torch.float32)
        model = build_model(info, o.device, dt).eval()
        ids = torch.randint(0, info.config.get("vocab_size", 100), (o.batch_size, o.seq_len), device=o.device)
        return self.benchmark_model(model_name, lambda: model(ids), o)

    def benchmark_batch(self, model_names: Sequence[str], options: Optional[BenchmarkOptions] = None) -> Dict[str, BenchmarkResult]:
        return {n: self.benchmark(n, options) for n in model_names}

    def compare(self, model_names: Sequence[str], options: Optional[ComparisonOptions] = None) -> ComparisonResult:
        o = options or ComparisonOptions()
        res = self.benchmark_batch(model_names, o.benchmark)
        return self.rank(res, o.metric, o.lower_is_better)

    @staticmethod
    def rank(results: Dict[str, BenchmarkResult], metric: str = "p50_ms", lower_is_better: bool = True) -> ComparisonResult:
        if not results:
            raise ValueError("nothing to compare")
        order = sorted(results, key=lambda k: results[k].summary()[metric], reverse=not lower_is_better)
        return ComparisonResult(metric, results, order, order[0])


class BenchmarkReporter:
    FORMATS = ("markdown", "json", "csv")

    def render(self, r: BenchmarkResult, fmt: str = "markdown") -> str:
        s = r.summary()
        if fmt == "json":
            return json.dumps(s, indent=1)
        if fmt == "csv":
            buf = io.StringIO()
            w = csv.DictWriter(buf, fieldnames=list(s))
            w.writeheader()
            w.writerow(s)
            return buf.getvalue()
        if fmt != "markdown":
            raise ValueError(f"unknown format {fmt!r}; one of {self.FORMATS}")
        return (f"## {r.model_name} on {r.device}\n\n| batch | seq | iterations | mean ms | p50 ms | p95 ms | p99 ms | tokens/s | peak MiB |\n"
                f"|---|---|---|---|---|---|---|---|---|\n| {r.batch_size} | {r.seq_len} | {r.iterations} | {r.mean_ms:.3f} | {r.p50_ms:.3f} | "
                f"{r.p95_ms:.3f} | {r.p99_ms:.3f} | {r.throughput:.0f} | {r.peak_memory_bytes / 2**20:.1f} |\n")

    def render_comparison(self, c: ComparisonResult, fmt: str = "markdown") -> str:
        rel = c.relative_to_winner()
        if fmt == "json":
            return json.dumps({"metric": c.metric, "winner": c.winner, "ranking": c.ranking, "results": {k: r.summary() for k, r in c.results.items()}}, indent=1)
        if fmt == "csv":
            buf = io.StringIO()
            w = csv.writer(buf)
            w.writerow(["rank", "model", c.metric, "relative"])
            for n, k in enumerate(c.ranking, 1):
                w.writerow([n, k, c.results[k].summary()[c.metric], rel[k]])
            return buf.getvalue()
        if fmt != "markdown":
            raise ValueError(f"unknown format {fmt!r}; one of {self.FORMATS}")
        lines = [f"## Comparison by {c.metric} (winner: {c.winner})", "", f"| rank | model | {c.metric} | relative |", "|---|---|---|---|"]
        lines += [f"| {n} | {k} | {c.results[k].summary()[c.metric]:.3f} | {rel[k]:.2f}x |" for n, k in enumerate(c.ranking, 1)]
        return "\n".join(lines) + "\n"

    def generate_report(self, r, path: str, fmt: str = "markdown"):
        text = self.render(r, fmt) if isinstance(r, BenchmarkResult) else self.render_comparison(r, fmt)
        with open(path, "w") as f:
            f.write(text)

    def print_result(self, r: BenchmarkResult, printer: Callable[[str], None] = print):
        printer(self.render(r))
