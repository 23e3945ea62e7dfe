"""Runtime compilation of fused element-wise chains: CUDA source text -> ``nvcc`` -> shared object -> launch.

The reference renders CUDA C from string templates per fused operator (one thread per element, scalar fp32:
src/MLFramework/Fusion/KernelCode/Cuda/CudaKernelTemplates.cs:8-160, CudaCodeGenerator / per-op snippets
Fusion/KernelCode/**), keeps compiled variants in a shape-keyed LRU cache and compiles lazily per shape variant
(Compilation/LazyCompilation*.cs, KernelCache*.cs), and searches thread-block shapes with an autotuner
(Fusion/Autotuning/**); it has no compiler attached, so none of that text ever runs.

Here the text is compiled and run. A chain such as ``relu(a * b + c)`` becomes ONE kernel for sm_100a:
16-byte loads and stores, fp32 arithmetic, a grid-stride loop over vectors with a scalar tail, ``UNROLL`` vectors
in flight per thread. ``NvccCompiler`` builds it into a shared object (kernel + a C launcher that takes raw pointers
and a stream) in a cache directory keyed by the hash of the source and the flags, so a second process or a second
run reuses the binary; ``FusedElementwise`` is the callable: it keeps one compiled variant per (chain, dtype,
configuration), picks the configuration per size bucket with the autotuner on first use when asked to, and falls back
to the same chain in PyTorch on tensors that are not on a GPU.

The hand-written kernels of ``csrc/`` stay the hot path; this module covers chains they do not.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import shutil
import subprocess
import tempfile
import threading
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .cache import Autotuner, LRUKernelCache, ShapeSignature, ShapeVariantGenerator

# kind -> (C expression over `v` (running value) and `x` (the extra operand), takes an extra operand)
SNIPPETS: Dict[str, Tuple[str, bool]] = {
    "add": ("v + x", True), "sub": ("v - x", True), "mul": ("v * x", True), "div": ("v / x", True),
    "maximum": ("fmaxf(v, x)", True), "minimum": ("fminf(v, x)", True),
    "relu": ("fmaxf(v, 0.f)", False), "sigmoid": ("1.f / (1.f + __expf(-v))", False), "tanh": ("tanhf(v)", False),
    "exp": ("__expf(v)", False), "log": ("__logf(v)", False), "sqrt": ("sqrtf(v)", False), "neg": ("-v", False),
    "abs": ("fabsf(v)", False), "square": ("v * v", False), "silu": ("v / (1.f + __expf(-v))", False),
    "leaky_relu": ("(v > 0.f ? v : 0.01f * v)", False),
    "gelu": ("0.5f * v * (1.f + tanhf(0.7978845608f * (v + 0.044715f * v * v * v)))", False),
}

_TORCH_OPS: Dict[str, Callable] = {
    "add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div, "maximum": torch.maximum, "minimum": torch.minimum,
    "relu": torch.relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh, "exp": torch.exp, "log": torch.log, "sqrt": torch.sqrt,
    "neg": torch.neg, "abs": torch.abs, "square": torch.square, "silu": torch.nn.functional.silu,
    "leaky_relu": lambda t: torch.nn.functional.leaky_relu(t, 0.01),
    "gelu": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
}

Chain = Sequence[str]


def chain_arity(chain: Chain) -> int:
    """Number of input tensors a chain reads: the running value plus one per binary step."""
    for k in chain:
        if k not in SNIPPETS:
            raise KeyError(f"no CUDA snippet for element-wise op '{k}'")
    return 1 + sum(1 for k in chain if SNIPPETS[k][1])


def eval_chain_torch(chain: Chain, inputs: Sequence[torch.Tensor]) -> torch.Tensor:
    """The chain in PyTorch (fp32 arithmetic, result in the inputs' dtype): the oracle and the CPU path."""
    v = inputs[0].float()
    nxt = 1
    for k in chain:
        if SNIPPETS[k][1]:
            v = _TORCH_OPS[k](v, inputs[nxt].float())
            nxt += 1
        else:
            v = _TORCH_OPS[k](v)
    return v.to(inputs[0].dtype)


@dataclass(frozen=True)
class KernelConfig:
    threads: int = 256
    unroll: int = 2              # 16-byte vectors in flight per thread and loop trip
    ctas_per_sm: int = 8         # grid = min(needed, SMs * ctas_per_sm)

    def key(self) -> str:
        return f"t{self.threads}u{self.unroll}c{self.ctas_per_sm}"

    def compile_key(self) -> str:
        """What the generated source depends on (the grid limit is a launch argument)."""
        return f"t{self.threads}u{self.unroll}"


def search_space() -> List[KernelConfig]:
    """Six compiled variants (threads x vectors in flight), each tried with two grid limits."""
    return [KernelConfig(t, u, c) for t in (256, 512) for u in (1, 2, 4) for c in (4, 8)]


class CudaChainSource:
    """Renders the complete translation unit of one fused chain."""

    def render(self, name: str, chain: Chain, dtype: torch.dtype, cfg: KernelConfig) -> str:
        n_in = chain_arity(chain)
        if dtype not in (torch.bfloat16, torch.float32, torch.float16):
            raise TypeError(f"unsupported element type {dtype}")
        T = {torch.bfloat16: "__nv_bfloat16", torch.float16: "__half", torch.float32: "float"}[dtype]
        V = 4 if dtype == torch.float32 else 8
        to_f = {torch.bfloat16: "__bfloat162float", torch.float16: "__half2float", torch.float32: ""}[dtype]
        from_f = {torch.bfloat16: "__float2bfloat16", torch.float16: "__float2half", torch.float32: ""}[dtype]
        steps, nxt = [], 1
        for k in chain:
            expr, binary = SNIPPETS[k]
            if binary:
                steps.append(f"    {{ const float x = X{nxt}; v = {expr}; }}")
                nxt += 1
            else:
                steps.append(f"    v = {expr};")
        params = ", ".join(f"const T* __restrict__ in{k}" for k in range(n_in))
        # the per-element body is a macro-free inline function over the operands of one element
        elem_args = ", ".join(f"float X{k}" for k in range(n_in))
        vec_loads = "\n".join(f"      Vec a{k} = *reinterpret_cast<const Vec*>(in{k} + i * V);" for k in range(n_in))
        elem_call_vec = ", ".join(f"{to_f}(a{k}.e[j])" for k in range(n_in))
        elem_call_tail = ", ".join(f"{to_f}(in{k}[i])" for k in range(n_in))
        body = "\n".join(steps)
        ptr_unpack = "\n".join(f"  const T* in{k} = static_cast<const T*>(ins[{k}]);" for k in range(n_in))
        call_args = ", ".join(f"in{k}" for k in range(n_in))
        align_checks = " || ".join([f"(reinterpret_cast<uintptr_t>(in{k}) & 15)" for k in range(n_in)] + ["(reinterpret_cast<uintptr_t>(out) & 15)"])
        return f"""// generated: fused element-wise chain {list(chain)} on {T}, {cfg.compile_key()}
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
using T = {T};
constexpr int V = {V};                 // elements per 16-byte access
constexpr int UNROLL = {cfg.unroll};
struct __align__(16) Vec {{ T e[V]; }};

__device__ __forceinline__ float chain_elem({elem_args}) {{
    float v = X0;
{body}
    return v;
}}

extern "C" __global__ void __launch_bounds__({cfg.threads}) {name}_kernel(T* __restrict__ out, {params}, long long n, int vec_ok) {{
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long nvec = vec_ok ? n / V : 0;
  for (long long i0 = tid; i0 < nvec; i0 += nthreads * UNROLL) {{
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {{
      const long long i = i0 + (long long)u * nthreads;
      if (i >= nvec) break;
{vec_loads}
      Vec r;
#pragma unroll
      for (int j = 0; j < V; ++j) r.e[j] = {from_f}(chain_elem({elem_call_vec}));
      *reinterpret_cast<Vec*>(out + i * V) = r;
    }}
  }}
  // scalar tail (and the whole range when a pointer is not 16-byte aligned)
  for (long long i = nvec * V + tid; i < n; i += nthreads)
    out[i] = {from_f}(chain_elem({elem_call_tail}));
}}

// C launcher: raw device pointers, element count, grid limit (SMs x CTAs per SM) and the stream to launch on.
extern "C" int {name}_launch(void* out_, const void* const* ins, long long n, int max_ctas, void* stream) {{
  T* out = static_cast<T*>(out_);
{ptr_unpack}
  if (n <= 0) return 0;
  const int vec_ok = ({align_checks}) ? 0 : 1;
  const long long work = vec_ok ? (n / V + UNROLL - 1) / UNROLL + (n % V) : n;
  long long grid = (work + {cfg.threads} - 1) / {cfg.threads};
  if (grid > max_ctas) grid = max_ctas;
  if (grid < 1) grid = 1;
  {name}_kernel<<<(unsigned)grid, {cfg.threads}, 0, static_cast<cudaStream_t>(stream)>>>(out, {call_args}, n, vec_ok);
  return (int)cudaGetLastError();
}}
"""


class CompileError(RuntimeError):
    pass


class NvccCompiler:
    """``nvcc`` as the back-end: source text -> shared object in a content-addressed cache directory."""

    FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--use_fast_math", "-lineinfo",
             "-shared", "-Xcompiler", "-fPIC"]

    def __init__(self, cache_dir: Optional[str] = None, nvcc: Optional[str] = None):
        self.cache_dir = Path(cache_dir or os.environ.get("MLF_JIT_CACHE") or Path(tempfile.gettempdir()) / "mlf_b200_jit")
        self.nvcc = nvcc or os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        self.compilations = 0
        self.cache_hits = 0

    def available(self) -> bool:
        return os.path.exists(self.nvcc)

    def digest(self, source: str) -> str:
        return hashlib.sha256((source + "\0" + " ".join(self.FLAGS)).encode()).hexdigest()[:24]

    def compile(self, source: str) -> Path:
        """Path of the shared object for ``source`` (built if no process has built it before)."""
        self.cache_dir.mkdir(parents=True, exist_ok=True)
        so = self.cache_dir / f"k_{self.digest(source)}.so"
        if so.exists():
            self.cache_hits += 1
            return so
        if not self.available():
            raise CompileError(f"nvcc not found at {self.nvcc}")
        with tempfile.TemporaryDirectory(dir=self.cache_dir) as td:
            cu = Path(td) / "k.cu"
            cu.write_text(source)
            tmp = Path(td) / "k.so"
            r = subprocess.run([self.nvcc, *self.FLAGS, "-o", str(tmp), str(cu)], capture_output=True, text=True)
            if r.returncode != 0 or not tmp.exists():
                raise CompileError(f"nvcc failed ({r.returncode}):\n{r.stderr[-4000:]}")
            os.replace(tmp, so)          # atomic: concurrent builders of the same source leave one complete file
        self.compilations += 1
        return so


class CompiledChain:
    """A loaded shared object of one chain variant."""

    def __init__(self, so: Path, name: str, n_in: int):
        self.path, self.name, self.n_in = so, name, n_in
        self._lib = C.CDLL(str(so))
        self._launch = getattr(self._lib, f"{name}_launch")
        self._launch.restype = C.c_int
        self._launch.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_longlong, C.c_int, C.c_void_p]

    def launch(self, out: torch.Tensor, inputs: Sequence[torch.Tensor], max_ctas: int, stream: Optional[int] = None):
        arr = (C.c_void_p * self.n_in)(*[t.data_ptr() for t in inputs])
        st = torch.cuda.current_stream(out.device).cuda_stream if stream is None else stream
        rc = self._launch(C.c_void_p(out.data_ptr()), arr, C.c_longlong(out.numel()), int(max_ctas), C.c_void_p(st))
        if rc != 0:
            raise RuntimeError(f"launch of {self.name} failed with CUDA error {rc}")


_default_compiler: Optional[NvccCompiler] = None
_compiler_lock = threading.Lock()


def default_compiler() -> NvccCompiler:
    global _default_compiler
    with _compiler_lock:
        if _default_compiler is None:
            _default_compiler = NvccCompiler()
        return _default_compiler


class FusedElementwise:
    """``out = chain(inputs)`` as one generated kernel. ``chain`` is a list of op names applied left to right to a
    running value that starts as ``inputs[0]``; every binary op consumes the next input tensor."""

    def __init__(self, chain: Chain, compiler: Optional[NvccCompiler] = None, autotune: bool = False,
                 default_config: Optional[KernelConfig] = None, cache_capacity: int = 64):
        self.chain = tuple(chain)
        self.n_in = chain_arity(self.chain)
        self.compiler = compiler or default_compiler()
        self.autotune = autotune
        self.default_config = default_config or KernelConfig()
        self.variants: LRUKernelCache = LRUKernelCache(cache_capacity)       # (dtype, config) -> CompiledChain
        self.chosen: Dict[str, KernelConfig] = {}                            # (dtype, size bucket) -> tuned config
        self.tuner = Autotuner()
        self._buckets = ShapeVariantGenerator.buckets(1 << 10, 1 << 32)
        self._src = CudaChainSource()

    def _name(self, dtype: torch.dtype, cfg: KernelConfig) -> str:
        h = hashlib.sha256(("|".join(self.chain) + str(dtype) + cfg.compile_key()).encode()).hexdigest()[:12]
        return f"fused_{h}"

    def source(self, dtype: torch.dtype, cfg: Optional[KernelConfig] = None) -> str:
        cfg = cfg or self.default_config
        return self._src.render(self._name(dtype, cfg), self.chain, dtype, cfg)

    def variant(self, dtype: torch.dtype, cfg: KernelConfig) -> CompiledChain:
        sig = ShapeSignature("fused:" + "|".join(self.chain), (), str(dtype), (cfg.compile_key(),))

        def build():
            name = self._name(dtype, cfg)
            so = self.compiler.compile(self._src.render(name, self.chain, dtype, cfg))
            return CompiledChain(so, name, self.n_in)
        return self.variants.get_or_create(sig, build)

    def precompile(self, dtype: torch.dtype, configs: Optional[Sequence[KernelConfig]] = None, workers: int = 6):
        """Build the variants of ``configs`` (default: the default configuration) ahead of the first call, in parallel
        (one ``nvcc`` process each)."""
        from concurrent.futures import ThreadPoolExecutor
        todo = {c.compile_key(): c for c in (configs or [self.default_config])}
        with ThreadPoolExecutor(max_workers=max(1, min(workers, len(todo)))) as ex:
            list(ex.map(lambda c: self.compiler.compile(self._src.render(self._name(dtype, c), self.chain, dtype, c)), todo.values()))
        for c in todo.values():
            self.variant(dtype, c)

    def _check(self, inputs: Sequence[torch.Tensor]):
        if len(inputs) != self.n_in:
            raise ValueError(f"chain {list(self.chain)} reads {self.n_in} tensors, got {len(inputs)}")
        a = inputs[0]
        for t in inputs[1:]:
            if t.shape != a.shape or t.dtype != a.dtype or t.device != a.device:
                raise ValueError("fused element-wise inputs must share shape, dtype and device (broadcast them first)")

    def __call__(self, *inputs: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        self._check(inputs)
        a = inputs[0]
        if not a.is_cuda:
            res = eval_chain_torch(self.chain, inputs)
            if out is not None:
                out.copy_(res)
                return out
            return res
        ins = [t.contiguous() for t in inputs]
        if out is None:
            out = torch.empty_like(ins[0])
        elif not out.is_contiguous() or out.shape != a.shape or out.dtype != a.dtype:
            raise ValueError("out must be a contiguous tensor of the inputs' shape and dtype")
        n = out.numel()
        cfg = self._config_for(a.dtype, n, ins, out)
        sms = torch.cuda.get_device_properties(a.device).multi_processor_count
        self.variant(a.dtype, cfg).launch(out, ins, sms * cfg.ctas_per_sm)
        return out

    def _config_for(self, dtype, n: int, ins, out) -> KernelConfig:
        if not self.autotune:
            return self.default_config
        bucket = ShapeVariantGenerator.bucket_for(max(n, 1 << 10), self._buckets)
        key = f"{dtype}:{bucket}"
        if key not in self.chosen:
            sms = torch.cuda.get_device_properties(out.device).multi_processor_count
            sig = ShapeSignature("fused:" + "|".join(self.chain), ((bucket,),), str(dtype), ())
            cands = [{"cfg": c} for c in search_space()]
            self.precompile(dtype, [c["cfg"] for c in cands])
            best = self.tuner.tune(sig, cands, lambda d: self.variant(dtype, d["cfg"]).launch(out, ins, sms * d["cfg"].ctas_per_sm))
            self.chosen[key] = best["cfg"]
        return self.chosen[key]


def compile_chain(chain: Chain, **kw) -> FusedElementwise:
    """A callable for the chain (compiled lazily, on the first GPU call of each dtype)."""
    return FusedElementwise(chain, **kw)
