"""Fusion planner: finds fusible patterns in a high-level graph and maps them to fused kernels.

Reference: src/MLFramework/Fusion/FusionEngine.cs:6-45, DefaultFusionRegistry.cs, pattern detectors for
element-wise chains / Conv+Activation / Conv+BatchNorm (Fusion/Patterns/*.cs), GraphTransformer.cs,
constraint validators (memory layout, precision, side effects, thread-block limits:
Fusion/Validation/**), decision logging (Fusion/Profiling/**), and a CUDA text generator whose
templates are one-thread-per-element scalar fp32 (Fusion/KernelCode/Cuda/CudaKernelTemplates.cs:8-160)
behind Triton / XLA adapter interfaces with no compiler attached (Fusion/Backends/*.cs).

Here the hot fused kernels exist, hand-written: a GEMM's epilogue takes bias, GELU, SwiGLU, residual add,
dGELU, dSwiGLU and accumulate; normalisation takes the residual; conv + batch-norm folds into the conv's
weights. The planner's job is to recognise those shapes in a graph and rewrite them to the fused op. Chains
of element-wise ops that the hand-written set does not cover are rewritten to one ``fused_elementwise`` op,
which the graph executor runs as ONE kernel generated, compiled with ``nvcc`` and cached at run time
(:mod:`ml_framework_b200.compiler.jit_cuda`); ``FusionEngine.compile_chain`` gives the callable directly.
``CudaSourceGenerator`` is the older text-only renderer kept for listings.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .ir import ELEMENTWISE, UNARY, HLGraph, Op


@dataclass
class FusionDecision:
    pattern: str
    ops: List[str]
    accepted: bool
    reason: str = ""


@dataclass
class FusionConstraints:
    max_chain_length: int = 16
    max_inputs: int = 8                      # pointer arguments of one fused element-wise kernel
    require_same_dtype: bool = True
    require_same_shape: bool = True


class FusionRegistry:
    def __init__(self):
        self.fusible_elementwise = set(ELEMENTWISE) | set(UNARY)
        self.gemm_epilogues = {"bias": "MLF_EPI_BIAS", "gelu": "MLF_EPI_GELU", "residual": "MLF_EPI_RESIDUAL"}
        self.patterns = ["linear_bias_gelu", "linear_residual", "conv_batchnorm", "conv_activation", "elementwise_chain"]

    def is_fusible(self, kind: str) -> bool:
        return kind in self.fusible_elementwise


class FusionEngine:
    def __init__(self, registry: Optional[FusionRegistry] = None, constraints: Optional[FusionConstraints] = None):
        self.reg, self.cons = registry or FusionRegistry(), constraints or FusionConstraints()
        self.decisions: List[FusionDecision] = []

    # ---- pattern: chains of element-wise ops with single-use intermediates
    def find_elementwise_chains(self, g: HLGraph) -> List[List[int]]:
        users = g.users()
        outs = set(g.outputs)
        chains, used = [], set()
        for i, o in enumerate(g.ops):
            if i in used or not self.reg.is_fusible(o.kind):
                continue
            chain, cur = [i], o
            while True:
                u = users.get(cur.output, [])
                if len(u) != 1 or cur.output in outs:
                    break
                nxt = g.ops[u[0]]
                if not self.reg.is_fusible(nxt.kind) or u[0] in used or nxt.inputs[0] != cur.output:
                    break
                if self.cons.require_same_shape and g.values[nxt.output].shape != g.values[o.output].shape:
                    break
                if self.cons.require_same_dtype and g.values[nxt.output].dtype != g.values[o.output].dtype:
                    break
                if len(chain) >= self.cons.max_chain_length:
                    break
                chain.append(u[0])
                cur = nxt
            if len(chain) > 1:
                n_in = sum(len(g.ops[k].inputs) for k in chain) - (len(chain) - 1)
                ok = n_in <= self.cons.max_inputs
                self.decisions.append(FusionDecision("elementwise_chain", [g.ops[k].output for k in chain], ok,
                                                     "" if ok else f"{n_in} inputs exceed limit {self.cons.max_inputs}"))
                if ok:
                    chains.append(chain)
                    used.update(chain)
        return chains

    def fuse_elementwise(self, g: HLGraph) -> int:
        chains = self.find_elementwise_chains(g)
        drop = set()
        for chain in chains:
            first, last = g.ops[chain[0]], g.ops[chain[-1]]
            spec, extra = [], []
            for n, k in enumerate(chain):
                o = g.ops[k]
                binary = len(o.inputs) == 2
                spec.append((o.kind, binary))
                if n == 0:
                    extra.extend(o.inputs[1:])
                elif binary:
                    extra.append(o.inputs[1])
            g.ops[chain[-1]] = Op("fused_elementwise", [first.inputs[0]] + extra, last.output, {"chain": spec})
            drop.update(chain[:-1])
        g.ops = [o for i, o in enumerate(g.ops) if i not in drop]
        return len(chains)

    # ---- pattern: linear (+bias) -> gelu, linear -> add residual: GEMM epilogues
    def find_gemm_epilogues(self, g: HLGraph) -> List[Tuple[int, int, str]]:
        users, found = g.users(), []
        for i, o in enumerate(g.ops):
            if o.kind not in ("linear", "matmul"):
                continue
            u = users.get(o.output, [])
            if len(u) != 1 or o.output in g.outputs:
                continue
            nxt = g.ops[u[0]]
            if nxt.kind == "gelu":
                found.append((i, u[0], "gelu"))
            elif nxt.kind == "add" and g.values[nxt.output].shape == g.values[o.output].shape:
                found.append((i, u[0], "residual"))
            if found and found[-1][0] == i:
                self.decisions.append(FusionDecision(f"gemm_{found[-1][2]}", [o.output, nxt.output], True))
        return found

    # ---- pattern: conv2d -> batchnorm (inference): fold into conv weights
    @staticmethod
    def fold_conv_batchnorm(w: torch.Tensor, b: Optional[torch.Tensor], gamma, beta, mean, var, eps: float = 1e-5):
        s = gamma / torch.sqrt(var + eps)
        w2 = w * s.view(-1, 1, 1, 1)
        b2 = (b if b is not None else torch.zeros_like(mean)) - mean
        return w2, b2 * s + beta

    @staticmethod
    def compile_chain(spec: Sequence[Tuple[str, bool]], **kw):
        """The callable of a fused element-wise chain (``spec`` as stored in a ``fused_elementwise`` op's attributes):
        one generated CUDA kernel on GPU tensors, the same chain in PyTorch elsewhere."""
        from .jit_cuda import compile_chain
        return compile_chain([kind for kind, _ in spec], **kw)

    def plan(self, g: HLGraph) -> Dict[str, object]:
        return {"gemm_epilogues": self.find_gemm_epilogues(g), "elementwise_chains": self.find_elementwise_chains(g),
                "decisions": list(self.decisions)}


class CudaSourceGenerator:
    """Element-wise chain -> CUDA source text: 128-bit loads and stores, fp32 math, grid-stride loop.
    The reference's template is one thread per element with scalar loads."""
    SNIPPETS = {"add": "{a} + {b}", "sub": "{a} - {b}", "mul": "{a} * {b}", "div": "{a} / {b}", "maximum": "fmaxf({a}, {b})",
                "minimum": "fminf({a}, {b})", "relu": "fmaxf({a}, 0.f)", "sigmoid": "1.f / (1.f + __expf(-{a}))", "tanh": "tanhf({a})",
                "exp": "__expf({a})", "log": "__logf({a})", "sqrt": "sqrtf({a})", "neg": "-{a}",
                "gelu": "0.5f * {a} * (1.f + tanhf(0.7978845608f * ({a} + 0.044715f * {a} * {a} * {a})))"}

    def generate(self, name: str, chain: Sequence[Tuple[str, bool]], dtype: str = "bf16") -> str:
        n_extra = sum(1 for _, b in chain if b)
        args = ", ".join([f"const T* __restrict__ in{k}" for k in range(n_extra + 1)])
        body, extra = [], 1
        for kind, binary in chain:
            if kind not in self.SNIPPETS:
                raise KeyError(f"no snippet for {kind}")
            expr = self.SNIPPETS[kind].format(a="v", b=f"x{extra}[j]" if binary else "")
            body.append(f"        v = {expr};")
            extra += int(binary)
        loads = "\n".join(f"      float x{k}[V]; load_vec(in{k} + i * V, x{k});" for k in range(n_extra + 1))
        T = "__nv_bfloat16" if dtype == "bf16" else "float"
        V = 8 if dtype == "bf16" else 4
        return f"""// generated: fused element-wise chain {[k for k, _ in chain]}
#include <cuda_bf16.h>
using T = {T};
constexpr int V = {V};   // elements per 16-byte access
__device__ inline void load_vec(const T* p, float (&f)[V]);   // 128-bit load + convert
__device__ inline void store_vec(T* p, const float (&f)[V]);  // convert + 128-bit store
extern "C" __global__ void __launch_bounds__(256) {name}(T* __restrict__ out, {args}, long long n) {{
  const long long nvec = n / V;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {{
{loads}
      float r[V];
#pragma unroll
      for (int j = 0; j < V; ++j) {{
        float v = x0[j];
{chr(10).join(body)}
        r[j] = v;
      }}
      store_vec(out + i * V, r);
  }}
}}
"""
