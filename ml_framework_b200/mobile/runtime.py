"""Mobile inference runtime: load a ``.mob`` model and run it; converter from ``torch.nn`` models with
graph optimisation and weight quantisation; benchmarking.

Reference: src/MobileRuntime/RuntimeMobileRuntime.cs:22-135 (LoadModel / Predict), Tensors/TensorOperations.cs
(CPU operator set), DefaultMemoryPool.cs, Benchmarking/*; converter CLI tools/MobileModelConverter
(``convert -i in -o out [-q int8|uint8|fp16]``: graph optimiser, constant folder, operator fuser, quantiser,
validator). The reference's accelerator back-end is a set of Metal dispatch wrappers; here the same
operators are CUDA kernels (``csrc/ops/mobile.cu``) when the model is loaded onto a GPU, PyTorch on the CPU.
"""
from __future__ import annotations

import ctypes as C
import time
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .format import MobModel, MobOperator, MobTensor, load_mob, save_mob


class MemoryPool:
    """Recycles activation buffers by element count between ``predict`` calls (the model's shapes repeat)."""

    def __init__(self, device):
        self.device, self._free, self.hits, self.misses = device, {}, 0, 0

    def get(self, shape: Sequence[int]) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        lst = self._free.get(n)
        if lst:
            self.hits += 1
            return lst.pop().view(*shape)
        self.misses += 1
        return torch.empty(*shape, dtype=torch.float32, device=self.device)

    def put(self, t: torch.Tensor):
        self._free.setdefault(t.numel(), []).append(t.reshape(-1))


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class MobileRuntime:
    def __init__(self, device: str = "cpu"):
        self.device = torch.device(device)
        self.model: Optional[MobModel] = None
        self.weights: Dict[str, torch.Tensor] = {}
        self.pool = MemoryPool(self.device)
        self.native = self.device.type == "cuda"

    # ---- loading
    def load_model(self, path_or_model) -> "MobileRuntime":
        m = load_mob(path_or_model) if isinstance(path_or_model, str) else path_or_model
        errs = m.validate()
        if errs:
            raise ValueError("invalid model: " + "; ".join(errs))
        self.model = m
        self.weights = {}
        for n, t in m.tensors.items():
            d = t.data
            if t.scale is not None:                              # stored quantised: expand once at load
                d = (d.float() - (t.zero_point or 0)) * t.scale
            self.weights[n] = d.float().contiguous().to(self.device)
        return self

    # ---- operators
    def _conv(self, x, op):
        a = op.attrs
        w = self.weights[op.inputs[1]]
        b = self.weights[op.inputs[2]] if len(op.inputs) > 2 else None
        st, pd, dl, g, relu = a.get("stride", 1), a.get("padding", 0), a.get("dilation", 1), a.get("groups", 1), a.get("relu", False)
        if self.native and w.shape[2] <= 7 and w.shape[3] <= 7 and st <= 4 and dl <= 2:
            from .. import _lib
            N, Cc, H, W = x.shape
            O, _, KH, KW = w.shape
            OH, OW = (H + 2 * pd - dl * (KH - 1) - 1) // st + 1, (W + 2 * pd - dl * (KW - 1) - 1) // st + 1
            out = self.pool.get((N, O, OH, OW))
            _lib.check(_lib.get().mlf_conv2d_f32(_p(out), _p(x.contiguous()), _p(w), _p(b), N, Cc, H, W, O, KH, KW, st, pd, dl, g, int(relu),
                                                 C.c_uint64(_lib.stream_handle())), "mlf_conv2d_f32")
            return out
        y = F.conv2d(x, w, b, st, pd, dl, g)
        return F.relu(y) if relu else y

    def _pool(self, x, op, mode):
        a = op.attrs
        k = a.get("kernel", 2)
        st, pd = a.get("stride", k), a.get("padding", 0)
        if mode == 1 and a.get("count_include_pad", False):
            mode = 2
        if self.native:
            from .. import _lib
            N, Cc, H, W = x.shape
            OH, OW = (H + 2 * pd - k) // st + 1, (W + 2 * pd - k) // st + 1
            out = self.pool.get((N, Cc, OH, OW))
            _lib.check(_lib.get().mlf_pool2d_f32(_p(out), _p(x.contiguous()), N * Cc, H, W, k, st, pd, mode, C.c_uint64(_lib.stream_handle())), "mlf_pool2d_f32")
            return out
        return F.max_pool2d(x, k, st, pd) if mode == 0 else F.avg_pool2d(x, k, st, pd, count_include_pad=(mode == 2))

    def _bn(self, x, op):
        g, b, m, v = (self.weights[n] for n in op.inputs[1:5])
        eps, relu = op.attrs.get("eps", 1e-5), op.attrs.get("relu", False)
        if self.native:
            from .. import _lib
            N, Cc = x.shape[:2]
            out = self.pool.get(tuple(x.shape))
            _lib.check(_lib.get().mlf_batchnorm_f32(_p(out), _p(x.contiguous()), _p(g), _p(b), _p(m), _p(v), C.c_float(eps), N, Cc,
                                                    x[0, 0].numel(), int(relu), C.c_uint64(_lib.stream_handle())), "mlf_batchnorm_f32")
            return out
        y = F.batch_norm(x, m, v, g, b, False, 0.0, eps)
        return F.relu(y) if relu else y

    def _fc(self, x, op):
        w = self.weights[op.inputs[1]]
        b = self.weights[op.inputs[2]] if len(op.inputs) > 2 else None
        relu = op.attrs.get("relu", False)
        x2 = x.reshape(x.shape[0], -1)
        if self.native:
            from .. import _lib
            out = self.pool.get((x2.shape[0], w.shape[0]))
            _lib.check(_lib.get().mlf_fc_f32(_p(out), _p(x2.contiguous()), _p(w), _p(b), x2.shape[0], x2.shape[1], w.shape[0], int(relu),
                                             C.c_uint64(_lib.stream_handle())), "mlf_fc_f32")
            return out
        y = F.linear(x2, w, b)
        return F.relu(y) if relu else y

    def _softmax(self, x, op):
        if self.native and op.attrs.get("dim", -1) in (-1, x.dim() - 1):
            from .. import _lib
            out = self.pool.get(tuple(x.shape))
            _lib.check(_lib.get().mlf_softmax_rows_f32(_p(out), _p(x.contiguous()), C.c_longlong(x.numel() // x.shape[-1]), x.shape[-1],
                                                       C.c_uint64(_lib.stream_handle())), "mlf_softmax_rows_f32")
            return out
        return torch.softmax(x, op.attrs.get("dim", -1))

    def _run_op(self, op: MobOperator, env: Dict[str, torch.Tensor]) -> torch.Tensor:
        get = lambda n: env[n] if n in env else self.weights[n]
        x = get(op.inputs[0])
        t = op.type
        if t == "conv2d": return self._conv(x, op)
        if t == "fully_connected": return self._fc(x, op)
        if t == "relu": return torch.relu(x)
        if t == "sigmoid": return torch.sigmoid(x)
        if t == "tanh": return torch.tanh(x)
        if t == "max_pool2d": return self._pool(x, op, 0)
        if t == "avg_pool2d": return self._pool(x, op, 1)
        if t == "global_avg_pool": return x.mean((2, 3), keepdim=True)
        if t == "batch_norm": return self._bn(x, op)
        if t == "softmax": return self._softmax(x, op)
        if t == "add": return x + get(op.inputs[1])
        if t == "mul": return x * get(op.inputs[1])
        if t == "flatten": return x.reshape(x.shape[0], -1)
        if t == "reshape": return x.reshape(op.attrs["shape"])
        if t == "concat": return torch.cat([get(n) for n in op.inputs], op.attrs.get("dim", 1))
        if t == "sub": return x - get(op.inputs[1])
        if t == "div": return x / get(op.inputs[1])
        if t == "matmul": return x @ get(op.inputs[1])
        if t in ("abs", "sqrt", "square", "log", "exp"): return getattr(torch, t)(x)
        if t in ("sum", "mean", "max", "min"):
            ax = op.attrs.get("axis")
            if ax is None:
                return getattr(x, t)().reshape(1)
            r = getattr(x, {"max": "amax", "min": "amin"}.get(t, t))(ax, keepdim=op.attrs.get("keepdims", False))
            return r
        if t == "transpose": return x.permute(op.attrs["perm"]).contiguous() if "perm" in op.attrs else x.transpose(-1, -2).contiguous()
        if t == "cast": return x.to(getattr(torch, op.attrs["dtype"]))
        if t == "copy": return x.clone()
        raise NotImplementedError(t)

    @torch.no_grad()
    def profile_operators(self, *inputs: torch.Tensor, iters: int = 5) -> List[Dict[str, object]]:
        """Time per operator (device-synchronised around every operator, so the sum exceeds an unprofiled ``predict``):
        ``[{index, type, output, mean_ms, share}]`` sorted by cost."""
        if self.model is None:
            raise RuntimeError("no model loaded")
        acc = [0.0] * len(self.model.operators)
        for _ in range(iters):
            env = {spec["name"]: x.to(self.device, torch.float32) for spec, x in zip(self.model.inputs, inputs)}
            for k, op in enumerate(self.model.operators):
                if self.native:
                    torch.cuda.synchronize()
                t0 = time.perf_counter()
                env[op.outputs[0]] = self._run_op(op, env)
                if self.native:
                    torch.cuda.synchronize()
                acc[k] += (time.perf_counter() - t0) * 1e3
        total = sum(acc) or 1.0
        rows = [{"index": k, "type": op.type, "output": op.outputs[0], "mean_ms": acc[k] / iters, "share": acc[k] / total}
                for k, op in enumerate(self.model.operators)]
        return sorted(rows, key=lambda r: -r["mean_ms"])

    @torch.no_grad()
    def predict(self, *inputs: torch.Tensor) -> List[torch.Tensor]:
        if self.model is None:
            raise RuntimeError("no model loaded")
        if len(inputs) != len(self.model.inputs):
            raise ValueError(f"model takes {len(self.model.inputs)} inputs, got {len(inputs)}")
        env = {spec["name"]: x.to(self.device, torch.float32) for spec, x in zip(self.model.inputs, inputs)}
        last_use = {}
        for k, op in enumerate(self.model.operators):
            for n in op.inputs:
                last_use[n] = k
        pooled = set()
        for k, op in enumerate(self.model.operators):
            out = self._run_op(op, env)
            env[op.outputs[0]] = out
            if self.native and op.type in ("conv2d", "fully_connected", "max_pool2d", "avg_pool2d", "batch_norm", "softmax"):
                pooled.add(op.outputs[0])
            for n in op.inputs:                                   # recycle buffers whose last reader just ran
                if last_use.get(n) == k and n in pooled and n not in self.model.outputs:
                    self.pool.put(env.pop(n))
                    pooled.discard(n)
        return [env[n].clone() if n in pooled else env[n] for n in self.model.outputs]

    def benchmark(self, *inputs: torch.Tensor, warmup: int = 3, iters: int = 20) -> Dict[str, float]:
        for _ in range(warmup):
            self.predict(*inputs)
        ts = []
        for _ in range(iters):
            if self.native:
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            self.predict(*inputs)
            if self.native:
                torch.cuda.synchronize()
            ts.append((time.perf_counter() - t0) * 1e3)
        ts.sort()
        return {"mean_ms": sum(ts) / len(ts), "p50_ms": ts[len(ts) // 2], "p99_ms": ts[min(len(ts) - 1, int(0.99 * len(ts)))],
                "pool_hits": self.pool.hits, "pool_misses": self.pool.misses}


# ------------------------------------------------------------------ converter
def convert_sequential(model: nn.Module, input_shape: Sequence[int], name: str = "model") -> MobModel:
    """Converts a chain of Conv2d / BatchNorm2d / ReLU / MaxPool2d / AvgPool2d / AdaptiveAvgPool2d(1) /
    Flatten / Linear / Softmax / Sigmoid / Tanh modules (``nn.Sequential`` or any module whose children run in order)."""
    ops: List[MobOperator] = []
    tensors: Dict[str, MobTensor] = {}
    cur = "input"

    def add_t(n, t):
        tensors[n] = MobTensor(n, t.detach().float().cpu().contiguous())
        return n
    for i, m in enumerate(model.children() if not isinstance(model, nn.Sequential) else model):
        out = f"t{i}"
        if isinstance(m, nn.Conv2d):
            if m.stride[0] != m.stride[1] or m.padding[0] != m.padding[1] or m.dilation[0] != m.dilation[1]:
                raise ValueError("conv2d: only square stride / padding / dilation are supported")
            ins = [cur, add_t(f"w{i}", m.weight)] + ([add_t(f"b{i}", m.bias)] if m.bias is not None else [])
            ops.append(MobOperator("conv2d", ins, [out], {"stride": m.stride[0], "padding": m.padding[0], "dilation": m.dilation[0], "groups": m.groups}))
        elif isinstance(m, nn.BatchNorm2d):
            ins = [cur, add_t(f"g{i}", m.weight if m.weight is not None else torch.ones(m.num_features)),
                   add_t(f"b{i}", m.bias if m.bias is not None else torch.zeros(m.num_features)), add_t(f"m{i}", m.running_mean), add_t(f"v{i}", m.running_var)]
            ops.append(MobOperator("batch_norm", ins, [out], {"eps": m.eps}))
        elif isinstance(m, nn.Linear):
            ins = [cur, add_t(f"w{i}", m.weight)] + ([add_t(f"b{i}", m.bias)] if m.bias is not None else [])
            ops.append(MobOperator("fully_connected", ins, [out]))
        elif isinstance(m, nn.ReLU): ops.append(MobOperator("relu", [cur], [out]))
        elif isinstance(m, nn.Sigmoid): ops.append(MobOperator("sigmoid", [cur], [out]))
        elif isinstance(m, nn.Tanh): ops.append(MobOperator("tanh", [cur], [out]))
        elif isinstance(m, nn.MaxPool2d):
            k = m.kernel_size if isinstance(m.kernel_size, int) else m.kernel_size[0]
            s = m.stride if isinstance(m.stride, int) else m.stride[0]
            pd = m.padding if isinstance(m.padding, int) else m.padding[0]
            ops.append(MobOperator("max_pool2d", [cur], [out], {"kernel": k, "stride": s, "padding": pd}))
        elif isinstance(m, nn.AvgPool2d):
            k = m.kernel_size if isinstance(m.kernel_size, int) else m.kernel_size[0]
            s = m.stride if isinstance(m.stride, int) else m.stride[0]
            pd = m.padding if isinstance(m.padding, int) else m.padding[0]
            ops.append(MobOperator("avg_pool2d", [cur], [out], {"kernel": k, "stride": s, "padding": pd, "count_include_pad": bool(m.count_include_pad)}))
        elif isinstance(m, nn.AdaptiveAvgPool2d): ops.append(MobOperator("global_avg_pool", [cur], [out]))
        elif isinstance(m, nn.Flatten): ops.append(MobOperator("flatten", [cur], [out]))
        elif isinstance(m, nn.Softmax): ops.append(MobOperator("softmax", [cur], [out], {"dim": -1}))
        elif isinstance(m, (nn.Dropout, nn.Identity)): continue
        else:
            raise NotImplementedError(f"no .mob operator for {type(m).__name__}")
        cur = out
    return MobModel([{"name": "input", "shape": list(input_shape)}], [cur], ops, tensors, {"name": name})


def optimize(model: MobModel) -> MobModel:
    """Operator fusion: conv + batch-norm folds into the conv's weights; conv / fc / batch-norm followed by
    ReLU sets the producer's ``relu`` flag. Dead tensors are dropped."""
    ops = list(model.operators)
    users: Dict[str, int] = {}
    for o in ops:
        for n in o.inputs:
            users[n] = users.get(n, 0) + 1
    out: List[MobOperator] = []
    i = 0
    while i < len(ops):
        o = ops[i]
        nxt = ops[i + 1] if i + 1 < len(ops) else None
        if o.type == "conv2d" and nxt is not None and nxt.type == "batch_norm" and nxt.inputs[0] == o.outputs[0] and users.get(o.outputs[0]) == 1:
            w = model.tensors[o.inputs[1]].data
            b = model.tensors[o.inputs[2]].data if len(o.inputs) > 2 else torch.zeros(w.shape[0])
            g, be, mu, var = (model.tensors[n].data for n in nxt.inputs[1:5])
            s = g / torch.sqrt(var + nxt.attrs.get("eps", 1e-5))
            wn, bn = f"{o.inputs[1]}.folded", f"{o.inputs[1]}.folded_bias"
            model.tensors[wn] = MobTensor(wn, w * s.view(-1, 1, 1, 1))
            model.tensors[bn] = MobTensor(bn, (b - mu) * s + be)
            o = MobOperator("conv2d", [o.inputs[0], wn, bn], list(nxt.outputs), dict(o.attrs))
            i += 1
            nxt = ops[i + 1] if i + 1 < len(ops) else None
        if o.type in ("conv2d", "fully_connected", "batch_norm") and nxt is not None and nxt.type == "relu" and nxt.inputs[0] == o.outputs[0] \
                and users.get(o.outputs[0], 1) == 1:
            o = MobOperator(o.type, o.inputs, list(nxt.outputs), dict(o.attrs, relu=True))
            i += 1
        out.append(o)
        i += 1
    used = {n for o in out for n in o.inputs}
    return MobModel(model.inputs, model.outputs, out, {k: v for k, v in model.tensors.items() if k in used}, dict(model.metadata, optimized=True))


def fold_constants(model: MobModel) -> MobModel:
    """Constant folder: an operator whose inputs are all stored tensors (no graph input reaches it) is evaluated once
    here and its result stored as a tensor; operators left without readers disappear with it."""
    rt = MobileRuntime("cpu")
    rt.model = model
    rt.weights = {n: (t.data.float() - (t.zero_point or 0)) * t.scale if t.scale is not None else t.data for n, t in model.tensors.items()}
    const = set(model.tensors)
    tensors = dict(model.tensors)
    kept: List[MobOperator] = []
    with torch.no_grad():
        for o in model.operators:
            if o.inputs and all(n in const for n in o.inputs) and o.type not in ("copy",):
                val = rt._run_op(o, {})
                rt.weights[o.outputs[0]] = val
                tensors[o.outputs[0]] = MobTensor(o.outputs[0], val)
                const.add(o.outputs[0])
            else:
                kept.append(o)
    used = {n for o in kept for n in o.inputs} | set(model.outputs)
    return MobModel(model.inputs, model.outputs, kept, {k: v for k, v in tensors.items() if k in used},
                    dict(model.metadata, constants_folded=len(model.operators) - len(kept)))


def quantize_weights(model: MobModel, mode: str = "int8") -> MobModel:
    """Stores conv / fc weights as int8 / uint8 (per tensor, affine) or fp16; biases and norm parameters stay fp32."""
    weight_names = {o.inputs[1] for o in model.operators if o.type in ("conv2d", "fully_connected")}
    new = {}
    for n, t in model.tensors.items():
        d = t.data
        if n not in weight_names or t.scale is not None:
            new[n] = t
        elif mode == "fp16":
            new[n] = MobTensor(n, d.half())
        elif mode == "int8":
            s = float(d.abs().max()) / 127.0 or 1.0
            new[n] = MobTensor(n, torch.round(d / s).clamp(-127, 127).to(torch.int8), s, 0)
        elif mode == "uint8":
            lo, hi = float(d.min()), float(d.max())
            s = (hi - lo) / 255.0 or 1.0
            zp = int(round(-lo / s))
            new[n] = MobTensor(n, (torch.round(d / s) + zp).clamp(0, 255).to(torch.uint8), s, zp)
        else:
            raise ValueError(f"unknown quantisation mode {mode!r}")
    return MobModel(model.inputs, model.outputs, model.operators, new, dict(model.metadata, quantization=mode))


def convert(in_path: str, out_path: str, quantize: Optional[str] = None, verbose: bool = False) -> MobModel:
    """``in_path``: a ``torch.save``'d ``{"model": nn.Sequential, "input_shape": [...]}`` or an existing ``.mob``."""
    if in_path.endswith(".mob"):
        m = load_mob(in_path)
    else:
        obj = torch.load(in_path, weights_only=False)
        m = convert_sequential(obj["model"].eval(), obj["input_shape"])
    n0 = len(m.operators)
    m = optimize(fold_constants(m))
    if quantize:
        m = quantize_weights(m, quantize)
    errs = m.validate()
    if errs:
        raise ValueError("; ".join(errs))
    save_mob(m, out_path)
    if verbose:
        print(f"{in_path} -> {out_path}: {n0} -> {len(m.operators)} operators, {len(m.tensors)} tensors, quantization={quantize}")
    return m
