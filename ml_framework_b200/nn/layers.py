"""Neural-network layers on ``torch.nn.Module`` whose forward/backward run the native kernels
for bf16 CUDA tensors (see :mod:`ml_framework_b200.ops.functional`) and plain PyTorch otherwise.

Module / Parameter containers are PyTorch's; they provide what the reference's ``Module``
(src/MLFramework/NN/Module.cs:10-56: Forward, GetParameters, GetNamedParameters,
SetRequiresGrad), ``Parameter`` gradient hooks (NN/Parameter.cs:41) and ``SequentialModule``
offer. ``Linear`` keeps the reference's weight layout ``[out, in]`` and Kaiming init
(src/MLFramework/Modules/Linear.cs:81-164).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as Fm


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype=None, device=None,
                 init_std: Optional[float] = None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        self.init_std = init_std
        self.reset_parameters()

    def reset_parameters(self):
        with torch.no_grad():
            if self.init_std is not None:
                self.weight.normal_(0.0, self.init_std)
            else:
                nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
            if self.bias is not None:
                self.bias.zero_()

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        return Fm.linear(x, self.weight, self.bias, residual)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))

    def forward(self, x):
        return Fm.layer_norm(x, self.weight, self.bias, self.eps)

    def with_skip(self, x):
        """``(norm(x), x)``: use the second value as the residual of the branch so that the backward adds the two
        gradients of x inside the normalisation's kernel."""
        return Fm.layer_norm_skip(x, self.weight, self.bias, self.eps)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x):
        return Fm.rms_norm(x, self.weight, self.eps)

    def with_skip(self, x):
        return Fm.rms_norm_skip(x, self.weight, self.eps)


class Embedding(nn.Module):
    """Token (+ optional learned position) embedding."""

    def __init__(self, num_embeddings: int, dim: int, max_positions: int = 0, dtype=None, device=None,
                 init_std: float = 0.02):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_embeddings, dim, dtype=dtype, device=device).normal_(0, init_std))
        self.pos_weight = (nn.Parameter(torch.empty(max_positions, dim, dtype=dtype, device=device).normal_(0, init_std))
                           if max_positions > 0 else None)

    def forward(self, ids: torch.Tensor, positions: Optional[torch.Tensor] = None):
        if self.pos_weight is not None and positions is None:
            positions = torch.arange(ids.shape[-1], device=ids.device).expand_as(ids)
        return Fm.embedding(ids, self.weight, positions if self.pos_weight is not None else None, self.pos_weight)


class GeluMLP(nn.Module):
    """fc1 -> tanh-GELU -> fc2 (GPT). The residual add is fused into fc2's epilogue."""

    def __init__(self, dim: int, hidden: int, dtype=None, device=None, init_std=0.02, out_init_std=None):
        super().__init__()
        self.fc1 = Linear(dim, hidden, True, dtype, device, init_std)
        self.fc2 = Linear(hidden, dim, True, dtype, device, out_init_std or init_std)

    def forward(self, x, residual=None):
        return Fm.mlp_gelu(x, self.fc1.weight, self.fc1.bias, self.fc2.weight, self.fc2.bias, residual)


class SwiGLUMLP(nn.Module):
    """(silu(x Wg) * x Wu) Wd (Llama). Gate and up projections live interleaved in one weight."""

    def __init__(self, dim: int, hidden: int, dtype=None, device=None, init_std=0.02, out_init_std=None):
        super().__init__()
        self.hidden = hidden
        self.gate_up = Linear(dim, 2 * hidden, False, dtype, device, init_std)   # row 2i gate_i, 2i+1 up_i
        self.down = Linear(hidden, dim, False, dtype, device, out_init_std or init_std)

    def forward(self, x, residual=None):
        return Fm.mlp_swiglu(x, self.gate_up.weight, self.down.weight, residual)

    @staticmethod
    def interleave(gate_w: torch.Tensor, up_w: torch.Tensor) -> torch.Tensor:
        return torch.stack([gate_w, up_w], dim=1).reshape(-1, gate_w.shape[1])


class SelfAttention(nn.Module):
    """Packed-QKV causal self-attention with optional GQA and RoPE; o-projection fuses the residual."""

    def __init__(self, dim: int, n_heads: int, n_kv_heads: Optional[int] = None, head_dim: Optional[int] = None,
                 bias: bool = True, rope_theta: Optional[float] = None, causal: bool = True, dtype=None, device=None,
                 init_std=0.02, out_init_std=None):
        super().__init__()
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads or n_heads
        self.head_dim = head_dim or dim // n_heads
        self.rope_theta, self.causal = rope_theta, causal
        qkv_out = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
        self.qkv = Linear(dim, qkv_out, bias, dtype, device, init_std)
        self.proj = Linear(self.n_heads * self.head_dim, dim, bias, dtype, device, out_init_std or init_std)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, positions=None):
        B, S, _ = x.shape
        qkv = self.qkv(x)
        a = Fm.attention_packed(qkv.reshape(B * S, -1), B, S, self.n_heads, self.n_kv_heads, self.head_dim, self.causal,
                                self.rope_theta, positions)
        return self.proj(a.view(B, S, -1), residual)


class Sequential(nn.Sequential):
    """``SequentialModule`` (src/MLFramework/NN/SequentialModule.cs)."""


class ReLU(nn.ReLU):
    pass
