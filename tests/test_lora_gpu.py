"""LoRA on the GPU: the fused adapter path (second product accumulated into the base product's output by the GEMM
epilogue) against an fp32 statement of the same layer; merge / unmerge; injection into a model."""
import pytest
import torch
import torch.nn as nn

from ml_framework_b200.nn.layers import Linear
from ml_framework_b200.nn.lora import LoraConfig, LoraInjector, LoraLinear

pytestmark = pytest.mark.gpu


def _ref(x, w, b, a, bm, s):
    return x @ w.t() + (b if b is not None else 0) + (x @ bm.t()) @ a.t() * s


@pytest.mark.parametrize("rank,bias", [(8, True), (16, False), (64, True)])
def test_lora_linear_fused_forward_backward_matches_fp32(rank, bias):
    torch.manual_seed(0)
    M, K, N = 512, 256, 384
    base = Linear(K, N, bias=bias, dtype=torch.bfloat16, device="cuda")
    lora = LoraLinear(base, LoraConfig(rank=rank, alpha=2 * rank))
    with torch.no_grad():
        lora.lora_B.copy_((torch.randn(rank, K, device="cuda") * 0.05).to(torch.bfloat16))
        lora.lora_A.copy_((torch.randn(N, rank, device="cuda") * 0.05).to(torch.bfloat16))
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    y = lora(x)
    g = (torch.randn(M, N, device="cuda") * 0.1).to(torch.bfloat16)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    ar, br = lora.lora_A.detach().float().requires_grad_(), lora.lora_B.detach().float().requires_grad_()
    yr = _ref(xr, base.weight.detach().float(), base.bias.detach().float() if bias else None, ar, br, lora.scaling)
    yr.backward(g.float())
    tol = dict(atol=3e-2, rtol=3e-2)
    assert torch.allclose(y.float(), yr, **tol)
    assert torch.allclose(x.grad.float(), xr.grad, **tol)
    assert torch.allclose(lora.lora_A.grad.float(), ar.grad, atol=5e-2, rtol=5e-2)
    assert torch.allclose(lora.lora_B.grad.float(), br.grad, atol=5e-2, rtol=5e-2)
    assert base.weight.grad is None                     # the base layer stays frozen
    # merge: same function with the adapter folded into the weight; unmerge restores the weight
    w0 = base.weight.detach().clone()
    lora.merge()
    ym = lora(x.detach())
    assert torch.allclose(ym.float(), yr.detach(), atol=6e-2, rtol=6e-2)
    lora.unmerge()
    assert torch.allclose(base.weight.float(), w0.float(), atol=2e-2)


def test_lora_injection_trains_only_the_adapters():
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = Linear(128, 128, dtype=torch.bfloat16, device="cuda")
            self.other = Linear(128, 64, dtype=torch.bfloat16, device="cuda")

        def forward(self, x):
            return self.other(self.q_proj(x))
    torch.manual_seed(1)
    net = Net()
    n = LoraInjector.inject(net, LoraConfig(rank=8, target_modules=("q_proj",)))
    assert n == ["q_proj"] and isinstance(net.q_proj, LoraLinear)
    for p in net.other.parameters():
        p.requires_grad_(False)
    x = torch.randn(64, 128, device="cuda").to(torch.bfloat16)
    tgt = torch.randn(64, 64, device="cuda")
    params = [p for p in net.parameters() if p.requires_grad]
    assert len(params) == 2
    opt = torch.optim.SGD(params, lr=0.5)
    losses = []
    for _ in range(10):
        opt.zero_grad()
        loss = (net(x).float() - tgt).pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
