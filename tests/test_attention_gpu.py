"""tcgen05 attention forward/backward against an fp32 PyTorch reference."""
import pytest
import torch

from ml_framework_b200.ops import native
from ml_framework_b200.ops.reference import attention_ref

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


@pytest.mark.parametrize("B,S,Hq,Hkv,causal", [(1, 128, 1, 1, True), (2, 256, 4, 4, True), (1, 320, 4, 2, True),
                                              (2, 200, 2, 2, False), (1, 1024, 8, 2, True)])
def test_flash_fwd(B, S, Hq, Hkv, causal):
    torch.manual_seed(0)
    D = 128
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
    q = qkv[:, :Hq * D].view(B * S, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(B * S, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(B * S, Hkv, D)
    out, lse = native.flash_fwd(q, k, v, B, S, causal=causal)
    ref, ref_lse = attention_ref(q.reshape(B, S, Hq, D), k.reshape(B, S, Hkv, D), v.reshape(B, S, Hkv, D), causal=causal)
    torch.cuda.synchronize()
    assert _rel(out.view(B, S, Hq, D), ref) < 2e-2
    assert (lse - ref_lse).abs().max().item() < 2e-2


@pytest.mark.parametrize("ws", [0, 1])
@pytest.mark.parametrize("B,S,Hq,Hkv,causal,amp", [(2, 256, 2, 2, True, 1.0), (1, 384, 2, 1, False, 1.0), (1, 320, 4, 2, True, 1.0),
                                                  (1, 2048, 4, 2, True, 1.0), (1, 1024, 2, 2, True, 4.0), (1, 1000, 2, 2, False, 4.0)])
def test_flash_fwd_kernel_variants(ws, B, S, Hq, Hkv, causal, amp):
    """Both forward kernels (single tile; two tiles ping-ponged with P in tensor memory) on the same inputs.
    ``amp`` scales Q so that row maxima grow quickly along the keys and the lazy rescale of O runs."""
    from ml_framework_b200 import _lib
    torch.manual_seed(2)
    D = 128
    q = (torch.randn(B * S, Hq, D, device="cuda") * amp).to(torch.bfloat16)
    k = torch.randn(B * S, Hkv, D, device="cuda").to(torch.bfloat16)
    v = torch.randn(B * S, Hkv, D, device="cuda").to(torch.bfloat16)
    _lib.get().mlf_set_flash_ws(ws)
    try:
        out, lse = native.flash_fwd(q, k, v, B, S, causal=causal)
        torch.cuda.synchronize()
    finally:
        _lib.get().mlf_set_flash_ws(1)
    ref, ref_lse = attention_ref(q.reshape(B, S, Hq, D), k.reshape(B, S, Hkv, D), v.reshape(B, S, Hkv, D), causal=causal)
    assert _rel(out.view(B, S, Hq, D), ref) < 2e-2
    assert (lse - ref_lse).abs().max().item() < 2e-2


@pytest.mark.parametrize("ws", [1, 0])
@pytest.mark.parametrize("B,S,Hq,Hkv,causal", [(1, 128, 1, 1, True), (2, 256, 4, 4, True), (1, 320, 4, 2, True),
                                              (1, 200, 2, 2, False), (1, 1024, 4, 2, True), (2, 640, 2, 1, False)])
def test_flash_bwd(ws, B, S, Hq, Hkv, causal):
    """Both backward kernels (128 x 64 tiles; 128 x 128 tiles with warpgroup roles) against autograd in fp32."""
    from ml_framework_b200 import _lib
    _lib.get().mlf_set_flash_bwd_ws(ws)
    try:
        _flash_bwd_case(B, S, Hq, Hkv, causal)
    finally:
        _lib.get().mlf_set_flash_bwd_ws(1)


def _flash_bwd_case(B, S, Hq, Hkv, causal):
    torch.manual_seed(1)
    D = 128
    q = torch.randn(B * S, Hq, D, device="cuda").to(torch.bfloat16)
    k = torch.randn(B * S, Hkv, D, device="cuda").to(torch.bfloat16)
    v = torch.randn(B * S, Hkv, D, device="cuda").to(torch.bfloat16)
    do = torch.randn(B * S, Hq, D, device="cuda").to(torch.bfloat16)
    out, lse = native.flash_fwd(q, k, v, B, S, causal=causal)
    dq, dk, dv = native.flash_bwd(q, k, v, out, do, lse, B, S, causal=causal)
    qf = q.float().reshape(B, S, Hq, D).requires_grad_()
    kf = k.float().reshape(B, S, Hkv, D).requires_grad_()
    vf = v.float().reshape(B, S, Hkv, D).requires_grad_()
    ref, _ = attention_ref(qf, kf, vf, causal=causal)
    ref.backward(do.float().reshape(B, S, Hq, D))
    torch.cuda.synchronize()
    assert _rel(dv.view(B, S, Hkv, D), vf.grad) < 3e-2
    assert _rel(dk.view(B, S, Hkv, D), kf.grad) < 3e-2
    assert _rel(dq.view(B, S, Hq, D), qf.grad) < 3e-2


@pytest.mark.parametrize("B,Sq,Skv,Hq,Hkv", [(1, 64, 64 + 512, 4, 2), (2, 200, 712, 2, 2), (1, 300, 300, 4, 1), (1, 17, 1041, 8, 2)])
def test_flash_fwd_prefix(B, Sq, Skv, Hq, Hkv):
    """A chunk of queries at the end of a longer key / value sequence (chunked prefill over a cached prefix)."""
    torch.manual_seed(2)
    D = 128
    q = torch.randn(B * Sq, Hq, D, device="cuda").to(torch.bfloat16)
    k = torch.randn(B * Skv, Hkv, D, device="cuda").to(torch.bfloat16)
    v = torch.randn(B * Skv, Hkv, D, device="cuda").to(torch.bfloat16)
    out = native.flash_fwd_prefix(q, k, v, B, Sq, Skv, causal=True)
    ref, _ = attention_ref(q.view(B, Sq, Hq, D), k.view(B, Skv, Hkv, D), v.view(B, Skv, Hkv, D), causal=True, start_pos=Skv - Sq)
    torch.cuda.synchronize()
    assert _rel(out.view(B, Sq, Hq, D), ref) < 2e-2
