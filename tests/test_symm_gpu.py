"""Peer-memory collectives with every "rank" buffer on one GPU (the kernels that move data never
wait on other ranks, so W emulated ranks can run one after the other)."""
import ctypes as C

import pytest
import torch

from ml_framework_b200 import _lib
from ml_framework_b200.dist.symm import SymmetricMemory, make_copy_segs, make_reduce_segs
from ml_framework_b200.ops.gemm import gemm, gemm_reference

pytestmark = pytest.mark.gpu


def test_reduce_scatter_with_unscale_and_overflow_flag():
    W, n = 4, 8 * 1000
    sm = SymmetricMemory(emulate_world=W)
    bufs = sm.alloc_emulated(n * 2)
    torch.manual_seed(0)
    data = [torch.randn(n, device="cuda").to(torch.bfloat16) for _ in range(W)]
    for r in range(W):
        bufs[r].view(torch.bfloat16, n).copy_(data[r])
    total = torch.stack([d.float() for d in data]).sum(0)
    per = n // W
    inv = torch.tensor(0.5, device="cuda")
    for r in range(W):
        out = torch.zeros(per, device="cuda")
        found = torch.zeros(1, dtype=torch.int32, device="cuda")
        ss = torch.zeros(1, device="cuda")
        segs = make_reduce_segs([(r * per, 0, per)], "cuda")
        sm.rs_reduce(bufs[r], segs, 1, out, per, rank=r, scale=0.25, scale_ptr=inv, found_inf=found, sumsq=ss)
        want = total[r * per:(r + 1) * per] * 0.125
        assert torch.allclose(out, want, atol=1e-5)
        assert found.item() == 0 and abs(ss.item() - want.pow(2).sum().item()) < 1e-2 * want.pow(2).sum().item()
    bufs[2].view(torch.bfloat16, n)[5] = float("inf")
    out = torch.zeros(per, device="cuda", dtype=torch.bfloat16)
    found = torch.zeros(1, dtype=torch.int32, device="cuda")
    sm.rs_reduce(bufs[0], make_reduce_segs([(0, 0, per)], "cuda"), 1, out, per, rank=0, found_inf=found)
    assert found.item() == 1
    sm.close()


def test_all_reduce_two_shot_and_one_shot():
    W, n = 4, 8 * 4096
    sm = SymmetricMemory(emulate_world=W)
    bufs = sm.alloc_emulated(n * 2)
    data = [torch.randn(n, device="cuda").to(torch.bfloat16) for _ in range(W)]
    want = torch.stack([d.float() for d in data]).sum(0)
    for r in range(W):
        bufs[r].view(torch.bfloat16, n).copy_(data[r])
    res = torch.randn(n, device="cuda").to(torch.bfloat16)
    out = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    sm.all_reduce_one_shot(bufs[1], out, n, residual=res, rank=1)
    assert torch.allclose(out.float(), want + res.float(), atol=0.1, rtol=2e-2)
    for r in range(W):
        sm.all_reduce_two_shot(bufs[r], n, scale=1.0 / W, rank=r)
    for r in range(W):
        assert torch.allclose(bufs[r].view(torch.bfloat16, n).float(), want / W, atol=0.05, rtol=2e-2)
    sm.close()


def test_gemm_with_piggybacked_copies_and_partial_sum():
    torch.manual_seed(1)
    M, N, K = 512, 512, 256
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
    src = [torch.randn(100_000 * 8, device="cuda").to(torch.bfloat16) for _ in range(3)]
    dst = [torch.zeros_like(s) for s in src]
    segs = make_copy_segs([(s.data_ptr(), d.data_ptr(), s.numel() * 2) for s, d in zip(src, dst)], "cuda")
    cm = _lib.GemmComm()
    cm.n_copy_ctas, cm.extra_segs, cm.n_extra = 6, segs.data_ptr(), 3
    out = gemm(a, b, comm=cm)
    ref, _ = gemm_reference(a, b)
    torch.cuda.synchronize()
    assert all(torch.equal(s, d) for s, d in zip(src, dst))
    assert (out.float() - ref).abs().max().item() < 0.05 * ref.abs().max().item()
    # standalone peer copy
    dst2 = [torch.zeros_like(s) for s in src]
    sm = SymmetricMemory(emulate_world=1)
    sm.peer_copy(make_copy_segs([(s.data_ptr(), d.data_ptr(), s.numel() * 2) for s, d in zip(src, dst2)], "cuda"), 3)
    assert all(torch.equal(s, d) for s, d in zip(src, dst2))
    # sum of W partial planes + bias + residual
    W, rows, cols = 4, 96, 256
    part = torch.randn(W, rows, cols, device="cuda").to(torch.bfloat16)
    bias = torch.randn(cols, device="cuda").to(torch.bfloat16)
    res = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    o = torch.empty(rows, cols, device="cuda", dtype=torch.bfloat16)
    rc = _lib.get().mlf_sum_partials(C.c_void_p(part.data_ptr()), W, C.c_longlong(rows), cols, C.c_void_p(o.data_ptr()),
                                     C.c_longlong(cols), C.c_void_p(bias.data_ptr()), C.c_void_p(res.data_ptr()),
                                     C.c_longlong(cols), C.c_uint64(_lib.stream_handle()))
    _lib.check(rc)
    want = part.float().sum(0) + bias.float() + res.float()
    assert torch.allclose(o.float(), want, atol=0.1, rtol=2e-2)
