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


def test_in_kernel_synchronised_reductions_single_rank():
    """World of one: the arrival / departure handshakes run against this rank's own signal pad, so the
    whole kernel (epoch bookkeeping included) is exercised on one GPU, several launches in a row."""
    sm = SymmetricMemory()
    n = 8 * 5000
    buf = sm.alloc(n * 2)
    flag = sm.alloc_flag()
    fl = flag.view(torch.int32, 1)
    x = torch.randn(n, device="cuda").to(torch.bfloat16)
    for it in range(3):
        buf.view(torch.bfloat16, n).copy_(x)
        out = torch.zeros(n // 2, device="cuda", dtype=torch.bfloat16)
        segs = make_reduce_segs([(n // 2, 0, n // 2)], "cuda")
        sm.rs_reduce_sync(buf, segs, 1, out, n // 2, scale=0.5, flag=flag, key="t")
        assert torch.allclose(out.float(), x[n // 2:].float() * 0.5, atol=1e-2, rtol=1e-2)
        sm.all_reduce_two_shot_sync(buf, n, scale=0.25, flag=flag, key="t")
        assert torch.allclose(buf.view(torch.bfloat16, n).float(), x.float() * 0.25, atol=1e-2, rtol=1e-2)
        assert fl.item() == 0
    # sum of partial planes with the arrival wait inside (world of one: a single plane), twice in a row
    rows, cols = 96, 256
    part = sm.alloc(rows * cols * 2)
    pv = part.view(torch.bfloat16, rows * cols).view(rows, cols)
    bias = torch.randn(cols, device="cuda").to(torch.bfloat16)
    res = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    for it in range(2):
        pv.copy_(torch.randn(rows, cols, device="cuda"))
        o = torch.empty(rows, cols, device="cuda", dtype=torch.bfloat16)
        sm.sum_partials_sync(part, rows, cols, o, bias, res)
        assert torch.allclose(o.float(), pv.float() + bias.float() + res.float(), atol=0.1, rtol=2e-2)
    buf.view(torch.bfloat16, n)[17] = float("nan")
    sm.all_reduce_two_shot_sync(buf, n, flag=flag, key="t")
    assert fl.item() == 1
    sm.check_status()
    sm.close()


def test_wait_on_a_silent_peer_runs_out_and_raises_timeout():
    """Emulated world of two on one GPU in which the "peer" never signals: with a small cycle budget the
    barrier kernel gives up, leaves ERR_WAIT_PEER_FLAG in the status word, and the host turns that into
    CommunicationTimeout; afterwards the context is intact and a barrier that is answered passes."""
    from ml_framework_b200.dist.process_group import CommunicationTimeout
    from ml_framework_b200.dist.symm import set_wait_budget_cycles
    lib = _lib.get()
    sm = SymmetricMemory(emulate_world=2)
    pads = sm.alloc_emulated(1024)
    set_wait_budget_cycles(2_000_000)
    try:
        _lib.check(lib.mlf_symm_barrier(pads[0].peer_table(), 0, 2, C.c_uint(1), C.c_uint64(_lib.stream_handle())))
        with pytest.raises(CommunicationTimeout):
            sm.check_status()
        assert _lib.read_status(True) == 0
        # the silent peer finally signals (written from the host side of the test), and the same wait passes
        pads[0].view(torch.int32, 256)[32] = 2
        _lib.check(lib.mlf_symm_barrier(pads[0].peer_table(), 0, 2, C.c_uint(2), C.c_uint64(_lib.stream_handle())))
        sm.check_status()
    finally:
        set_wait_budget_cycles(0)
    y = torch.ones(8, device="cuda") * 2
    assert y.sum().item() == 16.0
    sm.close()
