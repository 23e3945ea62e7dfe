"""Allocation-free column sum, called through its exported C symbol and compared with the
caller-buffer entry point on two calls in a row (the second call sees the first call's leftovers in
the built-in work buffer)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sym():
    from ml_framework_b200 import _lib
    lib = _lib.get()
    fn = lib.mlf_colsum_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_longlong, C.c_int, C.c_uint64]
    lib.mlf_colsum_static_max_cols.restype = C.c_int
    lib.mlf_colsum_static_setup.restype = C.c_int
    return lib, fn


def test_colsum_static_matches_caller_buffer_entry_point():
    from ml_framework_b200 import _lib
    from ml_framework_b200.ops import native
    lib, fn = _sym()
    torch.cuda.set_device(0)
    assert lib.mlf_colsum_static_setup() == 0, _lib.last_error() if hasattr(_lib, "last_error") else "setup failed"
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(7)
    # second call: fewer columns and other data, so stale sums from the first call would show
    for (M, N) in [(4096, 2048), (1000, 1000)]:
        pitch = (N + 7) // 8 * 8
        buf = torch.randn(M, pitch, device="cuda", dtype=torch.float32, generator=g).to(torch.bfloat16)
        dy = buf[:, :N]
        out = torch.empty(N, device="cuda", dtype=torch.bfloat16)
        rc = fn(out.data_ptr(), dy.data_ptr(), M, N, dy.stride(0), 0, st)
        assert rc == 0
        want = native.colsum(dy)
        ref = dy.float().sum(0)
        torch.cuda.synchronize()
        assert torch.allclose(out.float(), want.float(), rtol=2e-2, atol=2e-2 * ref.abs().max().item())
        assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item())
        # accumulate form: db += column sums
        rc = fn(out.data_ptr(), dy.data_ptr(), M, N, dy.stride(0), 1, st)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.allclose(out.float(), 2 * ref, rtol=3e-2, atol=3e-2 * ref.abs().max().item())


def test_colsum_static_rejects_oversize():
    lib, fn = _sym()
    n_max = lib.mlf_colsum_static_max_cols()
    assert n_max == 65536
    x = torch.zeros(8, 8, device="cuda", dtype=torch.bfloat16)
    rc = fn(x.data_ptr(), x.data_ptr(), 8, n_max + 8, n_max + 8, 0, 0)
    assert rc != 0
    lib.mlf_last_error.restype = C.c_char_p
    assert b"exceeds" in lib.mlf_last_error()
