"""tcgen05 GEMM against an fp32 PyTorch statement of the same product and epilogue."""
import pytest
import torch

from ml_framework_b200 import _lib
from ml_framework_b200.ops.gemm import gemm, gemm_reference

pytestmark = pytest.mark.gpu


def _mk(rows, k, mn, dev, scale=1.0):
    shape = (k, rows) if mn else (rows, k)
    return (torch.randn(shape, device=dev, dtype=torch.float32) * scale).to(torch.bfloat16)


def _check(out, ref, k):
    out = out.float()
    tol = 2e-2 * (k ** 0.5) * 0.05 + 2e-2
    err = (out - ref).abs().max().item()
    rel = err / (ref.abs().max().item() + 1e-6)
    assert rel < 1.5e-2 or err < tol, f"max abs err {err}, rel {rel}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_layouts(a_mn, b_mn, tile_n):
    torch.manual_seed(0)
    M, N, K = 384, 512, 320
    a = _mk(M, K, a_mn, "cuda")
    b = _mk(N, K, b_mn, "cuda")
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, tile_n=tile_n)
    ref, _ = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    _check(out, ref, K)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (200, 264, 72), (1000, 1336, 520), (8, 64, 4096), (2048, 2048, 2048)])
def test_shapes_and_tails(M, N, K):
    torch.manual_seed(1)
    a = _mk(M, K, False, "cuda")
    b = _mk(N, K, False, "cuda")
    out = gemm(a, b)
    ref, _ = gemm_reference(a, b)
    _check(out, ref, K)


def test_epilogues():
    torch.manual_seed(2)
    M, N, K = 512, 768, 256
    a = _mk(M, K, False, "cuda")
    b = _mk(N, K, False, "cuda", 0.1)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    # bias + gelu with the pre-activation stored
    pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b, bias=bias, aux_out=pre, flags=_lib.EPI_GELU | _lib.EPI_STORE_PRE)
    ref, refpre = gemm_reference(a, b, bias=bias, flags=_lib.EPI_BIAS | _lib.EPI_GELU)
    _check(out, ref, K)
    _check(pre, refpre, K)
    # bias + residual
    out = gemm(a, b, bias=bias, aux_in=res, flags=_lib.EPI_RESIDUAL)
    ref, _ = gemm_reference(a, b, bias=bias, aux_in=res, flags=_lib.EPI_BIAS | _lib.EPI_RESIDUAL)
    _check(out, ref, K)
    # dgelu multiply
    out = gemm(a, b, aux_in=res, flags=_lib.EPI_DGELU_MUL)
    ref, _ = gemm_reference(a, b, aux_in=res, flags=_lib.EPI_DGELU_MUL)
    _check(out, ref, K)
    # fp32 out with accumulation
    acc = torch.randn(M, N, device="cuda")
    acc0 = acc.clone()
    gemm(a, b, out=acc, flags=_lib.EPI_ACCUM, out_dtype=torch.float32, alpha=0.5)
    ref, _ = gemm_reference(a, b, flags=_lib.EPI_ACCUM, alpha=0.5, prev_out=acc0)
    _check(acc, ref, K)
    # swiglu and its derivative
    out = gemm(a, b, flags=_lib.EPI_SWIGLU)
    ref, _ = gemm_reference(a, b, flags=_lib.EPI_SWIGLU)
    assert out.shape == (M, N // 2)
    _check(out, ref, K)
    gu = torch.randn(M, 2 * N, device="cuda").to(torch.bfloat16)
    out = gemm(a, b, aux_in=gu, flags=_lib.EPI_DSWIGLU)
    ref, _ = gemm_reference(a, b, aux_in=gu, flags=_lib.EPI_DSWIGLU)
    assert out.shape == (M, 2 * N)
    _check(out, ref, K)


@pytest.mark.parametrize("tile_n", [256, 512])
def test_gather_and_scatter_emulated_ranks(tile_n):
    """The fused-communication paths with every 'peer' buffer on this GPU: one launch, copy
    CTAs and compute CTAs of the same grid, as the multi-GPU path runs them. tile_n 512 is the
    CTA-pair kernel."""
    import ctypes as C
    torch.manual_seed(3)
    W = 4
    M, N, K = 1024, 1024, 512
    a = _mk(M, K, False, "cuda")
    b = _mk(N, K, False, "cuda", 0.1)
    ref, _ = gemm_reference(a, b)
    for operand in (1, 2):
        full = a if operand == 1 else b
        rows = full.shape[0]
        shards = [full[r * rows // W:(r + 1) * rows // W].clone() for r in range(W)]
        gathered = torch.zeros_like(full)
        flag_rows = 256
        flags = torch.zeros(rows // flag_rows, dtype=torch.int32, device="cuda")
        counters = torch.zeros_like(flags)
        cm = _lib.GemmComm()
        cm.gather_operand, cm.world, cm.rank, cm.n_copy_ctas = operand, W, 1, 8
        cm.rows_per_rank, cm.flag_rows, cm.row_bytes = rows // W, flag_rows, K * 2
        for r in range(W):
            cm.src[r] = shards[r].data_ptr()
        cm.gathered, cm.flags, cm.counters = gathered.data_ptr(), flags.data_ptr(), counters.data_ptr()
        if operand == 1:
            out = gemm(shards[1], b, comm=cm, m_override=M, tile_n=tile_n)
        else:
            out = gemm(a, shards[1], comm=cm, n_override=N, tile_n=tile_n)
        torch.cuda.synchronize()
        assert torch.equal(gathered, full)
        _check(out, ref, K)
    # scatter: rows routed to per-owner partial buffers [W, rows_per_owner, N]
    parts = [torch.zeros(W, M // W, N, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    cm = _lib.GemmComm()
    cm.scatter_out, cm.rows_per_owner, cm.world, cm.rank = 1, M // W, W, 2
    for r in range(W):
        cm.out_peer[r] = parts[r].data_ptr()
    dummy = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    gemm(a, b, out=dummy, comm=cm, tile_n=tile_n)
    torch.cuda.synchronize()
    for r in range(W):
        _check(parts[r][2], ref[r * (M // W):(r + 1) * (M // W)], K)
        assert parts[r][0].abs().max().item() == 0


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_cta_pair_kernel(a_mn, b_mn):
    """tile_n=512 selects the 256 x 256 CTA-pair (cta_group::2) kernel."""
    torch.manual_seed(5)
    M, N, K = 1280, 768, 448
    a = _mk(M, K, a_mn, "cuda")
    b = _mk(N, K, b_mn, "cuda", 0.1)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, tile_n=512, bias=bias, flags=_lib.EPI_GELU)
    ref, _ = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, flags=_lib.EPI_BIAS | _lib.EPI_GELU)
    torch.cuda.synchronize()
    _check(out, ref, K)
    # odd sizes: M and N tails inside a pair tile
    a = _mk(1000, 320, False, "cuda")
    b = _mk(600, 320, False, "cuda")
    out = gemm(a, b, tile_n=512)
    ref, _ = gemm_reference(a, b)
    _check(out, ref, 320)


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(4096, 512, 8192, True, True), (768, 4096, 8192, True, True), (1024, 1024, 4096, False, False),
                                            (520, 1000, 2112, False, True)])
def test_split_k_and_accumulate_pair_kernel(M, N, K, a_mn, b_mn):
    """Few tiles and a long K: the CTA-pair kernel splits K and the splits meet in `out` through TMA reduction
    stores; with the accumulate flag the product is added to what `out` held."""
    torch.manual_seed(4)
    a = _mk(M, K, a_mn, "cuda", 0.25)
    b = _mk(N, K, b_mn, "cuda", 0.25)
    ref, _ = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    _check(out, ref, K)
    prev = (torch.randn(M, N, device="cuda") * ref.abs().mean()).to(torch.bfloat16)
    out2 = prev.clone()
    gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out2, flags=_lib.EPI_ACCUM)
    torch.cuda.synchronize()
    _check(out2, ref + prev.float(), K)


@pytest.mark.parametrize("route", ["fewrow", "split_k"])
@pytest.mark.parametrize("M,N,K", [(8, 4096, 4096), (33, 1096, 4096), (64, 6144, 4096), (100, 28672, 1024), (128, 4096, 14336),
                                   (200, 1024, 14336), (256, 3584, 4096)])
def test_few_rows_split_k(M, N, K, route):
    """A decode-step product (few rows, a large weight): up to 128 rows take the weight-as-M stream-K kernel, more rows
    (or that route switched off) the split-K CTA-pair route; also as an accumulation into the residual stream."""
    torch.manual_seed(6)
    _lib.get().mlf_set_gemm_fewrow(1 if route == "fewrow" else 0)
    try:
        _few_rows_case(M, N, K)
    finally:
        _lib.get().mlf_set_gemm_fewrow(1)


def _few_rows_case(M, N, K):
    a = _mk(M, K, False, "cuda", 0.25)
    b = _mk(N, K, False, "cuda", 0.25)
    ref, _ = gemm_reference(a, b)
    out = gemm(a, b)
    torch.cuda.synchronize()
    _check(out, ref, K)
    x = (torch.randn(M, N, device="cuda") * ref.abs().mean()).to(torch.bfloat16)
    x0 = x.clone()
    gemm(a, b, out=x, flags=_lib.EPI_ACCUM)
    torch.cuda.synchronize()
    _check(x, ref + x0.float(), K)
    assert _lib.read_status() == 0
