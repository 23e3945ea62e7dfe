"""Tensor-parallel kernels that can be checked on one GPU: the vocabulary-parallel cross-entropy with both "ranks"
run one after the other (their statistics exchanged through plain device buffers), and the one-rank path through the
public function."""
import ctypes as C

import pytest
import torch
import torch.nn.functional as F

from ml_framework_b200 import _lib
from ml_framework_b200.parallel import tensor_parallel as tpm

pytestmark = pytest.mark.gpu


def _reference(logits_full, targets, vocab, scale):
    lg = logits_full[:, :vocab].float().clone().requires_grad_()
    loss = F.cross_entropy(lg, targets, ignore_index=-100, reduction="sum") / targets.numel()
    loss.backward()
    return loss.item(), lg.grad * scale


@pytest.mark.parametrize("T,Vl,vocab", [(300, 1024, 2000), (64, 16128, 128256 // 4)])
def test_vocab_parallel_cross_entropy_two_emulated_ranks(T, Vl, vocab):
    W = 2
    vocab = min(vocab, W * Vl - 5)
    torch.manual_seed(0)
    full = (torch.randn(T, W * Vl, device="cuda") * 3).to(torch.bfloat16)
    tg = torch.randint(0, vocab, (T,), device="cuda")
    tg[3] = -100
    scale_t = torch.tensor(8.0, device="cuda")
    ref_loss, ref_grad = _reference(full, tg, vocab, 8.0)
    lib = _lib.get()
    st = lambda: C.c_uint64(_lib.stream_handle())  # noqa: E731
    shards = [full[:, r * Vl:(r + 1) * Vl].contiguous() for r in range(W)]
    stats = [torch.empty(T, 4, device="cuda") for _ in range(W)]
    for r in range(W):
        _lib.check(lib.mlf_vp_ce_stats(C.c_void_p(shards[r].data_ptr()), C.c_longlong(Vl), Vl, C.c_void_p(tg.data_ptr()), T,
                                       C.c_longlong(r * Vl), C.c_longlong(vocab), C.c_void_p(stats[r].data_ptr()), st()))
    table = (C.c_void_p * 8)(*[C.c_void_p(s.data_ptr()) for s in stats] + [None] * 6)
    for r in range(W):
        loss_sum = torch.zeros((), device="cuda")
        rows = torch.empty(T, device="cuda")
        _lib.check(lib.mlf_vp_ce_grad(C.c_void_p(shards[r].data_ptr()), C.c_longlong(Vl), Vl, C.c_void_p(tg.data_ptr()), T,
                                      C.c_longlong(r * Vl), C.c_longlong(vocab), table, None, None, W, r, 0, C.c_void_p(rows.data_ptr()),
                                      C.c_void_p(loss_sum.data_ptr()), C.c_float(1.0 / T), C.c_void_p(scale_t.data_ptr()),
                                      C.c_float(1.0 / T), st()))
        assert abs(loss_sum.item() - ref_loss) < 2e-3 * abs(ref_loss)
        assert rows[3].item() == 0.0
        want = torch.zeros(T, Vl, device="cuda")
        lo, hi = r * Vl, min((r + 1) * Vl, vocab)
        if hi > lo:
            want[:, :hi - lo] = ref_grad[:, lo:hi]
        got = shards[r].float()
        assert torch.allclose(got, want, atol=2e-3 * 8.0 / T + 1e-6, rtol=2e-2), (got - want).abs().max()


def test_vocab_parallel_lm_loss_single_rank_matches_dense_head():
    tp = tpm.TPContext(None)
    T, D, V = 256, 128, 1000
    torch.manual_seed(1)
    h = (torch.randn(T, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(1024, D, device="cuda") * 0.2).to(torch.bfloat16).requires_grad_()
    tg = torch.randint(0, V, (T,), device="cuda")
    loss = tpm.vocab_parallel_lm_loss(h, w, tg, tp, V)
    loss.backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    ref = F.cross_entropy(F.linear(hr, wr)[:, :V], tg)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-2 * ref.item()
    assert torch.allclose(h.grad.float(), hr.grad, atol=2e-4, rtol=5e-2)
    assert torch.allclose(w.grad.float(), wr.grad, atol=2e-4, rtol=5e-2)
