"""Bandwidth-bound kernels (norms, activations, optimizer, AMP, loss, embedding, RoPE) against
plain fp32 PyTorch statements of the same operations."""
import pytest
import torch

from ml_framework_b200.ops import native
from ml_framework_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _close(a, b, tol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert err <= tol * (b.abs().max().item() + 1e-3), f"max err {err} vs scale {b.abs().max().item()}"


@pytest.mark.parametrize("D", [256, 2048, 4096, 5120])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_bwd(D, rms):
    torch.manual_seed(0)
    rows = 301
    x = (torch.randn(rows, D, device="cuda") * 2 + 0.5).to(torch.bfloat16)
    g = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16)
    b = None if rms else (0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16)
    dy = torch.randn(rows, D, device="cuda").to(torch.bfloat16)
    y, mean, rstd = native.norm_fwd(x, g, b, 1e-5, rms)
    xf = x.float().requires_grad_()
    gf = g.float().requires_grad_()
    if rms:
        yr, _ = ref.rms_norm_ref(xf, gf, 1e-5)
    else:
        bf = b.float().requires_grad_()
        yr, _, _ = ref.layer_norm_ref(xf, gf, bf, 1e-5)
    _close(y, yr)
    yr.backward(dy.float())
    dx, dg, db = native.norm_bwd(x, dy, g, mean, rstd, rms)
    _close(dx, xf.grad)
    _close(dg, gf.grad, 3e-2)
    if not rms:
        _close(db, bf.grad, 3e-2)
    # the gradient of a skip connection added inside the kernel
    skip = torch.randn(rows, D, device="cuda").to(torch.bfloat16)
    dx2, _, _ = native.norm_bwd(x, dy, g, mean, rstd, rms, dx_add=skip)
    _close(dx2, xf.grad + skip.float())


def test_elementwise_and_reduce():
    torch.manual_seed(1)
    for dt in (torch.float32, torch.bfloat16):
        a = torch.randn(100003, device="cuda").to(dt)
        b = (torch.rand(100003, device="cuda") + 0.5).to(dt)
        for op, f in (("add", torch.add), ("sub", torch.sub), ("mul", torch.mul), ("div", torch.div)):
            _close(native.ew_binary(op, a, b), f(a.float(), b.float()))
        _close(native.ew_binary("mul", a, 0.5), a.float() * 0.5)
        for op, f in (("relu", torch.relu), ("sigmoid", torch.sigmoid), ("tanh", torch.tanh)):
            _close(native.ew_unary(op, a), f(a.float()))
        _close(native.reduce_all("sum", a), a.float().sum(), 2e-2)
        _close(native.reduce_all("max", a), a.float().max(), 1e-6)
        _close(native.reduce_all("min", a), a.float().min(), 1e-6)
        _close(native.reduce_all("mean", b), b.float().mean(), 1e-3)
        t = torch.empty(1001, device="cuda", dtype=dt)
        native.fill_(t, 3.0)
        assert (t.float() == 3.0).all()


def test_swiglu_gelu_colsum():
    torch.manual_seed(2)
    rows, F = 257, 1024
    for inter in (False, True):
        gu = torch.randn(rows, 2 * F, device="cuda").to(torch.bfloat16)
        d = torch.randn(rows, F, device="cuda").to(torch.bfloat16)
        guf = gu.float().requires_grad_()
        o = ref.swiglu_ref(guf, inter)
        _close(native.swiglu_fwd(gu, inter), o)
        o.backward(d.float())
        _close(native.swiglu_bwd(d, gu, inter), guf.grad)
    x = torch.randn(rows, F, device="cuda").to(torch.bfloat16)
    d = torch.randn(rows, F, device="cuda").to(torch.bfloat16)
    xf = x.float().requires_grad_()
    torch.nn.functional.gelu(xf, approximate="tanh").backward(d.float())
    _close(native.gelu_bwd(d, x), xf.grad)
    dy = torch.randn(1000, 776, device="cuda").to(torch.bfloat16)
    _close(native.colsum(dy), dy.float().sum(0), 2e-2)


def test_adamw_and_scaler():
    torch.manual_seed(3)
    n = 100001
    p = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    inv = torch.tensor(0.5, device="cuda")
    found = torch.zeros(1, device="cuda", dtype=torch.int32)
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
    for step in (1, 2, 3):
        g = torch.randn(n, device="cuda").to(torch.bfloat16)
        native.adamw_(p, m, v, g, pb, step=step, inv_scale=inv, found_inf=found, **hp)
        pr, mr, vr = ref.adamw_ref(pr, mr, vr, g.float() * 0.5, step=step, **hp)
    _close(p, pr, 1e-4)
    _close(pb, pr, 1e-2)
    # a raised found_inf flag skips the step
    found.fill_(1)
    before = p.clone()
    native.adamw_(p, m, v, g, pb, step=4, inv_scale=inv, found_inf=found, **hp)
    assert torch.equal(before, p)
    # unscale + overflow detection + norm
    grad = torch.randn(5000, device="cuda")
    found.zero_()
    ss = torch.zeros(1, device="cuda")
    g2 = grad.clone()
    native.amp_unscale_check_(g2, found, inv_scale=inv, sumsq=ss)
    _close(g2, grad * 0.5, 1e-6)
    _close(ss, (grad * 0.5).pow(2).sum(), 1e-3)
    assert found.item() == 0
    g2[17] = float("inf")
    native.amp_unscale_check_(g2, found, inv_scale=inv)
    assert found.item() == 1
    # read-only check of bf16 gradients (vector loads): clean, then one inf, then one nan in the unaligned tail
    found.zero_()
    gb = torch.randn(100003, device="cuda").to(torch.bfloat16)
    ss2 = torch.zeros(1, device="cuda")
    native.amp_unscale_check_(gb, found, inv_scale=inv, sumsq=ss2, write_back=False)
    assert found.item() == 0
    _close(ss2, (gb.float() * 0.5).pow(2).sum(), 1e-3)
    for bad_at, val in ((4321, float("inf")), (100001, float("nan"))):
        gbad = gb.clone()
        gbad[bad_at] = val
        found.zero_()
        native.amp_unscale_check_(gbad, found, inv_scale=inv, write_back=False)
        assert found.item() == 1
    # dynamic loss-scale state machine: back off on overflow, grow after `interval` clean steps
    scale = torch.tensor(1024.0, device="cuda")
    tracker = torch.zeros(1, device="cuda", dtype=torch.int32)
    native.scaler_update_(scale, tracker, found, growth=2.0, backoff=0.5, interval=2, min_scale=1.0, max_scale=2.0 ** 24)
    assert scale.item() == 512.0 and found.item() == 0
    native.scaler_update_(scale, tracker, found, growth=2.0, backoff=0.5, interval=2, min_scale=1.0, max_scale=2.0 ** 24)
    native.scaler_update_(scale, tracker, found, growth=2.0, backoff=0.5, interval=2, min_scale=1.0, max_scale=2.0 ** 24)
    assert scale.item() == 1024.0


@pytest.mark.parametrize("T,V,ld", [(64, 1000, 1024), (33, 50257, 50304), (16, 128256, 128256)])
def test_cross_entropy(T, V, ld):
    torch.manual_seed(4)
    logits = (torch.randn(T, ld, device="cuda") * 3).to(torch.bfloat16)
    tg = torch.randint(0, V, (T,), device="cuda")
    tg[3] = -100
    loss_ref, d_ref = ref.cross_entropy_ref(logits, tg, V, grad_scale=0.25)
    work = logits.clone()
    loss_rows, loss_sum = native.cross_entropy_(work, tg, V, grad_scale=0.25, loss_weight=1.0 / T)
    _close(loss_rows, loss_ref, 1e-2)
    _close(loss_sum, loss_ref.sum() / T, 1e-2)
    _close(work, d_ref, 2e-2)
    assert work[:, V:].abs().max().item() == 0 if ld > V else True


def test_embedding_and_rope():
    torch.manual_seed(5)
    V, D, T = 1000, 256, 513
    wte = torch.randn(V, D, device="cuda").to(torch.bfloat16)
    wpe = torch.randn(600, D, device="cuda").to(torch.bfloat16)
    ids = torch.randint(0, V, (T,), device="cuda")
    pos = torch.arange(T, device="cuda")
    out = native.embedding_fwd(ids, wte, pos, wpe)
    _close(out, wte[ids].float() + wpe[pos].float())
    d = torch.randn(T, D, device="cuda").to(torch.bfloat16)
    dw = native.embedding_bwd(d, ids, V)
    r = torch.zeros(V, D, device="cuda")
    r.index_add_(0, ids, d.float())
    _close(dw, r, 1e-3)
    x = torch.randn(T, 4, 128, device="cuda").to(torch.bfloat16)
    want = ref.rope_ref(x, pos, 500000.0)
    got = native.rope_(x.clone(), pos, 500000.0)
    _close(got, want)
    back = native.rope_(got.clone(), pos, 500000.0, inverse=True)
    _close(back, x, 3e-2)


@pytest.mark.parametrize("rows,D", [(5001, 2048), (1501, 2048), (64, 4096), (3001, 4096)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_whole_cta_rows(rows, D, rms):
    """Row counts that select each rows-per-CTA variant of the wide forward kernel."""
    torch.manual_seed(4)
    x = (torch.randn(rows, D, device="cuda") * 1.5 + 0.3).to(torch.bfloat16)
    g = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16)
    b = None if rms else (0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16)
    y, mean, rstd = native.norm_fwd(x, g, b, 1e-5, rms)
    if rms:
        yr, _ = ref.rms_norm_ref(x.float(), g.float(), 1e-5)
    else:
        yr, mr, rr = ref.layer_norm_ref(x.float(), g.float(), b.float(), 1e-5)
        assert (mean - mr.reshape(-1)).abs().max().item() < 1e-3
    _close(y, yr)
