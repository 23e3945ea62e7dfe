"""Functional transforms on CPU beyond the basic cases: every traceable operator of the jit tracer against eager
execution, what must refuse to trace, composition, chunked vmap, pmap collectives and its single-device form."""
import pytest
import torch

from ml_framework_b200.compiler import functional as Fn
from ml_framework_b200.dist.process_group import run_fake_world


def test_tracer_covers_reflected_operators_methods_and_torch_functions():
    def net(x, w):
        a = 2.0 - x                      # reflected subtraction
        b = 1.0 / (a * a + 3.0)          # reflected division, reflected and plain addition
        c = (-b).exp().log().tanh() + torch.sigmoid(x) * 0.5 + torch.sqrt(a * a)
        d = torch.maximum(c, x) - torch.minimum(c, x)
        e = torch.nn.functional.gelu(d, approximate="tanh") @ w.T
        f = e.reshape(-1, 2).transpose(0, 1).mean(dim=1, keepdim=True)
        s = torch.softmax(e, dim=-1).sum()
        return f, s, torch.neg(e).relu().sum(dim=0)
    torch.manual_seed(0)
    x, w = torch.randn(4, 6), torch.randn(6, 6)
    jf = Fn.jit(net)
    got, want = jf(x, w), net(x, w)
    assert jf.stats["traced"] == 1 and all(torch.allclose(g, t, atol=1e-5) for g, t in zip(got, want))
    g = jf.graph(x, w)
    kinds = {o.kind for o in g.ops}
    assert {"gelu", "softmax", "maximum", "minimum", "matmul", "transpose", "reshape"} <= kinds
    raw = Fn.jit(lambda t: (t * 1.0 + 0.0).relu(), optimize=False)
    assert "mul" in [o.kind for o in raw.graph(x).ops]                      # without the pass manager nothing is simplified

    @Fn.jit(name="decorated")
    def dec(t):
        return t * t
    assert dec.name == "decorated" and torch.equal(dec(x), x * x) and dec.__wrapped__(x).equal(x * x)


def test_what_cannot_be_traced_falls_back_and_says_why():
    x = torch.randn(3, 3)
    tr = None

    def probe(t):
        nonlocal tr
        tr = t
        return t
    Fn.jit(probe)(x)
    assert tr.shape == (3, 3) and tr.dtype == torch.float32 and tr.T.shape == (3, 3)
    for bad in (lambda t: bool(t), lambda t: float(t), lambda t: t.item(), lambda t: t.tolist(), lambda t: t + "s", lambda t: torch.fft.fft(t)):
        with pytest.raises(Fn.TraceError):
            bad(tr)
    const = Fn.jit(lambda t: torch.ones(2))                                  # returns nothing computed from its input
    assert torch.equal(const(x), torch.ones(2)) and const.stats["eager"] == 1 and const.graph(x) is None
    ctrl = Fn.jit(lambda t: t if t.sum() > 0 else -t)                        # control flow on a value
    assert torch.equal(ctrl(torch.ones(2)), torch.ones(2)) and ctrl.stats == {"traced": 0, "captured": 0, "eager": 1, "hits": 0}


def test_compose_grad_and_chunked_vmap():
    f = Fn.compose(lambda t: t + 1, lambda t: t * 3, torch.relu)
    assert torch.equal(f(torch.tensor([-2.0, 1.0])), torch.tensor([0.0, 6.0]))
    assert torch.allclose(Fn.grad(lambda t: (t ** 2).sum())(torch.tensor([1.0, -3.0])), torch.tensor([2.0, -6.0]))
    g, v = Fn.grad_and_value(lambda t: (t ** 3).sum())(torch.tensor([2.0]))
    assert float(g) == 12.0 and float(v) == 8.0
    xs = torch.randn(10, 4)
    per = lambda row: row.cumsum(0) * row.max()                              # noqa: E731
    want = torch.stack([per(r) for r in xs])
    assert torch.allclose(Fn.vmap(per, chunk_size=3)(xs), want, atol=1e-6)
    assert torch.allclose(Fn.vmap(per, chunk_size=3, fallback="loop")(xs), want, atol=1e-6)
    pair = Fn.vmap(lambda a, b: (a + b, a * b), in_axes=(0, 1))(torch.ones(3, 2), torch.full((2, 3), 2.0))
    assert torch.equal(pair[0], torch.full((3, 2), 3.0)) and torch.equal(pair[1], torch.full((3, 2), 2.0))
    with pytest.raises(ValueError):
        Fn.vmap(lambda a, b: a + b)(torch.ones(3, 2), torch.ones(4, 2))       # mapped sizes disagree


def test_pmap_collectives_single_device_form_and_errors():
    data = torch.arange(24.0).reshape(6, 4)

    def run(pg):
        def body(x):
            return x - Fn.pmax(x.max(), "m"), Fn.all_gather(x[:1], "m", axis=0), Fn.axis_index("m")
        shifted, firsts, idx = Fn.pmap(body, pg, axis_name="m", gather=False)(data)
        tup = Fn.pmap(lambda x: (x * 2, x.sum(1)), pg, axis_name="m")(data)
        rep = Fn.pmap(lambda x, s: x * s, pg, axis_name="m", in_axes=(0, None))(data, torch.tensor(0.5))
        cols = Fn.pmap(lambda x: x + 1, pg, axis_name="m", in_axes=1, out_axis=1)(data[:, :3])
        return shifted, firsts, idx, tup, rep, cols
    outs = run_fake_world(3, run)
    for r, (shifted, firsts, idx, tup, rep, cols) in enumerate(outs):
        assert idx == r and torch.equal(shifted, data[2 * r:2 * r + 2] - 23.0)
        assert torch.equal(firsts, data[[0, 2, 4]]) and torch.equal(tup[0], data * 2) and torch.equal(tup[1], data.sum(1))
        assert torch.equal(rep, data * 0.5) and torch.equal(cols, data[:, :3] + 1)
    solo = Fn.pmap(lambda x: Fn.psum(x, "i") + Fn.pmean(x, "i") + Fn.pmax(x, "i") + Fn.all_gather(x, "i") + Fn.axis_index("i"))
    assert torch.equal(solo(torch.ones(2)), torch.full((2,), 4.0))            # no group: one device, collectives are identities

    def bad(pg):
        with pytest.raises(ValueError):
            Fn.pmap(lambda x: x, pg)(torch.ones(5, 2))                         # 5 rows over 2 ranks
        return True
    assert run_fake_world(2, bad) == [True, True]
    with pytest.raises(NameError):
        Fn.axis_index("unbound")
