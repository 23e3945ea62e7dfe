"""Autograd utilities on CPU: custom functions against autograd's own derivatives, the function registry, nested and
persistent tapes, first- and higher-order derivative helpers against closed forms, validators, scaling helpers."""
import pytest
import torch
import torch.nn as nn

from ml_framework_b200.autograd import functional as A


def test_custom_functions_match_autograd_and_finite_differences():
    torch.manual_seed(0)
    x = torch.randn(3, 5, dtype=torch.float64, requires_grad=True)
    w = torch.randn(3, 5, dtype=torch.float64)
    (A.StableSoftmax().apply(x) * w).sum().backward()
    g1 = x.grad.clone()
    x.grad = None
    (torch.softmax(x, -1) * w).sum().backward()
    assert torch.allclose(g1, x.grad, atol=1e-10)
    big = torch.tensor([[1e4, 1e4 + 1.0, -1e4]], dtype=torch.float64)
    assert torch.isfinite(A.StableSoftmax().apply(big)).all()
    pred = torch.tensor([0.2, 1.7, -3.0, 0.9], requires_grad=True)
    tgt = torch.tensor([0.0, 0.0, 0.0, 1.0])
    loss = A.ClampedMSELoss(clamp=1.0).apply(pred, tgt)
    assert float(loss) == pytest.approx((0.04 + 1.0 + 1.0 + 0.01) / 4)
    loss.backward()
    assert torch.allclose(pred.grad, torch.tensor([0.1, 0.0, 0.0, -0.05]), atol=1e-6)      # clamped elements get no gradient
    ok, worst = A.GradientChecker.check_gradients(lambda a: A.StableSoftmax().apply(a)[:, 0].sum(), [torch.randn(2, 4)])
    assert ok, worst
    bad, _ = A.GradientChecker.check_gradients(lambda a: _WrongGrad().apply(a).sum(), [torch.randn(3)])
    assert not bad
    outs = A.StableSoftmax().apply_many([[torch.randn(2, 3)], [torch.randn(4, 3)]])
    assert [tuple(o.shape) for o in outs] == [(2, 3), (4, 3)]


class _WrongGrad(A.CustomFunction):
    def forward(self, ctx, x):
        return x * x

    def backward(self, ctx, g):
        return g                                                       # should be 2 x g


def test_engine_registry_and_backward():
    eng = A.AutogradEngine()
    eng.register_custom_function("ste", A.STEBinary())
    with pytest.raises(ValueError):
        eng.register_custom_function("ste", A.STEBinary())
    x = torch.tensor([-0.5, 3.0], requires_grad=True)
    y = eng.apply("ste", x)
    assert y.tolist() == [-1.0, 1.0]
    A.AutogradEngine.backward(y.sum(), retain_graph=True)
    A.AutogradEngine.backward(y.sum())
    assert x.grad.tolist() == [2.0, 0.0]
    with pytest.raises(KeyError):
        eng.apply("missing", x)


def test_tapes_nested_persistent_and_unused_sources():
    with A.GradientTape(persistent=True) as outer:
        x = outer.watch(torch.tensor(3.0))
        with A.GradientTape() as inner:
            inner.watch(x)
            y = x ** 3
            dy = inner.gradient(y, x, create_graph=True)                # 3 x^2, differentiable
        d2y = outer.gradient(dy, x)                                     # 6 x
        again = outer.gradient(y, x)                                    # persistent: a second query is allowed
    assert float(dy) == 27.0 and float(d2y) == 18.0 and float(again) == 27.0
    assert A.GradientTape._stack == []
    with torch.no_grad():
        with A.GradientTape() as t:                                     # the tape re-enables gradient recording
            a, b = t.watch(torch.tensor(2.0)), t.watch(torch.tensor(5.0))
            z = a * a
        ga, gb = t.gradient(z, [a, b])
    assert float(ga) == 4.0 and gb is None                              # b does not take part


def test_first_and_higher_order_helpers_against_closed_forms():
    f = lambda v: (v ** 2).sum() + v[0] * v[1]
    v = torch.tensor([1.0, -2.0, 0.5])
    assert torch.allclose(A.gradient(f, v), torch.tensor([0.0, -3.0, 1.0]))
    H = A.hessian(f, v)
    assert torch.allclose(H, torch.tensor([[2.0, 1.0, 0.0], [1.0, 2.0, 0.0], [0.0, 0.0, 2.0]]))
    u = torch.tensor([1.0, 1.0, 1.0])
    assert torch.allclose(A.hvp(f, v, u), H @ u)
    g = lambda t: torch.stack([t[0] * t[1], t[1] ** 2, t.sum()])
    J = torch.tensor([[-2.0, 1.0, 0.0], [0.0, -4.0, 0.0], [1.0, 1.0, 1.0]])
    for mode in ("auto", "forward", "reverse"):
        assert torch.allclose(A.jacobian(g, v, mode), J)
    out, tangent = A.jvp(g, v, u)
    assert torch.allclose(out, g(v)) and torch.allclose(tangent, J @ u)
    out2, cot = A.vjp(g, v, torch.tensor([1.0, 0.0, 2.0]))
    assert torch.allclose(out2, g(v)) and torch.allclose(cot, J.t() @ torch.tensor([1.0, 0.0, 2.0]))
    wide = A.jacobian(lambda t: t.sum().reshape(1), torch.ones(6))      # many inputs, one output: reverse mode is picked
    assert wide.shape == (1, 6) and torch.allclose(wide, torch.ones(1, 6))


def test_validator_exception_types_and_scaling_helpers():
    p = torch.zeros(2, 2)
    assert A.GradientValidator.validate(p, torch.ones(2, 2), "w")
    with pytest.raises(A.GradientTypeException):
        A.GradientValidator.validate(p, torch.ones(2, 2, dtype=torch.float64), "w")
    with pytest.raises(A.GradientInfException):
        A.GradientValidator.validate(p, torch.tensor([[1.0, float("inf")], [0.0, 0.0]]), "w")
    with pytest.raises(A.GradientShapeException) as e:
        A.GradientValidator.validate(p, torch.ones(3), "layer.w")
    assert "layer.w" in str(e.value)
    g = [torch.full((2,), 4.0), torch.full((3,), 8.0)]
    sc = A.scale_by_batch_size(g, batch_size=64, reference_batch_size=16)
    assert torch.allclose(sc[0], torch.full((2,), 1.0)) and torch.allclose(sc[1], torch.full((3,), 2.0))
    wa = A.weighted_average([[torch.tensor([1.0]), torch.tensor([10.0])], [torch.tensor([3.0]), torch.tensor([30.0])]], [1, 3])
    assert torch.allclose(wa[0], torch.tensor([2.5])) and torch.allclose(wa[1], torch.tensor([25.0]))
    with pytest.raises(ValueError):
        A.GradientAccumulator([nn.Parameter(torch.ones(1))], 0)
    w = nn.Parameter(torch.ones(2))
    acc = A.GradientAccumulator([w, nn.Parameter(torch.ones(1))], 3)    # the second parameter never gets a gradient
    done = []
    for k in range(3):
        (w * (k + 1)).sum().backward()
        done.append(acc.step())
    assert done == [False, False, True]
    acc.apply_gradients(average=False)
    assert torch.allclose(w.grad, torch.full((2,), 6.0)) and acc.count == 0
