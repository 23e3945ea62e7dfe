"""Options-driven Jacobians / Hessians, sparse / partial / regularised variants, eigenvalues, batched HVPs, numerical checks,
order tracking, function registry."""
import math

import pytest
import torch

from ml_framework_b200.autograd import higher_order as H
from ml_framework_b200.autograd.functional import STEBinary, StableSoftmax

torch.set_default_dtype(torch.float32)


def _quad(A):
    return lambda x: 0.5 * x @ A @ x


def test_jacobian_modes_chunks_and_validation():
    f = lambda x: torch.stack([x[0] * x[1], x[1].sin(), x.sum(), (x ** 2).sum()])       # noqa: E731
    x = torch.tensor([0.5, -1.2, 2.0], dtype=torch.float64)
    want = torch.tensor([[-1.2, 0.5, 0.0], [0.0, math.cos(-1.2), 0.0], [1.0, 1.0, 1.0], [1.0, -2.4, 4.0]], dtype=torch.float64)
    auto = H.jacobian_with_options(f, x)
    assert auto.mode_used == H.JacobianMode.FORWARD and torch.allclose(auto.jacobian, want) and auto.sweeps == 1
    rev = H.jacobian_with_options(f, x, H.JacobianOptions(H.JacobianMode.REVERSE, chunk_size=3, validate=True))
    assert rev.sweeps == 2 and torch.allclose(rev.jacobian, want) and rev.max_numerical_error < 1e-6
    wide = H.jacobian_with_options(lambda t: t.sum().reshape(1), torch.ones(5))
    assert wide.mode_used == H.JacobianMode.REVERSE
    assert torch.allclose(H.numerical_jacobian(f, x), want, atol=1e-7)
    broken = lambda t: t.detach() * 2 + t * 0          # noqa: E731  (autograd sees a zero Jacobian)
    with pytest.raises(ArithmeticError):
        H.jacobian_with_options(broken, x, H.JacobianOptions(validate=True))


def test_numerical_gradients_and_error_measures():
    x, y = torch.tensor([1.0, 2.0], dtype=torch.float64), torch.tensor([3.0, -1.0], dtype=torch.float64)
    g = H.numerical_gradients(lambda a, b: (a * b).sum() + (a ** 2).sum(), [x, y])
    assert torch.allclose(g[0], y + 2 * x, atol=1e-7) and torch.allclose(g[1], x, atol=1e-7)
    assert torch.allclose(H.numerical_gradient(lambda a: a.pow(3).sum(), x), 3 * x ** 2, atol=1e-6)
    a, b = torch.tensor([1.0, 0.0]), torch.tensor([1.0, 0.0])
    assert H.relative_error(a, b) == 0.0 and H.mean_squared_error(a, b + 1) == 1.0 and H.validate_gradient(a, b) and not H.validate_gradient(a, torch.zeros(3))
    assert abs(H.relative_error(torch.tensor([1.0]), torch.tensor([-1.0])) - 1.0) < 1e-12


def test_hessian_options_sparse_partial_regularised_eigen():
    A = torch.tensor([[4.0, 1.0, 0.0], [1.0, 3.0, 0.0], [0.0, 0.0, 2.0]], dtype=torch.float64)
    f = _quad(A)
    x = torch.tensor([0.3, -0.7, 1.1], dtype=torch.float64)
    r = H.hessian_with_options(f, x, H.HessianOptions(eigenvalues=True))
    assert torch.allclose(r.hessian, A) and r.nonzeros == 5 and abs(r.density - 5 / 9) < 1e-12 and r.is_positive_definite
    assert torch.allclose(r.eigenvalues, torch.linalg.eigvalsh(A)) and abs(r.condition_number - float(r.eigenvalues.max() / r.eigenvalues.min())) < 1e-9
    sp = H.sparse_hessian(f, x)
    assert sp.is_sparse and sp.hessian.is_sparse and sp.hessian._nnz() == 5 and torch.allclose(sp.hessian.to_dense(), A)
    assert torch.allclose(H.partial_hessian(f, x, [0, 2]), A[[0, 2]][:, [0, 2]]) and torch.allclose(H.hessian_with_options(f, x, H.HessianOptions(indices=[1])).hessian, A[1:2, 1:2])
    with pytest.raises(IndexError):
        H.partial_hessian(f, x, [5])
    assert torch.allclose(H.regularized_hessian(f, x, 0.5), A + 0.5 * torch.eye(3, dtype=torch.float64))
    Hm, ev = H.hessian_with_eigenvalues(lambda t: -t.pow(2).sum(), x)
    assert torch.allclose(ev, torch.full((3,), -2.0, dtype=torch.float64)) and H.hessian_with_options(lambda t: -t.pow(2).sum(), x, H.HessianOptions(eigenvalues=True)).is_positive_definite is False
    lam, v = H.top_eigenvalue(f, x, iters=200, tol=1e-10)
    assert abs(lam - float(torch.linalg.eigvalsh(A).max())) < 1e-5 and abs(float(v.norm()) - 1.0) < 1e-9
    assert H.top_eigenvalue(lambda t: t.sum(), x)[0] == 0.0
    assert torch.allclose(H.grad_of_grad(f, x), A.sum(0))


def test_hvp_batch_numerical_and_validation():
    A = torch.tensor([[2.0, 1.0], [1.0, 5.0]], dtype=torch.float64)
    f = lambda x: 0.5 * x @ A @ x + x.pow(4).sum()      # noqa: E731
    x = torch.tensor([0.5, -1.0], dtype=torch.float64)
    Hx = A + torch.diag(12 * x ** 2)
    vs = [torch.tensor([1.0, 0.0], dtype=torch.float64), torch.tensor([0.5, 2.0], dtype=torch.float64)]
    for opts in (None, H.HVPOptions(checkpoint=True), H.HVPOptions(validate=True)):
        out = H.hvp_batch(f, x, vs, opts)
        assert all(torch.allclose(o, Hx @ v) for o, v in zip(out, vs))
    assert H.hvp_batch(f, x, []) == [] and torch.allclose(H.numerical_hvp(f, x, vs[1]), Hx @ vs[1], atol=1e-6) and H.validate_hvp(f, x, vs[0])
    assert not H.validate_hvp(f, x, vs[0], analytical=torch.zeros(2, dtype=torch.float64))
    with pytest.raises(ArithmeticError):
        H.hvp_batch(lambda t: (t.detach() * t).sum() * t.sum(), x, vs, H.HVPOptions(validate=True, tolerance=1e-6))


def test_order_context_and_nth_derivative():
    ctx = H.HigherOrderContext(max_order=3)
    assert ctx.current_order == 0
    with ctx.order(target_order=2) as d1:
        assert d1 == 1 and ctx.create_graph
        with ctx.order() as d2:
            assert d2 == 2 and not ctx.create_graph
            with ctx.order():
                with pytest.raises(RecursionError):
                    with ctx.order():
                        pass
    assert ctx.current_order == 0
    with pytest.raises(RecursionError):
        with ctx.order(target_order=9):
            pass
    x = torch.tensor([0.3, 1.0], dtype=torch.float64)
    assert torch.allclose(ctx.nth_derivative(torch.sin, x, 3), -torch.cos(x)) and torch.allclose(ctx.nth_derivative(torch.sin, x, 0), torch.sin(x))
    with pytest.raises(RecursionError):
        ctx.nth_derivative(torch.sin, x, 4)
    with pytest.raises(ValueError):
        H.HigherOrderContext(0)


def test_function_registry():
    H.FunctionRegistry.clear_all()
    H.FunctionRegistry.register("ste", STEBinary)
    H.FunctionRegistry.register("softmax", StableSoftmax)
    assert H.FunctionRegistry.names() == ["softmax", "ste"] and H.FunctionRegistry.is_registered("ste") and H.FunctionRegistry.get_function_type("ste") is STEBinary
    x = torch.tensor([[1.0, 2.0, 3.0]], requires_grad=True)
    y = H.FunctionRegistry.apply_function("softmax", x, init_args=(-1,))
    assert torch.allclose(y, torch.softmax(x, -1)) and H.FunctionRegistry.create_instance("ste") is not H.FunctionRegistry.create_instance("ste")
    with pytest.raises(KeyError):
        H.FunctionRegistry.register("ste", STEBinary)
    H.FunctionRegistry.register("ste", StableSoftmax, overwrite=True)
    with pytest.raises(TypeError):
        H.FunctionRegistry.register("bad", dict)
    with pytest.raises(KeyError):
        H.FunctionRegistry.get_function_type("none")
    assert H.FunctionRegistry.unregister("ste") and not H.FunctionRegistry.unregister("ste")
    H.FunctionRegistry.clear_all()
    assert H.FunctionRegistry.names() == []


def test_jvp_vjp_products_options_batches_and_validation():
    from ml_framework_b200.autograd.higher_order import JacobianVectorProduct as JVP, JVPOptions, VectorJacobianProduct as VJP, VJPOptions
    torch.manual_seed(0)
    A = torch.randn(3, 4, dtype=torch.float64)
    f = lambda x: torch.tanh(A @ x)                                     # noqa: E731
    x, v, u = torch.randn(4, dtype=torch.float64), torch.randn(4, dtype=torch.float64), torch.randn(3, dtype=torch.float64)
    J = torch.autograd.functional.jacobian(f, x)
    torch.testing.assert_close(JVP.compute(f, x, v), J @ v)
    torch.testing.assert_close(VJP.compute(f, x, u), u @ J)
    torch.testing.assert_close(JVP.compute_jacobian(f, x), J)
    assert JVP.validate(f, x, v) and VJP.validate(f, x, u)
    torch.testing.assert_close(JVP.compute_numerical(f, x, v), J @ v, rtol=1e-6, atol=1e-8)
    # zero vectors short-circuit; buffers are filled in place
    calls = []
    g = lambda t: (calls.append(1), f(t))[1]                            # noqa: E731
    assert float(JVP.compute(g, x, torch.zeros_like(x)).abs().sum()) == 0 and float(VJP.compute(g, x, torch.zeros(3, dtype=torch.float64)).abs().sum()) == 0
    assert len(calls) == 1                                              # one plain forward for the shape; the pull-back needs none
    buf = torch.empty(3, dtype=torch.float64)
    assert JVP.compute(f, x, v, JVPOptions(output_buffer=buf)) is buf and torch.allclose(buf, J @ v)
    with pytest.raises(ValueError):
        JVP.compute(f, x, v, JVPOptions(output_buffer=torch.empty(2, dtype=torch.float64)))
    with pytest.raises(ValueError):
        JVP.compute(f, x, torch.ones(3, dtype=torch.float64))
    with pytest.raises(ValueError):
        VJP.compute(f, x, torch.ones(4, dtype=torch.float64))
    # caches
    JVP.clear_tangent_cache(); VJP.clear_gradient_cache()
    JVP.compute(f, x, v, JVPOptions(cache_tangents=True)); JVP.compute(f, x, v, JVPOptions(cache_tangents=True))
    VJP.compute(f, x, u, VJPOptions(cache_gradients=True))
    assert JVP.get_cache_size() == 1 and VJP.get_cache_size() == 1
    JVP.compute(f, x, v, JVPOptions(clear_cache=True))
    assert JVP.get_cache_size() == 0
    # batches: vectorised, chunked and looped agree
    vs = [torch.randn(4, dtype=torch.float64) for _ in range(5)]
    us = [torch.randn(3, dtype=torch.float64) for _ in range(5)]
    for opts_j, opts_v in ((None, None), (JVPOptions(max_parallel_tasks=2), VJPOptions(max_parallel_tasks=2)),
                           (JVPOptions(enable_parallel=False), VJPOptions(enable_parallel=False))):
        for got, vec in zip(JVP.compute_batch(f, x, vs, opts_j), vs):
            torch.testing.assert_close(got, J @ vec)
        for got, vec in zip(VJP.compute_batch(f, x, us, opts_v), us):
            torch.testing.assert_close(got, vec @ J)
    assert JVP.compute_batch(f, x, []) == [] and VJP.compute_batch(f, x, []) == []
    # several inputs
    h = lambda ts: ts[0] * ts[1].sin()                                  # noqa: E731
    a, b, t = torch.randn(4, dtype=torch.float64), torch.randn(4, dtype=torch.float64), torch.randn(4, dtype=torch.float64)
    torch.testing.assert_close(JVP.compute_multiple(h, [a, b], t, input_index=1), a * b.cos() * t)
    da, db = VJP.compute_multiple(h, [a, b], t)
    torch.testing.assert_close(da, t * b.sin()); torch.testing.assert_close(db, t * a * b.cos())
    with pytest.raises(IndexError):
        JVP.compute_multiple(h, [a, b], t, input_index=2)
