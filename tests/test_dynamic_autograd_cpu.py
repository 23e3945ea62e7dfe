"""Dynamic-shape autograd functions: shape rules on symbolic shapes, gradients against torch autograd."""
import pytest
import torch

from ml_framework_b200.autograd import dynamic as D
from ml_framework_b200.compiler.shapes import SymbolicDimension as Dim, SymbolicShape as Shape

B, S = Dim("batch", None, 1, 64), Dim("seq", None, 1, 128)


def _check(fn, inputs, ref):
    """fn through autograd == the same maths written in torch, values and gradients."""
    ins = [x.clone().requires_grad_(x.is_floating_point()) if isinstance(x, torch.Tensor) else x for x in inputs]
    rins = [x.clone().requires_grad_(x.is_floating_point()) if isinstance(x, torch.Tensor) else x for x in inputs]
    out, want = fn(*ins), ref(*rins)
    torch.testing.assert_close(out, want)
    w = torch.randn_like(want)
    (out * w).sum().backward()
    (want * w).sum().backward()
    for a, b in zip(ins, rins):
        if isinstance(a, torch.Tensor) and a.is_floating_point():
            torch.testing.assert_close(a.grad, b.grad, rtol=1e-4, atol=1e-5)


def test_shape_helpers_context_and_gradient_tensor():
    x = torch.zeros(4, 7, 8)
    s = D.shape_of(x, ["batch", "seq", None])
    assert repr(s) == "[4, 7, 8]" and D.shape_of(x).concrete() == (4, 7, 8)
    env = {}
    assert D.matches(Shape([B, S, 8]), (4, 7, 8), env) and env == {"batch": 4, "seq": 7}
    assert not D.matches(Shape([B, B]), (4, 5)) and D.matches(Shape([B, B]), (5, 5)) and not D.matches(Shape([B, 8]), (4, 9))
    assert not D.matches(Shape([B]), (100,)) and not D.matches(Shape([B, 8]), (4,))
    with pytest.raises(ValueError):
        D.shape_of(x, ["a"])
    with D.DynamicAutogradContext() as ctx:
        ctx.save_for_backward(x, x + 1)
        ctx.save_input_shape(Shape([B, S, 8]))
        ctx.save_output_shape(Shape([B, 8]))
        ctx.register_gradient_shape(0, Shape([B, 8]))
        assert ctx.saved_tensor_count == 2 and ctx.input_shape_count == 1 and ctx.get_output_shape(0) == Shape([B, 8])
        ctx.validate_gradient(0, (4, 8)); ctx.validate_gradient(0, Shape([B, 8]))
        with pytest.raises(ValueError):
            ctx.validate_gradient(0, (4, 9))
        with pytest.raises(KeyError):
            ctx.get_gradient_shape(3)
        with pytest.raises(IndexError):
            ctx.get_saved_tensor(2)
        assert "saved=2" in repr(ctx)
    with pytest.raises(RuntimeError):
        ctx.save_for_backward(x)
    t = D.DynamicGradientTensor(torch.ones(4, 8), Shape([B, 8]))
    t.accumulate_gradient(torch.ones(4, 8)); t.accumulate_gradient(torch.ones(4, 8))
    assert t.has_gradient and float(t.gradient.sum()) == 64 and "has_grad=True" in repr(t)
    with pytest.raises(ValueError):
        t.accumulate_gradient(torch.ones(8, 4))
    d = t.detach()
    with pytest.raises(RuntimeError):
        d.accumulate_gradient(torch.ones(4, 8))
    t.clear_gradient()
    assert not t.has_gradient
    with pytest.raises(ValueError):
        D.DynamicGradientTensor(torch.ones(4, 9), Shape([B, 8]))


def test_slice_and_pad():
    x = torch.randn(5, 9, 4)
    sl = D.DynamicSlice([1, 2, 0], Shape([3, S, 4]))                    # the symbolic extent runs to the end
    _check(sl, [x], lambda t: t[1:4, 2:, :])
    assert sl.get_output_shape([Shape([B, S, 4])]) == Shape([3, S, 4])
    with pytest.raises(ValueError):
        sl.get_output_shape([Shape([B, S])])
    with pytest.raises(ValueError):
        sl.validate_gradient_shape((3, 7, 5))
    with pytest.raises(IndexError):
        D.DynamicSlice([4, 0, 0], Shape([3, 9, 4])).forward(x)
    with pytest.raises(ValueError):
        D.DynamicSlice([], Shape([]))
    pad = D.DynamicPad([0, 0, 2, 3, 1, 0])
    _check(pad, [x], lambda t: torch.nn.functional.pad(t, [1, 0, 2, 3, 0, 0]))
    out = pad.get_output_shape([Shape([B, 9, 4])])
    assert str(out.dims[0]) == "batch" and out.dims[1].value == 14 and out.dims[2].value == 5
    grown = pad.get_output_shape([Shape([5, S, 4])]).dims[1]
    assert grown.name == "seq+5" and grown.min_value == 6 and grown.max_value == 133
    _check(D.DynamicPad([1, 1]), [x], lambda t: torch.nn.functional.pad(t, [0, 0, 0, 0, 1, 1]))
    for bad in ([1], [1, -1]):
        with pytest.raises(ValueError):
            D.DynamicPad(bad)


def test_mask_and_gather():
    x = torch.randn(3, 6, 2)
    lengths = torch.tensor([6, 2, 4])
    m = D.DynamicMask(S)

    def ref(t, ln):
        keep = (torch.arange(6)[None, :] < ln[:, None]).float()[..., None]
        return t * keep
    _check(m, [x, lengths], ref)
    assert m.get_output_shape([Shape([B, S, 2])]) == Shape([B, S, 2])
    with pytest.raises(ValueError):
        m.get_output_shape([Shape([B])])
    with pytest.raises(ValueError):
        D.DynamicMask(Dim("seq", 5)).forward(x, lengths)
    with pytest.raises(ValueError):
        D.DynamicMask(Dim("seq", None, 1, 4)).forward(x, lengths)
    g = D.DynamicGather(1)
    idx = torch.tensor([5, 0, 0, 3])                                   # a repeated index accumulates
    _check(g, [x, idx], lambda t, i: t.index_select(1, i))
    assert g.get_output_shape([Shape([B, S, 2]), Shape([Dim("picked")])]) == Shape([B, Dim("picked"), 2])
    assert D.DynamicGather(-1).get_output_shape([Shape([B, 7]), Shape([3])]) == Shape([B, 3])
    with pytest.raises(ValueError):
        g.get_output_shape([Shape([B, S]), Shape([2, 2])])
    with pytest.raises(ValueError):
        D.DynamicGather(4).get_output_shape([Shape([B, S]), Shape([2])])


def test_broadcast_and_reshape():
    x = torch.randn(1, 4, 1)
    bc = D.DynamicBroadcastBackward(Shape([1, 4, 1]), Shape([3, 2, 4, 5]))
    assert bc.broadcast_axes == [0, 1, 3]
    _check(bc, [x], lambda t: t.expand(3, 2, 4, 5).clone())
    like = torch.zeros(6, 4, 2)
    dyn = D.DynamicBroadcastBackward(Shape([1, 4, 1]), Shape([B, 4, S]))
    out = dyn.forward(x, like)
    assert out.shape == (6, 4, 2) and dyn.compute_grad(torch.ones(6, 4, 2), [x, like])[0].shape == (1, 4, 1)
    with pytest.raises(ValueError):
        bc.validate_gradient_shape((3, 2, 4, 6))
    with pytest.raises(ValueError):
        D.DynamicBroadcastBackward(Shape([2, 3, 4]), Shape([3, 4]))
    y = torch.randn(4, 6)
    rs = D.DynamicReshapeBackward(Shape([B, 6]), (-1, 3))
    _check(rs, [y], lambda t: t.reshape(-1, 3))
    assert rs.get_output_shape([Shape([4, 6])]) == Shape([8, 3]) and str(rs.get_output_shape([Shape([B, 6])]).dims[0]) == "inferred"
    with pytest.raises(ValueError):
        D.DynamicReshapeBackward(Shape([4, 6])).validate_gradient_shape((5, 5))
    with pytest.raises(ValueError):
        D.DynamicReshapeBackward(Shape([B, 7]), (-1,)).forward(y)


def test_matmul_and_conv2d():
    mm = D.DynamicMatMulBackward()
    a, b = torch.randn(2, 1, 5, 3), torch.randn(4, 3, 6)                # both batch axes broadcast
    _check(mm, [a, b], lambda p, q: p @ q)
    K = Dim("k")
    out = mm.get_output_shape([Shape([B, S, K]), Shape([K, 16])])
    assert out == Shape([B, S, 16])
    for bad in ([Shape([B, 8]), Shape([9, 4])], [Shape([B, Dim("p")]), Shape([Dim("q"), 4])], [Shape([8]), Shape([8, 4])]):
        with pytest.raises(ValueError):
            mm.get_output_shape(bad)
    cv = D.DynamicConv2DBackward(3, stride=2, padding=1, dilation=1)
    x, w, bias = torch.randn(2, 3, 9, 8), torch.randn(5, 3, 3, 3), torch.randn(5)
    _check(cv, [x, w, bias], lambda p, q, r: torch.nn.functional.conv2d(p, q, r, 2, 1, 1))
    _check(D.DynamicConv2DBackward((3, 1), dilation=(2, 1)), [x, torch.randn(4, 3, 3, 1)], lambda p, q: torch.nn.functional.conv2d(p, q, None, 1, 0, (2, 1)))
    H = Dim("h", None, 8, 64)
    s = cv.get_output_shape([Shape([B, 3, H, 32]), Shape([5, 3, 3, 3])])
    assert str(s.dims[0]) == "batch" and s.dims[1].value == 5 and s.dims[3].value == 16
    assert s.dims[2].name == "conv(h)" and (s.dims[2].min_value, s.dims[2].max_value) == (4, 32)
    for bad in ([Shape([B, 4, 8, 8]), Shape([5, 3, 3, 3])], [Shape([B, 3, 8, 8]), Shape([5, 3, 5, 5])], [Shape([B, 3, 1, 8]), Shape([5, 3, 3, 3])],
                [Shape([3, 8, 8]), Shape([5, 3, 3, 3])]):
        with pytest.raises(ValueError):
            D.DynamicConv2DBackward(3).get_output_shape(bad)
    with pytest.raises(ValueError):
        D.DynamicConv2DBackward(0)


def test_wrong_gradient_shape_is_caught_in_backward():
    class Liar(D.DynamicSlice):
        def expected_gradient_shape(self):
            return Shape([2, 2])

    x = torch.randn(4, 4, requires_grad=True)
    y = Liar([0, 0], Shape([3, 3]))(x)
    with pytest.raises(ValueError, match="does not match"):
        y.sum().backward()
