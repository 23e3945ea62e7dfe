"""Shape comparison / reshape checks, broadcast views, dimension bindings, symbolic tensors, constraint builder / validator, inference context."""
import pytest
import torch

from ml_framework_b200.compiler import shape_tools as S
from ml_framework_b200.compiler.shapes import ShapeInferenceEngine, ShapeMismatchException, SymbolicDimension, SymbolicShape


def test_factories_and_comparer():
    F, D = S.SymbolicShapeFactory, S.SymbolicDimensionFactory
    tok = F.tokens(4096, max_batch=64, max_len=2048)
    assert repr(tok) == "[batch, seq, 4096]" and tok[0].max_value == 64 and F.scalar().rank == 0 and F.matrix(2, 3).concrete() == (2, 3)
    assert repr(F.image(3)) == "[batch, 3, height, width]" and F.batched(7, 9).rank == 3 and D.create("n", 5).is_known and not D.bounded("k", 1, 8).is_known
    with pytest.raises(ValueError):
        D.bounded("k", 5, 2)
    C = S.ShapeComparer
    assert C.are_compatible(tok, F.from_concrete(8, 512, 4096)) and not C.are_compatible(tok, F.from_concrete(128, 512, 4096)) and not C.are_compatible(tok, F.from_concrete(8, 4096))
    assert C.are_compatible(SymbolicShape([D.bounded("a", 1, 4)]), SymbolicShape([D.bounded("b", 3, 9)])) and not C.are_compatible(SymbolicShape([D.bounded("a", 1, 2)]), SymbolicShape([D.bounded("b", 3, 9)]))
    assert C.are_equal(F.matrix(2, 3), F.from_concrete(2, 3)) and C.can_broadcast(F.from_concrete(4, 1, 3), F.from_concrete(5, 3)) and not C.can_broadcast(F.vector(4), F.vector(3))
    assert C.broadcast_shape(F.from_concrete(4, 1, 3), F.from_concrete(5, 3)).concrete() == (4, 5, 3) and C.numel(F.matrix(3, 4)) == 12 and C.numel(tok) is None
    assert C.can_reshape(F.matrix(6, 4), [3, -1]) and C.reshape(F.matrix(6, 4), [3, -1]).concrete() == (3, 8) and not C.can_reshape(F.matrix(6, 4), [5, -1]) and not C.can_reshape(F.matrix(6, 4), [-1, -1])
    assert not C.can_reshape(F.matrix(6, 4), [25]) and C.can_reshape(tok, [-1, 4096]) and repr(C.reshape(tok, [-1, 4096])) == "[inferred, 4096]"
    with pytest.raises(ShapeMismatchException):
        C.reshape(F.matrix(6, 4), [7, 7])


def test_broadcasted_tensor_is_a_zero_stride_view():
    src = torch.arange(3.0).view(1, 3)
    b = S.BroadcastedTensor(src, (2, 4, 3))
    assert b.shape == (2, 4, 3) and b.broadcast_sources() == [0, 1] and b.strides() == (0, 0, 1) and b.requires_materialization() and b.expansion_factor == 8
    v = b.view()
    assert v.data_ptr() == src.data_ptr() and v.stride() == (0, 0, 1) and torch.equal(b.materialize(), src.expand(2, 4, 3)) and b.materialize().is_contiguous()
    same = S.BroadcastedTensor(src, (1, 3))
    assert not same.requires_materialization() and same.broadcast_sources() == [] and "broadcast dims [0, 1]" in repr(b)
    for bad in ((2, 4, 5), (3,)):
        with pytest.raises(ShapeMismatchException):
            S.BroadcastedTensor(src, bad)


def test_bindings_and_symbolic_tensors():
    b = S.DimensionBindings({"batch": 8})
    b.register_binding("seq", 128)
    b.register_binding("seq", 128)
    assert b.get_binding("seq") == 128 and b.has_binding("batch") and b.bound_names() == ["batch", "seq"] and "batch=8" in repr(b)
    with pytest.raises(ValueError):
        b.register_binding("seq", 64)
    with pytest.raises(ValueError):
        b.register_binding("x", -1)
    c = b.clone()
    c.remove_binding("seq")
    other = S.DimensionBindings({"heads": 16})
    c.merge_from(other)
    assert c.bound_names() == ["batch", "heads"] and b.has_binding("seq") and not c.remove_binding("nope")
    shape = S.SymbolicShapeFactory.tokens(64)
    inf = S.DimensionBindings()
    inf.infer_from(shape, (4, 10, 64))
    assert inf.as_dict() == {"batch": 4, "seq": 10}
    with pytest.raises(ShapeMismatchException):
        inf.infer_from(shape, (4, 10, 65))
    with pytest.raises(ShapeMismatchException):
        inf.infer_from(shape, (4, 10))
    n = SymbolicDimension("n", None, 2, 16)
    t = S.SymbolicTensor(SymbolicShape([n, n, 3]), S.TensorFillType.ONES, torch.bfloat16, "attn")
    assert t.free_dimensions() == ["n"] and t.concrete_shape(4) == (4, 4, 3) and t.validate_shape() and "attn: [n, n, 3], bfloat16" in repr(t)
    assert t.can_instantiate_with(4, 4, 3) and not t.can_instantiate_with(4, 5, 3) and not t.can_instantiate_with(1, 1, 3) and not t.can_instantiate_with(4, 4, 2) and not t.can_instantiate_with(4, 4)
    x = t.to_concrete(bindings=S.DimensionBindings({"n": 5}))
    assert x.shape == (5, 5, 3) and x.dtype == torch.bfloat16 and float(x.sum()) == 75.0
    with pytest.raises(ValueError):
        t.concrete_shape()
    with pytest.raises(ValueError):
        t.concrete_shape(99)
    r = S.SymbolicTensor(S.SymbolicShapeFactory.matrix(2, 2), S.TensorFillType.RANDOM).to_concrete(generator=torch.Generator().manual_seed(0))
    assert r.shape == (2, 2) and float(r.abs().sum()) > 0 and float(S.SymbolicTensor(S.SymbolicShapeFactory.vector(3), S.TensorFillType.ZEROS).to_concrete().sum()) == 0.0


def test_constraint_builder_and_validator():
    cs = S.ShapeConstraintBuilder("seq").min(1).max(4096).modulo(8).equal_to("kv_seq").build()
    assert [S.describe_constraint(c) for c in cs] == ["1 <= seq <= 4096", "seq % 8 == 0", "seq == kv_seq"]
    v = S.ConstraintValidator()
    assert v.validate_all({"seq": 128, "kv_seq": 128}, cs) and v.violations({"seq": 130, "kv_seq": 128}, cs) == ["seq % 8 == 0 violated by seq=130", "seq == kv_seq violated by kv_seq=128, seq=130"]
    assert v.violations({"seq": 130, "kv_seq": 128}, cs) and (v.hits, v.misses) == (1, 2)
    assert v.validate_dimension(SymbolicDimension("seq", 8000), cs) is False and v.validate_dimension(SymbolicDimension("seq"), cs)
    shape = S.SymbolicShapeFactory.tokens(64)
    assert v.validate_shape(shape, (2, 16, 64), cs[:2]) == [] and "4096" in v.validate_shape(shape, (2, 8192, 64), cs[:2])[0]
    v.clear_cache()
    assert v.hits == 0
    b = S.ShapeConstraintBuilder("d").equal(64)
    assert S.describe_constraint(b.build()[0]) == "64 <= d <= 64" and b.reset().build() == []
    for bad in (lambda: S.ShapeConstraintBuilder("d").min(5).max(2), lambda: S.ShapeConstraintBuilder("d").range(3, 1), lambda: S.ShapeConstraintBuilder("d").modulo(0)):
        with pytest.raises(ValueError):
            bad()


def test_inference_context_memoises_per_operation():
    eng = ShapeInferenceEngine()
    ctx = S.InferenceContext({"x": SymbolicShape([SymbolicDimension("batch"), 16]), "w": SymbolicShape([32, 16])})
    y = ctx.infer(eng, "op0", "linear", ["x", "w"], "y")
    assert repr(y) == "[batch, 32]" and ctx.has_shape("y") and ctx.has_operation_results("op0") and ctx.get_operation_results("op0")[0] is y
    ctx.set_shape("w", SymbolicShape([8, 16]))
    assert ctx.infer(eng, "op0", "linear", ["x", "w"], "y") is y                 # memoised
    with pytest.raises(KeyError):
        ctx.infer(eng, "op1", "relu", ["missing"], "z")
    c2 = ctx.clone()
    c2.clear_operation_results()
    assert repr(c2.infer(eng, "op0", "linear", ["x", "w"], "y")) == "[batch, 8]" and ctx.get_operation_results("op0")[0] is y
    ctx.clear_tensor_shapes()
    assert not ctx.has_shape("x") and ctx.get_shape("x") is None
    ctx.clear()
    assert ctx.get_operation_results("op0") is None
    with pytest.raises(ValueError):
        ctx.set_shape("", y)
