"""Function combinators, transformation context / registry / typed transformations, jit cache control."""
import gc

import pytest
import torch

from ml_framework_b200.compiler import functional as F


def test_combinators():
    inc, dbl = (lambda x: x + 1), (lambda x: x * 2)
    assert F.pipe(3, inc, dbl) == 8 and F.compose(inc, dbl)(3) == 8 and F.pipe(5) == 5
    sub = lambda a, b: a - b                                           # noqa: E731
    assert F.partial(sub, 10)(3) == 7 and F.partial_second(sub, 10)(3) == -7
    add3 = lambda a, b, c: a + b + c                                   # noqa: E731
    assert F.curry(add3, 3)(1)(2)(3) == 6 and F.uncurry(F.curry(add3, 3))(1, 2, 3) == 6 and F.curry(sub)(5)(2) == 3
    with pytest.raises(ValueError):
        F.curry(sub, 0)
    assert F.identity("x") == "x" and F.constant(7)(1, 2, k=3) == 7
    seen = []
    assert F.tap(4, seen.append) == 4 and F.tap_if(5, False, seen.append) == 5 and F.tap_if(6, True, seen.append) == 6 and seen == [4, 6]


def test_context_inherits_and_shadows():
    root = F.TransformationContext()
    root.debug_mode = True
    root.set_metadata("axis", "data")
    child = root.create_child_context()
    child.set_metadata("chunk", 4)
    assert child.debug_mode and child.get_metadata("axis") == "data" and child.get_metadata("axis", search_parents=False) is None
    assert root.get_metadata("chunk", "none") == "none" and child.parent is root
    child.set_metadata("axis", "model")
    assert child.get_metadata("axis") == "model" and root.get_metadata("axis") == "data"
    assert (F.MeshAxisNames.DATA, F.MeshAxisNames.MODEL, F.MeshAxisNames.PIPELINE) == ("data", "model", "pipeline")


def test_registry_records_typed_transformations_and_purity():
    F.TransformationRegistry.clear()

    @F.tensor_function(input_shapes=["n"], output_shape="", description="sum of squares")
    def sq(x):
        return (x * x).sum()

    assert F.is_function_pure(sq) and sq.__tensor_function__["input_shapes"] == ("n",)
    batched = F.vectorize(sq)
    x = torch.arange(6.0).view(2, 3)
    torch.testing.assert_close(batched(x), (x * x).sum(1))
    compiled = F.compile_function(sq)
    torch.testing.assert_close(compiled(x[0]), (x[0] * x[0]).sum())
    F.vectorize(sq)                                                     # the same kind again is recorded once
    R = F.TransformationRegistry
    assert [t.name for t in R.get_transformations(sq)] == ["vmap", "jit"] and R.count() == 1 and R.total_transformation_count() == 2
    assert R.has_transformation_of_type(sq, F.TransformationType.COMPILATION)
    assert not R.has_transformation_of_type(sq, F.TransformationType.PARALLELIZATION)
    assert R.get_transformations_by_type(sq, F.TransformationType.VECTORIZATION)[0].in_axes == 0
    par = F.parallelize(sq, pg=None)
    assert callable(par) and R.has_transformation_of_type(sq, F.TransformationType.PARALLELIZATION)

    @F.tensor_function(is_pure=False)
    def logs(x):
        print(x)
        return x

    with pytest.raises(ValueError, match="impure"):
        F.vectorize(logs)
    with pytest.raises(TypeError):
        F.JITTransformation()(42)
    assert R.unregister(sq) and not R.unregister(sq) and not R.has_transformations(sq)
    ctx = F.TransformationContext()
    ctx.debug_mode = True
    F.VMapTransformation(context=ctx)(sq)
    assert ctx.get_metadata("last_applied") == ("vmap", "sq")
    # entries go when their function goes
    def temp(x):
        return x
    F.vectorize(temp)
    n = R.count()
    del temp
    gc.collect()
    assert R.count() == n - 1
    R.clear()
    assert R.count() == 0


def test_clear_jit_cache_forces_a_retrace():
    f = F.jit(lambda a, b: (a + b).relu())
    a, b = torch.randn(4), torch.randn(4)
    f(a, b); f(a, b)
    assert f.stats["traced"] == 1 and f.stats["hits"] == 1
    assert F.clear_jit_cache() >= 1
    torch.testing.assert_close(f(a, b), (a + b).relu())
    assert f.stats["traced"] == 2
