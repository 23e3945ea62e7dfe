"""Run-time compiled fused element-wise chains: source generation and the nvcc build are checked without a GPU, the
launch against an fp32 PyTorch statement of the chain on one."""
import os
import shutil

import pytest
import torch

from ml_framework_b200.compiler import jit_cuda as J

HAVE_NVCC = bool(shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"))


def test_chain_arity_reference_evaluation_and_validation():
    assert J.chain_arity(["mul", "add", "relu"]) == 3 and J.chain_arity(["gelu"]) == 1
    with pytest.raises(KeyError):
        J.chain_arity(["mul", "bessel"])
    torch.manual_seed(0)
    a, b, c = torch.randn(3, 257)
    f = J.compile_chain(["mul", "add", "relu", "square"])
    assert torch.allclose(f(a, b, c), torch.relu(a * b + c) ** 2)                 # CPU tensors: the PyTorch path
    out = torch.empty_like(a)
    assert f(a, b, c, out=out) is out and torch.allclose(out, torch.relu(a * b + c) ** 2)
    with pytest.raises(ValueError):
        f(a, b)                                                                    # the chain reads three tensors
    with pytest.raises(ValueError):
        f(a, b, c[:100])                                                           # shapes must agree


def test_generated_source_is_complete_and_specialised():
    f = J.compile_chain(["sub", "sigmoid", "maximum"])
    src = f.source(torch.bfloat16, J.KernelConfig(threads=512, unroll=4))
    assert "using T = __nv_bfloat16;" in src and "constexpr int UNROLL = 4;" in src and "__launch_bounds__(512)" in src
    assert src.count("const T* __restrict__ in") == 3 and "_launch(void* out_" in src and "fmaxf(v, x)" in src
    assert "constexpr int V = 4;" in f.source(torch.float32)
    with pytest.raises(TypeError):
        f.source(torch.int32)
    # the grid limit is a launch argument: it does not change the source, so variants are shared
    assert f.source(torch.float32, J.KernelConfig(ctas_per_sm=4)) == f.source(torch.float32, J.KernelConfig(ctas_per_sm=8))
    assert len({c.compile_key() for c in J.search_space()}) == 6 and len(J.search_space()) == 12


@pytest.mark.skipif(not HAVE_NVCC, reason="nvcc not installed")
def test_nvcc_builds_a_loadable_object_once_per_source(tmp_path):
    comp = J.NvccCompiler(cache_dir=str(tmp_path))
    f = J.FusedElementwise(["mul", "add", "gelu"], compiler=comp)
    v = f.variant(torch.bfloat16, f.default_config)                     # generate, compile for sm_100a, load
    assert v.path.exists() and v.n_in == 3 and comp.compilations == 1
    assert f.variant(torch.bfloat16, f.default_config) is v             # in-process cache
    g = J.FusedElementwise(["mul", "add", "gelu"], compiler=comp)
    g.variant(torch.bfloat16, g.default_config)                         # another object, same source: the file is reused
    assert comp.compilations == 1 and comp.cache_hits >= 1
    bad = "this is not CUDA"
    with pytest.raises(J.CompileError):
        comp.compile(bad)


def test_graph_executor_runs_fused_chain_op():
    from ml_framework_b200.compiler.ir import Op, _execute
    torch.manual_seed(1)
    a, b = torch.randn(2, 64)
    op = Op("fused_elementwise", ["a", "b"], "y", {"chain": [("mul", True), ("tanh", False), ("neg", False)]})
    assert torch.allclose(_execute(op, [a, b]), -torch.tanh(a * b))
    from ml_framework_b200.compiler.fusion import FusionEngine
    f = FusionEngine.compile_chain(op.attrs["chain"])
    assert torch.allclose(f(a, b), -torch.tanh(a * b))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_chain_kernel_matches_fp32_reference(dtype, tmp_path):
    if not J.NvccCompiler().available():
        pytest.skip("no nvcc on this machine: nothing to compile the generated source with")
    torch.manual_seed(2)
    comp = J.NvccCompiler(cache_dir=str(tmp_path))
    f = J.FusedElementwise(["mul", "add", "silu", "maximum"], compiler=comp)
    for n in (8 * 1024 * 1024 + 5, 1000, 7):                            # vector body + tail, small, tail only
        xs = [torch.randn(n, device="cuda").to(dtype) for _ in range(4)]
        ref = J.eval_chain_torch(f.chain, [x.float() for x in xs])
        out = f(*xs)
        torch.cuda.synchronize()
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        assert torch.allclose(out.float(), ref, atol=tol, rtol=tol)
    # operands that are not 16-byte aligned take the scalar path
    base = [torch.randn(4099, device="cuda").to(dtype) for _ in range(4)]
    xs = [t[1:] for t in base]
    out = torch.empty(4099, device="cuda", dtype=dtype)[1:]
    ref = J.eval_chain_torch(f.chain, [x.float() for x in xs])
    # views are contiguous but offset by one element
    f.variant(dtype, f.default_config).launch(out, xs, 148 * 8)
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), ref, atol=2e-2 if dtype == torch.bfloat16 else 1e-5, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5)
    assert comp.compilations == 1


@pytest.mark.gpu
def test_graph_fusion_pass_runs_the_generated_kernel_on_gpu():
    if not J.NvccCompiler().available():
        pytest.skip("no nvcc on this machine: nothing to compile the generated source with")
    from ml_framework_b200.compiler.ir import Op, _execute
    a, b = torch.randn(2, 4096, device="cuda").to(torch.bfloat16)
    op = Op("fused_elementwise", ["a", "b"], "y", {"chain": [("add", True), ("relu", False)]})
    y = _execute(op, [a, b])
    torch.cuda.synchronize()
    assert torch.allclose(y.float(), torch.relu(a.float() + b.float()), atol=2e-2, rtol=2e-2)
