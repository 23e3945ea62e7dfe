"""CUDA source templates: rendering, generation for the three patterns, compilation for sm_100a, index-arithmetic oracles."""
import os
import shutil

import pytest
import torch
import torch.nn.functional as F

from ml_framework_b200.compiler import cuda_templates as T
from ml_framework_b200.compiler.jit_cuda import NvccCompiler

HAVE_NVCC = bool(shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"))


def test_renderer_substitutes_and_rejects_unknown_names():
    r = T.SimpleTemplateRenderer()
    t = "a={{a}} {{#if flag}}on {{b}}{{/if}}{{#if off}}never{{/if}}"
    assert r.render(t, {"a": 1, "b": "x", "flag": True, "off": False}) == "a=1 on x" and r.variables(t) == ["a", "b", "flag", "off"]
    with pytest.raises(KeyError):
        r.render("{{missing}}", {})
    with pytest.raises(KeyError):
        r.render("{{#if c}}x{{/if}}", {})


def test_operation_snippets_and_specification_checks():
    G = T.CudaOperationCodeGenerator
    assert "leaky_relu" in G.supported() and G.expression("relu") == "fmaxf(v, 0.f)" and G.expression("add", "ld(in1, i)") == "v + ld(in1, i)"
    assert G.expression("maximum", "b") == "fmaxf(v, b)"
    with pytest.raises(ValueError):
        G.expression("add")
    with pytest.raises(ValueError):
        G.expression("relu", "x")
    with pytest.raises(KeyError):
        G.expression("erf")
    for bad in (dict(pattern="fft"), dict(pattern="linear", dtype=torch.int32), dict(pattern="linear", activation="swish"), dict(pattern="linear", threads=100),
                dict(pattern="linear", name="9bad")):
        with pytest.raises(ValueError):
            T.KernelSpecification(**bad).validate()


def test_generated_sources_have_the_expected_structure():
    gen = T.CudaKernelGenerator()
    conv = gen.generate(T.KernelSpecification("conv_activation", "conv_relu", torch.bfloat16, "relu"))
    assert "using T = __nv_bfloat16;" in conv and "conv_relu_launch" in conv and "fmaxf(v, 0.f)" in conv and "float acc = ld(bias, oc);" in conv and "{{" not in conv
    nb = gen.generate(T.KernelSpecification("conv_activation", "conv_plain", has_bias=False))
    assert "float acc = 0.f;" in nb and "using T = float;" in nb
    lin = gen.generate(T.KernelSpecification("linear", "fc_gelu", torch.float16, "gelu"))
    assert "__shfl_xor_sync" in lin and "+ ld(bias, o)" in lin and "__half2float" in lin
    g = gen.generate(T.KernelSpecification("generic", "bias_tanh_mul", torch.float32, "relu", chain=[("add", "column"), ("tanh", "none"), ("mul", "tensor")]))
    assert "v = v + ld(in1, col);" in g and "v = tanhf(v);" in g and "v = v * ld(in2, i);" in g and "(const T*)in[2]" in g and "const T* __restrict__ in2" in g
    with pytest.raises(ValueError):
        gen.generate(T.KernelSpecification("generic", chain=[("add", "row")]))
    gen.register_template("custom", "// {{kernel_name}}")
    assert "custom" in gen.templates


@pytest.mark.skipif(not HAVE_NVCC, reason="nvcc not installed")
def test_every_pattern_compiles_for_sm_100a(tmp_path):
    gen, cc = T.CudaKernelGenerator(), NvccCompiler(cache_dir=str(tmp_path))
    specs = [T.KernelSpecification("conv_activation", "conv_relu_bf16", torch.bfloat16, "relu"),
             T.KernelSpecification("linear", "fc_sigmoid_f16", torch.float16, "sigmoid", has_bias=False, threads=128),
             T.KernelSpecification("generic", "bias_gelu_f32", torch.float32, "none", chain=[("add", "column"), ("gelu", "none"), ("maximum", "tensor")])]
    for s in specs:
        so = gen.compile(s, cc)
        assert so.exists() and so.stat().st_size > 0
    assert cc.compilations == 3
    gen.compile(specs[0], cc)
    assert cc.cache_hits == 1


def test_index_arithmetic_oracles_match_torch():
    torch.manual_seed(0)
    x, w, b = torch.randn(2, 3, 6, 5), torch.randn(4, 3, 3, 2), torch.randn(4)
    for stride, pad in ((1, 0), (2, 1)):
        got = T.reference_conv_activation(x, w, b, stride, pad, "relu")
        assert torch.allclose(got, torch.relu(F.conv2d(x, w, b, stride, pad)), atol=1e-4)
    assert torch.allclose(T.reference_conv_activation(x, w, None, 1, 1, "none"), F.conv2d(x, w, None, 1, 1), atol=1e-4)
    a, col, full = torch.randn(4, 6), torch.randn(6), torch.randn(4, 6)
    got = T.reference_generic([("add", "column"), ("tanh", "none"), ("mul", "tensor")], [a, col, full], "relu")
    assert torch.allclose(got, torch.relu(torch.tanh(a + col) * full))
