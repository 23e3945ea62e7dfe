"""The fp32 PyTorch statements of the kernels (the CPU path and the GPU tests' oracle) against torch's own operators,
plus small model / layer helpers, engine state, FSDP shard accumulation, version-manager queries."""
import math

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from ml_framework_b200.ops import reference as R


def test_reference_norms_rope_swiglu_attention_and_loss_match_torch():
    torch.manual_seed(0)
    x, g, b = torch.randn(5, 16), torch.randn(16), torch.randn(16)
    y, mean, rstd = R.layer_norm_ref(x, g, b, 1e-5)
    assert torch.allclose(y, F.layer_norm(x, (16,), g, b, 1e-5), atol=1e-5)
    assert torch.allclose(mean, x.mean(-1), atol=1e-6) and torch.allclose(rstd, 1 / torch.sqrt(x.var(-1, unbiased=False) + 1e-5), atol=1e-5)
    assert torch.allclose(R.layer_norm_ref(x, g, None)[0], F.layer_norm(x, (16,), g, None), atol=1e-5)
    yr, rr = R.rms_norm_ref(x, g, 1e-6)
    assert torch.allclose(yr, F.rms_norm(x, (16,), g, 1e-6), atol=1e-5) and rr.shape == (5,)
    q = torch.randn(7, 2, 8)
    pos = torch.arange(7)
    rot = R.rope_ref(q, pos, 10000.0)
    assert torch.allclose(rot[0], q[0]) and torch.allclose(rot.norm(dim=-1), q.norm(dim=-1), atol=1e-5)      # a rotation
    assert torch.allclose(R.rope_ref(rot, pos, 10000.0, inverse=True), q, atol=1e-5)
    # relative property: <rope(q, i), rope(k, j)> depends on i - j only
    k = torch.randn(7, 2, 8)
    a = (R.rope_ref(q[:1].expand(7, 2, 8), pos, 100.0) * R.rope_ref(k[:1].expand(7, 2, 8), pos, 100.0)).sum(-1)
    assert torch.allclose(a, a[0].expand_as(a), atol=1e-5)
    gu = torch.randn(3, 12)
    assert torch.allclose(R.swiglu_ref(gu), F.silu(gu[:, :6]) * gu[:, 6:])
    assert torch.allclose(R.swiglu_ref(gu, interleaved=True), F.silu(gu[:, 0::2]) * gu[:, 1::2])
    B, S, Hq, Hkv, D = 2, 6, 4, 2, 8
    qq, kk, vv = torch.randn(B, S, Hq, D), torch.randn(B, S, Hkv, D), torch.randn(B, S, Hkv, D)
    out, lse = R.attention_ref(qq, kk, vv, causal=True)
    want = F.scaled_dot_product_attention(qq.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=True, enable_gqa=True)
    assert torch.allclose(out, want.transpose(1, 2), atol=1e-5) and lse.shape == (B, Hq, S)
    dec, _ = R.attention_ref(qq[:, -1:], kk, vv, causal=True, start_pos=S - 1)                                # one query at the end
    assert torch.allclose(dec[:, 0], out[:, -1], atol=1e-5)
    full, _ = R.attention_ref(qq, kk, vv, causal=False, scale=0.5)
    want = F.scaled_dot_product_attention(qq.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), scale=0.5, enable_gqa=True)
    assert torch.allclose(full, want.transpose(1, 2), atol=1e-5)
    logits = torch.randn(6, 12, requires_grad=True)
    tgt = torch.tensor([1, 3, -1, 0, 9, 2])
    loss, d = R.cross_entropy_ref(logits.detach(), tgt, vocab=10, grad_scale=2.0)
    ref = F.cross_entropy(logits[:, :10], tgt.clamp(min=0), reduction="none") * (tgt >= 0)
    assert torch.allclose(loss, ref.detach(), atol=1e-6)
    (ref.sum() * 2.0).backward()
    assert torch.allclose(d, logits.grad, atol=1e-6) and d[:, 10:].abs().sum() == 0 and d[2].abs().sum() == 0


def test_layer_helpers_model_presets_and_flop_counts():
    from ml_framework_b200.models.gpt import GPT, GPTConfig
    from ml_framework_b200.models.llama import LlamaConfig
    from ml_framework_b200.models.mlp import MLP
    from ml_framework_b200.nn.layers import Linear, SwiGLUMLP
    lin = Linear(8, 4, bias=True)
    assert "in_features=8, out_features=4, bias=True" in repr(lin)
    gate, up = torch.arange(6.0).view(3, 2), -torch.arange(6.0).view(3, 2)
    inter = SwiGLUMLP.interleave(gate, up)
    assert inter.shape == (6, 2) and torch.equal(inter[0::2], gate) and torch.equal(inter[1::2], up)
    mlp = SwiGLUMLP(8, 16)
    x = torch.randn(3, 8)
    w = mlp.gate_up.weight
    want = (F.silu(x @ w[0::2].t()) * (x @ w[1::2].t())) @ mlp.down.weight.t()
    assert torch.allclose(mlp(x), want, atol=1e-5) and torch.allclose(mlp(x, residual=x), want + x, atol=1e-5)
    m = MLP()
    assert m(torch.randn(2, 784)).shape == (2, 10)
    g13 = GPTConfig.gpt_1_3b()
    assert 1.2e9 < g13.num_params() < 1.5e9 and g13.flops_per_token(2048) > 6 * g13.num_params()
    tiny = GPTConfig.tiny()
    model = GPT(tiny)
    assert sum(p.numel() for p in model.parameters()) == tiny.num_params()
    l8, l13, lt = LlamaConfig.llama_8b(), LlamaConfig.llama_13b(), LlamaConfig.tiny()
    assert 7.5e9 < l8.num_params() < 8.5e9 and 12.5e9 < l13.num_params() < 13.5e9 and lt.num_params() < 1e8
    assert l8.flops_per_token(4096) > 6 * l8.num_params() * 0.9


def test_engine_state_dict_close_and_single_device_step():
    from ml_framework_b200.engine import EngineConfig, TrainEngine
    from ml_framework_b200.models.gpt import GPT, GPTConfig
    torch.manual_seed(0)
    cfg = GPTConfig.tiny()
    eng = TrainEngine(GPT(cfg), EngineConfig(strategy="ddp", lr=1e-3))           # one process: the strategy degrades to none
    assert eng.strategy == "none"
    ids, tgt = torch.randint(0, cfg.vocab_size, (2, 16)), torch.randint(0, cfg.vocab_size, (2, 16))
    l0 = float(eng.step(ids, tgt).detach())
    for _ in range(4):
        last = float(eng.step(ids, tgt).detach())
    assert last < l0 and eng.steps == 5
    sd = eng.state_dict()
    assert sd["steps"] == 5 and sd["optimizer"]["step"] >= 1 and "scaler" in sd
    eng.close()
    with pytest.raises(ValueError):
        EngineConfig(strategy="zero9").validate()
    with pytest.raises(ValueError):
        EngineConfig(lr=0.0).validate()


def test_fsdp_shard_accumulator_and_version_queries():
    from ml_framework_b200.parallel.fsdp_state import FSDPGradientAccumulator
    from ml_framework_b200.serving import versioning as V

    class FakeFSDP:
        grad_shards = torch.zeros(4, dtype=torch.bfloat16)
    f = FakeFSDP()
    acc = FSDPGradientAccumulator(f, 2)
    f.grad_shards.fill_(1.0)
    assert not acc.add_gradients()
    f.grad_shards.fill_(3.0)
    assert acc.add_gradients() and acc.is_complete()
    acc.apply()
    assert torch.equal(f.grad_shards, torch.full((4,), 2.0, dtype=torch.bfloat16)) and acc.count == 0 and not acc.is_complete()
    with pytest.raises(ValueError):
        FSDPGradientAccumulator(f, 0)
    m = V.ModelVersionManager()
    for v in ("1.0.0", "1.1.0", "2.0.0"):
        m.register("llm", v, lambda x: x)
    m.promote("llm", "1.0.0")
    assert m.production("llm") == "1.0.0" and m.in_state("llm", V.VersionState.REGISTERED) == ["1.1.0", "2.0.0"]
    assert m.production("other") is None
    mon = V.VersionMonitor({"error_rate": 0.5})
    for ok in (True, True, False, True):
        mon.record("llm", "1.0.0", 0.010, ok=ok)
    for ok in (True, False, False, False):
        mon.record("llm", "1.1.0", 0.030, ok=ok)
    diff = mon.compare("llm", "1.0.0", "1.1.0")
    assert diff["error_rate"] == pytest.approx(0.5) and diff["latency_mean_s"] == pytest.approx(0.020) and diff["requests"] == 0
    assert mon.check("llm", "1.0.0") == [] and mon.check("llm", "1.1.0")[0].metric == "error_rate"
