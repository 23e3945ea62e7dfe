"""AMP integrations: optimizer wrapper that reports skipped steps, overflow statistics, casts, precision rules, autograd function."""
import pytest
import torch
import torch.nn as nn

from ml_framework_b200.amp import integrations as A
from ml_framework_b200.amp.autocast import OpPrecision
from ml_framework_b200.amp.grad_scaler import DynamicLossScaler, DynamicScalerConfig
from ml_framework_b200.dist.process_group import run_fake_world


def test_wrapper_skips_on_overflow_backs_off_and_resumes():
    torch.manual_seed(0)
    lin = nn.Linear(4, 1)
    w = A.AmpOptimizerWrapper(torch.optim.SGD(lin.parameters(), lr=0.1), DynamicLossScaler(DynamicScalerConfig(initial_scale=1024.0, growth_interval=2)),
                              named_parameters=lin.named_parameters())
    x = torch.randn(8, 4)
    before = lin.weight.detach().clone()
    w.zero_grad()
    w.backward(lin(x).pow(2).mean())
    assert torch.allclose(lin.weight.grad, torch.autograd.grad(lin(x).pow(2).mean(), lin.weight)[0] * 1024, rtol=1e-5)
    assert w.step() is True and not torch.equal(lin.weight, before) and w.scale == 1024.0
    w.zero_grad()
    w.backward(lin(x).pow(2).mean())
    lin.weight.grad[0, 0] = float("inf")
    held = lin.weight.detach().clone()
    assert w.step() is False and torch.equal(lin.weight, held) and w.scale == 512.0
    s = w.stats
    assert (s.total_steps, s.overflow_steps, s.consecutive_overflows, s.last_overflow_step) == (2, 1, 1, 2) and s.overflow_parameters == {"weight": 1} and s.overflow_rate == 0.5
    for _ in range(2):
        w.zero_grad()
        w.backward(lin(x).pow(2).mean())
        assert w.step()
    assert w.scale == 1024.0 and w.stats.consecutive_overflows == 0 and w.stats.max_consecutive_overflows == 1
    sd = w.state_dict()
    w2 = A.AmpOptimizerHelper.wrap(torch.optim.SGD(lin.parameters(), lr=0.1))
    w2.load_state_dict(sd)
    assert w2.scale == 1024.0 and w2.stats.total_steps == 4
    clip = A.AmpOptimizerWrapper(torch.optim.SGD(lin.parameters(), lr=0.0), max_grad_norm=1e-3)
    clip.zero_grad()
    clip.backward(lin(x).pow(2).mean() * 100)
    clip.step()
    assert float(torch.cat([p.grad.reshape(-1) for p in lin.parameters()]).norm()) <= 1.001e-3


def test_wrapper_agrees_on_overflow_across_ranks():
    def run(pg):
        lin = nn.Linear(2, 1)
        w = A.AmpOptimizerWrapper(torch.optim.SGD(lin.parameters(), lr=0.1), process_group=pg)
        w.backward(lin(torch.ones(1, 2)).sum())
        if pg.rank == 1:
            lin.bias.grad.fill_(float("nan"))
        return w.step()
    assert run_fake_world(2, run) == [False, False]


def test_overflow_stats_scale_factor_and_casts():
    s = A.ScaleFactor(65536.0)
    assert s.inverse == 1 / 65536 and s.grow().value == 131072.0 and s.backoff().value == 32768.0 and s.is_power_of_two() and not A.ScaleFactor(3.0).is_power_of_two()
    assert A.ScaleFactor(2.0 ** 24).grow().value == 2.0 ** 24 and A.ScaleFactor(1.0).backoff().value == 1.0 and A.ScaleFactor(0.25).is_power_of_two()
    for bad in (0.0, -1.0, float("inf"), float("nan")):
        with pytest.raises(ValueError):
            A.ScaleFactor(bad)
    f, i = torch.ones(2), torch.ones(2, dtype=torch.int64)
    assert A.AmpCast.to_bf16(f).dtype == torch.bfloat16 and A.AmpCast.to_fp16(i) is i and A.AmpCast.to_fp32(f) is f
    nest = A.AmpCast.cast_all({"a": [f, i], "b": (f.half(), 3)}, torch.bfloat16)
    assert nest["a"][0].dtype == torch.bfloat16 and nest["a"][1].dtype == torch.int64 and nest["b"][0].dtype == torch.bfloat16 and nest["b"][1] == 3
    a, b, c = A.AmpCast.promote(f.half(), f.bfloat16(), i)
    assert a.dtype == b.dtype == torch.float32 and c.dtype == torch.int64 and A.AmpCast.promote(f.half(), f.half())[0].dtype == torch.float16
    assert A.is_low_precision(f.half()) and not A.is_low_precision(f) and A.dtype_bytes(torch.bfloat16) == 2
    mx, tiny, eps = A.dtype_range(torch.float16)
    assert mx == 65504.0 and eps == 2 ** -10 and A.would_overflow(torch.tensor([7e4]), torch.float16) and not A.would_overflow(torch.tensor([7e4]), torch.bfloat16)
    assert not A.would_overflow(torch.zeros(0), torch.float16)


def test_precision_rules_and_autocast_constructors():
    rules = [A.OpPrecisionRule("conv*", OpPrecision.LOWER), A.OpPrecisionRule("softmax", OpPrecision.FP32), A.OpPrecisionRule("conv_transpose", OpPrecision.FP32, priority=5)]
    r = A.OpPrecisionRule.resolve
    assert r(rules, "conv2d") == OpPrecision.LOWER and r(rules, "conv_transpose") == OpPrecision.FP32 and r(rules, "softmax") == OpPrecision.FP32 and r(rules, "gather") == OpPrecision.KEEP
    assert A.autocast_fp16().cfg.target_dtype == torch.float16 and A.autocast_bf16().cfg.target_dtype == torch.bfloat16


class _Square(A.AmpAutogradFunction):
    forward_dtype = torch.float32

    @staticmethod
    def amp_forward(ctx, x):
        ctx.save_for_backward(x)
        ctx.seen = x.dtype
        return x * x

    @staticmethod
    def amp_backward(ctx, g):
        (x,) = ctx.saved_tensors
        ctx.grad_dtype = g.dtype
        return 2 * x * g


def test_amp_autograd_function_applies_its_policy():
    x = torch.tensor([1.5, -2.0], dtype=torch.bfloat16, requires_grad=True)
    y = _Square.apply(x)
    assert y.dtype == torch.float32
    y.to(torch.bfloat16).sum().backward()
    assert x.grad.dtype == torch.bfloat16 and x.grad.tolist() == [3.0, -4.0]
    out = A.AmpAutogradHelper.run_in_fp32(lambda t: torch.softmax(t, -1), torch.randn(2, 3).half())
    assert out.dtype == torch.float16
    lin = nn.Linear(2, 1)
    lin(torch.ones(1, 2)).sum().backward()
    lin.bias.grad.fill_(float("inf"))
    assert A.AmpAutogradHelper.nonfinite_parameters(lin.named_parameters()) == ["bias"]


def test_master_copies_and_scaler_context():
    model = nn.Linear(3, 2).bfloat16()
    master = A.AmpOptimizerHelper.master_copy(model.parameters())
    assert all(m.dtype == torch.float32 and m.requires_grad for m in master)
    model(torch.ones(1, 3, dtype=torch.bfloat16)).float().sum().backward()
    A.AmpOptimizerHelper.copy_grads_to_master(model.parameters(), master)
    assert master[0].grad.dtype == torch.float32 and torch.equal(master[0].grad, model.weight.grad.float())
    with torch.no_grad():
        master[0].add_(1.0)
    A.AmpOptimizerHelper.copy_master_to_model(master, model.parameters())
    assert torch.equal(model.weight.float(), master[0].bfloat16().float())
    with A.grad_scaler_context() as ctx:
        l = ctx.scale(torch.tensor(2.0))
        assert float(l) == 2.0 * float(ctx.scaler.scale)
    static = A.AmpOptimizerHelper.wrap(torch.optim.SGD(model.parameters(), lr=0.1), A.AmpConfig(loss_scaling=False))
    assert static.scale == 1.0
