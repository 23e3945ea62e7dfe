"""Learning-rate schedulers, the autocast policy, kernel dtype selection, gradient utilities and the software
16-bit types, on CPU: closed forms, comparison with torch's own schedulers and conversions, state round trips."""
import math
import random

import numpy as np
import pytest
import torch

from ml_framework_b200.amp import autocast as A
from ml_framework_b200.amp import softfloat as S
from ml_framework_b200.optim import schedulers as L


def _torch_curve(make, steps, lr=0.1):
    p = torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([p], lr=lr)
    sch = make(opt)
    out = [opt.param_groups[0]["lr"]]
    for _ in range(steps):
        opt.step()
        sch.step()
        out.append(opt.param_groups[0]["lr"])
    return out


@pytest.mark.parametrize("ours,theirs", [
    (lambda: L.StepDecay(0.1, 5, 0.5), lambda o: torch.optim.lr_scheduler.StepLR(o, 5, 0.5)),
    (lambda: L.MultiStepDecay(0.1, [3, 7, 12], 0.1), lambda o: torch.optim.lr_scheduler.MultiStepLR(o, [3, 7, 12], 0.1)),
    (lambda: L.ExponentialDecay(0.1, 0.9), lambda o: torch.optim.lr_scheduler.ExponentialLR(o, 0.9)),
    (lambda: L.CosineAnnealing(0.1, 20, 0.001), lambda o: torch.optim.lr_scheduler.CosineAnnealingLR(o, 20, 0.001)),
    (lambda: L.CosineAnnealingWarmRestarts(0.1, 4, 2, 0.0), lambda o: torch.optim.lr_scheduler.CosineAnnealingWarmRestarts(o, 4, 2, 0.0)),
    (lambda: L.PolynomialDecay(0.1, 15, 0.0, 2.0), lambda o: torch.optim.lr_scheduler.PolynomialLR(o, 15, 2.0)),
])
def test_schedulers_follow_torch_curves(ours, theirs):
    s = ours()
    ref = _torch_curve(theirs, 20)
    got = [s.get_lr(0)] + [s.step() for _ in range(20)]
    assert got == pytest.approx(ref, rel=1e-6, abs=1e-9)


def test_warmup_cycles_plateau_and_composition():
    w = L.LinearWarmup(1.0, 10, after=L.CosineAnnealing(1.0, 100))
    assert w.get_lr(0) == 0.0 and w.get_lr(5) == pytest.approx(0.5) and w.get_lr(10) == pytest.approx(1.0)
    assert w.get_lr(110) == pytest.approx(0.0, abs=1e-12)
    c = L.ConstantWarmup(1.0, 3, 0.01)
    assert [c.get_lr(i) for i in range(5)] == [0.01, 0.01, 0.01, 1.0, 1.0]
    cyc = L.CyclicLR(0.1, 1.0, 4)
    assert cyc.get_lr(0) == pytest.approx(0.1) and cyc.get_lr(4) == pytest.approx(1.0) and cyc.get_lr(8) == pytest.approx(0.1)
    assert L.CyclicLR(0.1, 1.0, 4, mode="triangular2").get_lr(12) == pytest.approx(0.1 + 0.9 * 0.5)
    oc = L.OneCycle(1.0, 100)
    lrs = [oc.get_lr(i) for i in range(101)]
    assert lrs[0] == pytest.approx(1 / 25) and max(lrs) == pytest.approx(1.0) and lrs.index(max(lrs)) == 30
    assert lrs[-1] == pytest.approx(1 / 25 / 1e4) and all(a <= b + 1e-12 for a, b in zip(lrs[:30], lrs[1:31]))
    # plateau: a worse metric for more than `patience` steps cuts the rate, the cooldown holds it
    p = L.ReduceLROnPlateau(1.0, factor=0.5, patience=2, cooldown=1, min_lr=0.2)
    seq = [p.step(m) for m in (1.0, 0.9, 0.95, 0.95, 0.95, 0.95, 0.95, 0.95, 0.95, 0.95, 0.95, 0.95)]
    assert seq[:4] == [1.0, 1.0, 1.0, 1.0] and seq[4] == 0.5 and 0.25 in seq and min(seq) == 0.25 and p.step(0.95) >= 0.2
    assert L.ReduceLROnPlateau(1.0, mode="max", patience=0).step(1.0) == 1.0
    with pytest.raises(ValueError):
        L.ReduceLROnPlateau(1.0, factor=1.5)
    ch = L.ChainedScheduler(0.2, [L.StepDecay(1.0, 2, 0.5), L.ExponentialDecay(1.0, 0.9)])
    assert ch.get_lr(4) == pytest.approx(0.2 * 0.25 * 0.9 ** 4)
    sq = L.SequentialScheduler([L.ConstantLR(0.1), L.StepDecay(0.1, 2, 0.1), L.ConstantLR(0.5)], [3, 7])
    assert [round(sq.get_lr(i), 6) for i in (0, 2, 3, 5, 6, 7, 9)] == [0.1, 0.1, 0.1, 0.01, 0.01, 0.5, 0.5]
    with pytest.raises(ValueError):
        L.SequentialScheduler([L.ConstantLR(0.1), L.ConstantLR(0.2)], [1, 2])
    with pytest.raises(ValueError):
        L.StepDecay(0.1, 0)
    with pytest.raises(ValueError):
        L.ConstantLR(-1.0)


def test_scheduler_state_layerwise_rates_and_callback():
    s = L.CosineAnnealing(0.3, 50, 0.01)
    for _ in range(17):
        s.step()
    t = L.CosineAnnealing(1.0, 1)
    t.load_state_dict(s.state_dict())
    assert t.step_count == 17 and t.current_lr == pytest.approx(s.current_lr) and t.step() == pytest.approx(s.step())
    s.reset()
    assert s.current_lr == pytest.approx(0.3)
    lw = L.LayerWiseLRDecay(1.0, 4, 0.5)
    assert [lw.lr_for_layer(i) for i in range(4)] == [0.125, 0.25, 0.5, 1.0]
    ps = [(f"blocks.{i}.w", torch.nn.Parameter(torch.zeros(1))) for i in range(4)]
    groups = lw.param_groups(ps, lambda n: int(n.split(".")[1]))
    assert [g["lr"] for g in groups] == [0.125, 0.25, 0.5, 1.0] and all(len(g["params"]) == 1 for g in groups)
    d = L.DiscriminativeLR(0.1, {"embed": 0.1, "blocks.": 0.5, "blocks.3": 2.0})
    assert d.lr_for("embed.weight") == pytest.approx(0.01) and d.lr_for("blocks.1.w") == pytest.approx(0.05)
    assert d.lr_for("blocks.3.w") == pytest.approx(0.2) and d.lr_for("head") == pytest.approx(0.1)

    class Opt:
        lr = None

        def set_learning_rate(self, v):
            self.lr = v
    o = Opt()
    cb = L.LRSchedulerCallback(L.StepDecay(1.0, 2, 0.1), o)
    for b in range(4):
        cb.on_batch_end(b)
    assert o.lr == pytest.approx(0.01)
    o2 = Opt()
    cb2 = L.LRSchedulerCallback(L.ReduceLROnPlateau(1.0, factor=0.5, patience=0), o2, per_batch=False)
    cb2.on_batch_end(0)
    assert o2.lr is None

    class Ctx:
        val_loss = 1.0
    cb2.on_epoch_end(0, Ctx())
    cb2.on_epoch_end(1, Ctx())
    assert o2.lr == 0.5


def test_autocast_policy_registry_and_context():
    reg = A.AmpRegistry()
    cfg = A.AmpConfig.create_bf16()
    assert reg.rule("Linear") == A.OpPrecision.LOWER and reg.rule("softmax") == A.OpPrecision.FP32 and reg.rule("argsort") == A.OpPrecision.KEEP
    assert reg.get_forward_dtype("matmul", cfg) == torch.bfloat16 and reg.get_forward_dtype("layernorm", cfg) == torch.float32
    assert reg.get_forward_dtype("argsort", cfg, torch.float16) == torch.float16
    assert reg.get_backward_dtype("cross_entropy", cfg) == torch.float32
    reg.register_custom_op("my_op", torch.float16, torch.float32)
    assert reg.get_forward_dtype("MY_OP", cfg) == torch.float16 and reg.get_backward_dtype("my_op", cfg) == torch.float32
    reg.unregister("my_op")
    assert reg.get_forward_dtype("my_op", cfg) == torch.float32
    reg.register_blacklist("linear")
    assert reg.get_forward_dtype("linear", cfg) == torch.float32
    off = A.AmpConfig(enabled=False)
    assert reg.get_forward_dtype("matmul", off, torch.float32) == torch.float32
    assert A.AmpConfig.create_fp16().target_dtype == torch.float16 and cfg.initial_loss_scale == 8.0
    assert A.AutoCast.current() is None
    with A.AutoCast.bf16(device_type="cpu") as outer:
        assert A.AutoCast.current() is outer
        x = torch.randn(4, 4)
        assert outer.cast(x, "linear").dtype == torch.bfloat16 and outer.cast(x, "softmax").dtype == torch.float32
        assert outer.cast(torch.arange(3), "linear").dtype == torch.int64
        assert torch.mm(x, x).dtype == torch.bfloat16               # torch.autocast follows the same policy
        with A.AutoCast(A.AmpConfig(enabled=False), device_type="cpu") as inner:
            assert A.AutoCast.current() is inner and inner.cast(x, "linear").dtype == torch.float32
        assert A.AutoCast.current() is outer
    assert A.AutoCast.current() is None


def test_kernel_selector_gradient_utils_and_clipping():
    sel = A.KernelSelector()
    assert sel.get_kernel_dtype("linear", torch.bfloat16) == torch.bfloat16
    assert sel.get_kernel_dtype("linear", torch.float16) == torch.bfloat16          # no fp16 GEMM: the bf16 one serves
    assert sel.get_kernel_dtype("adamw", torch.bfloat16) == torch.float32
    assert sel.get_kernel_dtype("unknown_op", torch.bfloat16) == torch.float32
    best = sel.select_best_kernel("matmul")
    assert best.dtype == torch.bfloat16 and best.tensor_cores and sel.select_best_kernel("nope") is None
    sel.registry.register("linear", A.KernelCapability(torch.float8_e4m3fn, True, 32.0, available=False))
    assert sel.select_best_kernel("linear").dtype == torch.bfloat16                  # unavailable kernels are not chosen
    g = [torch.full((4,), 8.0), None, torch.full((2,), -4.0)]
    un = A.GradientUtils.unscale(g, 4.0)
    assert un[1] is None and torch.equal(un[0], torch.full((4,), 2.0)) and torch.equal(g[0], torch.full((4,), 8.0))
    A.GradientUtils.unscale_in_place(g, 2.0)
    assert torch.equal(g[2], torch.full((2,), -2.0))
    assert not A.GradientUtils.check_overflow(g)
    g[0][1] = float("inf")
    assert A.GradientUtils.check_overflow(g)
    assert A.GradientUtils.find_overflow_gradients({"a": g[0], "b": g[2], "c": None}) == ["a"]
    grads = [torch.tensor([3.0, 0.0]), torch.tensor([0.0, 4.0])]
    assert float(A.GradientClipper.global_norm(grads)) == pytest.approx(5.0)
    n = A.GradientClipper.clip_by_norm(grads, 1.0)
    assert float(n) == pytest.approx(5.0) and float(A.GradientClipper.global_norm(grads)) == pytest.approx(1.0, rel=1e-4)
    A.GradientClipper.clip_by_value(grads, 0.5)
    assert max(float(t.abs().max()) for t in grads) <= 0.5
    with pytest.raises(ValueError):
        A.GradientClipper.clip_by_norm(grads, 0.0)
    with pytest.raises(ValueError):
        A.GradientClipper.clip_by_value(grads, -1.0)
    assert float(A.GradientClipper.global_norm([])) == 0.0


def test_software_half_and_bfloat16_are_bit_exact():
    random.seed(0)
    vals = [random.uniform(-1, 1) * 10 ** random.uniform(-42, 38) for _ in range(5000)]
    vals += [0.0, -0.0, 1.0, 65504.0, 65519.9, 65520.0, 6e-8, 2.98e-8, 2.99e-8, 2 ** -24, 2 ** -25, 2 ** -14,
             2 ** -14 * (1 - 2 ** -11), 3.4e38, float("inf"), -float("inf")]
    t = torch.tensor(vals, dtype=torch.float32)
    hb = t.to(torch.float16).view(torch.int16).numpy().astype(np.uint16)
    bb = t.to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16)
    assert np.array_equal(np.array([S.float_to_half_bits(v) for v in t.tolist()], dtype=np.uint16), hb)
    assert np.array_equal(np.array([S.float_to_bfloat16_bits(v) for v in t.tolist()], dtype=np.uint16), bb)
    assert np.array_equal(S.to_bfloat16_bits(t.numpy()), bb) and np.array_equal(S.to_half_bits(t.numpy()), hb)
    assert np.array_equal(S.from_bfloat16_bits(bb), t.to(torch.bfloat16).float().numpy())
    assert np.array_equal(S.from_half_bits(hb), t.to(torch.float16).float().numpy())
    assert S.Half(float("nan")).is_nan() and S.BFloat16(float("nan")).is_nan() and S.Half(1e6).is_inf()
    assert float(S.Half(1.0) + S.Half(2 ** -11)) == 1.0 and float(S.Half(1.0) + S.Half(2 ** -10)) == 1.0 + 2 ** -10
    assert float(S.BFloat16(3.14159)) == 3.140625 and float(-S.Half(2.5)) == -2.5 and S.Half(0.5) < S.Half(0.75)
    assert float(S.BFloat16(2.0) * S.BFloat16(1.5) / S.BFloat16(4.0) - S.BFloat16(0.25)) == 0.5
    assert S.Half(1.5) == S.Half(1.5) and len({S.Half(1.5), S.Half(1.5), S.Half(2.0)}) == 2
    assert S.round_trip_error([1.0, 3.3, 1e-3, 123.456], "bfloat16") <= 2 ** -8
    assert S.round_trip_error([1.0, 3.3, 1e-3, 123.456], "half") <= 2 ** -11


def test_precision_helpers_gradient_layer_and_mixed_precision_checkpoints(tmp_path):
    import torch.nn as nn

    from ml_framework_b200.optim import mixed_precision as MP
    P = MP.Precision
    cap = MP.HardwareDetector.detect_capabilities()
    assert cap.supports_fp32 and cap is MP.HardwareDetector.detect_capabilities() and cap.is_bf16_available
    MP.HardwareDetector.reset_cache()
    assert MP.HardwareDetector.get_recommended_precision() in (P.FP32, P.BF16, P.FP16)
    t = torch.tensor([1.0, 70000.0])
    assert MP.PrecisionConverter.detect_precision(t) is P.FP32 and MP.PrecisionConverter.convert(t, P.BF16).dtype == torch.bfloat16
    assert MP.PrecisionConverter.convert(t, P.FP32) is t
    C = MP.PrecisionConverter.is_conversion_safe
    assert C(P.FP16, P.FP32) and C(P.FP32, P.BF16) and not C(P.FP32, P.FP16, t) and C(P.FP32, P.FP16, t[:1]) and not C(P.FP32, P.FP16)
    with pytest.raises(TypeError):
        MP.PrecisionConverter.convert(torch.tensor([1]), P.FP16)
    with pytest.raises(TypeError):
        MP.PrecisionConverter.detect_precision(torch.tensor([1.0], dtype=torch.float64))

    layer = MP.GradientConversionLayer(MP.MixedPrecisionOptions(initial_loss_scale=8.0, max_grad_norm=1.0, growth_interval=2))
    assert float(layer.scale_loss(torch.tensor(2.0))) == 16.0
    grads, skip = layer.process_gradients({"w": torch.full((4,), 16.0, dtype=torch.bfloat16)})
    assert not skip and grads["w"].dtype == torch.float32 and layer.last_gradient_norm == pytest.approx(4.0)
    assert float(grads["w"].norm()) == pytest.approx(1.0, rel=1e-4) and layer.clip_count == 1
    _, skip = layer.process_gradients({"w": torch.tensor([float("inf")])})
    assert skip and layer.loss_scale == 4.0                                            # backed off
    layer.process_gradients({"w": torch.tensor([0.1])}); layer.process_gradients({"w": torch.tensor([0.1])})
    st = layer.get_stats()
    assert layer.loss_scale == 8.0 and st.loss_scaler_stats.total_overflows == 1 and st.clip_count == 1 and "clip at 1" in str(st)
    layer.reset()
    assert layer.loss_scale == 8.0 and layer.clip_count == 0 and layer.get_stats().loss_scaler_stats.total_steps == 0

    torch.manual_seed(0)
    def make():
        torch.manual_seed(0)
        m = nn.Sequential(nn.Linear(4, 8), nn.LayerNorm(8), nn.Linear(8, 1))
        return m, MP.MixedPrecisionOptimizer(m, lambda ps: torch.optim.SGD(ps, 0.1, momentum=0.9), MP.MixedPrecisionOptions(precision="bf16"))
    x, y = torch.randn(16, 4), torch.randn(16, 1)

    def step(m, opt):
        opt.zero_grad()
        dt = next(m.parameters()).dtype
        loss = ((m(x.to(dt)).float() - y) ** 2).mean()
        opt.scale_loss(loss).backward()
        opt.step()
        return float(loss.detach())
    m1, o1 = make()
    for _ in range(3):
        step(m1, o1)
    M = MP.MixedPrecisionCheckpointManager
    ck = M.create_checkpoint(o1, {"note": "after 3"})
    assert M.validate_checkpoint(ck) and ck.step_count == 3 and ck.metadata == {"note": "after 3"} and ck.options["precision"] == "bf16"
    path = str(tmp_path / "mp.ckpt")
    M.save_checkpoint(ck, path)
    after = [step(m1, o1) for _ in range(3)]
    m2, o2 = make()
    loaded = M.load_and_restore(o2, path)
    assert loaded.step_count == 3 and o2.step_count == 3
    assert [step(m2, o2) for _ in range(3)] == after                                   # the run continues bit for bit
    broken = M.load_checkpoint(path)
    broken.master_weights["0.weight"][0, 0] = float("nan")
    assert not M.validate_checkpoint(broken)
    with pytest.raises(ValueError):
        M.restore_checkpoint(o2, broken)
    other = M.load_checkpoint(path)
    other.version = 9
    assert not M.validate_checkpoint(other)
    with pytest.raises(FileNotFoundError):
        M.load_checkpoint(str(tmp_path / "none"))
