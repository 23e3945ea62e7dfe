"""Configuration-driven quantisation: settings, per-layer overrides, PTQ with an accuracy guard, QAT wrapper,
conversion and verification, metrics and accuracy reports, CPU feature detection."""
import json

import pytest
import torch
import torch.nn as nn

from ml_framework_b200.quantization import config as Q
from ml_framework_b200.quantization.core import (EntropyCalibrator, MinMaxCalibrator, MovingAverageCalibrator, PercentileCalibrator,
                                                 QuantizationMode, QuantizedLinear, prepare_qat)


def _model(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 32), nn.ReLU(), nn.Linear(32, 4))


def _data(n=6, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(8, 16, generator=g) for _ in range(n)]


def test_config_presets_validation_and_factory():
    d, a, c = Q.QuantizationConfig.create_default(), Q.QuantizationConfig.create_aggressive(), Q.QuantizationConfig.create_conservative()
    assert d.validate() and a.accuracy_threshold == 0.05 and not a.fallback_to_fp32 and c.calibration_method is Q.CalibrationMethod.PERCENTILE
    assert "cal=min_max" in str(d) and Q.QuantizationType.UINT8.range() == (0, 255)
    for bad in (Q.QuantizationConfig(calibration_batch_size=0), Q.QuantizationConfig(accuracy_threshold=1.5),
                Q.QuantizationConfig(quantization_type=Q.QuantizationType.UINT8)):
        with pytest.raises(ValueError):
            bad.validate()
    f = Q.CalibratorFactory()
    kinds = {Q.CalibrationMethod.MIN_MAX: MinMaxCalibrator, Q.CalibrationMethod.ENTROPY: EntropyCalibrator,
             Q.CalibrationMethod.PERCENTILE: PercentileCalibrator, Q.CalibrationMethod.MOVING_AVERAGE: MovingAverageCalibrator}
    for m, k in kinds.items():
        assert isinstance(f.create(m), k)
    assert isinstance(f.create_percentile(99.0), PercentileCalibrator) and isinstance(f.create_moving_average(0.5), MovingAverageCalibrator)
    with pytest.raises(ValueError):
        f.create_percentile(10.0)


def test_layerwise_config():
    lw = Q.LayerwiseConfig()
    lw.set_layer_config("0", Q.QuantizationConfig.create_conservative())
    lw.disable_layer("4")
    lw.set_layer_mode("2", QuantizationMode.SYMMETRIC, QuantizationMode.ASYMMETRIC)
    assert lw.configured_layers == ["0", "4", "2"] and lw.get_disabled_layers() == ["4"] and lw.get_enabled_layers() == ["0", "2"]
    assert lw.get_effective_config("0").accuracy_threshold == 0.005 and lw.get_effective_config("9") is lw.global_config
    assert lw.is_layer_enabled("9") and not lw.is_layer_enabled("4") and lw.get_layer_config("9") is None
    assert lw.get_effective_config("2").activation_quantization is QuantizationMode.ASYMMETRIC
    assert lw.global_config.activation_quantization is QuantizationMode.SYMMETRIC          # the override copied, not aliased
    assert set(lw.get_layer_configuration_dictionary()) == {"0", "2"} and "4: off" in str(lw.get_layer_config("4"))
    twin = lw.clone()
    twin.enable_layer("4")
    assert not lw.is_layer_enabled("4") and twin.is_layer_enabled("4") and lw.validate()
    assert lw.remove_layer_config("0") and not lw.remove_layer_config("0")
    lw.clear_all_layer_configs()
    assert lw.configured_layers == []
    with pytest.raises(ValueError):
        lw.set_layer_config("", Q.QuantizationConfig())


def test_model_traversal():
    m = nn.Sequential(nn.Conv2d(3, 4, 3), nn.BatchNorm2d(4), nn.Flatten(), nn.Linear(4, 2))
    t = Q.ModelTraversal()
    assert [n for n, _ in t.get_all_layers(m)] == ["0", "1", "2", "3"]
    assert [n for n, _ in t.get_quantizable_layers(m)] == ["3"] and [n for n, _ in t.get_quantizable_layers(m, implemented_only=False)] == ["0", "3"]
    assert t.is_quantizable(m[0]) and not t.is_quantizable(m[1]) and t.supports_per_channel_quantization(m[3])
    assert t.get_layer_name(m, m[3]) == "3"
    with pytest.raises(KeyError):
        t.get_layer_name(m, nn.Linear(1, 1))


def test_static_and_dynamic_quantization_with_overrides_and_guard():
    ref = _model()
    data = _data()
    with torch.no_grad():
        want = torch.cat([ref(x) for x in data])

    def closeness(model):                                              # higher is better, 1.0 = identical
        with torch.no_grad():
            got = torch.cat([model(x) for x in data])
        return 1.0 - float((got - want).abs().mean() / want.abs().mean())

    lw = Q.LayerwiseConfig()
    lw.disable_layer("4")
    sq = Q.StaticQuantization()
    m = sq.quantize(_model(), data, layerwise=lw)
    assert isinstance(m[0], QuantizedLinear) and isinstance(m[2], QuantizedLinear) and isinstance(m[4], nn.Linear)
    assert sq.skipped_layers == ["4"] and sq.quantized_layers == ["0", "2"] and closeness(m) > 0.9
    assert m[0].act_qparams is not None
    with pytest.raises(ValueError, match="calibration batch"):
        Q.StaticQuantization().quantize(_model(), [])
    # a strict threshold sends layers back to fp32, a lax one keeps them
    strict = Q.StaticQuantization()
    ms = strict.quantize(_model(), data, Q.QuantizationConfig(accuracy_threshold=0.0, fallback_to_fp32=True), metric=closeness)
    assert strict.fallback_layers and all(isinstance(ms[int(n)], nn.Linear) for n in strict.fallback_layers)
    lax = Q.StaticQuantization()
    lax.quantize(_model(), data, Q.QuantizationConfig(accuracy_threshold=0.5), metric=closeness)
    assert lax.fallback_layers == [] and lax.quantized_layers == ["0", "2", "4"]
    dq = Q.DynamicQuantization()
    md = dq.quantize(_model(), Q.QuantizationConfig.create_aggressive())
    assert all(isinstance(md[i], QuantizedLinear) and md[i].act_qparams is None for i in (0, 2, 4)) and closeness(md) > 0.9
    # asymmetric activations after a ReLU use the range better: the zero point moves
    asym = Q.StaticQuantization().quantize(_model(), data, Q.QuantizationConfig(activation_quantization=QuantizationMode.ASYMMETRIC))
    assert int(asym[2].act_qparams.zero_point) == -128 and closeness(asym) > 0.9


def test_moving_average_statistics():
    s = Q.MovingAverageStatistics(0.5)
    s.update_batch([2.0, 4.0, 6.0])
    assert s.mean == 4.5 and (s.min, s.max, s.count) == (2.0, 6.0, 3) and s.variance == pytest.approx(8 / 3)
    s.update_tensor(torch.tensor([10.0, -2.0]))
    assert s.min == -2.0 and s.max == 10.0 and s.count == 5 and s.mean == pytest.approx(0.5 * 4.5 + 0.5 * 4.0)
    assert s.get_statistics()["count"] == 5
    s.reset()
    assert s.count == 0 and s.variance == 0.0
    with pytest.raises(ValueError):
        Q.MovingAverageStatistics(1.0)


def test_qat_wrapper_trains_observes_and_converts():
    torch.manual_seed(0)
    model = nn.Sequential(Q.QATModuleWrapper(nn.Linear(16, 32)), nn.ReLU(), Q.QATModuleWrapper(nn.Linear(32, 4)))
    conv = Q.QATModuleWrapper(nn.Conv2d(3, 4, 3, padding=1), Q.QuantizationConfig(enable_per_channel_quantization=False))
    assert conv(torch.randn(2, 3, 5, 5)).shape == (2, 4, 5, 5) and conv.weight_quantization_parameters.axis is None
    with pytest.raises(ValueError):
        Q.QATModuleWrapper(nn.ReLU())
    opt = torch.optim.SGD(model.parameters(), 0.05)
    x, y = torch.randn(64, 16), torch.randint(0, 4, (64,))
    first = None
    for _ in range(30):
        loss = nn.functional.cross_entropy(model(x), y)
        first = first or float(loss)
        opt.zero_grad(); loss.backward(); opt.step()
    assert float(loss) < first                                            # gradients pass the fake quantisers
    w0 = model[0]
    a, w = w0.get_activation_observer_statistics(), w0.get_weight_observer_statistics()
    assert a.count == 30 * 64 * 16 and a.min < 0 < a.max and w.count == 30 * 32 * 16 and w0.get_fake_quantization_node_count() == 2
    wq, qp = w0.quantize_weights()
    assert wq.dtype == torch.int8 and qp.axis == 0 and w0.activation_quantization_parameters is not None
    params = Q.ModelConversion.extract_trained_parameters(model)
    assert set(params) == {"0", "2"} and params["0"] is not None
    res = Q.ModelConversion.convert_with_report(model)
    r = res.report
    assert r.success and r.quantized_layers == 2 and r.source_fake_quant_nodes == 4 and r.weight_scale_range[0] > 0 and r.duration_s >= 0
    assert r.activation_scale_range[1] >= r.activation_scale_range[0] > 0
    q = res.quantized_model
    model.eval()
    ver = Q.ModelConversion.verify_quantized_model(q, model, x)
    assert ver.success and len(ver.passed_checks) == 7, ver.failed_checks
    agree = float((q(x).argmax(-1) == model(x).argmax(-1)).float().mean())
    assert agree > 0.9
    w0.reset_observers()
    assert w0.get_activation_observer_statistics() is None and w0.activation_quantization_parameters is None
    # failures are reported, not raised
    bad = Q.ModelConversion.convert_with_report(_model())
    assert not bad.report.success and "no QAT layers" in bad.report.error_message and bad.quantized_model is None
    with pytest.raises(RuntimeError):
        Q.ModelConversion.convert_to_quantized(_model())
    also = Q.ModelConversion.convert_to_quantized(prepare_qat(_model()))     # the package's own QAT layers convert too
    assert sum(isinstance(m, QuantizedLinear) for m in also.modules()) == 3
    failed = Q.ModelConversion.verify_quantized_model(_model())
    assert not failed.success and "has quantized layers" in failed.failed_checks


def test_metrics():
    logits = torch.tensor([[0.1, 0.7, 0.2], [0.5, 0.3, 0.2], [0.2, 0.3, 0.5]])
    target = torch.tensor([1, 1, 0])
    t1, t2 = Q.TopKAccuracy(1), Q.TopKAccuracy(2)
    t1.update(logits, target); t2.update(logits, target); t2.update(logits, target)
    assert t1.compute() == pytest.approx(1 / 3) and t2.compute() == pytest.approx(2 / 3) and t2.name == "top2_accuracy"
    ce = Q.CrossEntropyLoss()
    ce.update(logits, target)
    assert ce.compute() == pytest.approx(float(nn.functional.cross_entropy(logits, target))) and not ce.higher_is_better
    a, b = torch.tensor([1.0, 2.0, 3.0]), torch.tensor([1.0, 4.0, 0.0])
    mae, rmse = Q.MAE(), Q.RMSE()
    mae.update(a, b); rmse.update(a, b)
    assert mae.compute() == pytest.approx(5 / 3) and rmse.compute() == pytest.approx((13 / 3) ** 0.5)
    mae.reset()
    assert mae.compute() == 0.0
    with pytest.raises(ValueError):
        Q.TopKAccuracy(0)


def test_accuracy_comparison_and_reporter(tmp_path):
    torch.manual_seed(0)
    fp = _model()
    xs = _data(4)
    data = [(x, fp(x).argmax(-1)) for x in xs]                           # the float model is right by construction
    q = Q.DynamicQuantization().quantize(_model())
    cmp = Q.AccuracyComparison(Q.TopKAccuracy(1))
    rep = cmp.compare_models(fp, q, data, threshold=0.2, per_layer=True)
    assert rep.fp32_accuracy == 1.0 and 0.8 <= rep.quantized_accuracy <= 1.0 and rep.is_acceptable
    assert [r.layer_name for r in rep.per_layer_results] and len(rep.per_layer_results) == 3
    assert all(isinstance(m, nn.Linear) for m in (fp[0], fp[2], fp[4]))   # the one-at-a-time swaps were undone
    assert cmp.get_accuracy_delta(rep) == pytest.approx(rep.accuracy_drop) and cmp.get_per_layer_metrics(rep) == rep.per_layer_results
    impacts = [r.accuracy_impact for r in rep.per_layer_results]
    assert impacts == sorted(impacts, reverse=True)
    rep.per_layer_results[0].is_sensitive = True
    rep.per_layer_results[0].recommended_action = "keep in fp32"
    R = Q.AccuracyReporter()
    text = R.generate_text_report(rep)
    assert "Result:     ACCEPTABLE" in text and "SENSITIVE" in text and f"Keep in fp32: {rep.per_layer_results[0].layer_name}" in text
    js = json.loads(R.generate_json_report(rep))
    assert js["is_acceptable"] and js["recommended_fp32_layers"] == [rep.per_layer_results[0].layer_name] and len(js["quantizable_layers"]) == 2
    md = R.generate_markdown_report(rep)
    assert md.startswith("# Quantisation accuracy report") and "| yes | keep in fp32 |" in md
    for fmt, ext in ((Q.ReportFormat.TEXT, "txt"), (Q.ReportFormat.JSON, "json"), (Q.ReportFormat.MARKDOWN, "md")):
        p = tmp_path / f"r.{ext}"
        R.save_report(rep, str(p), fmt)
        assert p.read_text()
    loss_cmp = Q.AccuracyComparison(Q.CrossEntropyLoss())
    lrep = loss_cmp.compare_models(fp, q, data, threshold=10.0)
    assert loss_cmp.get_accuracy_delta(lrep) == pytest.approx(lrep.quantized_accuracy - lrep.fp32_accuracy) and lrep.is_acceptable
    strict = cmp.compare_models(fp, q, data, threshold=-1.0)
    assert not strict.is_acceptable and "NOT ACCEPTABLE" in R.generate_text_report(strict)


def test_cpu_feature_detection_from_flag_sets():
    assert Q.X86FeatureDetection.is_available() != Q.ARMFeatureDetection.is_available() or not Q.X86FeatureDetection.is_available()
    flags = {"sse4_1", "avx2", "avx512f", "avx512_vnni", "fma"}
    assert Q.X86FeatureDetection.get_detected_features(flags) == ["sse4_1", "avx2", "avx512f", "avx512_vnni"]
    assert Q.X86FeatureDetection.has_int8_dot_product(flags) and not Q.X86FeatureDetection.has_int8_dot_product({"avx2"})
    assert Q.ARMFeatureDetection.get_detected_features({"asimd", "asimddp", "aes"}) == ["asimd", "asimddp"]
    assert Q.ARMFeatureDetection.has_int8_dot_product({"i8mm"}) and not Q.ARMFeatureDetection.has_int8_dot_product({"asimd"})
    assert isinstance(Q.X86FeatureDetection.get_detected_features(), list)
