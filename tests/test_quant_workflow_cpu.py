"""Per-channel helpers, calibration process, evaluation / regression / report, sensitivity plan, QAT schedule and checkpointing."""
import json

import pytest
import torch
import torch.nn as nn

from ml_framework_b200.quantization import workflow as Q
from ml_framework_b200.quantization.core import FakeQuantize, QuantizedLinear, prepare_qat


def _clf(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 10))


def _data(n=6, bs=8, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(bs, 16, generator=g), torch.randint(0, 10, (bs,), generator=g)) for _ in range(n)]


def test_per_channel_round_trip_beats_per_tensor_on_uneven_rows():
    torch.manual_seed(0)
    w = torch.randn(8, 3, 3, 3) * torch.logspace(-2, 1, 8).view(8, 1, 1, 1)
    qp = Q.PerChannelOperations.qparams(w, axis=0)
    q = Q.PerChannelOperations.quantize(w, qp)
    assert q.dtype == torch.int8 and q.shape == w.shape and qp.scale.shape == (8,)
    back = Q.PerChannelOperations.dequantize(q, qp)
    assert (back - w).abs().max() <= qp.scale.max() * 0.51
    e = Q.PerChannelOperations.error(w)
    assert e["per_channel_sqnr_db"] > e["per_tensor_sqnr_db"] + 5 and e["per_channel_rmse"] < e["per_tensor_rmse"]
    w2 = torch.randn(4, 6)
    qp1 = Q.PerChannelOperations.qparams(w2, axis=1)
    assert qp1.scale.shape == (6,) and torch.allclose(Q.PerChannelOperations.dequantize(Q.PerChannelOperations.quantize(w2, qp1, 1), qp1, 1), w2, atol=float(qp1.scale.max()))


def test_calibration_process_stops_on_convergence_and_quantizes():
    m = _clf()
    same = [(torch.ones(4, 16), torch.zeros(4, dtype=torch.long))] * 20
    cals, res = Q.CalibrationProcess(tolerance=1e-3, patience=2).run(m, same)
    assert res.converged and res.batches == 3 and res.samples == 12 and set(res.ranges) == {"0", "2"} and res.ranges["0"] == (1.0, 1.0)
    cals, res = Q.CalibrationProcess(max_batches=4).run(m, _data(10))
    assert not res.converged and res.batches == 4 and m.training
    qm, res = Q.CalibrationProcess().quantize(_clf(), _data(3))
    assert isinstance(qm[0], QuantizedLinear) and qm[0].act_qparams is not None and res.batches == 3
    assert Q.CalibrationProcess().run(_clf(), [])[1].ranges == {}


def test_evaluation_regression_detector_and_report():
    fp = _clf()
    data = _data()
    for x, y in data:                                   # make the task learnable: labels from the model itself
        y.copy_(fp(x).argmax(-1))
    qm, _ = Q.CalibrationProcess().quantize(_clf(), data)
    rep = Q.build_report("clf", fp, qm, data)
    assert rep.baseline.top1 == 1.0 and rep.quantized.top1 > 0.9 and rep.quantized.sqnr_db > 25 and rep.quantized.samples == 48
    assert rep.regressions == [] and 2.5 < rep.compression_ratio < 4.0
    md = rep.to_markdown()
    assert "# Quantisation report: clf" in md and "regressions: none" in md and json.loads(rep.to_json())["compression_ratio"] == rep.compression_ratio
    bad = Q.EvaluationMetrics(top1=0.5, cross_entropy=2.0, sqnr_db=5.0)
    found = Q.RegressionDetector(Q.RegressionThresholds(0.01, 0.05, 20.0)).check(Q.EvaluationMetrics(top1=0.9, cross_entropy=1.0), bad)
    assert [f.metric for f in found] == ["top1", "cross_entropy", "sqnr_db"]
    rep.regressions = found
    assert "top1 (0.9000 -> 0.5000, limit 0.01)" in rep.to_markdown() and json.loads(rep.to_json())["regressions"][2]["baseline"] is None
    nolab = Q.ModelEvaluator().evaluate(fp, [torch.randn(4, 16)])
    assert nolab.top1 is None and nolab.samples == 4


def test_sensitivity_analysis_and_mixed_precision_plan():
    fp = _clf()
    data = _data()
    for x, y in data:
        y.copy_(fp(x).argmax(-1))
    metric = lambda m: -Q.ModelEvaluator().evaluate(m, data).cross_entropy      # noqa: E731
    sens = Q.PerLayerSensitivityAnalyzer().analyze(fp, metric)
    assert {s.layer for s in sens} == {"0", "2"} and sens[0].metric_drop >= sens[1].metric_drop and all(s.weight_sqnr_db > 30 for s in sens)
    assert isinstance(fp[0], nn.Linear)                                         # restored
    fake = [Q.LayerSensitivity("big", 0.02, 40, 1_000_000), Q.LayerSensitivity("small_bad", 0.05, 30, 1000), Q.LayerSensitivity("free", -0.01, 45, 5000)]
    plan = Q.PerLayerSensitivityAnalyzer.plan(fake, max_total_drop=0.03)
    assert plan.quantize == ["free", "big"] and plan.keep_full_precision == ["small_bad"] and abs(plan.estimated_drop - 0.02) < 1e-12
    rep = Q.build_report("clf", fp, fp, data[:1], sensitivity=sens)
    assert "| layer | metric drop |" in rep.to_markdown()


def test_qat_schedule_and_checkpointing(tmp_path):
    model = prepare_qat(nn.Sequential(nn.Linear(8, 8), nn.BatchNorm1d(8), nn.ReLU(), nn.Linear(8, 2)))
    integ = Q.QATTrainingIntegration(model, Q.QATSchedule(observer_warmup_steps=2, freeze_observers_after=4, freeze_batchnorm_after=5))
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    fq = integ.fake_quant_modules()
    assert len(fq) == 2 and not fq[0].fake_quant_enabled and fq[0].observer_enabled
    states = []
    for step in range(6):
        model.train()
        integ._apply()
        loss = model(torch.randn(16, 8)).sum()
        opt.zero_grad()
        loss.backward()
        opt.step()
        integ.on_step_end()
        states.append((integ.state()["fake_quant_enabled"], integ.state()["observers_enabled"], model[1].training))
    assert states == [(False, True, True), (True, True, True), (True, True, True), (True, False, True), (True, False, False), (True, False, False)]
    lo_frozen = fq[0].cal.lo.clone()
    model.train()
    integ._apply()
    model(torch.randn(16, 8) * 100)
    assert torch.equal(fq[0].cal.lo, lo_frozen)                                 # observers are frozen
    p = str(tmp_path / "qat.pt")
    Q.QATCheckpointing.save(p, model, integ, opt)
    fresh = prepare_qat(nn.Sequential(nn.Linear(8, 8), nn.BatchNorm1d(8), nn.ReLU(), nn.Linear(8, 2)))
    integ2 = Q.QATTrainingIntegration(fresh, Q.QATSchedule(2, 4, 5))
    opt2 = torch.optim.SGD(fresh.parameters(), lr=0.5)
    assert Q.QATCheckpointing.load(p, fresh, integ2, opt2) == 6 and integ2.step_count == 6
    fq2 = integ2.fake_quant_modules()
    assert torch.equal(fq2[0].cal.lo, lo_frozen) and fq2[0].fake_quant_enabled and not fq2[0].observer_enabled and opt2.param_groups[0]["lr"] == 0.01
    x = torch.randn(4, 8)
    model.eval(); fresh.eval()
    assert torch.allclose(model(x), fresh(x))
    with pytest.raises(KeyError):
        Q.QATCheckpointing.load(p, prepare_qat(nn.Sequential(nn.Linear(8, 8))))
