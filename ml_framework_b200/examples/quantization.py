"""Quantization examples: post-training (static and dynamic), calibrator comparison, per-layer
selection from a sensitivity analysis, and a quantization-aware training quick start. They follow the
topics of the reference's examples (src/Examples/Quantization: PTQ / QAT quick starts, calibration,
per-layer quantization, sensitivity analysis).

    python -m ml_framework_b200.examples.quantization [name ...]
"""
from __future__ import annotations

import copy
import sys
from typing import Dict

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..quantization import core as Q


def _problem(seed: int = 0, device: str = "cpu"):
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(512, 16, generator=g)
    W = torch.randn(16, 4, generator=g)
    y = (X @ W).argmax(1)
    net = nn.Sequential(nn.Linear(16, 64), nn.ReLU(), nn.Linear(64, 64), nn.ReLU(), nn.Linear(64, 4))
    torch.manual_seed(seed)
    opt = torch.optim.Adam(net.parameters(), lr=1e-2)
    for _ in range(150):
        opt.zero_grad()
        F.cross_entropy(net(X), y).backward()
        opt.step()
    return net.to(device).eval(), X.to(device), y.to(device)


def _acc(net, X, y) -> float:
    with torch.no_grad():
        return Q.top_k_accuracy(net(X), y, 1)


def ptq_quickstart(device: str = "cpu") -> Dict[str, float]:
    net, X, y = _problem(device=device)
    base = _acc(net, X, y)
    dyn = Q.PTQQuantizer().quantize_dynamic(copy.deepcopy(net))
    sta = Q.PTQQuantizer().quantize_static(copy.deepcopy(net), [X[i:i + 64] for i in range(0, 256, 64)])
    with torch.no_grad():
        sqnr = Q.sqnr_db(net(X), sta(X))
    rep = Q.detect_regression(base, _acc(sta, X, y), tolerance=0.05)
    return {"fp32_accuracy": base, "dynamic_int8_accuracy": _acc(dyn, X, y), "static_int8_accuracy": _acc(sta, X, y),
            "static_sqnr_db": sqnr, "regressed": float(rep.regressed)}


def calibration(device: str = "cpu") -> Dict[str, float]:
    """The four calibrators on one heavy-tailed activation tensor: range chosen and reconstruction error."""
    g = torch.Generator().manual_seed(1)
    x = torch.randn(4096, generator=g)
    x[::512] *= 20            # outliers
    x = x.to(device)
    out = {}
    for name, cal in [("minmax", Q.MinMaxCalibrator()), ("moving_average", Q.MovingAverageCalibrator(0.9)),
                      ("percentile", Q.PercentileCalibrator(99.9)), ("entropy", Q.EntropyCalibrator())]:
        for chunk in x.chunk(8):
            cal.observe(chunk)
        qp = cal.qparams()
        out[name + "_rmse"] = Q.rmse(x, Q.dequantize(Q.quantize(x, qp), qp))
    return out


def sensitivity_and_per_layer(device: str = "cpu") -> Dict[str, float]:
    """Ranks the layers by accuracy drop when quantised alone, then quantises all but the most sensitive."""
    net, X, y = _problem(device=device)
    ranking = Q.sensitivity_analysis(net, [X], lambda m: _acc(m, X, y))
    keep = ranking[0][0]
    mixed = Q.PTQQuantizer(skip=(keep,)).quantize_dynamic(copy.deepcopy(net))
    return {"most_sensitive_layer": float(keep), "drop_when_quantised_alone": ranking[0][1], "fp32_accuracy": _acc(net, X, y),
            "mixed_precision_accuracy": _acc(mixed, X, y)}


def qat_quickstart(device: str = "cpu") -> Dict[str, float]:
    net, X, y = _problem(device=device)
    base = _acc(net, X, y)
    qat = Q.prepare_qat(copy.deepcopy(net)).train()
    opt = torch.optim.Adam(qat.parameters(), lr=2e-3)
    for _ in range(60):
        opt.zero_grad()
        F.cross_entropy(qat(X), y).backward()
        opt.step()
    int8 = Q.convert_qat(qat.eval())
    return {"fp32_accuracy": base, "qat_int8_accuracy": _acc(int8, X, y)}


EXAMPLES = {"ptq_quickstart": ptq_quickstart, "calibration": calibration, "sensitivity_and_per_layer": sensitivity_and_per_layer,
            "qat_quickstart": qat_quickstart}


def main(argv=None):
    names = list(argv if argv is not None else sys.argv[1:]) or list(EXAMPLES)
    for n in names:
        print(n, EXAMPLES[n]())


if __name__ == "__main__":
    main()
