"""The shipped examples run end to end on CPU and reach the outcome each one demonstrates."""
from ml_framework_b200.examples import higher_order as H
from ml_framework_b200.examples import quantization as QZ


def test_higher_order_examples():
    r = H.maml(steps=12)
    assert r["meta_loss_last"] < r["meta_loss_first"] * 1.2
    r = H.neural_ode(steps=40)
    assert r["loss_last"] < 0.1 * r["loss_first"]
    r = H.newton()
    assert r["f_end"] < 1e-6
    r = H.natural_gradient(steps=20)
    assert r["loss_last"] < 0.2 and r["accuracy"] > 0.95
    r = H.adversarial_robustness()
    assert r["clean_accuracy"] > 0.9 and r["fgsm_accuracy"] > 0.7
    r = H.sharpness()
    assert r["top_eigenvalue_before"] > 0 and r["top_eigenvalue_after"] > 0


def test_quantization_examples():
    r = QZ.ptq_quickstart()
    assert r["static_int8_accuracy"] > 0.95 and r["static_sqnr_db"] > 25 and r["regressed"] == 0.0
    r = QZ.calibration()
    assert all(v > 0 for v in r.values())
    r = QZ.sensitivity_and_per_layer()
    assert r["mixed_precision_accuracy"] > 0.95
    r = QZ.qat_quickstart()
    assert r["qat_int8_accuracy"] > 0.95
