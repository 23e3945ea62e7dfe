"""Data-type facts, shape validator, tensor / device conveniences."""
import pytest
import torch

from ml_framework_b200 import core as K
from ml_framework_b200.core import DataType as DT, DataTypeInfo as I


def test_data_type_facts():
    assert I.size_of(DT.BFLOAT16) == 2 and I.size_of(DT.FLOAT8_E4M3) == 1 and I.name(DT.INT64) == "int64" and DT.from_torch(torch.float16) == DT.FLOAT16 and DT.BOOL.torch == torch.bool
    assert I.max_value(DT.FLOAT16) == 65504.0 and I.min_value(DT.INT8) == -128.0 and I.max_value(DT.BOOL) == 1.0 and I.epsilon(DT.BFLOAT16) == 2 ** -7 and I.epsilon(DT.INT32) == 1.0
    assert I.supports_nan(DT.FLOAT32) and not I.supports_nan(DT.INT32) and I.supports_infinity(DT.FLOAT8_E5M2) and not I.supports_infinity(DT.FLOAT8_E4M3)
    assert I.precision(DT.FLOAT32) == 6 and I.precision(DT.BFLOAT16) == 2 and I.precision(DT.FLOAT16) == 3 and I.precision(DT.INT8) == 2
    assert I.dynamic_range_db(DT.BFLOAT16) > I.dynamic_range_db(DT.FLOAT16) > 180 and abs(I.dynamic_range_db(DT.INT8) - 42.08) < 0.01
    assert I.tensor_core_input(DT.BFLOAT16) and not I.tensor_core_input(DT.FLOAT64) and I.is_integer(DT.UINT8) and not I.is_integer(DT.BOOL) and I.is_floating_point(DT.FLOAT8_E5M2)
    c = I.can_cast_losslessly
    assert c(DT.FLOAT16, DT.FLOAT32) and c(DT.BFLOAT16, DT.FLOAT32) and not c(DT.FLOAT32, DT.BFLOAT16) and not c(DT.FLOAT16, DT.BFLOAT16) and not c(DT.BFLOAT16, DT.FLOAT16)
    assert c(DT.INT8, DT.INT32) and not c(DT.INT32, DT.INT8) and not c(DT.UINT8, DT.INT8) and c(DT.INT16, DT.FLOAT32) and not c(DT.INT64, DT.FLOAT32) and not c(DT.FLOAT32, DT.INT64) and c(DT.INT8, DT.INT8)


def test_shape_validator():
    V = K.ShapeValidator
    assert V.validate_matrix_multiply([8, 2, 3], [3, 5]) and V.validate("matmul", [2, 3], [3, 4]).is_valid
    r = V.validate_matrix_multiply([2, 3], [4, 3])
    assert not r and "inner dimensions differ" in r.message and r.suggestions[0] == "transpose the second operand"
    assert "rank >= 2" in V.validate_matrix_multiply([3], [3, 2]).message and "do not broadcast" in V.validate_matrix_multiply([2, 4, 3], [3, 3, 5]).message
    assert V.validate_conv2d([1, 3, 32, 32], [8, 3, 3, 3], padding=1) and V.validate("conv2d", [1, 4, 8, 8], [6, 2, 3, 3], groups=2)
    assert "channels" in V.validate_conv2d([1, 3, 8, 8], [8, 4, 3, 3]).message and "exceeds the padded input" in V.validate_conv2d([1, 3, 2, 2], [8, 3, 5, 5]).message
    assert "ranks" in V.validate_conv2d([3, 8, 8], [8, 3, 3, 3]).message and "groups" in V.validate_conv2d([1, 4, 8, 8], [5, 2, 3, 3], groups=2).message
    assert V.validate_concat([[2, 3], [4, 3]], 0) and V.validate("concat", [2, 3], [2, 5], axis=-1)
    assert "outside axis 0" in V.validate_concat([[2, 3], [4, 5]], 0).message and "out of range" in V.validate_concat([[2, 3]], 2).message and "rank" in V.validate_concat([[2, 3], [2]], 0).message
    assert not V.validate_concat([], 0) and V.validate_broadcast([4, 1, 3], [5, 3]) and "dimension -1" in V.validate("add", [4, 3], [4, 2]).message
    assert "no shape rule" in V.validate("fft", [2]).message and K.ValidationResult.ok().is_valid


def test_tensor_device_conveniences():
    from ml_framework_b200.hal.core import Device, DeviceType
    t = torch.arange(6.0).view(2, 3).t()
    assert K.device_pointer(t) == t.data_ptr() and K.with_data_pointer(t, lambda p: p != 0)
    z = K.zeros_on((2, 2), "cpu", DT.BFLOAT16)
    assert z.dtype == torch.bfloat16 and float(z.sum()) == 0.0
    a = K.from_array([1, 2, 3, 4], "cpu", DT.INT32, shape=(2, 2))
    assert a.dtype == torch.int32 and a.tolist() == [[1, 2], [3, 4]] and K.to_device(a, "cpu").device.type == "cpu"
