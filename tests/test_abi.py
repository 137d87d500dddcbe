"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares, and
rejects bad arguments before touching a device (no compute call is made here)."""
import ctypes
import os
import re

import pytest

from ngraph_b200 import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200_kernels.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"B200_API\s+[\w\s\*]+?\b(b200_\w+)\s*\(", text)


def test_header_declares_entry_points():
    names = declared_symbols()
    assert len(names) >= 12 and len(set(names)) == len(names)
    for must in ("b200_quantize", "b200_dequantize", "b200_qgemm", "b200_qconv"):
        assert must in names


@pytest.mark.parametrize("name", declared_symbols())
def test_library_exports(name):
    assert hasattr(lib.LIB, name), "libb200_kernels.so does not export " + name


def test_status_strings():
    assert lib.LIB.b200_status_string(0) == b"ok"
    for code in (-1, -2, -3, -4, 1):
        assert lib.LIB.b200_status_string(code) not in (b"ok", b"unknown status")


def test_argument_validation_without_device():
    i64 = ctypes.c_int64
    shape = (i64 * 9)(*([2] * 9))
    axes = (i64 * 2)(1, 1)
    # rank beyond B200_MAX_RANK, bad round mode, duplicate axes, bad dtype: all rejected on the host
    assert lib.LIB.b200_quantize(None, None, None, None, lib.U8, shape, 9, None, 0, 4, None) == -1
    assert lib.LIB.b200_quantize(None, None, None, None, lib.U8, shape, 2, None, 0, 11, None) == -1
    assert lib.LIB.b200_quantize(None, None, None, None, lib.U8, shape, 2, axes, 2, 4, None) == -1
    assert lib.LIB.b200_quantize(None, None, None, None, lib.F32, shape, 2, None, 0, 4, None) == -1
    assert lib.LIB.b200_dequantize(None, None, None, None, lib.U8, shape, 2, None, 0, None) == -1  # null data
    # empty tensors are a no-op
    empty = (i64 * 2)(0, 5)
    assert lib.LIB.b200_quantize(None, None, None, None, lib.U8, empty, 2, None, 0, 4, None) == 0
    e = lib.Epilogue()
    assert lib.LIB.b200_qgemm(None, lib.U8, None, None, 4, 4, 16, ctypes.byref(e), None) == -1  # no scale
    cp = lib.ConvParams(1, 8, 8, 64, 64, 3, 3, 0, 1, 1, 1, 1, 1, 1, 1)
    p, q = i64(), i64()
    assert lib.LIB.b200_qconv_out_shape(ctypes.byref(cp), ctypes.byref(p), ctypes.byref(q)) == -1  # stride 0
    cp.stride_h = 1
    assert lib.LIB.b200_qconv_out_shape(ctypes.byref(cp), ctypes.byref(p), ctypes.byref(q)) == 0
    assert (p.value, q.value) == (8, 8)


def test_argument_validation_of_the_glue_entry_points():
    """the f32 glue, Concat and zero-point entry points: bad arguments are refused on the host, empty work is a no-op"""
    L = lib.LIB
    i64 = ctypes.c_int64
    assert L.b200_f32_binary(99, None, None, None, 4, None) == -1            # unknown op
    assert L.b200_f32_binary(0, None, None, None, 0, None) == 0              # nothing to do
    assert L.b200_f32_binary(0, None, None, None, 4, None) == -1             # null operands
    assert L.b200_f32_binary_periodic(0, None, None, None, 8, 0, 0, None) == -1   # period 0
    assert L.b200_f32_unary(-1, None, None, 4, None) == -1
    assert L.b200_softmax_rows_f32(None, None, -1, 4, None) == -1
    assert L.b200_softmax_rows_f32(None, None, 0, 4, None) == 0
    assert L.b200_layer_norm_rows_f32(None, None, None, None, 3, 4, ctypes.c_float(1e-5), None) == -1
    assert L.b200_gelu_f32(None, None, 0, None) == 0
    assert L.b200_bmm_f32(None, None, None, 1, -1, 4, 4, None) == -1
    assert L.b200_copy_rows(None, None, 2, 8, 4, None) == -1                 # pitch shorter than a row
    assert L.b200_copy_rows(None, None, 0, 8, 8, None) == 0
    shape, axes = (i64 * 2)(4, 5), (i64 * 2)(1, 1)
    assert L.b200_reduce_f32(7, None, None, shape, 2, axes, 1, None) == -1   # unknown reduction
    assert L.b200_reduce_f32(0, None, None, shape, 2, axes, 2, None) == -1   # an axis named twice
    assert L.b200_strided_sums(None, lib.F32, None, 1, 1, 1, 1, 1, 1, None) == -1  # only u8 / i8 are summed
    e = lib.Epilogue()
    e.round_half_away, e.out_type = 2, lib.U8                                # raw accumulators exist as int32 only
    assert L.b200_qgemm(None, lib.U8, None, None, 4, 4, 16, ctypes.byref(e), None) == -1
    assert L.b200_requant_zero_points(None, None, None, None, ctypes.byref(e), None, None) == -1
