"""The C restatement (oracle/ngraph_oracle.c: ora_qdot_core / ora_qconv_core) with NON-ZERO input and filter zero points
against nGraph's INTERPRETER on the same seeded inputs: reference::dot (dot.hpp:134-159) and reference::convolution
(convolution.hpp:236-258) subtract the zero points before they multiply and skip padded taps.  Both run on the CPU; the
device path for the same cases is checked in tests/test_plugin.py::test_quantized_*_with_zero_points."""
import numpy as np
import pytest

ng = pytest.importorskip("ngraph_b200.ngraph_api")
from oracle import interpreter, ref  # noqa: E402

pytestmark = pytest.mark.skipif(not interpreter.available(), reason="nGraph host library / INTERPRETER not built here")


@pytest.mark.parametrize("za,zb", [(128, 0), (0, -5), (37, 11)])
def test_dot_with_zero_points(za, zb):
    rng = np.random.default_rng(za * 7 + zb + 50)
    a = rng.integers(0, 256, size=(9, 96)).astype(np.uint8)
    b = rng.integers(-127, 128, size=(96, 7)).astype(np.int8)
    for out_dtype, so, zo in ((np.int8, 2000.0, 3), (np.int32, 0.5, -4)):
        pa, pb = ng.parameter(np.uint8, a.shape), ng.parameter(np.int8, b.shape)
        fn = ng.Function([ng.quantized_dot(pa, pb, 0.5, za, 0.25, zb, so, zo, out_dtype)], [pa, pb])
        want = interpreter.backend().compile(fn).run(a, b)[0]
        got = ref.qdot_core(a, b, np.float32(0.5), za, np.float32(0.25), zb, np.float32(so), zo, out_dtype)
        np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("za,zf", [(128, 0), (0, 9), (100, -7)])
@pytest.mark.parametrize("stride,pad_below,pad_above,dilation", [((1, 1), (1, 1), (1, 1), (1, 1)), ((2, 2), (2, 1), (0, 2), (2, 1))])
def test_convolution_with_zero_points(za, zf, stride, pad_below, pad_above, dilation):
    rng = np.random.default_rng(za + zf + 60)
    ds, fs = (2, 5, 9, 8), (4, 5, 3, 3)
    data = rng.integers(0, 256, size=ds).astype(np.uint8)
    filt = rng.integers(-127, 128, size=fs).astype(np.int8)
    cs = ref.conv_shape(ds, fs, stride, pad_below, pad_above, dilation)
    for out_dtype, so, zo in ((np.int32, 1.0, 5), (np.int8, 4000.0, -2)):
        d, f = ng.parameter(np.uint8, ds), ng.parameter(np.int8, fs)
        fn = ng.Function([ng.quantized_convolution(d, f, 1.0, za, 1.0, zf, so, zo, out_dtype, stride=stride, dilation=dilation,
                                                   pad_below=pad_below, pad_above=pad_above)], [d, f])
        want = interpreter.backend().compile(fn).run(data, filt)[0]
        got = ref.qconv_core(data, filt, cs, np.float32(1.0), za, np.float32(1.0), zf, np.float32(so), zo, out_dtype)
        np.testing.assert_array_equal(got, want)
