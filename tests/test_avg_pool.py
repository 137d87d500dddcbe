"""op::v0::AvgPool on the device: f32 with any window / stride / padding / include_padding, the op applied to u8 / i8 directly
(the reference's one-byte instantiation, whose running sum wraps), and Dequantize -> AvgPool(window) -> Quantize as one
kernel.  Through the plugin against nGraph's INTERPRETER (runtime/reference/avg_pool.hpp:160-236), bit for bit; ceil-mode
windows, which INTERPRETER refuses, against the numpy restatement of the same loop (oracle/glue.py)."""
import ctypes

import numpy as np
import pytest

ng = pytest.importorskip("ngraph_b200.ngraph_api")
from oracle import glue, interpreter  # noqa: E402

needs_ngraph = pytest.mark.skipif(not interpreter.available(), reason="nGraph host library / INTERPRETER not built here")

GEOMETRIES = [((3, 3), (2, 2), (1, 1), (1, 1), False), ((3, 3), (2, 2), (1, 1), (1, 1), True), ((2, 3), (1, 2), (0, 1), (1, 0), True),
              ((5, 4), (5, 4), (0, 0), (0, 0), False), ((7, 7), (1, 1), (0, 0), (0, 0), False), ((3, 3), (1, 1), (1, 1), (1, 1), False)]


@pytest.fixture(scope="module")
def backends():
    ng.load_b200()
    return ng.Backend("B200"), interpreter.backend()


def bits(a):
    return np.where(a == 0, 0.0, a).astype(np.float32).view(np.uint32)


def test_geometries_without_a_counted_element_are_refused_on_the_host():
    """the reference throws "AvgPool elements == 0"; the C ABI refuses the geometry before any launch"""
    from ngraph_b200 import lib
    P = lib.PoolParams
    ok = P(1, 16, 8, 8, 4, 4, 2, 2, 2, 2, 0, 0, 0, 0, 0)
    assert lib.LIB.b200_avgpool_f32_nchw(None, None, ctypes.byref(ok), None) == -1       # null tensors
    empty = P(0, 16, 8, 8, 4, 4, 2, 2, 2, 2, 0, 0, 0, 0, 0)
    assert lib.LIB.b200_avgpool_f32_nchw(None, None, ctypes.byref(empty), None) == 0     # nothing to do
    too_far = P(1, 16, 8, 8, 6, 4, 2, 2, 2, 2, 0, 0, 0, 0, 0)                            # window row 5 starts at h = 10 >= 8
    assert lib.LIB.b200_avgpool_f32_nchw(None, None, ctypes.byref(too_far), None) == -1
    all_padding = P(1, 16, 8, 8, 5, 5, 1, 1, 2, 2, 1, 1, 1, 1, 0)                        # first window covers padding only
    assert lib.LIB.b200_avgpool_nhwc_bytes(None, None, lib.U8, ctypes.byref(all_padding), None) == -1
    assert lib.LIB.b200_avgpool_nhwc_bytes(None, None, lib.F32, ctypes.byref(ok), None) == -1   # one-byte types only
    assert lib.LIB.b200_avgpool_q_nhwc(None, lib.U8, None, lib.I32, None, None, ctypes.byref(ok), None) == -1


@pytest.mark.gpu
@needs_ngraph
@pytest.mark.parametrize("window,stride,pad_below,pad_above,include_padding", GEOMETRIES)
def test_f32_avg_pool_matches_interpreter(backends, window, stride, pad_below, pad_above, include_padding):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((3, 5, 13, 11)) * 50).astype(np.float32)
    p = ng.parameter(np.float32, x.shape)
    fn = ng.Function([ng.avg_pool(p, window, stride, pad_below, pad_above, include_padding)], [p])
    got, exp = backends[0].compile(fn).run(x)[0], backends[1].compile(fn).run(x)[0]
    assert got.shape == exp.shape
    np.testing.assert_array_equal(bits(got), bits(exp))


@pytest.mark.gpu
@needs_ngraph
@pytest.mark.parametrize("dtype", [np.uint8, np.int8])
@pytest.mark.parametrize("window,stride,pad_below,pad_above,include_padding", GEOMETRIES)
def test_one_byte_avg_pool_wraps_like_the_reference(backends, dtype, window, stride, pad_below, pad_above, include_padding):
    rng = np.random.default_rng(2)
    x = rng.integers(np.iinfo(dtype).min, np.iinfo(dtype).max + 1, size=(2, 24, 13, 11)).astype(dtype)
    p = ng.parameter(dtype, x.shape)
    fn = ng.Function([ng.avg_pool(p, window, stride, pad_below, pad_above, include_padding)], [p])
    got, exp = backends[0].compile(fn).run(x)[0], backends[1].compile(fn).run(x)[0]
    np.testing.assert_array_equal(got, exp)
    np.testing.assert_array_equal(got, glue.avg_pool(x, window, stride, pad_below, pad_above, include_padding))


@pytest.mark.gpu
@needs_ngraph
@pytest.mark.parametrize("in_dtype,out_dtype", [(np.uint8, np.uint8), (np.int8, np.int8), (np.uint8, np.int8)])
@pytest.mark.parametrize("window,stride,pad_below,pad_above,include_padding", GEOMETRIES[:5])
def test_dequantize_avg_pool_quantize_runs_as_one_kernel(backends, in_dtype, out_dtype, window, stride, pad_below, pad_above, include_padding):
    """the graph the CPU backend's construct_qavg_pool starts from (cpu_fusion.cpp:2160-2200), with a window"""
    rng = np.random.default_rng(3)
    x = rng.integers(np.iinfo(in_dtype).min, np.iinfo(in_dtype).max + 1, size=(2, 32, 14, 14)).astype(in_dtype)
    p = ng.parameter(in_dtype, x.shape)
    f = ng.avg_pool(ng.dequantize(p, np.float32(0.037), in_dtype(0)), window, stride, pad_below, pad_above, include_padding)
    fn = ng.Function([ng.quantize(f, np.float32(0.021), out_dtype(0), out_dtype)], [p])
    exe = backends[0].compile(fn, perf=True)
    got, exp = exe.run(x)[0], backends[1].compile(fn).run(x)[0]
    np.testing.assert_array_equal(got, exp)
    steps = [n.split(":")[0] for n, _, _ in exe.performance_data()]
    assert "AvgPool" not in steps and "Dequantize" not in steps, steps   # folded into the Quantize node's one kernel


@pytest.mark.gpu
@needs_ngraph
def test_ceil_mode_counts_only_positions_of_the_padded_image(backends):
    rng = np.random.default_rng(4)
    x = (rng.standard_normal((2, 3, 14, 12)) * 10).astype(np.float32)
    p = ng.parameter(np.float32, x.shape)
    for pad, include in (((0, 0), False), ((1, 1), True), ((1, 1), False)):
        fn = ng.Function([ng.avg_pool(p, (3, 3), (2, 2), pad, pad, include, ceil_mode=True)], [p])
        got = backends[0].compile(fn).run(x)[0]
        out_hw = tuple(-(-(x.shape[2 + i] + 2 * pad[i] - 3) // 2) + 1 for i in (0, 1))
        assert got.shape[2:] == out_hw
        np.testing.assert_array_equal(bits(got), bits(glue.avg_pool(x, (3, 3), (2, 2), pad, pad, include, out_hw=out_hw)))
