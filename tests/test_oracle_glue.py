"""oracle/glue.py (numpy restatements of the f32 reference kernels used between the int8 ops) against nGraph's
INTERPRETER on seeded inputs, all on the CPU: Sum (Kahan), Softmax, LayerNorm, Gelu, BatchMatMul."""
import numpy as np
import pytest

ng = pytest.importorskip("ngraph_b200.ngraph_api")
from oracle import glue, interpreter  # noqa: E402

pytestmark = pytest.mark.skipif(not interpreter.available(), reason="nGraph host library / INTERPRETER not built here")


def run(fn, *arrays):
    return interpreter.backend().compile(fn).run(*arrays)[0]


def bits(a):
    return np.where(a == 0, 0.0, a).astype(np.float32).view(np.uint32)


def test_kahan_sum_matches_reference_sum():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((37, 768)) * 100).astype(np.float32)
    p = ng.parameter(np.float32, x.shape)
    want = run(ng.Function([ng.reduce_sum(p, (1,))], [p]), x)
    np.testing.assert_array_equal(bits(glue.kahan_sum(x)), bits(want))
    assert not np.array_equal(bits(x.sum(axis=1, dtype=np.float32)), bits(want))  # a plain float32 sum is a different number


def test_softmax_matches_reference_softmax():
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((50, 96)) * 4).astype(np.float32)
    p = ng.parameter(np.float32, x.shape)
    want = run(ng.Function([ng.softmax(p, (1,))], [p]), x)
    got = glue.softmax(x)
    # exp: the host library's float routine against double-then-round; equal in all but a few last bits per million
    assert (bits(got) != bits(want)).mean() < 1e-3
    np.testing.assert_allclose(got, want, rtol=2e-7, atol=0)


def test_layer_norm_matches_the_decomposition_on_interpreter():
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((24, 768)) * 3 + 1).astype(np.float32)
    g, b = rng.standard_normal(768).astype(np.float32), rng.standard_normal(768).astype(np.float32)
    p = ng.parameter(np.float32, x.shape)
    want = run(ng.Function([ng.layer_norm(p, g, b)], [p]), x)
    np.testing.assert_array_equal(bits(glue.layer_norm(x, g, b)), bits(want))


def test_gelu_matches_the_decomposition_on_interpreter():
    x = np.linspace(-6, 6, 4001).astype(np.float32)
    p = ng.parameter(np.float32, x.shape)
    want = run(ng.Function([ng.gelu(p)], [p]), x)
    got = glue.gelu(x)
    assert (bits(got) != bits(want)).mean() < 5e-2  # erf: the host float routine (about 1 ulp) against double-then-round
    np.testing.assert_allclose(got, want, rtol=3e-7, atol=2e-7)  # 1 + erf cancels for very negative x: compare absolutely there


def test_batch_mat_mul_is_close_to_the_reference_and_more_exact():
    """reference::dot accumulates f32 products in f32 (dot.hpp:108-160); the device and this restatement accumulate in double
    and round once, which is the more exact of the two: both are compared with an exact (float64) product"""
    rng = np.random.default_rng(3)
    a, b = rng.standard_normal((3, 17, 96)).astype(np.float32), rng.standard_normal((3, 96, 21)).astype(np.float32)
    pa, pb = ng.parameter(np.float32, a.shape), ng.parameter(np.float32, b.shape)
    ref = run(ng.Function([ng.batch_mat_mul(pa, pb)], [pa, pb]), a, b)
    got = glue.batch_mat_mul(a, b)
    exact = np.einsum("bmk,bkn->bmn", a.astype(np.float64), b.astype(np.float64))
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-5)
    assert np.abs(got - exact).max() <= np.abs(ref - exact).max()


@pytest.mark.parametrize("dtype", [np.float32, np.uint8, np.int8])
@pytest.mark.parametrize("window,stride,pad_below,pad_above,include_padding",
                         [((3, 3), (2, 2), (1, 1), (1, 1), False), ((3, 3), (2, 2), (1, 1), (1, 1), True),
                          ((2, 3), (1, 2), (0, 1), (1, 0), True), ((5, 4), (5, 4), (0, 0), (0, 0), False), ((12, 10), (1, 1), (0, 0), (0, 0), False)])
def test_avg_pool_matches_reference_avg_pool(dtype, window, stride, pad_below, pad_above, include_padding):
    """f32 and the one-byte instantiations (whose running sum wraps in the element type) against INTERPRETER"""
    rng = np.random.default_rng(5)
    shape = (2, 3, 12, 10)
    x = (rng.standard_normal(shape) * 50).astype(np.float32) if dtype == np.float32 else \
        rng.integers(np.iinfo(dtype).min, np.iinfo(dtype).max + 1, size=shape).astype(dtype)
    p = ng.parameter(dtype, shape)
    want = run(ng.Function([ng.avg_pool(p, window, stride, pad_below, pad_above, include_padding)], [p]), x)
    got = glue.avg_pool(x, window, stride, pad_below, pad_above, include_padding)
    assert got.shape == want.shape
    if dtype == np.float32:
        np.testing.assert_array_equal(bits(got), bits(want))
    else:
        np.testing.assert_array_equal(got, want)
