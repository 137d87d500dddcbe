"""The plugin's quantisation fusion (ngraph_b200/backend/quant_fusion.cpp), the counterpart of the rewrites nGraph's CPU
backend keeps in CPUQuantFusion (src/ngraph/runtime/cpu/pass/cpu_fusion.cpp:2025-2609; its tests are
test/cpu_fusion.in.cpp:2475-2990: the same graph with the pass on and off must agree).

CPU tests run the plugin's graph passes on un-fused graphs without a device and check WHAT was rewritten; for the
rewrites that never change a value (MaxPool and Concat hoisted above Dequantize, Dequantize->Quantize dropped) they
also run the graph before and after on nGraph's INTERPRETER and compare bits.  GPU tests run the un-fused graph through
Backend::create("B200") and compare with the fused arithmetic (the decomposition on INTERPRETER), bit for bit."""
import os

import numpy as np
import pytest

ng = pytest.importorskip("ngraph_b200.ngraph_api")
from oracle import interpreter  # noqa: E402

pytestmark = pytest.mark.skipif(not interpreter.available(), reason="nGraph host library / INTERPRETER not built here")

RNE = 4
DS, FS = (2, 32, 9, 9), (48, 32, 3, 3)
GEOM = dict(pad_below=(1, 1))


@pytest.fixture(scope="module")
def plugin():
    ng.load_b200()
    return ng


def names(fn):
    return ng.function_op_names(fn, lowered=False)


def ops(fn):
    """op names in execution order without Parameters and Constants"""
    return [n for n in names(fn) if n not in ("Parameter", "Constant")]


def conv_inputs(seed=0):
    rng = np.random.default_rng(seed)
    data = rng.integers(0, 256, size=DS).astype(np.uint8)
    filt = rng.integers(-127, 128, size=FS).astype(np.int8)
    bias = rng.integers(-1000, 1000, size=FS[0]).astype(np.int32)
    sigma = np.sqrt(FS[1] * FS[2] * FS[3]) * 74 * 147
    return rng, data, filt, bias, sigma


# ------------------------------------------------------------------------------------------------ graphs
def conv_bias_relu_graph(filt, bias, scale, dq_scale=0.05, zp=0, second_user=False):
    d = ng.parameter(np.uint8, DS)
    c = ng.quantized_conv_bias(d, filt, bias, scale, False, **GEOM)
    y = ng.relu(ng.dequantize(c, dq_scale, zp))
    results = [y, ng.convert(c, np.uint8)] if second_user else [y]
    return ng.Function(results, [d])


def core_conv_relu_graph(filt, si, sf, so, out_zp=0):
    d = ng.parameter(np.uint8, DS)
    c = ng.quantized_convolution(d, filt, si, 0, sf, 0, so, out_zp, np.int8, **GEOM)
    return ng.Function([ng.relu(ng.dequantize(c, so, out_zp))], [d])


def conv_add_graph(filt, bias, scale, s_left, s_right, sum_dtype, out_shape, quantize_after=None):
    d, s = ng.parameter(np.uint8, DS), ng.parameter(sum_dtype, out_shape)
    left = ng.dequantize(ng.quantized_conv_bias(d, filt, bias, scale, False, **GEOM), s_left, 0)
    right = ng.dequantize(s, s_right, 0)
    y = ng.relu(ng.add(right, left))  # the convolution on the right-hand side of the Add: either order has to match
    if quantize_after is not None:
        y = ng.quantize(y, quantize_after, 0, np.uint8, round_mode=RNE)
    return ng.Function([y], [d, s])


def max_pool_graph(dtype, scale, zp, shape=(2, 16, 10, 10)):
    x = ng.parameter(dtype, shape)
    return ng.Function([ng.max_pool(ng.dequantize(x, scale, zp), (3, 3), (2, 2), (1, 1))], [x])


def concat_graph(scales, shapes=((2, 16, 5, 5), (2, 32, 5, 5), (2, 16, 5, 5)), axis=1, dtype=np.uint8):
    xs = [ng.parameter(dtype, s) for s in shapes]
    return ng.Function([ng.concat([ng.dequantize(x, sc, 0) for x, sc in zip(xs, scales)], axis)], xs)


def dq_q_graph(s1, s2, mode=RNE, dtype=np.uint8, shape=(3, 500)):
    x = ng.parameter(dtype, shape)
    y = ng.quantize(ng.dequantize(x, s1, 0), s2, 0, dtype, round_mode=mode)
    return ng.Function([ng.dequantize(y, s2, 0)], [x])


# ------------------------------------------------------------------------------------------------ CPU: structure
def test_conv_bias_relu_is_fused(plugin):
    _, _, filt, bias, sigma = conv_inputs()
    before = conv_bias_relu_graph(filt, bias, np.float32([30 / sigma]))
    assert "Relu" in names(before)
    after = names(ng.after_b200_passes(before))
    assert "Relu" not in after and after.count("QuantizedConvolutionBias") == 1 and ops(ng.after_b200_passes(before))[-2] == "Dequantize"
    # a non-zero zero point, or a second reader of the convolution, keeps the graph as it was
    assert "Relu" in names(ng.after_b200_passes(conv_bias_relu_graph(filt, bias, np.float32([30 / sigma]), zp=3)))
    assert "Relu" in names(ng.after_b200_passes(conv_bias_relu_graph(filt, bias, np.float32([30 / sigma]), second_user=True)))
    # a negative Dequantize scale: Relu no longer commutes with it
    assert "Relu" in names(ng.after_b200_passes(conv_bias_relu_graph(filt, bias, np.float32([30 / sigma]), dq_scale=-0.05)))


def test_core_conv_relu_becomes_quantized_convolution_relu(plugin):
    _, _, filt, _, sigma = conv_inputs()
    after = names(ng.after_b200_passes(core_conv_relu_graph(filt, 0.02, 0.005, np.float32(0.02 * 0.005 * sigma / 30))))
    assert "QuantizedConvolutionRelu" in after and "Relu" not in after and "QuantizedConvolution" not in after
    assert "Multiply" not in after and "Divide" not in after  # the requantisation scale was folded into a Constant
    after = names(ng.after_b200_passes(core_conv_relu_graph(filt, 0.02, 0.005, 0.3, out_zp=1)))
    assert "QuantizedConvolutionRelu" not in after and "Relu" in after


@pytest.mark.parametrize("sum_dtype,fused_op", [(np.uint8, "QuantizedConvolutionBiasAdd"), (np.int8, "QuantizedConvolutionBiasSignedAdd")])
def test_conv_bias_add_relu_is_fused(plugin, sum_dtype, fused_op):
    _, _, filt, bias, sigma = conv_inputs()
    out_shape = (DS[0], FS[0], DS[2], DS[3])
    after = names(ng.after_b200_passes(conv_add_graph(filt, bias, np.float32([30 / sigma]), 0.05, 0.04, sum_dtype, out_shape)))
    assert fused_op in after and "Relu" not in after and "Add" not in after and "Divide" not in after
    assert ("Convert" in after) == (sum_dtype == np.int8)
    # followed by a Quantize with the same scale, the Dequantize / Quantize pair disappears too
    after = names(ng.after_b200_passes(conv_add_graph(filt, bias, np.float32([30 / sigma]), 0.05, 0.04, sum_dtype, out_shape,
                                                      quantize_after=0.05)))
    assert fused_op in after and "Quantize" not in after and "Dequantize" not in after
    # a summand of another shape cannot be the fused op's sum input
    bad = names(ng.after_b200_passes(conv_add_graph(filt, bias, np.float32([30 / sigma]), 0.05, 0.04, sum_dtype, (1,) + out_shape[1:])))
    assert fused_op not in bad and "Relu" in bad


def test_switch_named_like_the_cpu_backends_knob(plugin):
    _, _, filt, bias, sigma = conv_inputs()
    fn = conv_bias_relu_graph(filt, bias, np.float32([30 / sigma]))
    old = os.environ.get("NGRAPH_PASS_ENABLES")
    os.environ["NGRAPH_PASS_ENABLES"] = "B200QuantFusion:0"
    try:
        assert "Relu" in names(ng.after_b200_passes(fn))
        os.environ["NGRAPH_PASS_ENABLES"] = "B200QuantFusion:1"
        assert "Relu" not in names(ng.after_b200_passes(fn))
    finally:
        if old is None:
            del os.environ["NGRAPH_PASS_ENABLES"]
        else:
            os.environ["NGRAPH_PASS_ENABLES"] = old


# ------------------------------------------------------------------------------------------------ CPU: exact rewrites
def run_interpreter(fn, inputs):
    return interpreter.backend().compile(fn).run(*inputs)[0]


@pytest.mark.parametrize("dtype,zp", [(np.uint8, 0), (np.uint8, 7), (np.int8, -3)])
def test_max_pool_moves_above_dequantize_without_changing_a_bit(plugin, dtype, zp):
    before = max_pool_graph(dtype, 0.037, zp)
    after = ng.after_b200_passes(before)
    assert ops(after) == ["MaxPool", "Dequantize", "Result"]
    x = np.random.default_rng(1).integers(np.iinfo(dtype).min, np.iinfo(dtype).max + 1, size=(2, 16, 10, 10)).astype(dtype)
    np.testing.assert_array_equal(run_interpreter(after, [x]).view(np.uint32), run_interpreter(before, [x]).view(np.uint32))
    # a negative scale reverses the order of values: left alone
    assert ops(ng.after_b200_passes(max_pool_graph(dtype, -0.037, zp))) == ["Dequantize", "MaxPool", "Result"]
    # a scale so large that code * scale overflows: the dequantised values no longer compare like the codes
    assert ops(ng.after_b200_passes(max_pool_graph(dtype, 3.0e37, zp))) == ["Dequantize", "MaxPool", "Result"]


def test_concat_moves_above_dequantize_without_changing_a_bit(plugin):
    before = concat_graph([0.02, 0.02, 0.02])
    after = ng.after_b200_passes(before)
    got = names(after)
    assert got.count("Dequantize") == 1 and ops(after) == ["Concat", "Dequantize", "Result"]
    rng = np.random.default_rng(2)
    xs = [rng.integers(0, 256, size=p.shape).astype(np.uint8) for p in before.params]
    np.testing.assert_array_equal(run_interpreter(after, xs).view(np.uint32), run_interpreter(before, xs).view(np.uint32))
    assert names(ng.after_b200_passes(concat_graph([0.02, 0.03, 0.02]))).count("Dequantize") == 3  # scales differ


def test_dequantize_quantize_pair_is_dropped_only_when_exact(plugin):
    before = dq_q_graph(0.0371, 0.0371)
    after = ng.after_b200_passes(before)
    assert names(after).count("Dequantize") == 1 and "Quantize" not in names(after)
    x = np.arange(1500, dtype=np.int64).reshape(3, 500).astype(np.uint8)
    np.testing.assert_array_equal(run_interpreter(after, [x]).view(np.uint32), run_interpreter(before, [x]).view(np.uint32))
    assert "Quantize" in names(ng.after_b200_passes(dq_q_graph(0.0371, 0.05)))          # another scale
    assert "Quantize" in names(ng.after_b200_passes(dq_q_graph(0.0371, 0.0371, mode=8)))  # ROUND_DOWN is not a nearest mode
    # 255 * scale overflows to +inf, the original Quantize then saturates: not an identity any more
    assert "Quantize" in names(ng.after_b200_passes(dq_q_graph(3.0e37, 3.0e37)))
    assert "Quantize" in names(ng.after_b200_passes(dq_q_graph(1.0e-38, 1.0e-38)))      # products go subnormal


def test_a_graph_of_fused_ops_is_left_alone(plugin):
    _, _, filt, bias, sigma = conv_inputs()
    d = ng.parameter(np.uint8, DS)
    fn = ng.Function([ng.dequantize(ng.quantized_conv_bias(d, filt, bias, np.float32([30 / sigma]), True, **GEOM), 0.05, 0)], [d])
    assert names(ng.after_b200_passes(fn)) == names(fn)


# ------------------------------------------------------------------------------------------------ GPU
@pytest.fixture(scope="module")
def backends(plugin):
    return ng.Backend("B200"), interpreter.backend()


def bits(a):
    return np.where(a == 0, 0.0, a).astype(np.float32).view(np.uint32)


@pytest.mark.gpu
def test_unfused_conv_bias_relu_runs_as_the_fused_kernel(backends):
    b200, ref = backends
    _, data, filt, bias, sigma = conv_inputs(3)
    scale = np.float32([30 / sigma])
    exe = b200.compile(conv_bias_relu_graph(filt, bias, scale), perf=True)
    got = exe.run(data)[0]
    assert not any(n.startswith("Relu") for n, _, _ in exe.performance_data())
    d = ng.parameter(np.uint8, DS)
    fused = interpreter.decomposed_conv(d, ng.constant(filt), ng.constant(bias), ng.constant(scale), np.uint8, True, **GEOM)
    exp = ref.compile(ng.Function([ng.dequantize(fused, 0.05, 0)], [d])).run(data)[0]
    np.testing.assert_array_equal(bits(got), bits(exp))
    # and, like the reference's own fusion tests, the un-fused arithmetic agrees wherever i8 did not clip
    d2 = ng.parameter(np.uint8, DS)
    plain = interpreter.decomposed_conv(d2, ng.constant(filt), ng.constant(bias), ng.constant(scale), np.int8, False, **GEOM)
    unfused = ref.compile(ng.Function([ng.relu(ng.dequantize(plain, 0.05, 0))], [d2])).run(data)[0]
    keep = unfused < 127 * 0.05
    np.testing.assert_array_equal(bits(got[keep]), bits(unfused[keep]))
    assert keep.mean() > 0.9


@pytest.mark.gpu
def test_unfused_core_conv_relu(backends):
    b200, ref = backends
    _, data, filt, _, sigma = conv_inputs(4)
    si, sf = np.float32(0.02), np.float32(0.005)
    so = np.float32(si * sf * np.float32(sigma) / np.float32(30))
    got = b200.compile(core_conv_relu_graph(filt, si, sf, so)).run(data)[0]
    requant = np.float32(np.float32(si * sf) / so)
    d = ng.parameter(np.uint8, DS)
    fused = interpreter.decomposed_conv(d, ng.constant(filt), None, ng.constant(np.float32([requant])), np.uint8, True, **GEOM)
    exp = ref.compile(ng.Function([ng.dequantize(fused, so, 0)], [d])).run(data)[0]
    np.testing.assert_array_equal(bits(got), bits(exp))


@pytest.mark.gpu
@pytest.mark.parametrize("sum_dtype", [np.uint8, np.int8])
def test_unfused_residual_block_tail(backends, sum_dtype):
    b200, ref = backends
    rng, data, filt, bias, sigma = conv_inputs(5)
    scale = np.float32([30 / sigma])
    out_shape = (DS[0], FS[0], DS[2], DS[3])
    hi = 128 if sum_dtype == np.int8 else 256
    summand = rng.integers(hi - 256, hi, size=out_shape).astype(sum_dtype)
    s_left, s_right = np.float32(0.05), np.float32(0.04)
    exe = b200.compile(conv_add_graph(filt, bias, scale, s_left, s_right, sum_dtype, out_shape, quantize_after=s_left), perf=True)
    got = exe.run(data, summand)[0]
    steps = [n.split(":")[0] for n, _, _ in exe.performance_data()]
    assert "Relu" not in steps and "Add" not in steps and "Quantize" not in steps and "Dequantize" not in steps
    d, s = ng.parameter(np.uint8, DS), ng.parameter(sum_dtype, out_shape)
    fused = interpreter.decomposed_conv(d, ng.constant(filt), ng.constant(bias), ng.constant(scale), np.uint8, True,
                                        sum_in=s, sum_scale=ng.constant(np.float32([s_right / s_left])), signed=sum_dtype == np.int8,
                                        **GEOM)
    exp = ref.compile(ng.Function([fused], [d, s])).run(data, summand)[0]
    np.testing.assert_array_equal(got, exp)


@pytest.mark.gpu
def test_hoisted_max_pool_and_concat_on_the_device(backends):
    b200, ref = backends
    rng = np.random.default_rng(6)
    for dtype, zp in ((np.uint8, 0), (np.int8, -3)):
        fn = max_pool_graph(dtype, 0.037, zp, shape=(2, 32, 14, 14))
        x = rng.integers(np.iinfo(dtype).min, np.iinfo(dtype).max + 1, size=(2, 32, 14, 14)).astype(dtype)
        np.testing.assert_array_equal(bits(b200.compile(fn).run(x)[0]), bits(ref.compile(fn).run(x)[0]))
    for axis, shapes in ((1, ((2, 16, 5, 5), (2, 32, 5, 5), (2, 16, 5, 5))), (3, ((2, 3, 5, 1), (2, 3, 5, 6))), (0, ((1, 8), (3, 8)))):
        fn = concat_graph([0.02] * len(shapes), shapes, axis)
        xs = [rng.integers(0, 256, size=s).astype(np.uint8) for s in shapes]
        exe = b200.compile(fn, perf=True)
        np.testing.assert_array_equal(bits(exe.run(*xs)[0]), bits(ref.compile(fn).run(*xs)[0]))
        assert sum(n.startswith("Dequantize") for n, _, _ in exe.performance_data()) == 1
    # Concat of f32 values that did not come from Dequantize ops runs as it is
    a, b = ng.parameter(np.float32, (4, 3)), ng.parameter(np.float32, (4, 5))
    fn = ng.Function([ng.concat([a, b], 1)], [a, b])
    xa, xb = rng.standard_normal((4, 3)).astype(np.float32), rng.standard_normal((4, 5)).astype(np.float32)
    np.testing.assert_array_equal(b200.compile(fn).run(xa, xb)[0], np.concatenate([xa, xb], 1))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.uint8, np.int8])
def test_quantized_concat_builder_graph(backends, dtype):
    """builder::QuantizedConcatBuilder (src/ngraph/builder/quantized_concat_builder.cpp:28-79): Dequantize / Quantize each
    operand to the scale of the widest range, then Concat; the ranges are run-time values here, like in the
    reference's tests (test/builder_quantization.cpp:847-944), so the scale arithmetic (Concat, Min, Max, Abs, Maximum,
    Divide) runs on the device as well."""
    b200, ref = backends
    shapes = ((2, 2), (3, 2), (3, 2))
    xs = [ng.parameter(dtype, s) for s in shapes]
    mins = [ng.parameter(np.float32, (1,)) for _ in shapes]
    maxs = [ng.parameter(np.float32, (1,)) for _ in shapes]
    fn = ng.Function([ng.quantized_concat(xs, mins, maxs, 0)], xs + mins + maxs)
    # the reference's own vectors: equal ranges leave every value as it is
    lo = -2 if dtype == np.int8 else 2
    data = [np.array([lo, 4, 8, 16], dtype).reshape(2, 2), np.array([lo, 2, 4, 8, 16, 15], dtype).reshape(3, 2),
            np.array([lo, 3, 5, 7, 11, 16], dtype).reshape(3, 2)]
    same = [np.float32([2.0])] * 3 + [np.float32([16.0])] * 3
    got = b200.compile(fn).run(*data, *same)[0]
    np.testing.assert_array_equal(got, np.concatenate(data, 0))
    # different ranges: every operand is rescaled; INTERPRETER runs the same graph
    rng = np.random.default_rng(8)
    big = ((40, 16), (25, 16), (70, 16))
    xs = [ng.parameter(dtype, s) for s in big]
    fn = ng.Function([ng.quantized_concat(xs, mins, maxs, 0)], xs + mins + maxs)
    data = [rng.integers(np.iinfo(dtype).min, np.iinfo(dtype).max + 1, size=s).astype(dtype) for s in big]
    ranges = [np.float32([-1.5]), np.float32([-6.0]), np.float32([-0.25]), np.float32([3.0]), np.float32([5.5]), np.float32([9.75])]
    np.testing.assert_array_equal(b200.compile(fn).run(*data, *ranges)[0], ref.compile(fn).run(*data, *ranges)[0])


@pytest.mark.parametrize("seed", range(6))
def test_exact_rewrites_compose_on_random_graphs(plugin, seed):
    """Random small graphs built from the three rewrites that must not change a bit (Dequantize -> MaxPool, Dequantize... ->
    Concat, Dequantize -> Quantize), nested in random order with random scales: the graph after the plugin's passes gives
    the INTERPRETER the same bytes as the graph before them, and has lost at least one f32 op."""
    rng = np.random.default_rng(seed)
    scales = [np.float32(s) for s in (0.02, 0.037, 0.11)]
    params, data = [], []

    def leaf(shape):
        p = ng.parameter(np.uint8, shape)
        params.append(p)
        data.append(rng.integers(0, 256, size=shape).astype(np.uint8))
        return p

    def dequantized(depth, shape, s):
        """an f32 value of `shape` whose integer source was (or will be) quantized with scale s"""
        kind = rng.integers(0, 3) if depth > 0 else 3
        if kind == 0:      # MaxPool over a larger dequantized tensor
            src = (shape[0], shape[1], shape[2] * 2, shape[3] * 2)
            return ng.max_pool(dequantized(depth - 1, src, s), (2, 2), (2, 2))
        if kind == 1:      # Concat of two dequantized halves along the channels
            half = (shape[0], shape[1] // 2, shape[2], shape[3])
            return ng.concat([dequantized(depth - 1, half, s), dequantized(depth - 1, half, s)], 1)
        if kind == 2:      # a Quantize / Dequantize round trip in between, sometimes with another scale (not removable)
            s2 = s if rng.random() < 0.7 else scales[int(rng.integers(0, 3))]
            q = ng.quantize(dequantized(depth - 1, shape, s), s2, 0, np.uint8, round_mode=RNE)
            return ng.dequantize(q, s2, 0)
        return ng.dequantize(leaf(shape), s, 0)

    y = dequantized(3, (1, 32, 4, 4), scales[int(rng.integers(0, 3))])
    before = ng.Function([y], params)
    after = ng.after_b200_passes(before)
    got, want = run_interpreter(after, data), run_interpreter(before, data)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    f32_ops = lambda fn: sum(n in ("Dequantize", "Quantize") for n in names(fn))
    assert f32_ops(after) <= f32_ops(before)
