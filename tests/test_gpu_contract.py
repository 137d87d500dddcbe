"""Parity of the tcgen05 int8 contractions (b200_qgemm / b200_qconv through the C ABI) with the
golden fixtures and with the CPU oracle on seeded inputs.  Integer outputs bit-exact; f32 outputs
bit-exact too (the epilogue is the same sequence of IEEE single operations)."""
import numpy as np
import pytest
import torch

from oracle import ref
from tests.fixtures import NP, blob, f32_from_bits, interpreter_cases, reference_tests, typed

pytestmark = pytest.mark.gpu

FUSED_CONV = ("QuantizedConvolutionBias", "QuantizedConvolutionBiasRelu", "QuantizedConvolutionBiasAdd",
              "QuantizedConvolutionBiasSignedAdd", "QuantizedConvolutionRelu")
TDT = {np.dtype(np.uint8): torch.uint8, np.dtype(np.int8): torch.int8, np.dtype(np.int32): torch.int32,
       np.dtype(np.float32): torch.float32}


@pytest.fixture(scope="module")
def ops():
    from ngraph_b200 import ops as o
    return o


@pytest.fixture(autouse=True)
def device_status_clean():
    yield
    from ngraph_b200 import lib
    lib.device_status()


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def pad_k(a, mult=16):
    """Zero-pad the reduction (last) axis to a multiple of 16 bytes (zeros do not change the sums)."""
    k = a.shape[-1]
    kp = (k + mult - 1) // mult * mult
    if kp == k:
        return a
    out = np.zeros(a.shape[:-1] + (kp,), a.dtype)
    out[..., :k] = a
    return out


def same_f32(got, exp):
    np.testing.assert_array_equal(np.where(got == 0, 0.0, got).view(np.uint32), np.where(exp == 0, 0.0, exp).view(np.uint32))


def nhwc(a):
    return np.ascontiguousarray(a.transpose(0, 2, 3, 1))


def run_conv(ops, data_nchw, filt_kcrs, bias, scale, cs, out_dt, relu, sum_in=None, sum_scale=None, core=False, out_zp=0,
             packed=False):
    cp = ops.conv_params((cs.N, cs.H, cs.W, cs.C), (cs.K, cs.R, cs.S, cs.C), (cs.stride_h, cs.stride_w),
                         (cs.pad_h, cs.pad_w), (cs.pad_h_above, cs.pad_w_above), (cs.dil_h, cs.dil_w))
    out = ops.qconv(dev(nhwc(data_nchw)), dev(nhwc(filt_kcrs)), dev(np.atleast_1d(scale).astype(np.float32)),
                    TDT[np.dtype(out_dt)], cp, bias=dev(bias), relu=relu,
                    sum_in=None if sum_in is None else dev(nhwc(sum_in)),
                    sum_scale=None if sum_in is None else dev(np.array([sum_scale], np.float32)), core=core, out_zp=out_zp,
                    packed=packed)
    return out.cpu().numpy().transpose(0, 3, 1, 2)


# ---------------------------------------------------------------- fixtures
def test_reference_quantized_dot_bias_vectors(ops):
    for case in reference_tests("QuantizedDotBias"):
        out_dt = NP[case["expected"]["dtype"]]
        a = pad_k(typed(case["data"], case["shape_a"]))
        w = pad_k(typed(case["weights"], case["shape_b"]))
        got = ops.qgemm(dev(a), dev(w), dev(np.array([f32_from_bits(case["scale_bits"])], np.float32)), TDT[np.dtype(out_dt)],
                        bias=dev(typed(case["bias"])), relu=case["relu"]).cpu().numpy()
        np.testing.assert_array_equal(got.ravel(), typed(case["expected"]), err_msg=case["name"])


def test_reference_quantized_dot_vectors(ops):
    for case in reference_tests("QuantizedDot"):
        c = case["consts"]
        if c["input_zero_point"] or c["filter_zero_point"]:
            continue  # non-zero input zero points are outside the tensor-core path (none among the reference's vectors)
        a = pad_k(typed(case["a"], case["shape_a"]))
        w = pad_k(np.ascontiguousarray(typed(case["b"], case["shape_b"]).T))
        scale = np.float32(c["input_scale"]) * np.float32(c["filter_scale"]) / np.float32(c["output_scale"])
        out_dt = NP[case["expected"]["dtype"]]
        got = ops.qgemm(dev(a), dev(w), dev(np.array([scale], np.float32)), TDT[np.dtype(out_dt)], core=True,
                        out_zp=c["output_zero_point"]).cpu().numpy()
        np.testing.assert_array_equal(got.ravel(), typed(case["expected"]), err_msg=case["name"])


def test_reference_quantized_convolution_vectors(ops):
    """test/backend/quantized_convolution.in.cpp: one input channel (zero-padded to 64 for the tensor cores), i8 and u8 filters"""
    for case in reference_tests("QuantizedConvolution"):
        if case["uses_builder"]:
            v = [x[1] for x in case["f32_consts"]]
            f32 = np.float32
            sd, sf, so = f32(max(abs(v[0]), abs(v[1]))) / f32(255), f32(max(abs(v[2]), abs(v[3]))) / f32(127), \
                f32(max(abs(v[4]), abs(v[5]))) / f32(127)
            zo = 0
        else:
            c = case["consts"]
            if c["input_zero_point"] or c["filter_zero_point"]:
                continue
            sd, sf, so, zo = np.float32(c["input_scale"]), np.float32(c["filter_scale"]), np.float32(c["output_scale"]), c["output_zero_point"]
        data, filt = typed(case["a"], case["shape_a"]), typed(case["b"], case["shape_b"])
        n, ch, h, w = data.shape
        dpad = np.zeros((n, 64, h, w), data.dtype)
        dpad[:, :ch] = data
        fpad = np.zeros((filt.shape[0], 64) + filt.shape[2:], filt.dtype)
        fpad[:, :ch] = filt
        cs = ref.conv_shape(dpad.shape, fpad.shape, case["stride"], case["pad_below"], case["pad_above"], case["dilation"])
        out_dt = NP[case["expected"]["dtype"]]
        got = run_conv(ops, dpad, fpad, None, np.float32(sd * sf / so), cs, out_dt, False, core=True, out_zp=zo)
        np.testing.assert_array_equal(got.ravel(), typed(case["expected"]), err_msg=case["name"])


def test_interpreter_fused_dot(ops):
    for case in interpreter_cases("QuantizedDotBias"):
        i = {k: blob(v) for k, v in case["inputs"].items()}
        exp = blob(case["outputs"]["y"])
        got = ops.qgemm(dev(i["data"]), dev(i["weights"]), dev(i["scale"]), TDT[exp.dtype], bias=dev(i["bias"]),
                        relu=bool(case["attrs"]["relu"])).cpu().numpy()
        if exp.dtype == np.float32:
            same_f32(got, exp)
        else:
            np.testing.assert_array_equal(got, exp, err_msg=case["name"])


def test_interpreter_fused_convolution(ops):
    for case in interpreter_cases(FUSED_CONV):
        i = {k: blob(v) for k, v in case["inputs"].items()}
        a = case["attrs"]
        exp = blob(case["outputs"]["y"])
        cs = ref.conv_shape(i["data"].shape, i["filters"].shape, a["stride"], a["pad_below"], a["pad_above"], a["dilation"])
        signed = case["op"] == "QuantizedConvolutionBiasSignedAdd"
        out_dt = np.int8 if signed else exp.dtype
        kw = {}
        if "sum_in" in i:
            kw = dict(sum_in=i["sum_in"], sum_scale=i["sum_scale"].ravel()[0])
        got = run_conv(ops, i["data"], i["filters"], i.get("bias"), i["scale"], cs, out_dt, bool(a["relu"]), **kw)
        np.testing.assert_array_equal(got.astype(exp.dtype), exp, err_msg=case["name"])


# ---------------------------------------------------------------- seeded, against the oracle
GEMM_SHAPES = [(1, 16, 16), (7, 10, 48), (128, 128, 128), (129, 65, 144), (300, 1000, 2048), (256, 1024, 1024),
               (513, 272, 400)]


@pytest.mark.parametrize("mnk", GEMM_SHAPES)
@pytest.mark.parametrize("a_signed", [False, True])
def test_qgemm_vs_oracle(ops, mnk, a_signed):
    m, n, k = mnk
    rng = np.random.default_rng(m * 31 + n * 7 + k + a_signed)
    a = rng.integers(-128, 128, size=(m, k)).astype(np.int8) if a_signed else rng.integers(0, 256, size=(m, k)).astype(np.uint8)
    w = rng.integers(-127, 128, size=(n, k)).astype(np.int8)
    bias = rng.integers(-1000, 1001, size=n).astype(np.int32)
    acc_sigma = np.sqrt(k) * 74 * (74 if a_signed else 147)
    for per_channel in (False, True):
        scale = (np.exp(rng.uniform(np.log(0.5), np.log(2.0), size=n if per_channel else 1)) * 40.0 / acc_sigma).astype(np.float32)
        for out_dt, relu in ((np.uint8, True), (np.int8, False), (np.float32, False), (np.float32, True), (np.int32, False)):
            exp = ref.qgemm_fused(a, w, bias, scale, out_dt, relu=relu)
            for packed in (False, True):  # plain [N,K] weights through TMA / the packed image through bulk copies
                got = ops.qgemm(dev(a), dev(w), dev(scale), TDT[np.dtype(out_dt)], bias=dev(bias), relu=relu, packed=packed).cpu().numpy()
                if out_dt == np.float32:
                    same_f32(got, exp)
                else:
                    np.testing.assert_array_equal(got, exp, err_msg="%s %s relu=%d packed=%d" % (mnk, out_dt, relu, packed))
    # core contract (QuantizedDot): half-away rounding, output zero point, saturation
    scale1 = np.float32(30.0 / acc_sigma)
    for out_dt, zp in ((np.int8, 3), (np.uint8, 100), (np.int32, -5)):
        exp = ref.qgemm_core(a, w, scale1, zp, out_dt)
        got = ops.qgemm(dev(a), dev(w), dev(np.array([scale1], np.float32)), TDT[np.dtype(out_dt)], core=True, out_zp=zp).cpu().numpy()
        np.testing.assert_array_equal(got, exp, err_msg="core %s %s" % (mnk, out_dt))


@pytest.mark.parametrize("k,a_signed", [(64, False), (128, False), (192, False), (128, True), (256, True)])
def test_short_reductions_with_small_and_large_biases(ops, k, a_signed):
    """Extreme operands (every product at its largest magnitude, both signs) with biases that bring accumulator + bias to the
    edge of +-2^22, just beyond it and far beyond (up to +-2^30), side by side in one launch, with and without a residual:
    the int32 sum, its conversion to float and the saturation must hold over the whole int32 range, not only for the
    magnitudes random data produces."""
    rng = np.random.default_rng(k + a_signed)
    m, n = 384, 512
    a = (rng.integers(-128, 128, size=(m, k)).astype(np.int8) if a_signed else rng.integers(0, 256, size=(m, k)).astype(np.uint8))
    w = rng.integers(-128, 128, size=(n, k)).astype(np.int8)
    a[0], a[1] = (-128 if a_signed else 255), (127 if a_signed else 255)   # rows of extreme activations
    w[0::64], w[1::64] = -128, 127                                            # columns of extreme weights in every 64-column block
    bound = k * (128 if a_signed else 255) * 128
    room = (1 << 22) - 1 - bound
    bias = rng.integers(-1000, 1001, size=n).astype(np.int64)
    if room > 0:
        bias[0:64] = rng.integers(-room, room + 1, size=64)        # everything the guarantee admits
        bias[0], bias[1] = -room, room                             # ... up to the very edge, on the extreme columns
        bias[64:128] = rng.integers(-room, room + 1, size=64)
        bias[70] = room + 1                                        # one bias just beyond: this block converts the usual way
    bias[128:192] = rng.integers(-(1 << 30), 1 << 30, size=64)     # far beyond
    bias = bias.astype(np.int32)
    scale = (np.exp(rng.uniform(np.log(0.5), np.log(2.0), size=n)) * 3e-5).astype(np.float32)
    s = rng.integers(0, 256, size=(m, n)).astype(np.uint8)
    for out_dt, relu in ((np.uint8, True), (np.int8, False), (np.int8, True)):
        for sum_in in (None, s):
            kw = {} if sum_in is None else {"sum_in": sum_in, "sum_scale": np.float32(0.41)}
            exp = ref.qgemm_fused(a, w, bias, scale, out_dt, relu=relu, **kw)
            dkw = {} if sum_in is None else {"sum_in": dev(sum_in), "sum_scale": dev(np.array([0.41], np.float32))}
            got = ops.qgemm(dev(a), dev(w), dev(scale), TDT[np.dtype(out_dt)], bias=dev(bias), relu=relu, **dkw).cpu().numpy()
            np.testing.assert_array_equal(got, exp, err_msg="k=%d %s relu=%d sum=%s" % (k, out_dt, relu, sum_in is not None))


def test_qgemm_sum_input(ops):
    rng = np.random.default_rng(5)
    m, n, k = 2000, 96, 256  # enough outputs that a product fused with the residual addition (one rounding) would show
    a = rng.integers(0, 256, size=(m, k)).astype(np.uint8)
    w = rng.integers(-127, 128, size=(n, k)).astype(np.int8)
    bias = rng.integers(-1000, 1001, size=n).astype(np.int32)
    scale = np.full(n, 2e-4, np.float32)
    for sdt in (np.uint8, np.int8):
        s = rng.integers(np.iinfo(sdt).min, np.iinfo(sdt).max + 1, size=(m, n)).astype(sdt)
        for out_dt, relu in ((np.uint8, True), (np.int8, False), (np.int8, True)):
            exp = ref.qgemm_fused(a, w, bias, scale, out_dt, relu=relu, sum_in=s, sum_scale=np.float32(0.37))
            got = ops.qgemm(dev(a), dev(w), dev(scale), TDT[np.dtype(out_dt)], bias=dev(bias), relu=relu, sum_in=dev(s),
                            sum_scale=dev(np.array([0.37], np.float32))).cpu().numpy()
            np.testing.assert_array_equal(got, exp)


CONV_CASES = [
    # N, C, H, W, K, R, S, stride, pad_below, pad_above, dilation
    (2, 64, 8, 8, 64, 3, 3, (1, 1), (1, 1), (1, 1), (1, 1)),
    (3, 64, 7, 7, 32, 3, 3, (1, 1), (1, 1), (1, 1), (1, 1)),
    (2, 128, 14, 14, 96, 1, 1, (1, 1), (0, 0), (0, 0), (1, 1)),
    (2, 128, 14, 14, 256, 1, 1, (2, 2), (0, 0), (0, 0), (1, 1)),
    (2, 64, 15, 13, 64, 3, 3, (2, 2), (1, 1), (1, 1), (1, 1)),
    (1, 64, 12, 12, 16, 3, 3, (1, 1), (2, 2), (2, 2), (2, 2)),
    (2, 256, 9, 9, 40, 3, 3, (1, 2), (1, 0), (0, 1), (1, 1)),
    (5, 64, 5, 6, 8, 5, 3, (1, 1), (2, 1), (2, 1), (1, 1)),
    (4, 128, 10, 10, 320, 3, 3, (1, 1), (1, 1), (1, 1), (1, 1)),   # three column tiles, the last one ragged
    (40, 64, 16, 16, 192, 1, 1, (1, 1), (0, 0), (0, 0), (1, 1)),   # 80 row tiles x width 192
]


@pytest.mark.parametrize("cfg", CONV_CASES)
def test_qconv_vs_oracle(ops, cfg):
    n, c, h, w, k, r, s, stride, pb, pa, dil = cfg
    rng = np.random.default_rng(hash(cfg) % (2 ** 31))
    data = rng.integers(0, 256, size=(n, c, h, w)).astype(np.uint8)
    filt = rng.integers(-127, 128, size=(k, c, r, s)).astype(np.int8)
    bias = rng.integers(-1000, 1001, size=k).astype(np.int32)
    cs = ref.conv_shape(data.shape, filt.shape, stride, pb, pa, dil)
    acc_sigma = np.sqrt(c * r * s) * 74 * 147
    scale = (np.exp(rng.uniform(np.log(0.5), np.log(2.0), size=k)) * 60.0 / acc_sigma).astype(np.float32)
    p, q = ref.conv_out_hw(cs)
    for out_dt, relu in ((np.uint8, True), (np.int8, False)):
        exp = ref.qconv_fused(data, filt, bias, scale, cs, out_dt, relu=relu)
        for packed in (False, True):
            got = run_conv(ops, data, filt, bias, scale, cs, out_dt, relu, packed=packed)
            np.testing.assert_array_equal(got, exp, err_msg="%s packed=%d" % (cfg, packed))
    sum_u8 = rng.integers(0, 256, size=(n, k, p, q)).astype(np.uint8)
    exp = ref.qconv_fused(data, filt, bias, scale, cs, np.uint8, relu=True, sum_in=sum_u8, sum_scale=np.float32(0.61))
    for packed in (False, True):
        got = run_conv(ops, data, filt, bias, scale, cs, np.uint8, True, sum_in=sum_u8, sum_scale=0.61, packed=packed)
        np.testing.assert_array_equal(got, exp, err_msg="add %s packed=%d" % (cfg, packed))
    sum_i8 = rng.integers(-128, 128, size=(n, k, p, q)).astype(np.int8)
    exp = ref.qconv_fused(data, filt, bias, scale[:1], cs, np.int8, relu=True, sum_in=sum_i8, sum_scale=np.float32(1.3))
    got = run_conv(ops, data, filt, bias, scale[:1], cs, np.int8, True, sum_in=sum_i8, sum_scale=1.3)
    np.testing.assert_array_equal(got, exp, err_msg="signed add " + str(cfg))
    # core contract: QuantizedConvolution -> i32 with unit scales (raw accumulators) and -> i8 requantised
    exp = ref.qconv_core(data, filt, cs, 1.0, 0, 1.0, 0, 1.0, 0, np.int32)
    got = run_conv(ops, data, filt, None, np.float32(1.0), cs, np.int32, False, core=True)
    np.testing.assert_array_equal(got, exp, err_msg="core i32 " + str(cfg))


def test_qconv_baseline_layer(ops):
    """The single-convolution workload: QuantizedConvolutionBias+Relu, u8 [32,64,56,56] * i8 [64,64,3,3], per-channel
    scales, i32 bias, stride 1 pad 1 -> u8.  The oracle runs on a batch slice (a few seconds); the rest
    of the batch is checked through linearity in the batch index (each image is independent)."""
    rng = np.random.default_rng(3)
    data = rng.integers(0, 256, size=(32, 64, 56, 56)).astype(np.uint8)
    filt = rng.integers(-127, 128, size=(64, 64, 3, 3)).astype(np.int8)
    bias = rng.integers(-1000, 1001, size=64).astype(np.int32)
    sf = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), size=64)).astype(np.float32)
    scale = (np.float32(0.02) * sf / np.float32(0.05)).astype(np.float32)
    cs = ref.conv_shape(data.shape, filt.shape, (1, 1), (1, 1), (1, 1), (1, 1))
    got = run_conv(ops, data, filt, bias, scale, cs, np.uint8, True)
    sl = [0, 17, 31]
    cs1 = ref.conv_shape((len(sl),) + data.shape[1:], filt.shape, (1, 1), (1, 1), (1, 1), (1, 1))
    exp = ref.qconv_fused(data[sl], filt, bias, scale, cs1, np.uint8, relu=True)
    np.testing.assert_array_equal(got[sl], exp)
    # batch independence: running images one by one through the device gives the same bytes
    for b in (5, 20):
        cs_b = ref.conv_shape((1,) + data.shape[1:], filt.shape, (1, 1), (1, 1), (1, 1), (1, 1))
        one = run_conv(ops, data[b:b + 1], filt, bias, scale, cs_b, np.uint8, True)
        np.testing.assert_array_equal(one[0], got[b])


def test_layout_and_pooling(ops):
    rng = np.random.default_rng(11)
    x = rng.integers(0, 256, size=(3, 5, 7, 9)).astype(np.uint8)
    y = ops.nchw_to_nhwc(dev(x), 16).cpu().numpy()
    assert y.shape == (3, 7, 9, 16)
    np.testing.assert_array_equal(y[..., :5], x.transpose(0, 2, 3, 1))
    assert not y[..., 5:].any()
    np.testing.assert_array_equal(ops.nhwc_to_nchw(dev(y), 5).cpu().numpy(), x)
    m = rng.integers(-128, 128, size=(37, 70)).astype(np.int8)
    np.testing.assert_array_equal(ops.transpose_u8(dev(m)).cpu().numpy(), m.T)
    for case in interpreter_cases("MaxPool"):
        a = case["attrs"]
        xi = blob(case["inputs"]["x"])
        got = ops.maxpool_nhwc(dev(nhwc(xi)), a["window"], a["stride"], a["pad_below"], a["pad_above"]).cpu().numpy()
        np.testing.assert_array_equal(got.transpose(0, 3, 1, 2), blob(case["outputs"]["y"]))
    for case in interpreter_cases("GlobalAvgPoolQ"):
        i = {k: blob(v) for k, v in case["inputs"].items()}
        got = ops.global_avgpool_q(dev(nhwc(i["x"])), dev(i["s_in"].reshape(1)), dev(i["s_out"].reshape(1))).cpu().numpy()
        np.testing.assert_array_equal(got, blob(case["outputs"]["y"]).reshape(got.shape))
    big = rng.integers(0, 256, size=(4, 64, 30, 30)).astype(np.uint8)
    got = ops.maxpool_nhwc(dev(nhwc(big)), (3, 3), (2, 2), (1, 1), (1, 1)).cpu().numpy()
    np.testing.assert_array_equal(got.transpose(0, 3, 1, 2), ref.maxpool_u8(big, (3, 3), (2, 2), (1, 1), (1, 1)))
    # odd output widths and asymmetric padding through the two-outputs-per-thread form of the 3x3 / stride 2 window
    for shape, pb, pa in (((2, 32, 29, 33), (1, 1), (1, 1)), ((3, 16, 18, 21), (0, 1), (1, 0)), ((1, 64, 112, 112), (1, 1), (1, 1))):
        xs = rng.integers(0, 256, size=shape).astype(np.uint8)
        got = ops.maxpool_nhwc(dev(nhwc(xs)), (3, 3), (2, 2), pb, pa).cpu().numpy()
        np.testing.assert_array_equal(got.transpose(0, 3, 1, 2), ref.maxpool_u8(xs, (3, 3), (2, 2), pb, pa), err_msg=str(shape))


# ---------------------------------------------------------------- stride-2 small-channel stem (space-to-depth path)
STEM_CASES = [
    # N, C, H, W, K, R, S, pad_below, pad_above, data dtype
    (2, 3, 32, 32, 64, 7, 7, (3, 3), (3, 3), np.int8),     # the ResNet stem geometry, small image
    (1, 3, 224, 224, 64, 7, 7, (3, 3), (3, 3), np.uint8),  # full ResNet stem
    (3, 1, 17, 23, 16, 3, 3, (1, 1), (1, 1), np.uint8),    # odd sizes, one channel
    (2, 4, 20, 18, 32, 5, 7, (2, 3), (1, 2), np.uint8),    # asymmetric padding, four channels
    (2, 2, 16, 16, 24, 8, 8, (0, 0), (0, 0), np.int8),     # even filter without padding
    (1, 3, 9, 9, 8, 7, 7, (2, 2), (3, 3), np.uint8),       # even padding below
    (2, 3, 20, 140, 64, 7, 7, (3, 3), (3, 3), np.int8),    # 70 output columns: one partly filled 128-pixel row tile
    (1, 4, 12, 300, 32, 5, 5, (2, 2), (2, 2), np.uint8),   # 150 output columns: two row tiles, the second ragged
]


@pytest.mark.parametrize("case", STEM_CASES, ids=lambda c: "x".join(str(v) for v in c[:7]))
def test_qconv_stem_vs_oracle(ops, case):
    n, c, h, w, k, r, s, pb, pa, dt = case
    rng = np.random.default_rng(hash(case[:7]) & 0xFFFF)
    info = np.iinfo(dt)
    data = rng.integers(info.min, info.max + 1, (n, c, h, w)).astype(dt)
    filt = rng.integers(-127, 128, (k, c, r, s)).astype(np.int8)
    bias = rng.integers(-2000, 2000, k).astype(np.int32)
    scale = (rng.uniform(0.5, 1.5, k) * 255.0 / (c * r * s * 127 * 40)).astype(np.float32)
    cs = ref.conv_shape(data.shape, filt.shape, (2, 2), pb, pa)
    for out_dt, relu in ((np.uint8, True), (np.int8, False)):
        exp = ref.qconv_fused(data, filt, bias, scale, cs, out_dt, relu=relu)
        got = ops.qconv_stem(dev(data), filt, dev(scale), TDT[np.dtype(out_dt)], pb, pa, bias=dev(bias), relu=relu)
        np.testing.assert_array_equal(got.cpu().numpy().transpose(0, 3, 1, 2), exp)


def test_stem_rejects_wide_filters(ops):
    from ngraph_b200 import lib
    with pytest.raises(lib.B200Error):
        ops.stem_geometry(32, 32, 9, 9, (0, 0), (0, 0))


@pytest.mark.parametrize("q_np", [np.uint8, np.int8])
def test_stem_pack_with_fused_quantize(ops, q_np):
    """b200_stem_pack_input_f32 == b200_quantize followed by b200_stem_pack_input, every round mode."""
    from ngraph_b200.lib import LIB, check
    rng = np.random.default_rng(17)
    n, c, h, w = 2, 3, 37, 41
    x = (rng.standard_normal((n, c, h, w)) * 60).astype(np.float32)
    x.flat[:64] = (np.arange(64) - 32) * 0.5 * 0.7  # exact .5 ties after the division by 0.7
    xd = dev(x)
    scale = dev(np.array([0.7], np.float32))
    zp = dev(np.array([3], q_np))
    p, q, hc, wc, rc = ops.stem_geometry(h, w, 7, 7, (3, 3), (3, 3))
    st = torch.cuda.current_stream().cuda_stream
    for mode in range(9):
        qx = ops.quantize(xd, scale, zp, round_mode=mode)
        want = torch.empty((n, hc, wc, 16), dtype=torch.uint8, device="cuda")
        check(LIB.b200_stem_pack_input(qx.data_ptr(), want.data_ptr(), n, c, h, w, 7, 7, 3, 3, 3, 3, st), "pack")
        got = torch.full((n, hc, wc, 16), 99, dtype=torch.uint8, device="cuda")
        check(LIB.b200_stem_pack_input_f32(xd.data_ptr(), scale.data_ptr(), zp.data_ptr(), 0 if q_np == np.uint8 else 1, mode,
                                           got.data_ptr(), n, c, h, w, 7, 7, 3, 3, 3, 3, st), "pack f32")
        assert torch.equal(got, want), "round mode %d" % mode


HALO_CASES = [
    # N, C, H, W, K, R, S, pad: stride 1, weights small enough to stay in shared memory -> the patch-with-halo path
    (2, 64, 56, 56, 64, 3, 3, (1, 1)),    # the 56x56 64 -> 64 layer geometry, small batch
    (3, 64, 31, 45, 64, 3, 3, (1, 1)),    # ragged in both directions
    (2, 64, 20, 33, 32, 3, 3, (0, 0)),    # no padding
    (1, 128, 17, 64, 32, 3, 3, (1, 1)),   # 128-byte rows
    (2, 64, 12, 40, 48, 5, 3, (2, 1)),    # 5 x 3 filter
]


@pytest.mark.parametrize("case", HALO_CASES, ids=lambda c: "x".join(str(v) for v in c[:7]))
def test_qconv_halo_path_vs_oracle(ops, case):
    n, c, h, w, k, r, s, pad = case
    rng = np.random.default_rng(hash(case[:7]) & 0xFFFF)
    data = rng.integers(0, 256, (n, c, h, w)).astype(np.uint8)
    filt = rng.integers(-127, 128, (k, c, r, s)).astype(np.int8)
    bias = rng.integers(-1000, 1001, k).astype(np.int32)
    cs = ref.conv_shape(data.shape, filt.shape, (1, 1), pad, pad)
    scale = (np.exp(rng.uniform(np.log(0.5), np.log(2.0), k)) * 60.0 / (np.sqrt(c * r * s) * 74 * 147)).astype(np.float32)
    p, q = ref.conv_out_hw(cs)
    exp = ref.qconv_fused(data, filt, bias, scale, cs, np.uint8, relu=True)
    for packed in (False, True):
        got = run_conv(ops, data, filt, bias, scale, cs, np.uint8, True, packed=packed)
        np.testing.assert_array_equal(got, exp, err_msg="packed=%d" % packed)
    sum_u8 = rng.integers(0, 256, (n, k, p, q)).astype(np.uint8)
    exp = ref.qconv_fused(data, filt, bias, scale, cs, np.uint8, relu=True, sum_in=sum_u8, sum_scale=np.float32(0.4))
    got = run_conv(ops, data, filt, bias, scale, cs, np.uint8, True, sum_in=sum_u8, sum_scale=0.4)
    np.testing.assert_array_equal(got, exp, err_msg="residual")
    exp = ref.qconv_core(data, filt, cs, 1.0, 0, 1.0, 0, 1.0, 0, np.int32)
    got = run_conv(ops, data, filt, None, np.float32(1.0), cs, np.int32, False, core=True)
    np.testing.assert_array_equal(got, exp, err_msg="core i32")


# ---------------------------------------------------------------- two row tiles per CTA sharing each B stage
@pytest.mark.parametrize("m,n,k", [(24576, 768, 3072), (24576 + 100, 768, 3072), (8192, 1024, 4096)])
def test_large_qgemm_with_paired_row_tiles(ops, m, n, k):
    """Problems large enough that a CTA takes two 128-row tiles at a time (they share every weight stage): every output type
    the kernel has a store path for, against the oracle on rows taken from first / second tiles of pairs, from the ragged last
    tile and from the tile that only exists as padding of an odd tile count."""
    rng = np.random.default_rng(m + n + k)
    a = rng.integers(0, 256, size=(m, k)).astype(np.uint8)
    w = rng.integers(-127, 128, size=(n, k)).astype(np.int8)
    bias = rng.integers(-1000, 1001, size=n).astype(np.int32)
    scale = (np.exp(rng.uniform(np.log(0.5), np.log(2.0), size=n)) * 40.0 / (np.sqrt(k) * 74 * 147)).astype(np.float32)
    rows = np.concatenate([np.arange(0, 40), np.arange(128 + 90, 128 + 130), np.arange(5 * 256 + 120, 5 * 256 + 140),
                           np.arange((m // 128 - 1) * 128 - 8, m)])
    ad, wd, sd, bd = dev(a), dev(w), dev(scale), dev(bias)
    for out_dt, relu in ((np.uint8, True), (np.float32, False), (np.int8, False), (np.int32, False)):
        exp = ref.qgemm_fused(a[rows], w, bias, scale, out_dt, relu=relu)
        for packed in (True, False):
            got = ops.qgemm(ad, wd, sd, TDT[np.dtype(out_dt)], bias=bd, relu=relu, packed=packed)[torch.from_numpy(rows).cuda()].cpu().numpy()
            if out_dt == np.float32:
                same_f32(got, exp)
            else:
                np.testing.assert_array_equal(got, exp, err_msg="%s relu=%d packed=%d" % (out_dt, relu, packed))


@pytest.mark.parametrize("n,c,hw,k,r", [(128, 128, 28, 128, 3), (128, 256, 14, 256, 3), (65, 256, 14, 256, 3), (128, 512, 7, 512, 3)])
def test_large_qconv_at_full_batch(ops, n, c, hw, k, r):
    """ResNet-50 layer shapes at batch 128 (and an odd count of row tiles), where tile width and scheduling are chosen for a
    full device: images from the first, a middle and the last tiles against the oracle, with and without a residual input"""
    rng = np.random.default_rng(n + c + hw)
    data = rng.integers(0, 256, size=(n, c, hw, hw)).astype(np.uint8)
    filt = rng.integers(-127, 128, size=(k, c, r, r)).astype(np.int8)
    bias = rng.integers(-1000, 1001, size=k).astype(np.int32)
    scale = (np.exp(rng.uniform(np.log(0.5), np.log(2.0), size=k)) * 60.0 / (np.sqrt(c * r * r) * 74 * 147)).astype(np.float32)
    pad = (r // 2, r // 2)
    cs = ref.conv_shape(data.shape, filt.shape, (1, 1), pad, pad, (1, 1))
    sl = [0, 1, n // 2, n - 2, n - 1]
    cs_s = ref.conv_shape((len(sl),) + data.shape[1:], filt.shape, (1, 1), pad, pad, (1, 1))
    got = run_conv(ops, data, filt, bias, scale, cs, np.uint8, True, packed=True)
    np.testing.assert_array_equal(got[sl], ref.qconv_fused(data[sl], filt, bias, scale, cs_s, np.uint8, relu=True))
    sum_u8 = rng.integers(0, 256, size=(n, k, hw, hw)).astype(np.uint8)
    got = run_conv(ops, data, filt, bias, scale, cs, np.uint8, True, sum_in=sum_u8, sum_scale=0.61, packed=True)
    np.testing.assert_array_equal(got[sl], ref.qconv_fused(data[sl], filt, bias, scale, cs_s, np.uint8, relu=True, sum_in=sum_u8[sl],
                                                           sum_scale=np.float32(0.61)))


def test_repeated_calls_reuse_the_launch_plan_not_the_data(ops):
    """The entry points keep the launch set-up of an argument list they have seen (tile choice, tensor maps, shared-memory
    plan).  Same pointers with new contents must give new results; same contents at other addresses the same results."""
    rng = np.random.default_rng(17)
    a = rng.integers(0, 256, size=(300, 256)).astype(np.uint8)
    w = rng.integers(-127, 128, size=(96, 256)).astype(np.int8)
    scale = np.full(96, 3e-4, np.float32)
    ad, wd, sd = dev(a), dev(w), dev(scale)
    out = torch.empty((300, 96), dtype=torch.uint8, device="cuda")
    for _ in range(3):
        ops.qgemm(ad, wd, sd, torch.uint8, relu=True, out=out)
    np.testing.assert_array_equal(out.cpu().numpy(), ref.qgemm_fused(a, w, None, scale, np.uint8, relu=True))
    a2 = rng.integers(0, 256, size=a.shape).astype(np.uint8)
    ad.copy_(torch.from_numpy(a2))  # same address, other bytes
    ops.qgemm(ad, wd, sd, torch.uint8, relu=True, out=out)
    np.testing.assert_array_equal(out.cpu().numpy(), ref.qgemm_fused(a2, w, None, scale, np.uint8, relu=True))
    other = ops.qgemm(dev(a2), dev(w), dev(scale), torch.uint8, relu=True)  # other addresses, same bytes
    assert torch.equal(other, out)
    data = rng.integers(0, 256, size=(2, 64, 12, 12)).astype(np.uint8)
    filt = rng.integers(-127, 128, size=(64, 64, 3, 3)).astype(np.int8)
    bias = rng.integers(-1000, 1001, size=64).astype(np.int32)
    cs = ref.conv_shape(data.shape, filt.shape, (1, 1), (1, 1), (1, 1), (1, 1))
    first = run_conv(ops, data, filt, bias, scale[:64], cs, np.uint8, True)
    again = run_conv(ops, data, filt, bias, scale[:64], cs, np.uint8, True)
    np.testing.assert_array_equal(first, again)
    np.testing.assert_array_equal(first, ref.qconv_fused(data, filt, bias, scale[:64], cs, np.uint8, relu=True))
