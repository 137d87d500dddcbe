"""The nGraph backend plugin (libb200_backend.so) driven the way any nGraph client drives a backend:
build a Function, Backend::create("B200"), compile, create_tensor, write, call_with_validate, read.
GPU tests run the same Function (or, for the fused ops INTERPRETER lacks, its decomposition) on
nGraph's own INTERPRETER backend in the same process and compare: integers bit-exact, f32 bit-exact."""
import ctypes
import os

import numpy as np
import pytest

from tests.fixtures import blob, interpreter_cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ng = pytest.importorskip("ngraph_b200.ngraph_api")
from oracle import interpreter
from oracle import ref as ref_c  # noqa: E402

needs_ngraph = pytest.mark.skipif(not interpreter.available(), reason="nGraph host library / INTERPRETER not built here")


# ---------------------------------------------------------------- CPU: boundary and harness
def test_plugin_exports_registration_symbol():
    path = os.path.join(ROOT, "ngraph_b200", "libb200_backend.so")
    if not os.path.exists(path):
        pytest.skip("plugin not built (needs nGraph headers)")
    ng.capi()  # libngraph must be in the process before the plugin resolves its symbols
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    assert hasattr(lib, "ngraph_register_b200_backend")


def test_plugin_exports_nothing_but_the_registration_symbol():
    """BackendManager finds a backend by dlsym of ngraph_register_<name>_backend (backend_manager.cpp:105-113): that is the
    plugin's whole C ABI.  Its dynamic symbol table holds no other function or object of its own (weak template / inline
    instantiations the C++ runtime may merge across libraries do not count)."""
    import shutil
    import subprocess
    path = os.path.join(ROOT, "ngraph_b200", "libb200_backend.so")
    if not os.path.exists(path) or not shutil.which("nm"):
        pytest.skip("plugin not built, or no nm")
    rows = subprocess.check_output(["nm", "-D", "--defined-only", path], text=True).split("\n")
    strong = [r.split() for r in rows if r.strip() and r.split()[-2] in ("T", "D", "B", "R")]
    assert [r[-1] for r in strong] == ["ngraph_register_b200_backend"], strong


@needs_ngraph
def test_backend_registers_and_fails_loudly_without_a_device():
    import torch
    ng.load_b200()
    assert "B200" in ng.registered_backends()
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(ng.NgraphError):
        ng.Backend("B200")  # no CUDA device: creation raises, nothing falls back to the host


@needs_ngraph
def test_bogus_backend_name_raises():
    with pytest.raises(ng.NgraphError):
        ng.Backend("NO_SUCH_BACKEND")


@needs_ngraph
def test_decomposed_oracle_graphs_match_fixtures():
    """oracle/interpreter.py's decompositions, run on INTERPRETER here, reproduce the committed fixtures."""
    be = interpreter.backend()
    for case in interpreter_cases("QuantizedDotBias")[:4]:
        i = {k: blob(v) for k, v in case["inputs"].items()}
        exp = blob(case["outputs"]["y"])
        x, w = ng.parameter(np.uint8, i["data"].shape), ng.parameter(np.int8, i["weights"].shape)
        b, s = ng.parameter(np.int32, i["bias"].shape), ng.parameter(np.float32, i["scale"].shape)
        y = interpreter.decomposed_dot_bias(x, w, b, s, exp.dtype, bool(case["attrs"]["relu"]))
        got = be.compile(ng.Function([y], [x, w, b, s])).run(i["data"], i["weights"], i["bias"], i["scale"])[0]
        np.testing.assert_array_equal(got.view(np.uint8), exp.view(np.uint8), err_msg=case["name"])
    for case in interpreter_cases("QuantizedConvolutionBiasAdd")[:2] + interpreter_cases("QuantizedConvolutionBiasSignedAdd")[:1]:
        i = {k: blob(v) for k, v in case["inputs"].items()}
        a = case["attrs"]
        exp = blob(case["outputs"]["y"])
        d, f = ng.parameter(np.uint8, i["data"].shape), ng.parameter(np.int8, i["filters"].shape)
        b, s = ng.parameter(np.int32, i["bias"].shape), ng.parameter(np.float32, i["scale"].shape)
        sm, ss = ng.parameter(i["sum_in"].dtype, i["sum_in"].shape), ng.parameter(np.float32, i["sum_scale"].shape)
        y = interpreter.decomposed_conv(d, f, b, s, exp.dtype, True, a["stride"], a["dilation"], a["pad_below"], a["pad_above"],
                                        sum_in=sm, sum_scale=ss, signed=case["op"].endswith("SignedAdd"))
        got = be.compile(ng.Function([y], [d, f, b, s, sm, ss])).run(i["data"], i["filters"], i["bias"], i["scale"],
                                                                      i["sum_in"], i["sum_scale"])[0]
        np.testing.assert_array_equal(got, exp, err_msg=case["name"])


# ---------------------------------------------------------------- GPU: B200 vs INTERPRETER, same process
@pytest.fixture(scope="module")
def backends():
    ng.load_b200()
    return ng.Backend("B200"), interpreter.backend()


def run_both(backends, fn_b200, fn_ref, inputs):
    b200, ref = backends
    got = b200.compile(fn_b200).run(*inputs)
    exp = ref.compile(fn_ref).run(*inputs)
    return got, exp


def same_bits(got, exp, msg=""):
    assert got.dtype == exp.dtype and got.shape == exp.shape, (got.dtype, exp.dtype, got.shape, exp.shape)
    if got.dtype == np.float32:
        g, e = np.where(got == 0, 0.0, got).astype(np.float32), np.where(exp == 0, 0.0, exp).astype(np.float32)
        np.testing.assert_array_equal(g.view(np.uint32), e.view(np.uint32), err_msg=msg)
    else:
        np.testing.assert_array_equal(got, exp, err_msg=msg)


@pytest.mark.gpu
@needs_ngraph
@pytest.mark.parametrize("mode", range(9))
def test_quantize_dequantize_graph(backends, mode):
    rng = np.random.default_rng(mode)
    x = (rng.standard_normal((2, 64, 16, 16)) * 3).astype(np.float32)
    x.ravel()[::7] = (np.round(x.ravel()[::7] / 0.05) + 0.5) * np.float32(0.05)
    for dtype, zp, axes in ((np.uint8, 128, ()), (np.int8, 0, ()), (np.uint8, None, (1,)), (np.int8, None, (1,))):
        ss = tuple(x.shape[a] for a in axes)
        scale = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=ss)).astype(np.float32) if axes else np.float32(0.05)
        zpa = np.full(ss, 7, dtype) if zp is None else np.array(zp, dtype)
        p = ng.parameter(np.float32, x.shape)
        q = ng.quantize(p, scale, zpa, dtype, axes, mode)
        dq = ng.dequantize(q, scale, zpa, axes)
        fn = ng.Function([q, dq], [p])
        got, exp = run_both(backends, fn, fn, [x])
        same_bits(got[0], exp[0], "quantize %s %s" % (dtype, axes))
        same_bits(got[1], exp[1], "dequantize %s %s" % (dtype, axes))


@pytest.mark.gpu
@needs_ngraph
def test_dynamic_scale_parameters(backends):
    """scale and zero point as run-time tensors (test/backend/quantize_dequantize.in.cpp:981-1056)."""
    x = np.array([0, 3, 128, 255], np.uint8)
    p, s, z = ng.parameter(np.uint8, (4,)), ng.parameter(np.float32, ()), ng.parameter(np.uint8, ())
    fn = ng.Function([ng.dequantize(p, s, z)], [p, s, z])
    got, exp = run_both(backends, fn, fn, [x, np.float32(2), np.uint8(128)])
    same_bits(got[0], exp[0])
    np.testing.assert_array_equal(got[0], np.array([-256, -250, 0, 254], np.float32))


@pytest.mark.gpu
@needs_ngraph
def test_quantized_dot_core(backends):
    # INTERPRETER implements u8 x i8 -> i8 and -> i32 only (int_executable.hpp:1573-1644)
    rng = np.random.default_rng(1)
    a = rng.integers(0, 256, size=(37, 64)).astype(np.uint8)
    b = rng.integers(-127, 128, size=(64, 24)).astype(np.int8)
    for out_dtype, so, zo in ((np.int8, 3000.0, 3), (np.int32, 0.5, -4)):
        pa, pb = ng.parameter(np.uint8, a.shape), ng.parameter(np.int8, b.shape)
        fn = ng.Function([ng.quantized_dot(pa, pb, 0.5, 0, 0.25, 0, so, zo, out_dtype)], [pa, pb])
        got, exp = run_both(backends, fn, fn, [a, b])
        same_bits(got[0], exp[0], str(out_dtype))
        # and with B as a Constant (transposed once at compile time)
        fn2 = ng.Function([ng.quantized_dot(pa, ng.constant(b), 0.5, 0, 0.25, 0, so, zo, out_dtype)], [pa])
        got2 = backends[0].compile(fn2).run(a)
        same_bits(got2[0], exp[0], "constant B " + str(out_dtype))
    # u8 x u8 (INTERPRETER: -> u8 and -> i32), run-time and constant B
    bu = rng.integers(0, 256, size=(64, 24)).astype(np.uint8)
    for out_dtype, so, zo in ((np.uint8, 9000.0, 5), (np.int32, 0.5, 7)):
        pa, pb = ng.parameter(np.uint8, a.shape), ng.parameter(np.uint8, bu.shape)
        fn = ng.Function([ng.quantized_dot(pa, pb, 0.5, 0, 0.25, 0, so, zo, out_dtype)], [pa, pb])
        got, exp = run_both(backends, fn, fn, [a, bu])
        same_bits(got[0], exp[0], "u8 x u8 " + str(out_dtype))
        fn2 = ng.Function([ng.quantized_dot(pa, ng.constant(bu), 0.5, 0, 0.25, 0, so, zo, out_dtype)], [pa])
        same_bits(backends[0].compile(fn2).run(a)[0], exp[0], "u8 x u8 constant B " + str(out_dtype))


@pytest.mark.gpu
@needs_ngraph
@pytest.mark.parametrize("za,zb", [(128, 0), (0, -5), (37, 11)])
def test_quantized_dot_with_zero_points(backends, za, zb):
    """sum_k (a - za) * (b - zb) of reference::dot (dot.hpp:134-159): the device subtracts the rank-one terms from exact
    int32 accumulators.  Large K on purpose: the accumulators pass 2^24, where a float would lose bits."""
    rng = np.random.default_rng(za * 7 + zb + 100)
    a = rng.integers(0, 256, size=(45, 2048)).astype(np.uint8)
    b = rng.integers(-127, 128, size=(2048, 40)).astype(np.int8)
    b[:, 0] = 127  # a column that drives the raw sum far beyond 2^24
    for out_dtype, so, zo in ((np.int8, 40000.0, 3), (np.int32, 0.5, -4)):
        pa, pb = ng.parameter(np.uint8, a.shape), ng.parameter(np.int8, b.shape)
        fn = ng.Function([ng.quantized_dot(pa, pb, 0.5, za, 0.25, zb, so, zo, out_dtype)], [pa, pb])
        got, exp = run_both(backends, fn, fn, [a, b])
        same_bits(got[0], exp[0], str(out_dtype))
        fn2 = ng.Function([ng.quantized_dot(pa, ng.constant(b), 0.5, za, 0.25, zb, so, zo, out_dtype)], [pa])
        same_bits(backends[0].compile(fn2).run(a)[0], exp[0], "constant B " + str(out_dtype))
    if zb >= 0:
        bu = rng.integers(0, 256, size=(2048, 40)).astype(np.uint8)
        pa, pb = ng.parameter(np.uint8, a.shape), ng.parameter(np.uint8, bu.shape)
        fn = ng.Function([ng.quantized_dot(pa, pb, 0.5, za, 0.25, zb, 0.5, 9, np.int32)], [pa, pb])
        got, exp = run_both(backends, fn, fn, [a, bu])
        same_bits(got[0], exp[0], "u8 x u8")


@pytest.mark.gpu
@needs_ngraph
@pytest.mark.parametrize("za,zf", [(128, 0), (0, 9), (100, -7)])
@pytest.mark.parametrize("geom", [dict(pad_below=(1, 1)), dict(stride=(2, 2), pad_below=(2, 1), pad_above=(0, 2), dilation=(2, 1)), dict()])
def test_quantized_convolution_with_zero_points(backends, za, zf, geom):
    """reference::convolution (convolution.hpp:236-258) skips the taps that fall into the padding, so the correction
    terms depend on where the output pixel sits; borders, strides and dilation are all exercised."""
    rng = np.random.default_rng(za + zf + len(geom) + 100)
    for channels in (64, 48):  # 48: padded to the kernels' channel granule on the device (constant filters only)
        ds, fs = (2, channels, 9, 8), (24, channels, 3, 3)
        data = rng.integers(0, 256, size=ds).astype(np.uint8)
        filt = rng.integers(-127, 128, size=fs).astype(np.int8)
        for out_dtype, so, zo in ((np.int32, 1.0, 5), (np.int8, 60000.0, -2)):
            d, f = ng.parameter(np.uint8, ds), ng.parameter(np.int8, fs)
            fn = ng.Function([ng.quantized_convolution(d, f, 1.0, za, 1.0, zf, so, zo, out_dtype, **geom)], [d, f])
            exp = backends[1].compile(fn).run(data, filt)[0]
            if channels % 64 == 0:
                same_bits(backends[0].compile(fn).run(data, filt)[0], exp, str(out_dtype))
            fn2 = ng.Function([ng.quantized_convolution(d, ng.constant(filt), 1.0, za, 1.0, zf, so, zo, out_dtype, **geom)], [d])
            same_bits(backends[0].compile(fn2).run(data)[0], exp, "constant filters %d %s" % (channels, out_dtype))


@pytest.mark.gpu
@needs_ngraph
def test_quantized_dot_bias(backends):
    rng = np.random.default_rng(2)
    x = rng.integers(0, 256, size=(50, 128)).astype(np.uint8)
    w = rng.integers(-127, 128, size=(40, 128)).astype(np.int8)
    bias = rng.integers(-1000, 1000, size=40).astype(np.int32)
    for per_channel in (False, True):
        scale = (np.exp(rng.uniform(-1, 1, size=40 if per_channel else 1)) * 3e-4).astype(np.float32)
        for requant, relu in ((False, False), (False, True), (True, False), (True, True)):
            out_dtype = (np.uint8 if relu else np.int8) if requant else np.float32
            px = ng.parameter(np.uint8, x.shape)
            ps = ng.parameter(np.float32, scale.shape)  # the scale is a run-time tensor
            fused = ng.Function([ng.quantized_dot_bias(px, w, bias, ps, requant, relu)], [px, ps])
            px2, ps2 = ng.parameter(np.uint8, x.shape), ng.parameter(np.float32, scale.shape)
            ref = ng.Function([interpreter.decomposed_dot_bias(px2, ng.constant(w), ng.constant(bias), ps2, out_dtype, relu)],
                              [px2, ps2])
            got, exp = run_both(backends, fused, ref, [x, scale])
            same_bits(got[0], exp[0], "requant %s relu %s" % (requant, relu))


@pytest.mark.gpu
@needs_ngraph
@pytest.mark.parametrize("act_dtype", [np.uint8, np.int8])
@pytest.mark.parametrize("out_scale", [0.05, 5.0])
def test_baseline_quantized_dot_bias_layer(backends, act_dtype, out_scale):
    """The single-layer workload as a graph: X f32 [256,1024] ~N(0,1) -> Quantize(0.02, zp 0, RNE) -> QuantizedDotBias+Relu with
    W i8 [1024,1024] (scale 0.01), bias f32 ~N(0,0.1) quantised to i32 with scale 0.02*0.01, requantised with
    0.02*0.01/out_scale.  out_scale 0.05 is the config as written (most outputs saturate); 5.0 is its non-saturating twin
    that exercises the rounding.  u8 activations are the reference-runnable variant, i8 the one the workload names."""
    rng = np.random.default_rng(1)
    x = rng.standard_normal((256, 1024)).astype(np.float32)
    w = rng.integers(-127, 128, size=(1024, 1024)).astype(np.int8)
    bias_f = (rng.standard_normal(1024) * 0.1).astype(np.float32)
    s_in, s_w = np.float32(0.02), np.float32(0.01)
    bias = ref_c.quantize(bias_f, np.float32(s_in * s_w), np.int32(0))
    scale = np.array([np.float32(np.float32(s_in * s_w) / np.float32(out_scale))], np.float32)
    zp = act_dtype(0)

    def build(fused):
        px = ng.parameter(np.float32, x.shape)
        q = ng.quantize(px, s_in, zp, act_dtype)
        if fused:
            return ng.Function([ng.quantized_dot_bias(q, w, bias, scale, True, True)], [px])
        return ng.Function([interpreter.decomposed_dot_bias(q, ng.constant(w), ng.constant(bias), ng.constant(scale), np.uint8, True)],
                           [px])

    got, exp = run_both(backends, build(True), build(False), [x])
    same_bits(got[0], exp[0])
    saturated = float((got[0] == 255).mean())
    assert (saturated > 0.15) if out_scale == 0.05 else (saturated < 0.01)  # half of the outputs are negative -> 0 after ReLU


CONVS = [
    # data NCHW, filters KCRS, stride, pad_below, pad_above, dilation
    ((2, 64, 9, 9), (32, 64, 3, 3), (1, 1), (1, 1), (1, 1), (1, 1)),
    ((2, 128, 8, 8), (64, 128, 1, 1), (2, 2), (0, 0), (0, 0), (1, 1)),
    ((1, 64, 11, 10), (16, 64, 3, 3), (2, 2), (1, 1), (1, 1), (1, 1)),
    ((2, 3, 20, 20), (8, 3, 7, 7), (2, 2), (3, 3), (3, 3), (1, 1)),      # small-channel stem path
    ((2, 16, 6, 6), (8, 16, 3, 3), (1, 1), (1, 1), (1, 1), (1, 1)),      # channels padded to 64 on the device
]


@pytest.mark.gpu
@needs_ngraph
@pytest.mark.parametrize("cfg", CONVS)
def test_fused_convolutions(backends, cfg):
    ds, fs, stride, pb, pa, dil = cfg
    rng = np.random.default_rng(sum(ds) + sum(fs))
    data = rng.integers(0, 256, size=ds).astype(np.uint8)
    filt = rng.integers(-127, 128, size=fs).astype(np.int8)
    bias = rng.integers(-1000, 1000, size=fs[0]).astype(np.int32)
    sigma = np.sqrt(fs[1] * fs[2] * fs[3]) * 74 * 147
    geom = dict(stride=stride, dilation=dil, pad_below=pb, pad_above=pa)
    for per_channel in (False, True):
        scale = (np.exp(rng.uniform(-0.7, 0.7, size=fs[0] if per_channel else 1)) * 60.0 / sigma).astype(np.float32)
        for relu in (False, True):
            out_dtype = np.uint8 if relu else np.int8
            d = ng.parameter(np.uint8, ds)
            fused = ng.Function([ng.quantized_conv_bias(d, filt, bias, scale, relu, **geom)], [d])
            d2 = ng.parameter(np.uint8, ds)
            ref = ng.Function([interpreter.decomposed_conv(d2, ng.constant(filt), ng.constant(bias), ng.constant(scale),
                                                           out_dtype, relu, **geom)], [d2])
            got, exp = run_both(backends, fused, ref, [data])
            same_bits(got[0], exp[0], "bias relu=%s per_channel=%s" % (relu, per_channel))
    # QuantizedConvolutionRelu (no bias)
    d = ng.parameter(np.uint8, ds)
    fused = ng.Function([ng.quantized_conv_relu(d, filt, scale, **geom)], [d])
    d2 = ng.parameter(np.uint8, ds)
    ref = ng.Function([interpreter.decomposed_conv(d2, ng.constant(filt), None, ng.constant(scale), np.uint8, True, **geom)], [d2])
    got, exp = run_both(backends, fused, ref, [data])
    same_bits(got[0], exp[0], "conv relu")
    # BiasAdd (u8 sum) and BiasSignedAdd (i8 sum, i8 result converted to u8 as the builder does)
    os_ = exp[0].shape
    for signed in (False, True):
        sdt = np.int8 if signed else np.uint8
        s_in = rng.integers(np.iinfo(sdt).min, np.iinfo(sdt).max + 1, size=os_).astype(sdt)
        ssc = np.array([0.73], np.float32)
        d, sm = ng.parameter(np.uint8, ds), ng.parameter(sdt, os_)
        y = ng.quantized_conv_bias_add(d, filt, bias, sm, scale, ssc, True, signed, **geom)
        if signed:
            y = ng.convert(y, np.uint8)
        fused = ng.Function([y], [d, sm])
        d2, sm2 = ng.parameter(np.uint8, ds), ng.parameter(sdt, os_)
        ref = ng.Function([interpreter.decomposed_conv(d2, ng.constant(filt), ng.constant(bias), ng.constant(scale), np.uint8, True,
                                                       sum_in=sm2, sum_scale=ng.constant(ssc), signed=signed, **geom)], [d2, sm2])
        got, exp2 = run_both(backends, fused, ref, [data, s_in])
        same_bits(got[0], exp2[0], "add signed=%s" % signed)


@pytest.mark.gpu
@needs_ngraph
def test_core_quantized_convolution(backends):
    rng = np.random.default_rng(5)
    ds, fs = (2, 64, 7, 7), (24, 64, 3, 3)
    data = rng.integers(0, 256, size=ds).astype(np.uint8)
    filt = rng.integers(-127, 128, size=fs).astype(np.int8)
    for out_dtype, so, zo in ((np.int32, 1.0, 0), (np.int8, 12000.0, 2)):  # INTERPRETER: u8 x i8 -> i8 / i32 only; keep in range (it wraps)
        d, f = ng.parameter(np.uint8, ds), ng.parameter(np.int8, fs)
        fn = ng.Function([ng.quantized_convolution(d, f, 1.0, 0, 1.0, 0, so, zo, out_dtype, pad_below=(1, 1))], [d, f])
        got, exp = run_both(backends, fn, fn, [data, filt])
        same_bits(got[0], exp[0], str(out_dtype))
    # u8 filters (the reference's quantized_conv_int32_output test is u8 x u8)
    filt_u = rng.integers(0, 256, size=fs).astype(np.uint8)
    for out_dtype, so, zo in ((np.int32, 1.0, 0), (np.uint8, 100000.0, 3)):  # in range: the INTERPRETER wraps, the device saturates
        d, f = ng.parameter(np.uint8, ds), ng.parameter(np.uint8, fs)
        fn = ng.Function([ng.quantized_convolution(d, f, 1.0, 0, 1.0, 0, so, zo, out_dtype, pad_below=(1, 1))], [d, f])
        got, exp = run_both(backends, fn, fn, [data, filt_u])
        same_bits(got[0], exp[0], "u8 filters " + str(out_dtype))
        fn2 = ng.Function([ng.quantized_convolution(d, ng.constant(filt_u), 1.0, 0, 1.0, 0, so, zo, out_dtype, pad_below=(1, 1))], [d])
        same_bits(backends[0].compile(fn2).run(data)[0], exp[0], "u8 constant filters " + str(out_dtype))


@pytest.mark.gpu
@needs_ngraph
def test_small_network_with_pooling_head(backends):
    """Quantize -> conv+relu -> maxpool -> conv+add+relu -> Dequantize/AvgPool/Quantize head -> QuantizedDot -> Dequantize:
    the shape of the int8 ResNet graphs, end to end through both backends."""
    rng = np.random.default_rng(8)
    x = rng.standard_normal((4, 64, 12, 12)).astype(np.float32)
    w1 = rng.integers(-127, 128, size=(64, 64, 3, 3)).astype(np.int8)
    w2 = rng.integers(-127, 128, size=(64, 64, 1, 1)).astype(np.int8)
    b1 = rng.integers(-500, 500, size=64).astype(np.int32)
    s1 = (np.exp(rng.uniform(-0.5, 0.5, size=64)) * 2e-4).astype(np.float32)
    s2 = (np.exp(rng.uniform(-0.5, 0.5, size=64)) * 6e-4).astype(np.float32)
    wd = rng.integers(-127, 128, size=(64, 10)).astype(np.int8)

    def build(fused):
        p = ng.parameter(np.float32, x.shape)
        q = ng.quantize(p, np.float32(0.02), np.uint8(0), np.uint8)
        if fused:
            c1 = ng.quantized_conv_bias(q, w1, b1, s1, True, pad_below=(1, 1))
        else:
            c1 = interpreter.decomposed_conv(q, ng.constant(w1), ng.constant(b1), ng.constant(s1), np.uint8, True, pad_below=(1, 1))
        mp = ng.max_pool(c1, (3, 3), (2, 2), (1, 1))
        if fused:
            c2 = ng.quantized_conv_bias_add(mp, w2, b1, mp, s2, np.array([0.5], np.float32), True, False)
        else:
            c2 = interpreter.decomposed_conv(mp, ng.constant(w2), ng.constant(b1), ng.constant(s2), np.uint8, True, sum_in=mp,
                                             sum_scale=ng.constant(np.array([0.5], np.float32)))
        hw = c2.shape[2:]
        pooled = ng.quantize(ng.avg_pool(ng.dequantize(c2, np.float32(0.05), np.uint8(0)), hw), np.float32(0.04), np.uint8(0), np.uint8)
        flat = ng.reshape(pooled, (0, 1, 2, 3), (x.shape[0], 64))
        logits = ng.quantized_dot(flat, ng.constant(wd), 0.04, 0, 0.01, 0, 0.5, 0, np.int8)
        return ng.Function([ng.dequantize(logits, np.float32(0.5), np.int8(0)), c2], [p])

    got, exp = run_both(backends, build(True), build(False), [x])
    same_bits(got[1], exp[1], "feature map")
    same_bits(got[0], exp[0], "logits")


@pytest.mark.gpu
@needs_ngraph
@pytest.mark.parametrize("dtype", [np.uint8, np.int8])
@pytest.mark.parametrize("hw,window,stride,pad,ceil_mode", [((14, 12), (3, 3), (2, 2), (0, 0), True), ((14, 12), (3, 3), (2, 2), (1, 1), True),
                                                            ((15, 9), (2, 2), (2, 2), (0, 0), True), ((12, 12), (3, 3), (2, 2), (1, 1), False),
                                                            ((7, 10), (3, 2), (3, 2), (0, 1), True)])
def test_max_pool_with_ceil_mode_and_odd_sizes(backends, dtype, hw, window, stride, pad, ceil_mode):
    """u8 / i8 MaxPool whose last window hangs over the (padded) input when the output extent is rounded up: the device writes
    the node's own output shape and takes the maximum over the taps that exist, the rule of reference::max_pool
    (max_pool.hpp:124-236).  INTERPRETER itself refuses such windows ("The end corner is out of bounds"), so the expected
    values come from that rule restated in numpy; where INTERPRETER does run the graph it must agree as well."""
    rng = np.random.default_rng(31)
    x = rng.integers(np.iinfo(dtype).min, np.iinfo(dtype).max + 1, size=(2, 32) + hw).astype(dtype)
    p = ng.parameter(dtype, x.shape)
    fn = ng.Function([ng.max_pool(p, window, stride, pad, pad, ceil_mode=ceil_mode)], [p])
    got = backends[0].compile(fn).run(x)[0]
    div = (lambda a, b: -(-a // b)) if ceil_mode else (lambda a, b: a // b)
    P, Q = (div(hw[i] + 2 * pad[i] - window[i], stride[i]) + 1 for i in (0, 1))
    assert got.shape == (2, 32, P, Q)
    want = np.empty_like(got)
    for i in range(P):
        for j in range(Q):
            h0, w0 = i * stride[0] - pad[0], j * stride[1] - pad[1]
            want[:, :, i, j] = x[:, :, max(h0, 0):min(h0 + window[0], hw[0]), max(w0, 0):min(w0 + window[1], hw[1])].max(axis=(2, 3))
    np.testing.assert_array_equal(got, want)
    try:
        exp = backends[1].compile(fn).run(x)[0]
    except ng.NgraphError:
        assert ceil_mode
    else:
        np.testing.assert_array_equal(got, exp)


@pytest.mark.gpu
@needs_ngraph
def test_numpy_style_broadcasting_in_elementwise_ops(backends):
    """op::v1 binary ops broadcast their operands NumPy-style; compile() makes the broadcasts explicit
    (pass::ImplicitBroadcastElimination) before it lowers"""
    rng = np.random.default_rng(12)
    a, b, c = ng.parameter(np.float32, (4, 3, 5)), ng.parameter(np.float32, (5,)), ng.parameter(np.float32, (3, 1))
    fn = ng.Function([ng.multiply(ng.add(a, b), c)], [a, b, c])
    xs = [rng.standard_normal(p.shape).astype(np.float32) for p in (a, b, c)]
    got, exp = run_both(backends, fn, fn, xs)
    same_bits(got[0], exp[0])
    np.testing.assert_array_equal(got[0], ((xs[0] + xs[1]) * xs[2]).astype(np.float32))


@pytest.mark.gpu
@needs_ngraph
def test_broadcast_operands_are_read_in_place(backends):
    """Broadcast(small constant or tensor) along new leading axes feeding an elementwise op: no copy is made, the result is
    the same (large enough that ConstantFolding would otherwise have expanded the constant)"""
    rng = np.random.default_rng(13)
    x = ng.parameter(np.float32, (300, 256))
    row = rng.standard_normal(256).astype(np.float32)
    s = ng.parameter(np.float32, ())
    y = ng.add(x, ng.broadcast(ng.constant(row), (300, 256), (0,)))                  # bias row
    y = ng.multiply(ng.broadcast(s, (300, 256), (0, 1)), y)                          # run-time scalar on the left
    y = ng.add(y, ng.broadcast(ng.constant(np.float32(0.5)), (300, 256), (0, 1)))    # constant scalar
    fn = ng.Function([y], [x, s])
    xs = [rng.standard_normal((300, 256)).astype(np.float32), np.float32(1.7) * np.ones((), np.float32)]
    exe = backends[0].compile(fn, perf=True)
    got = exe.run(*xs)[0]
    same_bits(got, backends[1].compile(fn).run(*xs)[0])
    assert not any(n.startswith("Broadcast") and us > 0 for n, us, _ in exe.performance_data())


@pytest.mark.gpu
@needs_ngraph
def test_api_contract(backends):
    """create_tensor / validate / foreign tensors / unsupported ops (test/backend/api.in.cpp,
    validate_call.in.cpp, unhandled_op.in.cpp restated)."""
    b200, ref = backends
    p = ng.parameter(np.float32, (2, 3))
    fn = ng.Function([ng.quantize(p, np.float32(1), np.uint8(0), np.uint8)], [p])
    exe = b200.compile(fn)
    good_in, good_out = b200.create_tensor(np.float32, (2, 3)), b200.create_tensor(np.uint8, (2, 3))
    good_in.write(np.arange(6, dtype=np.float32))
    exe.call([good_out], [good_in])
    np.testing.assert_array_equal(good_out.read().ravel(), np.arange(6, dtype=np.uint8))
    with pytest.raises(ng.NgraphError):  # wrong input count
        exe.call([good_out], [good_in, good_in])
    with pytest.raises(ng.NgraphError):  # wrong input type
        exe.call([good_out], [b200.create_tensor(np.int32, (2, 3))])
    with pytest.raises(ng.NgraphError):  # wrong input shape
        exe.call([good_out], [b200.create_tensor(np.float32, (3, 2))])
    with pytest.raises(ng.NgraphError):  # wrong output type
        exe.call([b200.create_tensor(np.float32, (2, 3))], [good_in])
    with pytest.raises(ng.NgraphError):  # a tensor created by another backend
        exe.call([good_out], [ref.create_tensor(np.float32, (2, 3))])
    with pytest.raises(ng.NgraphError):  # an op outside the quantized path is rejected at compile, no host fallback
        q, f = ng.parameter(np.float32, (1, 2, 4, 4)), ng.parameter(np.float32, (3, 2, 1, 1))
        b200.compile(ng.Function([ng.convolution(q, f)], [q, f]))  # a float convolution is not part of the quantized path
    # per-node performance counters
    exe2 = b200.compile(ng.Function([ng.quantize(p, np.float32(1), np.uint8(0), np.uint8)], [p]), perf=True)
    exe2.call([good_out], [good_in])
    names = [n for n, us, calls in exe2.performance_data()]
    assert any(n.startswith("Quantize") for n in names)


@pytest.mark.gpu
@needs_ngraph
@pytest.mark.parametrize("data_dilation,pad_below,pad_above,stride,dilation",
                         [((2, 2), (1, 1), (1, 1), (1, 1), (1, 1)),     # zero pixels between neighbours
                          ((1, 1), (-1, -2), (0, -1), (1, 1), (1, 1)),   # negative padding crops the input
                          ((2, 3), (-1, 0), (2, -2), (2, 1), (1, 1)),    # both, with a stride
                          ((3, 2), (2, 2), (-3, 1), (1, 1), (2, 1))])    # and with a dilated window
def test_convolution_data_dilation_and_negative_padding(backends, data_dilation, pad_below, pad_above, stride, dilation):
    """legal in every convolution op (reference::general_convolution walks the dilated, signed-padded input and skips what is
    not a source coordinate, convolution.hpp:59-265): QuantizedConvolution -> i32 and the fused QuantizedConvolutionBias+Relu"""
    rng = np.random.default_rng(21)
    ds, fs = (2, 64, 9, 11), (32, 64, 3, 3)
    data = rng.integers(0, 256, size=ds).astype(np.uint8)
    filt = rng.integers(-127, 128, size=fs).astype(np.int8)
    geometry = dict(stride=stride, dilation=dilation, pad_below=pad_below, pad_above=pad_above, data_dilation=data_dilation)
    d = ng.parameter(np.uint8, ds)
    core = ng.Function([ng.quantized_convolution(d, ng.constant(filt), 1.0, 0, 1.0, 0, 1.0, 0, np.int32, **geometry)], [d])
    got, exp = run_both(backends, core, core, [data])
    same_bits(got[0], exp[0], "core")
    assert np.abs(exp[0]).max() > 0
    bias = rng.integers(-500, 500, size=32).astype(np.int32)
    scale = (np.exp(rng.uniform(-0.5, 0.5, size=32)) * 2e-4).astype(np.float32)
    fused = ng.Function([ng.quantized_conv_bias(d, filt, bias, scale, True, **geometry)], [d])
    plain = ng.Function([interpreter.decomposed_conv(d, ng.constant(filt), ng.constant(bias), ng.constant(scale), np.uint8, True, **geometry)], [d])
    got, exp = run_both(backends, fused, plain, [data])
    same_bits(got[0], exp[0], "fused")


@pytest.mark.gpu
@needs_ngraph
def test_chrome_trace_events(tmp_path):
    """NGRAPH_ENABLE_TRACING (src/ngraph/chrome_trace.hpp:77-130): like INTERPRETER's call (int_executable.cpp:122,171) the
    plugin's call writes one Duration for the call and one per executed step, category "B200".  The switch is read when
    libngraph is loaded, so the traced run is a process of its own."""
    import json
    import subprocess
    import sys
    script = (
        "import sys, numpy as np\n"
        "sys.path.insert(0, %r)\n"
        "from ngraph_b200 import ngraph_api as ng\n"
        "b = ng.Backend('B200')\n"
        "p = ng.parameter(np.float32, (4, 64))\n"
        "q = ng.quantize(p, np.float32(0.05), np.array(128, np.uint8), np.uint8, (), 4)\n"
        "fn = ng.Function([ng.dequantize(q, np.float32(0.05), np.array(128, np.uint8), ())], [p])\n"
        "out = b.compile(fn).run(np.ones((4, 64), np.float32))\n"
        "assert out[0].shape == (4, 64)\n" % ROOT)
    env = dict(os.environ, NGRAPH_ENABLE_TRACING="1")
    done = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=600, cwd=str(tmp_path), env=env)
    assert done.returncode == 0, done.stderr[-2000:]
    text = (tmp_path / "runtime_event_trace.json").read_text()
    # the file is a JSON array that the library closes at exit; tolerate a missing bracket
    text = text.strip().rstrip(",")
    if not text.endswith("]"):
        text += "]"
    events = [e for e in json.loads(text) if e.get("cat") == "B200"]
    names = [e["name"] for e in events]
    assert "call" in names and "Quantize" in names and "Dequantize" in names, names
    step = [e for e in events if e["name"] == "Quantize"][0]
    assert step["args"]["kernel"] and step["dur"] >= 0
