"""Pins the CPU oracle (oracle/ngraph_oracle.c) against
  (1) the known-answer vectors of the reference's own tests (tests/golden/reference_tests.json) and
  (2) outputs of the reference's INTERPRETER backend on seeded inputs
      (tests/golden/interpreter_cases.json).
Integer outputs must be bit-exact; f32 outputs bit-exact as well (single multiply)."""
import numpy as np
import pytest

from oracle import ref
from tests.fixtures import NP, blob, f32_from_bits, interpreter_cases, reference_tests, typed

FUSED_CONV = ("QuantizedConvolutionBias", "QuantizedConvolutionBiasRelu", "QuantizedConvolutionBiasAdd",
              "QuantizedConvolutionBiasSignedAdd", "QuantizedConvolutionRelu")


def ids(cases):
    return [c["name"] for c in cases]


# ---------------------------------------------------------------- reference's own test vectors
@pytest.mark.parametrize("case", reference_tests(("Quantize", "Dequantize")), ids=ids(reference_tests(("Quantize", "Dequantize"))))
def test_reference_quantize_dequantize_vectors(case):
    if "f64" in (case["input_type"], case["output_type"]):
        pytest.skip("f64 Quantize/Dequantize is outside the f32 hot path")
    shape, ss = case["shape"], case["scale_shape"]
    if case["op"] == "Quantize":
        qt = NP[case["output_type"]]
        got = ref.quantize(np.array(case["x"], np.float32).reshape(shape), np.array(case["scale"], np.float32).reshape(ss),
                           np.array(case["zero_point"], qt).reshape(ss), case["axes"], case["round_mode"])
        assert got.dtype == qt
        np.testing.assert_array_equal(got.ravel(), np.array(case["expected"], qt))
    else:
        qt = NP[case["input_type"]]
        got = ref.dequantize(np.array(case["x"], qt).reshape(shape), np.array(case["scale"], np.float32).reshape(ss),
                             np.array(case["zero_point"], qt).reshape(ss), case["axes"])
        np.testing.assert_array_equal(got.ravel(), np.array(case["expected"], np.float32))


@pytest.mark.parametrize("case", reference_tests("QuantizedDot"), ids=ids(reference_tests("QuantizedDot")))
def test_reference_quantized_dot_vectors(case):
    c = case["consts"]
    got = ref.qdot_core(typed(case["a"], case["shape_a"]), typed(case["b"], case["shape_b"]), c["input_scale"],
                        c["input_zero_point"], c["filter_scale"], c["filter_zero_point"], c["output_scale"],
                        c["output_zero_point"], NP[case["expected"]["dtype"]])
    np.testing.assert_array_equal(got.ravel(), typed(case["expected"]))


@pytest.mark.parametrize("case", reference_tests("QuantizedConvolution"), ids=ids(reference_tests("QuantizedConvolution")))
def test_reference_quantized_convolution_vectors(case):
    cs = ref.conv_shape(case["shape_a"], case["shape_b"], case["stride"], case["pad_below"], case["pad_above"],
                        case["dilation"])
    if case["uses_builder"]:
        # builder: scale = max(|min|,|max|) / 255 (u8) or 127 (i8), src/ngraph/builder/quantization_utils.cpp:33-79
        v = [x[1] for x in case["f32_consts"]]
        f32 = np.float32
        sd = f32(max(abs(v[0]), abs(v[1]))) / f32(255)
        sf = f32(max(abs(v[2]), abs(v[3]))) / f32(127)
        so = f32(max(abs(v[4]), abs(v[5]))) / f32(127)
        got = ref.qconv_core(typed(case["a"], case["shape_a"]), typed(case["b"], case["shape_b"]), cs, sd, 0, sf, 0, so,
                             0, NP[case["expected"]["dtype"]])
    else:
        c = case["consts"]
        got = ref.qconv_core(typed(case["a"], case["shape_a"]), typed(case["b"], case["shape_b"]), cs, c["input_scale"],
                             c["input_zero_point"], c["filter_scale"], c["filter_zero_point"], c["output_scale"],
                             c["output_zero_point"], NP[case["expected"]["dtype"]])
    np.testing.assert_array_equal(got.ravel(), typed(case["expected"]))


@pytest.mark.parametrize("case", reference_tests(FUSED_CONV), ids=ids(reference_tests(FUSED_CONV)))
def test_reference_fused_convolution_vectors(case):
    """The oneDNN-computed expectations of test/builder_quantization.cpp pin scale -> sum -> relu ->
    round-half-even -> saturate (the Add/SignedAdd cases contain exact .5 ties)."""
    cs = ref.conv_shape(case["shape_a"], case["shape_b"], (1, 1), case["pad_below"], case["pad_above"])
    signed = case["op"] == "QuantizedConvolutionBiasSignedAdd"
    out_dt = np.int8 if (signed or not case["relu"]) else np.uint8
    kw = {}
    if "sum_in" in case:
        p, q = ref.conv_out_hw(cs)
        kw = dict(sum_in=typed(case["sum_in"], (cs.N, cs.K, p, q)), sum_scale=f32_from_bits(case["sum_scale_bits"]))
    got = ref.qconv_fused(typed(case["data"], case["shape_a"]), typed(case["filters"], case["shape_b"]),
                          typed(case["bias"]), f32_from_bits(case["scale_bits"]), cs, out_dt, relu=case["relu"], **kw)
    exp = typed(case["expected"])
    np.testing.assert_array_equal(got.ravel().astype(exp.dtype), exp)


@pytest.mark.parametrize("case", reference_tests("QuantizedDotBias"), ids=ids(reference_tests("QuantizedDotBias")))
def test_reference_quantized_dot_bias_vectors(case):
    out_dt = NP[case["expected"]["dtype"]]
    got = ref.qgemm_fused(typed(case["data"], case["shape_a"]), typed(case["weights"], case["shape_b"]),
                          typed(case["bias"]), f32_from_bits(case["scale_bits"]), out_dt, relu=case["relu"])
    exp = typed(case["expected"])
    if out_dt == np.float32:
        np.testing.assert_array_equal(got.ravel(), exp)  # exact fp32 equality (-0.0 == 0.0)
    else:
        np.testing.assert_array_equal(got.ravel(), exp)


# ---------------------------------------------------------------- INTERPRETER outputs on seeded inputs
def _axes(c):
    return c["attrs"]["axes"]


@pytest.mark.parametrize("case", interpreter_cases("Quantize"), ids=ids(interpreter_cases("Quantize")))
def test_interpreter_quantize(case):
    i = {k: blob(v) for k, v in case["inputs"].items()}
    got = ref.quantize(i["x"], i["scale"], i["zero_point"], _axes(case), case["attrs"]["round_mode"])
    np.testing.assert_array_equal(got, blob(case["outputs"]["y"]))


@pytest.mark.parametrize("case", interpreter_cases("Dequantize"), ids=ids(interpreter_cases("Dequantize")))
def test_interpreter_dequantize(case):
    i = {k: blob(v) for k, v in case["inputs"].items()}
    got = ref.dequantize(i["x"], i["scale"], i["zero_point"], _axes(case))
    np.testing.assert_array_equal(got.view(np.uint32), blob(case["outputs"]["y"]).view(np.uint32))


@pytest.mark.parametrize("case", interpreter_cases("QuantizedDot"), ids=ids(interpreter_cases("QuantizedDot")))
def test_interpreter_quantized_dot(case):
    i = {k: blob(v) for k, v in case["inputs"].items()}
    a = case["attrs"]
    exp = blob(case["outputs"]["y"])
    got = ref.qdot_core(i["a"], i["b"], i["sa"], a["za"], i["sb"], a["zb"], i["so"], a["zo"], exp.dtype)
    np.testing.assert_array_equal(got, exp)


def conv_shape_of(case):
    a = case["attrs"]
    return ref.conv_shape(case["inputs"]["data"]["shape"], case["inputs"]["filters"]["shape"], a["stride"],
                          a["pad_below"], a["pad_above"], a["dilation"])


@pytest.mark.parametrize("case", interpreter_cases("QuantizedConvolution"), ids=ids(interpreter_cases("QuantizedConvolution")))
def test_interpreter_quantized_convolution(case):
    i = {k: blob(v) for k, v in case["inputs"].items()}
    a = case["attrs"]
    exp = blob(case["outputs"]["y"])
    got = ref.qconv_core(i["data"], i["filters"], conv_shape_of(case), i["sd"], a["zd"], i["sf"], a["zf"], i["so"],
                         a["zo"], exp.dtype)
    np.testing.assert_array_equal(got, exp)


@pytest.mark.parametrize("case", interpreter_cases("QuantizedDotBias"), ids=ids(interpreter_cases("QuantizedDotBias")))
def test_interpreter_fused_dot(case):
    i = {k: blob(v) for k, v in case["inputs"].items()}
    exp = blob(case["outputs"]["y"])
    got = ref.qgemm_fused(i["data"], i["weights"], i["bias"], i["scale"], exp.dtype, relu=bool(case["attrs"]["relu"]))
    if exp.dtype == np.float32:
        np.testing.assert_array_equal(got.view(np.uint32) & 0x7FFFFFFF | (got.view(np.uint32) & 0x80000000) * (got != 0),
                                      exp.view(np.uint32) & 0x7FFFFFFF | (exp.view(np.uint32) & 0x80000000) * (exp != 0))
    else:
        np.testing.assert_array_equal(got, exp)


@pytest.mark.parametrize("case", interpreter_cases(FUSED_CONV), ids=ids(interpreter_cases(FUSED_CONV)))
def test_interpreter_fused_convolution(case):
    i = {k: blob(v) for k, v in case["inputs"].items()}
    exp = blob(case["outputs"]["y"])
    signed = case["op"] == "QuantizedConvolutionBiasSignedAdd"
    out_dt = np.int8 if signed else exp.dtype
    kw = {}
    if "sum_in" in i:
        kw = dict(sum_in=i["sum_in"], sum_scale=i["sum_scale"].ravel()[0])
    got = ref.qconv_fused(i["data"], i["filters"], i.get("bias"), i["scale"], conv_shape_of(case), out_dt,
                          relu=bool(case["attrs"]["relu"]), **kw)
    np.testing.assert_array_equal(got.astype(exp.dtype), exp)


def test_interpreter_pooling():
    for case in interpreter_cases("MaxPool"):
        a = case["attrs"]
        got = ref.maxpool_u8(blob(case["inputs"]["x"]), a["window"], a["stride"], a["pad_below"], a["pad_above"])
        np.testing.assert_array_equal(got, blob(case["outputs"]["y"]))
    for case in interpreter_cases("GlobalAvgPoolQ"):
        i = {k: blob(v) for k, v in case["inputs"].items()}
        got = ref.global_avgpool_q(i["x"], i["s_in"], i["s_out"])
        np.testing.assert_array_equal(got, blob(case["outputs"]["y"]))
