#!/usr/bin/env python3
"""Regenerates the fixtures in this directory.  Needs the nGraph reference checkout.

    python tests/golden/make_golden.py [--ref /path/to/ngraph]

1. ``interpreter_cases.json``: seeded cases run through the reference's own INTERPRETER
   backend by ``oracle/_ref/gen_golden`` (built by ``make -C oracle ref``).
2. ``reference_tests.json``: the known-answer vectors of the reference's own tests for
   this path, read out of its test sources as text:
     test/backend/quantize_dequantize.in.cpp   Quantize / Dequantize, all round modes
     test/backend/quantized_dot.in.cpp         QuantizedDot
     test/backend/quantized_convolution.in.cpp QuantizedConvolution
     test/builder_quantization.cpp             fused ops (results computed by oneDNN there)
   For the builder tests the scale constants are obtained by running nGraph's own builder +
   ConstantFolding on the test's min/max ranges (``gen_golden scales``).

The fixtures are data; the tests never read the reference checkout.
"""
import argparse
import json
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
GEN = os.path.join(ROOT, "oracle", "_ref", "gen_golden")

ET = {"element::f32": "f32", "element::f64": "f64", "element::u8": "u8", "element::i8": "i8",
      "element::i32": "i32"}
CT = {"float": "f32", "double": "f64", "uint8_t": "u8", "int8_t": "i8", "int32_t": "i32"}
LIMITS = {"u8": (0, 255), "i8": (-128, 127), "i32": (-2 ** 31, 2 ** 31 - 1)}
ROUND = ["ROUND_NEAREST_TOWARD_INFINITY", "ROUND_NEAREST_TOWARD_ZERO", "ROUND_NEAREST_UPWARD",
         "ROUND_NEAREST_DOWNWARD", "ROUND_NEAREST_TOWARD_EVEN", "ROUND_TOWARD_INFINITY", "ROUND_TOWARD_ZERO",
         "ROUND_UP", "ROUND_DOWN"]


def split_tests(text, macro):
    """name -> body for every TEST-like macro in a gtest source."""
    out = {}
    for m in re.finditer(macro + r"\(([^,]+),\s*(\w+)\)\s*\{", text):
        start = m.end()
        depth, i = 1, start
        while depth:
            depth += {"{": 1, "}": -1}.get(text[i], 0)
            i += 1
        out[m.group(2)] = text[start:i - 1]
    return out


def strip_comments(body):
    return re.sub(r"//[^\n]*", "", body)


def numbers(src, env=None):
    src = src.replace("\n", " ").strip()
    if not src:
        return []
    vals = []
    for tok in src.split(","):
        tok = tok.strip()
        if not tok:
            continue
        tok = re.sub(r"(?<=[0-9.])f\b", "", tok)
        vals.append(eval(tok, {"__builtins__": {}}, env or {}))  # plain arithmetic literals only
    return vals


def shape_of(body, name):
    m = re.search(r"Shape\s+" + name + r"\s*=?\s*(?:\{([^}]*)\})?\s*;", body)
    if not m:
        raise KeyError(name)
    return [int(v) for v in numbers(m.group(1) or "")]


def parse_qdq(name, body):
    body = strip_comments(body)
    it = ET[re.search(r"auto input_type = (element::\w+);", body).group(1)]
    ot = ET[re.search(r"auto output_type = (element::\w+);", body).group(1)]
    quant = ot != "f32" and ot != "f64"
    qt = ot if quant else it
    env = {}
    if qt in LIMITS:
        env = {"max": LIMITS[qt][1], "min": LIMITS[qt][0]}
    axes = re.search(r"AxisSet quantization_axes(?:\{([^}]*)\})?;", body)
    case = {
        "name": name, "op": "Quantize" if quant else "Dequantize", "input_type": it, "output_type": ot,
        "shape": shape_of(body, "input_shape"), "scale_shape": shape_of(body, "scale_offset_shape"),
        "axes": [int(v) for v in numbers(axes.group(1) or "")],
    }
    rm = re.search(r"RoundMode::(ROUND_\w+);", body)
    if rm:
        case["round_mode"] = ROUND.index(rm.group(1))
    consts = re.findall(r"auto (\w+) =\s*op::v0::Constant::create\(\s*\w+,\s*\w+,\s*\{([^}]*)\}\)", body)
    for cname, vals in consts:
        case[cname] = numbers(vals, env)
    for var, vals in re.findall(r"copy_data\((\w+),\s*vector<\w+>\{([^}]*)\}\)", body):
        case[{"Scale": "scale", "Offset": "offset"}.get(var, var)] = numbers(vals, env)
    exp = re.search(r"vector<output_c_type>\{([^}]*)\}\)?,\s*read_vector", body, re.S)
    case["expected"] = numbers(exp.group(1), env)
    if "offset" in case:
        case["zero_point"] = case.pop("offset")
    return case


def parse_vectors(body):
    out = {}
    for ctype, name, vals in re.findall(r"vector<(\w+)>\s+(\w+)\s*=\s*\{([^}]*)\};", body):
        out[name] = {"dtype": CT[ctype], "data": numbers(vals)}
    return out


def parse_qdot(name, body):
    body = strip_comments(body)
    vec = parse_vectors(body)
    consts = dict((n, (ET[t], numbers(v)[0])) for n, t, v in
                  re.findall(r"auto (\w+) = op::v0::Constant::create\((element::\w+), Shape\{\}, \{([^}]*)\}\)", body))
    exp = re.search(r"EXPECT_EQ\(\(vector<(\w+)>\{([^}]*)\}\)", body)
    return {"name": name, "op": "QuantizedDot", "a": vec["a_data"], "b": vec["b_data"],
            "shape_a": shape_of(body, "shape_a"), "shape_b": shape_of(body, "shape_b"),
            "consts": {k: v[1] for k, v in consts.items()},
            "expected": {"dtype": CT[exp.group(1)], "data": numbers(exp.group(2))}}


def parse_qconv(name, body):
    body = strip_comments(body)
    vec = parse_vectors(body)
    exp = re.search(r"EXPECT_EQ\(\(vector<(\w+)>\{([^}]*)\}\)", body)
    case = {"name": name, "op": "QuantizedConvolution", "a": vec["a_data"], "b": vec["b_data"],
            "shape_a": shape_of(body, "shape_a"), "shape_b": shape_of(body, "shape_b"),
            "shape_r": shape_of(body, "shape_r"),
            "expected": {"dtype": CT[exp.group(1)], "data": numbers(exp.group(2))}}
    f32c = re.findall(r"auto (\w+) = op::v0::Constant::create\(element::f32, Shape\{1?\}, \{([^}]*)\}\)", body)
    case["f32_consts"] = [[n, numbers(v)[0]] for n, v in f32c]
    allc = re.findall(r"auto (\w+) = op::v0::Constant::create\((element::\w+), Shape\{1?\}, \{([^}]*)\}\)", body)
    case["consts"] = {n: numbers(v)[0] for n, t, v in allc}
    case["uses_builder"] = "QuantizedConvolutionBuilder" in body
    floats = [numbers(v)[0] for v in re.findall(r"copy_data\(\w+, vector<float>\{([^}]*)\}\)", body)]
    if not case["uses_builder"] and len(floats) == 3:  # scales arrive as run-time tensors: in, filter, out
        zps = [numbers(v)[0] for n, t, v in allc if t != "element::f32"]
        case["consts"] = {"input_scale": floats[0], "filter_scale": floats[1], "output_scale": floats[2],
                          "input_zero_point": zps[0], "filter_zero_point": zps[1], "output_zero_point": zps[2]}
    if case["uses_builder"]:  # min/max ranges arrive as run-time tensors
        case["f32_consts"] = [["range%d" % i, numbers(v)[0]] for i, v in
                              enumerate(re.findall(r"copy_data\(\w+, vector<float>\{([^}]*)\}\)", body))]
    pads = re.findall(r"CoordinateDiff\{(\d+),\s*(\d+)\}", body)
    strides = re.findall(r"Strides\{(\d+),\s*(\d+)\}", body)
    case["pad_below"] = [int(v) for v in pads[0]] if pads else [0, 0]
    case["pad_above"] = [int(v) for v in pads[1]] if len(pads) > 1 else case["pad_below"]
    case["stride"] = [int(v) for v in strides[0]] if strides else [1, 1]
    case["dilation"] = [int(v) for v in strides[1]] if len(strides) > 1 else [1, 1]
    return case


BUILDER_TESTS = ["scaled_QC_with_bias", "scaled_QC_with_bias_and_relu", "scaled_QC_with_bias_add_and_relu",
                 "scaled_QC_with_bias_signed_add_and_relu"]


def builder_scales(builder, requantize, relu, ranges):
    out = subprocess.check_output([GEN, "scales", builder, str(int(requantize)), str(int(relu))] +
                                  [repr(float(v)) for v in ranges])
    return json.loads(out)


def parse_builder_conv(name, body):
    body = strip_comments(body)
    vec = parse_vectors(body)
    builder = re.search(r"ngraph::builder::(\w+)\(", body).group(1)
    ranges = [numbers(v)[0] for v in
              re.findall(r"auto [A-Z] = op::v0::Constant::create\(element::f32, Shape\{1?\}, \{([^}]*)\}\)", body)]
    call = body[body.index("ngraph::builder::"):]
    call = call[:call.index(";")]
    relu = bool(re.search(r",\s*true\)\s*$", call.strip()))
    exp = re.search(r"EXPECT_EQ\(\(vector<(\w+)>\{([^}]*)\}\)", body)
    sc = builder_scales(builder, True, relu, ranges)
    pads = re.findall(r"CoordinateDiff\{(\d+),\s*(\d+)\}", body)
    case = {"name": name, "op": sc["op"], "builder": builder, "relu": relu, "ranges": ranges,
            "data": vec["a_data"], "filters": vec["b_data"], "bias": vec["c_data"],
            "shape_a": shape_of(body, "shape_a"), "shape_b": shape_of(body, "shape_b"),
            "pad_below": [int(v) for v in pads[0]], "pad_above": [int(v) for v in pads[1]],
            "scale_bits": sc["scale_bits"],
            "expected": {"dtype": CT[exp.group(1)], "data": numbers(exp.group(2))}}
    if "conv_2_data" in vec:
        case["sum_in"] = vec["conv_2_data"]
        case["sum_scale_bits"] = sc["sum_scale_bits"]
    return case


def parse_builder_dot(body):
    body = strip_comments(body)
    vec = parse_vectors(body)
    ranges = [numbers(v)[0] for v in re.findall(r"copy_data\(\w+, vector<float>\{([^}]*)\}\)", body)]
    exps = re.findall(r"EXPECT_EQ\(\(vector<(\w+)>\{([^}]*)\}\)", body, re.S)
    modes = [(False, False), (False, True), (True, False), (True, True)]
    cases = []
    for (requant, relu), (ctype, vals) in zip(modes, exps):
        sc = builder_scales("QuantizedDotBiasBuilder", requant, relu, ranges)
        data = numbers(vals)
        cases.append({"name": "dynamic_scaled_QD_with_bias_rq%d_relu%d" % (requant, relu), "op": "QuantizedDotBias",
                      "requantize": requant, "relu": relu, "ranges": ranges, "data": vec["a_data"],
                      "weights": vec["b_data"], "bias": vec["c_data"], "shape_a": shape_of(body, "shape_a"),
                      "shape_b": shape_of(body, "shape_b"), "scale_bits": sc["scale_bits"],
                      "expected": {"dtype": CT[ctype], "data": data}})
    return cases


def main():
    ap = argparse.ArgumentParser()
    from ngraph_b200.build import ngraph_checkout
    ap.add_argument("--ref", default=ngraph_checkout(), help="root of the nGraph checkout (default: $NGRAPH_REF or the reference build recipe's)")
    args = ap.parse_args()
    if not os.path.exists(GEN):
        sys.exit("build the reference first: make -C oracle ref")
    subprocess.check_call([GEN, "interp", os.path.join(HERE, "interpreter_cases.json")])

    cases = []
    read = lambda rel: open(os.path.join(args.ref, rel)).read()
    for name, body in split_tests(read("test/backend/quantize_dequantize.in.cpp"), "NGRAPH_TEST").items():
        cases.append(dict(parse_qdq(name, body), source="test/backend/quantize_dequantize.in.cpp"))
    for name, body in split_tests(read("test/backend/quantized_dot.in.cpp"), "NGRAPH_TEST").items():
        cases.append(dict(parse_qdot(name, body), source="test/backend/quantized_dot.in.cpp"))
    for name, body in split_tests(read("test/backend/quantized_convolution.in.cpp"), "NGRAPH_TEST").items():
        cases.append(dict(parse_qconv(name, body), source="test/backend/quantized_convolution.in.cpp"))
    btests = split_tests(read("test/builder_quantization.cpp"), "TEST")
    for name in BUILDER_TESTS:
        cases.append(dict(parse_builder_conv(name, btests[name]), source="test/builder_quantization.cpp"))
    for c in parse_builder_dot(btests["dynamic_scaled_QD_with_bias"]):
        cases.append(dict(c, source="test/builder_quantization.cpp"))
    with open(os.path.join(HERE, "reference_tests.json"), "w") as f:
        json.dump(cases, f, indent=0, separators=(",", ":"))
        f.write("\n")
    print("wrote %d reference test cases" % len(cases))


if __name__ == "__main__":
    main()
