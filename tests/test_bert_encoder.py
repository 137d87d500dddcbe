"""In miniature and at full width: an int8 BERT-base-shaped encoder (QuantizedDotBias with per-channel i8 weights and
dynamic per-tensor i8 activation scales; softmax, LayerNorm, GELU and residual adds in f32) through the B200 plugin
against nGraph's INTERPRETER on the decomposed graph.  The CPU part checks the graph itself; the GPU part the parity."""
import collections

import numpy as np
import pytest

from oracle import interpreter

needs_reference = pytest.mark.skipif(not interpreter.available(), reason="nGraph reference libraries are not built")

DIMS = dict(layers=2, hidden=64, heads=4, ffn=128, seq=16, batch=2, vocab=100)


def _inputs(dims, seed):
    rng = np.random.default_rng(seed)
    m = dims["batch"] * dims["seq"]
    ids = rng.integers(0, dims["vocab"], m).astype(np.int32)
    seg = np.zeros((dims["batch"], dims["seq"]), np.int32)
    for b in range(dims["batch"]):
        seg[b, rng.integers(1, dims["seq"]):] = 1  # segment ids 0/1 split at a random position
    return ids, seg.reshape(m)


@needs_reference
def test_graph_lowering_uses_only_supported_ops():
    from ngraph_b200 import ngraph_api as ng
    fn = ng.bert_encoder(seed=3, **DIMS)
    ops = collections.Counter(ng.function_op_names(fn, lowered=True))
    assert ops["QuantizedDotBias"] == 6 * DIMS["layers"] and ops["Quantize"] == 6 * DIMS["layers"]
    assert ops["Softmax"] == DIMS["layers"] and ops["BatchMatMul"] == 2 * DIMS["layers"]
    supported = {"Parameter", "Constant", "Result", "Quantize", "QuantizedDotBias", "Add", "Subtract", "Multiply", "Divide", "Abs",
                 "Max", "Sum", "Sqrt", "Erf", "Broadcast", "Reshape", "Softmax", "BatchMatMul", "Gather"}
    assert set(ops) <= supported, set(ops) - supported


@needs_reference
def test_interpreter_runs_the_decomposed_encoder():
    from ngraph_b200 import ngraph_api as ng
    fn = ng.bert_encoder(seed=3, decomposed=True, **DIMS)
    out = interpreter.backend().compile(fn).run(*_inputs(DIMS, 0))[0]
    assert out.shape == (DIMS["batch"] * DIMS["seq"], DIMS["hidden"]) and np.isfinite(out).all()
    # LayerNorm output: every row is normalised before the affine step, so it cannot be constant
    assert out.std() > 0.1


@pytest.mark.gpu
@needs_reference
@pytest.mark.parametrize("dims", [DIMS, dict(layers=1, hidden=128, heads=2, ffn=256, seq=24, batch=3, vocab=50),
                                  dict(layers=2, hidden=256, heads=4, ffn=1024, seq=32, batch=2, vocab=500)])
def test_encoder_matches_interpreter(dims):
    from ngraph_b200 import ngraph_api as ng
    ng.load_b200()
    ids, seg = _inputs(dims, 1)
    want = interpreter.backend().compile(ng.bert_encoder(seed=5, decomposed=True, **dims)).run(ids, seg)[0]
    got = ng.Backend("B200").compile(ng.bert_encoder(seed=5, **dims)).run(ids, seg)[0]
    # every op reproduces the reference arithmetic (exp / erf up to the last bit), so the outputs agree far inside 1e-5
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)


def _golden_case(name):
    """(dims, ids, segments, INTERPRETER output) of one case of tests/golden/model_outputs.npz; make_model_golden.py holds the
    recipe (one encoder layer at BERT-base width: minutes of INTERPRETER time, hence computed once and committed).  With
    B200_LIVE_ORACLE set the INTERPRETER runs again instead."""
    import importlib.util
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_model_golden", os.path.join(here, "golden", "make_model_golden.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    c = gen.BERT_CASES[name]
    dims = dict(gen.BERT, seq=c["seq"], batch=c["batch"])
    ids, seg = gen.bert_inputs(c["seq"], c["batch"], gen.BERT["vocab"], c["input_seed"])
    if os.environ.get("B200_LIVE_ORACLE"):
        from ngraph_b200 import ngraph_api as ng
        want = interpreter.backend().compile(ng.bert_encoder(seed=c["model_seed"], decomposed=True, **dims)).run(ids, seg)[0]
    else:
        want = np.load(os.path.join(here, "golden", "model_outputs.npz"))[name]
    return dims, c["model_seed"], ids, seg, want


@pytest.mark.gpu
@needs_reference
@pytest.mark.parametrize("case", ["bert768_seq384", "bert768_seq128_b2"])
def test_bert_base_width_layer_matches_interpreter(case):
    """One encoder layer at BERT-base width (hidden 768, 12 heads, FFN 3072) on a 384-token sequence, and on two 128-token
    sequences: every QuantizedDotBias at its real K and N, softmax rows of 384, LayerNorm rows of 768, with the dynamic
    activation scales taken over tensors of the real size.  Bound: 1e-5 relative to the output's largest magnitude per
    element (LayerNorm output, values of order 1); the measured error is printed."""
    from ngraph_b200 import ngraph_api as ng
    ng.load_b200()
    dims, model_seed, ids, seg, want = _golden_case(case)
    got = ng.Backend("B200").compile(ng.bert_encoder(seed=model_seed, **dims)).run(ids, seg)[0]
    assert got.shape == want.shape == (dims["batch"] * dims["seq"], dims["hidden"])
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    rel = err / np.maximum(np.abs(want.astype(np.float64)), 1.0)
    print("%s: max abs err %.3g, max rel err %.3g, %d of %d elements differ in bits"
          % (case, err.max(), rel.max(), int((got.view(np.uint32) != want.view(np.uint32)).sum()), got.size))
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
@needs_reference
def test_bert_base_width_runs_and_repeats():
    """BERT-base widths (hidden 768, 12 heads, FFN 3072) at a short sequence: too large for the INTERPRETER in a test,
    so the plugin is checked against itself (two compilations, same seed: identical bits) and for sane LayerNorm output."""
    from ngraph_b200 import ngraph_api as ng
    ng.load_b200()
    dims = dict(layers=2, hidden=768, heads=12, ffn=3072, seq=128, batch=4, vocab=30522)
    ids, seg = _inputs(dims, 9)
    be = ng.Backend("B200")
    a = be.compile(ng.bert_encoder(seed=2, **dims)).run(ids, seg)[0]
    b = be.compile(ng.bert_encoder(seed=2, **dims)).run(ids, seg)[0]
    assert np.isfinite(a).all() and np.array_equal(a, b)
    assert 0.5 < a.std() < 2.0


@pytest.mark.gpu
@needs_reference
def test_full_width_encoder_commutes_with_a_permutation_of_the_batch():
    """At BERT-base width (hidden 768, 12 heads, FFN 3072, seq 384) the INTERPRETER would need hours, so the check is a
    property the arithmetic guarantees: every op acts per token or per sequence, and the dynamic activation scales are
    maxima over the whole tensor, which do not depend on the order of the sequences.  Reordering the sequences of the
    batch therefore reorders the output rows and changes no bit; the run is also repeatable."""
    from ngraph_b200 import ngraph_api as ng
    ng.load_b200()
    dims = dict(layers=2, hidden=768, heads=12, ffn=3072, seq=384, batch=6, vocab=30522)
    ids, seg = _inputs(dims, 2)
    exe = ng.Backend("B200").compile(ng.bert_encoder(seed=7, **dims))
    out = exe.run(ids, seg)[0]
    assert np.isfinite(out).all() and 0.5 < out.std() < 2.0
    np.testing.assert_array_equal(exe.run(ids, seg)[0].view(np.uint32), out.view(np.uint32))
    perm = np.array([4, 0, 5, 2, 1, 3])
    rows = lambda a, width: a.reshape(dims["batch"], dims["seq"], *width)[perm].reshape(a.shape)
    out_p = exe.run(rows(ids, ()), rows(seg, ()))[0]
    np.testing.assert_array_equal(out_p.view(np.uint32), rows(out, (dims["hidden"],)).view(np.uint32))


@needs_reference
def test_plugin_keeps_layer_norm_and_gelu_whole_and_constants_small():
    """compile()'s graph passes, without a device: LayerNorm and Gelu stay single ops (one kernel each on the device), and
    the bias rows / scalar factors that are broadcast to [tokens, features] are NOT folded into constants of that size."""
    from ngraph_b200 import ngraph_api as ng
    dims = dict(layers=1, hidden=768, heads=12, ffn=3072, seq=384, batch=4, vocab=1000)  # 1536 tokens: above the folding fence
    fn = ng.bert_encoder(seed=3, **dims)
    ops = collections.Counter(ng.function_op_names(ng.after_b200_passes(fn), lowered=False))
    assert ops["LayerNorm"] == 3 and ops["Gelu"] == 1 and ops["Sum"] == 0 and ops["Erf"] == 0
    assert ops["Broadcast"] >= 7 and ops["StopGradient"] == 0   # bias rows and the attention factor stay Broadcast nodes
    plain = collections.Counter(ng.function_op_names(ng.after_b200_passes(fn, decompose_all=True), lowered=False))
    assert plain["LayerNorm"] == 0 and plain["Gelu"] == 0 and plain["Sum"] == 9 and plain["Erf"] == 1
