"""Executable::save / Backend::load of the B200 plugin (src/ngraph/runtime/executable.hpp:76-78, backend.hpp:122-125; the
INTERPRETER's version is int_executable.cpp:345-352 + int_backend.cpp:81-110).  The container is a cpio archive holding the
lowered Function in the plugin's own binary form (nGraph's JSON serializer is not part of a JSON-less build) and the device
constant image compile() built (packed filter / weight images, folded scales).

CPU: the binary Function form round-trips every graph family of the quantized path - same op list, and bit-identical
outputs on INTERPRETER before and after.  GPU: a saved and re-loaded executable gives the logits of the original one bit for
bit without repeating the host-side packing, and damaged containers are refused."""
import os

import numpy as np
import pytest

ng = pytest.importorskip("ngraph_b200.ngraph_api")
from oracle import interpreter  # noqa: E402

needs_ngraph = pytest.mark.skipif(not interpreter.available(), reason="nGraph host library / INTERPRETER not built here")


def small_network(fused=True):
    rng = np.random.default_rng(8)
    shape = (2, 64, 12, 12)
    w1 = rng.integers(-127, 128, size=(64, 64, 3, 3)).astype(np.int8)
    w2 = rng.integers(-127, 128, size=(64, 64, 1, 1)).astype(np.int8)
    b1 = rng.integers(-500, 500, size=64).astype(np.int32)
    s1 = (np.exp(rng.uniform(-0.5, 0.5, size=64)) * 2e-4).astype(np.float32)
    s2 = (np.exp(rng.uniform(-0.5, 0.5, size=64)) * 6e-4).astype(np.float32)
    wd = rng.integers(-127, 128, size=(64, 10)).astype(np.int8)
    p = ng.parameter(np.float32, shape)
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
    pooled = ng.quantize(ng.avg_pool(ng.dequantize(c2, np.float32(0.05), np.uint8(0)), c2.shape[2:]), np.float32(0.04), np.uint8(0), np.uint8)
    flat = ng.reshape(pooled, (0, 1, 2, 3), (shape[0], 64))
    logits = ng.quantized_dot(flat, ng.constant(wd), 0.04, 0, 0.01, 0, 0.5, 0, np.int8)
    fn = ng.Function([ng.dequantize(logits, np.float32(0.5), np.int8(0)), c2], [p])
    return fn, [rng.standard_normal(shape).astype(np.float32)]


def bits(a):
    return a.view(np.uint32) if a.dtype == np.float32 else a


@needs_ngraph
def test_function_form_round_trips_the_decomposed_network_on_interpreter():
    fn, xs = small_network(fused=False)
    copy, nbytes = ng.function_roundtrip(fn)
    assert nbytes > 64 * 64 * 9  # the filters travel with the model
    assert ng.function_op_names(copy, lowered=False) == ng.function_op_names(fn, lowered=False)
    ref = interpreter.backend()
    for a, b in zip(ref.compile(fn).run(*xs), ref.compile(copy).run(*xs)):
        np.testing.assert_array_equal(bits(a), bits(b))


@needs_ngraph
def test_function_form_round_trips_the_lowered_graphs():
    """what save() actually writes: the graphs after the plugin's passes (fused ops, LayerNorm / Gelu kept whole)"""
    fn, _ = small_network(fused=True)
    enc = ng.bert_encoder(seed=3, layers=1, hidden=64, heads=4, ffn=128, seq=16, batch=2, vocab=100)
    for f in (fn, enc):
        lowered = ng.after_b200_passes(f)
        copy, _ = ng.function_roundtrip(lowered)
        assert ng.function_op_names(copy, lowered=False) == ng.function_op_names(lowered, lowered=False)
        again, _ = ng.function_roundtrip(copy)  # writing the copy gives the same op list again
        assert ng.function_op_names(again, lowered=False) == ng.function_op_names(lowered, lowered=False)


@needs_ngraph
def test_function_form_round_trips_the_decomposed_encoder_bit_for_bit():
    dims = dict(layers=1, hidden=64, heads=4, ffn=128, seq=16, batch=2, vocab=100)
    fn = ng.bert_encoder(seed=3, decomposed=True, **dims)
    copy, _ = ng.function_roundtrip(fn)
    rng = np.random.default_rng(0)
    ids, seg = rng.integers(0, 100, 32).astype(np.int32), (rng.random(32) < 0.5).astype(np.int32)
    ref = interpreter.backend()
    np.testing.assert_array_equal(bits(ref.compile(fn).run(ids, seg)[0]), bits(ref.compile(copy).run(ids, seg)[0]))


@needs_ngraph
def test_ops_outside_the_plugins_set_are_refused():
    a = ng.parameter(np.float32, (2, 3))
    with pytest.raises(ng.NgraphError, match="cannot save"):
        ng.function_roundtrip(ng.Function([ng.tanh(a)], [a]))


@pytest.mark.gpu
@needs_ngraph
def test_saved_executable_loads_and_gives_the_same_bits(tmp_path):
    ng.load_b200()
    be = ng.Backend("B200")
    fn, xs = small_network(fused=True)
    exe = be.compile(fn)
    want = exe.run(*xs)
    path = tmp_path / "small.b200"
    exe.save(path)
    assert os.path.getsize(path) > 64 * 64 * 9
    loaded = be.load(path, fn)
    got = loaded.run(*xs)
    for g, w in zip(got, want):
        np.testing.assert_array_equal(bits(g), bits(w))
    # and against the reference itself
    exp = interpreter.backend().compile(small_network(fused=False)[0]).run(*xs)
    for g, e in zip(got, exp):
        np.testing.assert_array_equal(bits(g), bits(e))
    # a second backend object (what a fresh process would create) loads the same file
    again = ng.Backend("B200").load(path, fn).run(*xs)
    np.testing.assert_array_equal(bits(again[0]), bits(want[0]))
    # damaged containers are refused: a flipped byte inside the constant image, a truncated file
    raw = bytearray(open(path, "rb").read())
    raw[len(raw) // 2] ^= 0x40
    bad = tmp_path / "bad.b200"
    bad.write_bytes(bytes(raw))
    with pytest.raises(ng.NgraphError):
        be.load(bad, fn)
    bad.write_bytes(bytes(raw[:len(raw) // 3]))
    with pytest.raises(ng.NgraphError):
        be.load(bad, fn)


@pytest.mark.gpu
@needs_ngraph
def test_saved_resnet50_and_encoder_load_bit_identically_and_faster(tmp_path):
    import time
    from ngraph_b200.harness.resnet50_int8 import QuantizedResNet50, synthetic_images
    ng.load_b200()
    be = ng.Backend("B200")
    model = QuantizedResNet50(seed=0, calibration_batch=2, calibration_size=64)
    fn, _ = model.build(ng, 2, fused=True, image_hw=(64, 64))
    x = synthetic_images(2, 5, 224)[:, :, :64, :64]
    t0 = time.time()
    exe = be.compile(fn)
    t_compile = time.time() - t0
    want = exe.run(x)[0]
    path = tmp_path / "resnet50.b200"
    exe.save(path)
    t0 = time.time()
    loaded = be.load(path, fn)
    t_load = time.time() - t0
    np.testing.assert_array_equal(bits(loaded.run(x)[0]), bits(want))
    print("ResNet-50: compile %.2f s, load %.2f s, file %.1f MB" % (t_compile, t_load, os.path.getsize(path) / 1e6))
    dims = dict(layers=2, hidden=256, heads=4, ffn=1024, seq=32, batch=2, vocab=500)
    enc = ng.bert_encoder(seed=5, **dims)
    rng = np.random.default_rng(1)
    ids, seg = rng.integers(0, 500, 64).astype(np.int32), (rng.random(64) < 0.5).astype(np.int32)
    e1 = be.compile(enc)
    e1.save(tmp_path / "enc.b200")
    np.testing.assert_array_equal(bits(be.load(tmp_path / "enc.b200", enc).run(ids, seg)[0]), bits(e1.run(ids, seg)[0]))
