"""int8 ResNet-50 v1.5 (the headline graph) through the B200 plugin against nGraph's INTERPRETER.

INTERPRETER needs ~40 s per 224x224 image: parity runs on reduced spatial sizes (the network is fully
convolutional up to the pooling head; every layer, channel count, stride, residual join and the head are
exercised), on ONE image at the full 224x224 size (all 1000 logits, bit for bit, alone and inside a batch
of two), and batch independence is checked at 224x224 on the device."""
import os

import numpy as np
import pytest

ng = pytest.importorskip("ngraph_b200.ngraph_api")
from ngraph_b200.harness.resnet50_int8 import QuantizedResNet50, conv_specs, synthetic_images  # noqa: E402
from oracle import interpreter  # noqa: E402

needs_ngraph = pytest.mark.skipif(not interpreter.available(), reason="nGraph host library / INTERPRETER not built here")


@pytest.fixture(scope="module")
def model():
    return QuantizedResNet50(seed=0, calibration_batch=2, calibration_size=64)


def test_layer_table():
    specs = conv_specs()
    assert len(specs) == 53
    assert sum(1 for s in specs if s[7]) == 16       # residual joins
    assert sum(1 for s in specs if s[3] == 3) == 16  # 3x3 convolutions


def test_mac_count(model):
    assert abs(model.macs_per_image() / 1e9 - 4.089) < 0.01  # ResNet-50 v1.5 at 224x224


@needs_ngraph
def test_fused_graph_is_what_a_quantizing_client_builds(model):
    fn, _ = model.build(ng, 2, fused=True, image_hw=(32, 32))
    assert ng.capi().ngc_function_op_count(fn.h) > 200


@needs_ngraph
def test_framework_style_graph_is_fused_back_by_the_plugin(model):
    """Every convolution written as QuantizedConvolutionBias -> Dequantize -> [Add] -> Relu -> Quantize (what a bridge emits
    before backend fusion): the plugin's graph passes must arrive at the op mix of the hand-fused graph, without a device."""
    import collections
    ng.load_b200()
    loose, _ = model.build(ng, 2, framework_style=True, image_hw=(32, 32))
    fused, _ = model.build(ng, 2, fused=True, image_hw=(32, 32))
    before = collections.Counter(ng.function_op_names(loose, lowered=False))
    assert before["Relu"] == 49 and before["Add"] == 16 and before["QuantizedConvolutionBiasAdd"] == 0
    got = collections.Counter(ng.function_op_names(ng.after_b200_passes(loose), lowered=False))
    want = collections.Counter(ng.function_op_names(ng.after_b200_passes(fused), lowered=False))
    for op in ("QuantizedConvolutionBias", "QuantizedConvolutionBiasAdd", "QuantizedConvolutionBiasSignedAdd", "Convert", "MaxPool",
               "Quantize", "Dequantize", "QuantizedDot", "AvgPool", "Relu", "Add", "Divide"):
        assert got[op] == want[op], (op, got[op], want[op])
    assert got["Relu"] == 0 and got["QuantizedConvolutionBiasAdd"] + got["QuantizedConvolutionBiasSignedAdd"] == 16


@pytest.mark.gpu
@needs_ngraph
def test_framework_style_graph_gives_the_fused_graphs_logits(model):
    ng.load_b200()
    b200 = ng.Backend("B200")
    x = synthetic_images(2, 9, 224)[:, :, :64, :64]
    loose, _ = model.build(ng, 2, framework_style=True, image_hw=(64, 64))
    fused, _ = model.build(ng, 2, fused=True, image_hw=(64, 64))
    exe = b200.compile(loose, perf=True)
    got = exe.run(x)[0]
    np.testing.assert_array_equal(got.view(np.uint32), b200.compile(fused).run(x)[0].view(np.uint32))
    assert not any(n.split(":")[0] in ("Relu", "Add") for n, _, _ in exe.performance_data())


@pytest.mark.gpu
@needs_ngraph
def test_resnet50_parity_with_interpreter(model):
    ng.load_b200()
    b200, ref = ng.Backend("B200"), interpreter.backend()
    for hw, batch in (((32, 32), 2), ((64, 96), 1)):
        x = synthetic_images(batch, 7, 224)[:, :, :hw[0], :hw[1]]
        fused, _ = model.build(ng, batch, fused=True, image_hw=hw)
        plain, _ = model.build(ng, batch, fused=False, decomposed=interpreter, image_hw=hw)
        got = b200.compile(fused).run(x)[0]
        exp = ref.compile(plain).run(x)[0]
        assert got.shape == exp.shape == (batch, 1000)
        np.testing.assert_array_equal(got.view(np.uint32), exp.view(np.uint32), err_msg=str(hw))
        assert np.abs(exp).max() > 0


def _full_size_reference(model):
    """INTERPRETER's logits for image 0 of synthetic_images(2, 11): the committed fixture (tests/golden/make_model_golden.py wrote
    it with the INTERPRETER built from the reference sources, a minute of CPU), or a live INTERPRETER run of the decomposed graph
    when B200_LIVE_ORACLE is set."""
    x = synthetic_images(2, 11, 224)
    if os.environ.get("B200_LIVE_ORACLE"):
        plain, _ = model.build(ng, 1, fused=False, decomposed=interpreter)
        return x, interpreter.backend().compile(plain).run(x[:1])[0]
    return x, np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "model_outputs.npz"))["resnet50_224_logits"]


@pytest.mark.gpu
@needs_ngraph
def test_resnet50_full_size_image_matches_interpreter(model):
    """One 224x224 image through every layer at its real geometry (112/56/28/14/7-wide maps, ragged last tiles,
    halo tiles at the image border): all 1000 logits equal INTERPRETER's bit for bit, whether the image is run
    alone or as either member of a batch of two."""
    ng.load_b200()
    b200 = ng.Backend("B200")
    x, exp = _full_size_reference(model)
    assert exp.shape == (1, 1000) and np.abs(exp).max() > 0 and len(np.unique(exp)) > 20
    alone = b200.compile(model.build(ng, 1, fused=True)[0]).run(x[:1])[0]
    np.testing.assert_array_equal(alone.view(np.uint32), exp.view(np.uint32))
    pair = b200.compile(model.build(ng, 2, fused=True)[0])
    np.testing.assert_array_equal(pair.run(x)[0][:1].view(np.uint32), exp.view(np.uint32))
    np.testing.assert_array_equal(pair.run(x[::-1].copy())[0][1:].view(np.uint32), exp.view(np.uint32))


@pytest.mark.gpu
@needs_ngraph
def test_resnet50_full_size_batch_independence(model):
    """224x224, batch 8: every image's logits equal the ones it gets when run alone (batch 1) - the
    size-independent property that stands in for a full-size oracle run."""
    ng.load_b200()
    b200 = ng.Backend("B200")
    x = synthetic_images(8, 9, 224)
    all_at_once = b200.compile(model.build(ng, 8, fused=True)[0]).run(x)[0]
    one = b200.compile(model.build(ng, 1, fused=True)[0])
    for i in (0, 3, 7):
        np.testing.assert_array_equal(one.run(x[i:i + 1])[0][0], all_at_once[i])
