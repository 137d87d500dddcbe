"""ngraph_b200.nbench: the serial and the double-buffered benchmark loops of nGraph's nbench
(src/tools/nbench/benchmark.cpp:85-190, benchmark_pipelined.cpp) over the public runtime API.  On CPU they drive nGraph's
INTERPRETER backend; on the GPU the B200 plugin, where both loops must return what a plain call returns."""
import numpy as np
import pytest

ng = pytest.importorskip("ngraph_b200.ngraph_api")
from oracle import interpreter  # noqa: E402
from ngraph_b200 import nbench  # noqa: E402

pytestmark = pytest.mark.skipif(not interpreter.available(), reason="nGraph host library / INTERPRETER not built here")


def quantize_roundtrip(shape=(4, 16, 9, 9)):
    x = ng.parameter(np.float32, shape)
    q = ng.quantize(x, 0.05, 128, np.uint8, round_mode=4)
    return ng.Function([ng.dequantize(q, 0.05, 128), q], [x])


def expected(x):
    q = np.clip(np.rint(x / np.float32(0.05)) + 128, 0, 255).astype(np.uint8)
    return ((q.astype(np.int32) - 128).astype(np.float32) * np.float32(0.05)).astype(np.float32), q


def test_serial_loop_on_interpreter():
    r = nbench.run_benchmark(quantize_roundtrip(), "INTERPRETER", iterations=3, warmup=1, timing_detail=True)
    assert r["ms_per_iteration"] > 0 and r["compile_ms"] >= 0
    want = expected(r["inputs"][0])
    np.testing.assert_array_equal(r["results"][1], want[1])
    np.testing.assert_array_equal(r["results"][0], want[0])
    assert any(name.startswith("Quantize") for name, _, _ in r["performance_data"])
    lines = []
    nbench.print_timing_detail(r["performance_data"], lines.append)
    assert lines[0].startswith("----") and any("Quantize" in l for l in lines)


def test_no_copy_data_still_produces_results():
    r = nbench.run_benchmark(quantize_roundtrip(), "INTERPRETER", iterations=2, warmup=0, copy_data=False)
    np.testing.assert_array_equal(r["results"][1], expected(r["inputs"][0])[1])


def test_pipelined_loop_on_interpreter():
    r = nbench.run_benchmark_pipelined(quantize_roundtrip(), "INTERPRETER", iterations=5, warmup=2)
    assert r["ms_per_iteration"] > 0
    for stage in range(2):  # each pipeline stage has its own host data and its own tensors
        np.testing.assert_array_equal(r["results"][stage][1], expected(r["inputs"][stage][0])[1])
    assert not np.array_equal(r["inputs"][0][0], r["inputs"][1][0])


def test_pipelined_loop_reports_a_failing_call():
    with pytest.raises(ng.NgraphError):
        nbench.run_benchmark_pipelined(quantize_roundtrip(), "NO_SUCH_BACKEND", iterations=2)


@pytest.mark.gpu
@pytest.mark.parametrize("model", ["qdot", "qconv"])
def test_both_loops_on_the_plugin(model):
    ng.load_b200()
    function, bounds = nbench.build_model(model, 8 if model == "qconv" else 64)
    serial = nbench.run_benchmark(function, "B200", iterations=4, warmup=1, timing_detail=True, int_high=bounds)
    piped = nbench.run_benchmark_pipelined(function, "B200", iterations=6, warmup=2, int_high=bounds)
    plain = ng.Backend("B200").compile(function).run(*serial["inputs"])[0]
    np.testing.assert_array_equal(serial["results"][0], plain)
    for stage in range(2):
        want = ng.Backend("B200").compile(function).run(*piped["inputs"][stage])[0]
        np.testing.assert_array_equal(piped["results"][stage][0], want)
    assert serial["performance_data"]


@pytest.mark.gpu
def test_command_line_prints_what_nbench_prints():
    lines = []
    nbench.main(["--model", "qdot", "-b", "B200", "-i", "3", "-w", "1", "--double_buffer", "--timing_detail"], out=lines.append)
    assert lines[0].startswith("compile time: ") and lines[1].endswith("ms per iteration")
    assert any("QuantizedDotBias" in l for l in lines)
