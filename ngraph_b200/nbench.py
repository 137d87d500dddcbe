"""nbench for this repository: the two benchmark loops of nGraph's own tool, driving any registered backend through the
public runtime API (Backend::create -> compile -> create tensors -> write / call / read).

    python -m ngraph_b200.nbench --model resnet50 -b B200 -i 50 -w 5 [--double_buffer] [--no_copy_data] [--timing_detail]

`run_benchmark` follows src/tools/nbench/benchmark.cpp:85-190: host data is made once, then every iteration writes each
input tensor (unless --no_copy_data), calls the executable and reads each result; the clock starts after the warm-up
iterations.  `run_benchmark_pipelined` follows src/tools/nbench/benchmark_pipelined.cpp: two host threads, each with its
own set of tensors from Executable::create_input_tensor(i, 2) / create_output_tensor(i, 2); a thread writes its inputs
while the other thread's call runs, then takes its turn.  nGraph's nbench reads a serialized Function from a file; the
models here are built in-process instead (the JSON serializer is not part of this build), which is the only difference
in what is measured."""
import argparse
import threading
import time

import numpy as np

from . import ngraph_api as ng


def random_init(spec, rng, high=None):
    """host data for one Parameter, like nbench's random_init (benchmark_utils.cpp): uniform values of the element type"""
    dt = np.dtype(spec.dtype)
    if dt == np.float32:
        return rng.uniform(-1.0, 1.0, size=spec.shape).astype(np.float32)
    info = np.iinfo(dt)
    lo, hi = (0, high) if high is not None else (max(info.min, -128), min(info.max, 255) + 1)
    return rng.integers(lo, hi, size=spec.shape).astype(dt)


def _host_data(function, rng, int_high):
    """int_high: None, or one exclusive upper bound per Parameter (None where the full range is fine)"""
    bounds = list(int_high) if int_high is not None else [None] * len(function.params)
    return [np.ascontiguousarray(random_init(p, rng, b)) for p, b in zip(function.params, bounds)]


def run_benchmark(function, backend_name, iterations, warmup=1, copy_data=True, timing_detail=False, seed=0, int_high=None):
    """the serial loop: returns a dict with compile_ms, ms_per_iteration, the last results and the performance counters"""
    t = time.perf_counter()
    backend = ng.Backend(backend_name)
    exe = backend.compile(function, perf=timing_detail)
    compile_ms = (time.perf_counter() - t) * 1e3
    rng = np.random.default_rng(seed)
    data = _host_data(function, rng, int_high)
    args = [ng.Tensor(backend, p.dtype, p.shape) for p in function.params]
    for tensor, host in zip(args, data):
        tensor.write(host)
    results = [ng.Tensor(backend, r.dtype, r.shape) for r in function.results]
    out = [np.empty(r.shape, np.dtype(r.dtype)) for r in function.results]
    start = None
    for i in range(iterations + warmup):
        if i == warmup:
            start = time.perf_counter()
        if copy_data:
            for tensor, host in zip(args, data):
                tensor.write_ptr(host.ctypes.data, host.nbytes)
        exe.call(results, args, validate=False)
        if copy_data:
            for tensor, host in zip(results, out):
                tensor.read_ptr(host.ctypes.data, host.nbytes)
    if not copy_data:  # the device may still be running: reading the results once ends the timed region
        for tensor, host in zip(results, out):
            tensor.read_ptr(host.ctypes.data, host.nbytes)
    total_ms = (time.perf_counter() - start) * 1e3
    return {"compile_ms": compile_ms, "ms_per_iteration": total_ms / iterations, "results": out, "inputs": data,
            "performance_data": exe.performance_data() if timing_detail else []}


def run_benchmark_pipelined(function, backend_name, iterations, warmup=1, timing_detail=False, seed=0, int_high=None):
    """the double-buffered loop (nbench --double_buffer): two threads, pipeline depth 2"""
    depth = 2
    t = time.perf_counter()
    backend = ng.Backend(backend_name)
    exe = backend.compile(function, perf=timing_detail)
    compile_ms = (time.perf_counter() - t) * 1e3
    rng = np.random.default_rng(seed)
    data = [_host_data(function, rng, int_high) for _ in range(depth)]
    out = [[np.empty(r.shape, np.dtype(r.dtype)) for r in function.results] for _ in range(depth)]
    ins = [exe.create_input_tensors(i, depth) for i in range(len(function.params))]
    outs = [exe.create_output_tensors(i, depth) for i in range(len(function.results))]
    state = {"iteration": 0, "start": None, "stop": None, "error": None}
    turn = threading.Condition()
    total = iterations + warmup

    def stage(s):
        args, results = [t[s] for t in ins], [t[s] for t in outs]
        written = False
        try:
            while True:
                if not written:  # while the other stage's call may still be running
                    for tensor, host in zip(args, data[s]):
                        tensor.write_ptr(host.ctypes.data, host.nbytes)
                    written = True
                with turn:
                    while state["iteration"] < total and (state["iteration"] & 1) != s and state["error"] is None:
                        turn.wait()
                    if state["iteration"] >= total or state["error"] is not None:
                        return
                    if state["iteration"] == warmup:
                        state["start"] = time.perf_counter()
                    exe.call(results, args, validate=False)
                    state["iteration"] += 1
                    last = state["iteration"] == total
                    written = False
                    turn.notify_all()
                for tensor, host in zip(results, out[s]):
                    tensor.read_ptr(host.ctypes.data, host.nbytes)
                if last:
                    state["stop"] = time.perf_counter()
        except Exception as e:  # surfaces in the caller; the other stage must not wait for ever
            with turn:
                state["error"] = e
                turn.notify_all()

    threads = [threading.Thread(target=stage, args=(s,)) for s in range(depth)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    if state["error"] is not None:
        raise state["error"]
    stop = state["stop"] if state["stop"] is not None else time.perf_counter()
    return {"compile_ms": compile_ms, "ms_per_iteration": (stop - state["start"]) * 1e3 / iterations, "results": out, "inputs": data,
            "performance_data": exe.performance_data() if timing_detail else []}


# ------------------------------------------------------------------------------------------------ models
def build_model(name, batch):
    """(Function, per-Parameter exclusive upper bounds for integer inputs that index something, or None)"""
    if name == "resnet50":
        from .harness.resnet50_int8 import QuantizedResNet50
        return QuantizedResNet50(seed=0, calibration_batch=8).build(ng, batch or 128, fused=True)[0], None
    if name == "bert":
        return ng.bert_encoder(layers=12, hidden=768, heads=12, ffn=3072, seq=384, batch=batch or 64, vocab=30522, seed=1), [30522, 2]
    rng = np.random.default_rng(0)
    if name == "qdot":  # the single-layer workload: QuantizedDotBias + Relu, u8 [M,1024] x i8 [1024,1024]
        m = batch or 256
        x = ng.parameter(np.uint8, (m, 1024))
        w = rng.integers(-127, 128, size=(1024, 1024)).astype(np.int8)
        bias = rng.integers(-1000, 1001, size=1024).astype(np.int32)
        return ng.Function([ng.quantized_dot_bias(x, w, bias, np.float32([0.004]), True, True)], [x]), None
    if name == "qconv":  # the single-convolution workload: QuantizedConvolutionBias + Relu, 64 -> 64 channels, 3x3, 56x56
        n = batch or 32
        x = ng.parameter(np.uint8, (n, 64, 56, 56))
        w = rng.integers(-127, 128, size=(64, 64, 3, 3)).astype(np.int8)
        bias = rng.integers(-1000, 1001, size=64).astype(np.int32)
        scale = (0.02 * np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), 64)) / 0.05).astype(np.float32)
        return ng.Function([ng.quantized_conv_bias(x, w, bias, scale, True, pad_below=(1, 1))], [x]), None
    raise ValueError("unknown model " + name)


def print_timing_detail(rows, out):
    """per-op totals like nbench's --timing_detail table"""
    by_op = {}
    for name, us, calls in rows:
        op = name.split(":")[0]
        t, c = by_op.get(op, (0, 0))
        by_op[op] = (t + us, c + 1)
    total = sum(t for t, _ in by_op.values()) or 1
    out("---- Aggregate times per op type ----")
    for op, (t, c) in sorted(by_op.items(), key=lambda kv: -kv[1][0]):
        out("%-40s %6d nodes %12d us %5.1f%%" % (op, c, t, 100.0 * t / total))


def main(argv=None, out=print):
    ap = argparse.ArgumentParser(prog="nbench", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, choices=["resnet50", "bert", "qdot", "qconv"])
    ap.add_argument("-b", "--backend", default="B200")
    ap.add_argument("-i", "--iterations", type=int, default=10)
    ap.add_argument("-w", "--warmup_iterations", type=int, default=1)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--timing_detail", action="store_true")
    ap.add_argument("--no_copy_data", action="store_true")
    ap.add_argument("--double_buffer", action="store_true")
    a = ap.parse_args(argv)
    if a.backend.split(":")[0] == "B200":
        ng.load_b200()
    function, int_high = build_model(a.model, a.batch)
    if a.double_buffer:
        r = run_benchmark_pipelined(function, a.backend, a.iterations, a.warmup_iterations, a.timing_detail, int_high=int_high)
    else:
        r = run_benchmark(function, a.backend, a.iterations, a.warmup_iterations, not a.no_copy_data, a.timing_detail, int_high=int_high)
    out("compile time: %.0fms" % r["compile_ms"])
    out("%.4fms per iteration" % r["ms_per_iteration"])
    if a.timing_detail:
        print_timing_detail(r["performance_data"], out)
    return r


if __name__ == "__main__":
    main()
