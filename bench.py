#!/usr/bin/env python3
"""Benchmark of the B200 quantized-inference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl b200|reference]

Prints ONE JSON line (rank 0).  Workloads (synthetic, seeded; shapes from the baseline configs):

  resnet50  (default) int8 ResNet-50 v1.5, batch 128 per GPU, as an nGraph Function compiled and run
            through the B200 backend plugin (Backend::create("B200:<dev>") -> compile -> call).
            value = images/s with the input tensor resident in HBM; e2e = the same through
            Tensor::write (pinned host -> device) + call + Tensor::read (logits -> host) every step.
  qconv     one QuantizedConvolutionBias+Relu layer, u8 [B,64,56,56] * i8 [64,64,3,3] (C ABI directly)
  qdot      one QuantizedDotBias+Relu layer, u8 [M,1024] x i8 [1024,1024]              (C ABI directly)
  quantize  Quantize f32 -> u8, per tensor, [B,64,256,256]                             (C ABI directly)

--impl reference times nGraph's own CPU implementation of the same path on the host cores: the
INTERPRETER backend (reference kernels) on the decomposed graph, one process per core, each on a
bounded sample (an image strip) sized from --steps so the run ends within minutes.
"""
import argparse
import json
import os
import pickle
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measure_int8_peak(torch, n=8192, reps=10):
    """Dense int8 tensor-core peak of this GPU, measured now: (1) cuBLASLt's int8 -> int32 GEMM (torch._int_mm; off the product
    path, used only as the roofline's denominator) and (2) this library's own b200_qgemm, both n^3, best of `reps` single launches
    timed with CUDA events (a burst figure, like the bf16 burst figure of MEASURED_PEAKS.json)."""
    from ngraph_b200 import ops
    out = {"n": n, "cublaslt_int8_tops": None, "own_qgemm_tops": None}

    def best(fn):
        fn()
        torch.cuda.synchronize()
        b = 1e30
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            b = min(b, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (b * 1e-3) / 1e12

    a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device="cuda")
    b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device="cuda")
    try:
        out["cublaslt_int8_tops"] = best(lambda: torch._int_mm(a, b))
    except Exception as e:  # the probe is optional: without it the own kernel's figure (or 2 x bf16) stands in
        out["cublaslt_error"] = str(e)[:120]
    au = a.view(torch.uint8)
    s = torch.full((1,), 1e-5, device="cuda")
    o = torch.empty((n, n), dtype=torch.uint8, device="cuda")
    out["own_qgemm_tops"] = best(lambda: ops.qgemm(au, b, s, torch.uint8, relu=True, out=o))
    del a, b, au, o
    torch.cuda.empty_cache()
    return out


def int8_peak(peaks, probe):
    """(peak TOP/s, text saying where it comes from): the larger of the two measured int8 figures; 2 x the measured bf16 burst
    figure only when no int8 GEMM could be timed"""
    cands = [(probe.get("cublaslt_int8_tops"), "measured in this run: cuBLASLt int8 GEMM %d^3, best of 10" % probe["n"]),
             (probe.get("own_qgemm_tops"), "measured in this run: b200_qgemm %d^3, best of 10" % probe["n"])]
    cands = [c for c in cands if c[0]]
    if cands:
        return max(cands)
    return 2.0 * peaks["bf16_tflops"], peaks["source"] + ": 2 x bf16 burst (no int8 GEMM could be timed)"


class ClockSampler:
    """Samples SM clocks / throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [v.strip() for v in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 - 0.05 <= t <= t1 + 0.15 and len(r) >= 7] or [r for _, r in self.rows if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "reasons": reasons, "samples": len(rows)}


# ------------------------------------------------------------------------------------------ CPU reference (INTERPRETER)
def _patch_for(budget_s):
    """largest image patch (h, w) one INTERPRETER pass gets through within budget_s (~38 s per full 224x224 image,
    time proportional to the area; 32 is the network's total stride, so no side goes below it)"""
    for h, w in ((224, 224), (128, 224), (96, 224), (64, 224), (32, 224), (32, 112), (32, 64), (32, 32)):
        if 38.0 * h * w / (224 * 224) <= budget_s:
            return h, w
    return 32, 32


def cpu_worker(pickle_path, patch, reps):
    """child process: INTERPRETER on the decomposed ResNet-50 graph over one image patch, `reps` passes"""
    from ngraph_b200 import ngraph_api as ng
    from ngraph_b200.harness.resnet50_int8 import synthetic_images
    from oracle import interpreter
    h, w = (int(v) for v in patch.split("x"))
    model = pickle.load(open(pickle_path, "rb"))
    fn, _ = model.build(ng, 1, fused=False, decomposed=interpreter, image_hw=(h, w))
    be = interpreter.backend()
    exe = be.compile(fn)
    x = synthetic_images(1, 77, 224)[:, :, :h, :w]
    tin, tout = ng.Tensor(be, np.float32, x.shape), ng.Tensor(be, np.float32, (1, model.classes))
    tin.write(x)
    times = []
    for _ in range(reps):
        t0 = time.time()
        exe.call([tout], [tin])
        times.append(time.time() - t0)
    out = tout.read()
    print(json.dumps({"seconds": times, "logit_bits": out.view(np.uint32).ravel().tolist()}))


def cpu_reference_rate(model, budget_s, procs=None, reps=1):
    """images/s of nGraph's reference kernels (INTERPRETER) over `procs` processes, each on one image patch, for each
    of `reps` passes: (rates per pass, procs, sample text, patch, first worker's result)"""
    procs = procs or max(1, os.cpu_count() or 1)
    h, w = _patch_for(budget_s)
    with tempfile.NamedTemporaryFile(suffix=".pkl", delete=False) as f:
        pickle.dump(model, f)
        path = f.name
    try:
        cmd = [sys.executable, os.path.abspath(__file__), "--cpu-worker", path, "%dx%d" % (h, w), str(reps)]
        ps = [subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, cwd=ROOT) for _ in range(procs)]
        outs = [p.communicate() for p in ps]
    finally:
        os.unlink(path)
    res = []
    for (o, e), p in zip(outs, ps):
        if p.returncode != 0:
            raise RuntimeError("INTERPRETER worker failed: " + e[-500:])
        res.append(json.loads(o.strip().splitlines()[-1]))
    frac = model.macs_per_image((h, w)) / model.macs_per_image()
    rates = [procs * frac / max(r["seconds"][i] for r in res) for i in range(reps)]
    sample = "INTERPRETER (nGraph reference kernels) on the decomposed graph, %d processes x one %dx%d patch (%.4f image by MACs), " \
             "%.1f s per pass" % (procs, h, w, frac, max(r["seconds"][-1] for r in res))
    return rates, procs, sample, (h, w), res[0]


# ------------------------------------------------------------------------------------------ workloads
class ResNet50:
    name, metric, unit = "resnet50", "int8 ResNet-50 v1.5 inference throughput", "img/s"
    dtype, bound = "u8*i8->i32 (f32 in, f32 logits out)", "tensor"

    def __init__(self, batch=128, pipeline=2):
        self.batch = batch
        self.pipeline = pipeline
        self.model = None

    def describe(self, world=1):
        return {"workload": "int8 ResNet-50 v1.5, nGraph Function through the B200 backend plugin: 53 QuantizedConvolutionBias"
                            "(+Relu/+Add+Relu), u8 MaxPool, Dequantize/AvgPool/Quantize head, QuantizedDot 2048->1000, Dequantize",
                "batch_per_gpu": self.batch, "global_batch": self.batch * world, "input": "f32 NCHW [B,3,224,224] normalised",
                "weights": "random He-normal, per-channel i8; activation scales from a seeded 8-image calibration",
                "parallelism": "batch-sharded replicas, outputs gathered with NCCL all_gather",
                "pipeline_depth": self.pipeline,
                "pipeline": ("%d executables of the same Function on %d CUDA streams, steps rotate over them: %d batches "
                             "in flight per GPU" % (self.pipeline, self.pipeline, self.pipeline)) if self.pipeline > 1
                            else "one executable, one stream",
                "l2": "per-step activation working set (~2 GB) >> 126 MB L2"}

    def build_model(self):
        from ngraph_b200.harness.resnet50_int8 import QuantizedResNet50
        if self.model is None:
            self.model = QuantizedResNet50(seed=0, calibration_batch=8)
        return self.model

    def setup(self, torch, rank, local_rank, world):
        from ngraph_b200 import ngraph_api as ng
        from ngraph_b200.harness.resnet50_int8 import synthetic_images
        from ngraph_b200 import sharding
        self.torch, self.ng, self.world, self.sharding = torch, ng, world, sharding
        model = self.build_model()
        ng.load_b200()
        stream = torch.cuda.current_stream().cuda_stream
        self.backend = ng.Backend("B200:%d,stream=%d" % (local_rank, stream))
        self.fn, _ = model.build(ng, self.batch, fused=True)
        self.exe = self.backend.compile(self.fn)
        x = synthetic_images(min(self.batch, 16), 100 + rank)
        x = np.tile(x, ((self.batch + x.shape[0] - 1) // x.shape[0], 1, 1, 1))[:self.batch]
        self.x_dev = torch.from_numpy(x).cuda()
        # two result buffers: with several GPUs the gather of step i runs on a stream of its own beside step i + 1
        self.nbuf = max(2, self.pipeline)
        self.logits2 = [torch.empty((self.batch, model.classes), dtype=torch.float32, device="cuda") for _ in range(self.nbuf)]
        self.t_out2 = [self.backend.create_tensor(np.float32, tuple(b.shape), b.data_ptr()) for b in self.logits2]
        self.logits, self.t_out = self.logits2[0], self.t_out2[0]
        self.t_in = self.backend.create_tensor(np.float32, x.shape, self.x_dev.data_ptr())
        self.gather_stream = torch.cuda.Stream() if world > 1 else None
        self.step_i = 0
        self.logits_read = [None] * self.nbuf
        # Pipeline depth 2, on the client side and through the public API only: a second Backend on a second CUDA stream
        # compiles the same Function, and the timed steps alternate between the two executables, so that two batches are in
        # flight and the tail of one batch's kernels overlaps the head of the other's (what nGraph's own nbench does with
        # --double_buffer for the copies).  Every step is still one [B,3,224,224] batch through the unchanged graph.
        self.lane_streams = [torch.cuda.current_stream()] + [torch.cuda.Stream() for _ in range(self.pipeline - 1)]
        self.lane_exe, self.lane_in, self.lane_out, self.lane_backends = [self.exe], [self.t_in], [self.t_out2[0]], [self.backend]
        from concurrent.futures import ThreadPoolExecutor
        self.lane_threads = [ThreadPoolExecutor(max_workers=1) for _ in range(self.pipeline)]
        self.lane_pending = [[] for _ in range(self.pipeline)]
        self.gather_due = None
        for lane in range(1, self.pipeline):
            b2 = ng.Backend("B200:%d,stream=%d" % (local_rank, self.lane_streams[lane].cuda_stream))
            self.lane_backends.append(b2)
            self.lane_exe.append(b2.compile(self.fn))
            self.lane_in.append(b2.create_tensor(np.float32, x.shape, self.x_dev.data_ptr()))  # the same resident input, read only
            self.lane_out.append(b2.create_tensor(np.float32, tuple(self.logits2[lane].shape), self.logits2[lane].data_ptr()))
        # end-to-end loop: two input tensors, so that Tensor::write of the next batch (copy stream) overlaps the
        # kernels of the current one; the pipelined-tensor pattern of nGraph's own nbench
        self.x_pipe = [torch.empty_like(self.x_dev) for _ in range(2)]
        self.t_pipe = [self.backend.create_tensor(np.float32, x.shape, b.data_ptr()) for b in self.x_pipe]
        self.e2e_i = 0
        self.e2e_primed = False
        self.pin_in = torch.from_numpy(x).pin_memory()
        self.pin_out = torch.empty((self.batch, model.classes), dtype=torch.float32).pin_memory()
        self.gathered = torch.empty((world * self.batch, model.classes), dtype=torch.float32, device="cuda") if world > 1 else None

    def units_per_step(self):
        return float(self.batch)

    def _gather_beside_next_step(self, logits, producer_stream=None):
        """the one collective of the path (NCCL all_gather of this step's logits), on its own stream, ordered after the
        kernels that produced them; the next step's kernels do not wait for it"""
        torch = self.torch
        done = torch.cuda.Event()
        done.record(producer_stream if producer_stream is not None else torch.cuda.current_stream())
        with torch.cuda.stream(self.gather_stream):
            self.gather_stream.wait_event(done)
            self.sharding.gather_rows(logits, [self.batch] * self.world, out=self.gathered)
            read = torch.cuda.Event()
            read.record()
        return read  # the buffer may be written again after this event

    def step(self):
        k = self.step_i % self.nbuf
        self.step_i += 1
        lane = k if self.pipeline > 1 else 0
        st = self.lane_streams[lane]
        if self.gathered is not None and self.logits_read[k] is not None:
            st.wait_event(self.logits_read[k])  # the gather of two steps ago has read this buffer
        out = self.lane_out[lane] if self.pipeline > 1 else self.t_out2[k]
        if self.pipeline > 1:
            # one host thread per lane issues that lane's launches (Executable::call only enqueues; ctypes releases the
            # interpreter lock for its duration), so neither stream waits for the other's 58 launches to be issued
            issued = self.lane_threads[lane].submit(self.lane_exe[lane].call, [out], [self.lane_in[lane]], False)
            self.lane_pending[lane].append(issued)
            if self.gathered is not None:
                # the collectives stay on this thread, in step order on every rank: the gather of the PREVIOUS step goes out
                # now (its launches have been issued by the time this step's have been handed over)
                self._flush_gather()
                self.gather_due = (issued, k, st)
            return
        self.lane_exe[lane].call([out], [self.lane_in[lane]], validate=False)
        if self.gathered is not None:
            self.logits_read[k] = self._gather_beside_next_step(self.logits2[k], st)

    def _flush_gather(self):
        if self.gather_due is not None:
            issued, k, st = self.gather_due
            issued.result()
            self.logits_read[k] = self._gather_beside_next_step(self.logits2[k], st)
            self.gather_due = None

    def begin(self):
        """the second lane starts no earlier than the timed region's opening event on the first"""
        for st in self.lane_streams[1:]:
            st.wait_stream(self.lane_streams[0])

    def finish(self):
        """joins the second lane and the gather stream: the timed region ends when the last steps' logits are there"""
        for pending in self.lane_pending:
            for f in pending:
                f.result()
            del pending[:]
        if self.gathered is not None:
            self._flush_gather()
        for st in self.lane_streams[1:]:
            self.torch.cuda.current_stream().wait_stream(st)
        if self.gather_stream is not None:
            self.torch.cuda.current_stream().wait_stream(self.gather_stream)

    def step_e2e(self):
        """One batch end to end through the plugin's public API: Tensor::write of the batch (pinned host memory),
        Executable::call, Tensor::read of the logits.  Two host threads and two input tensors, the scheme of nGraph's
        nbench --double_buffer (src/tools/nbench/benchmark_pipelined.cpp): while this thread calls the executable on
        batch i and reads its logits, the other writes batch i+1 into the second tensor (Tensor::write returns when the
        copy is done, so a single thread could not start it before it has finished enqueueing the kernels).  Every batch
        is written exactly once and read exactly once."""
        nbytes = self.pin_in.numel() * 4
        cur = self.e2e_i & 1
        if not self.e2e_primed:
            from concurrent.futures import ThreadPoolExecutor
            self.writer = ThreadPoolExecutor(max_workers=1)
            self.t_pipe[cur].write_ptr(self.pin_in.data_ptr(), nbytes)
            self.e2e_primed = True
        # the other tensor is free: the call that read it was waited for by the previous step's read
        pending = self.writer.submit(self.t_pipe[cur ^ 1].write_ptr, self.pin_in.data_ptr(), nbytes)
        if self.gathered is not None and self.logits_read[0] is not None:
            self.torch.cuda.current_stream().wait_event(self.logits_read[0])
        self.exe.call([self.t_out], [self.t_pipe[cur]], validate=False)
        if self.gathered is not None:
            self.logits_read[0] = self._gather_beside_next_step(self.logits)
        self.t_out.read_ptr(self.pin_out.data_ptr(), self.pin_out.numel() * 4)
        pending.result()
        self.e2e_i += 1

    def io_bytes(self):
        return self.pin_in.numel() * 4, self.pin_out.numel() * 4

    def roofline(self, peaks, per_step_ms, probe):
        """dominant kernel = the tcgen05 contraction kernel (all convolutions + the dot).  achieved = the step's int8 ops / the
        part of the TIMED step that kernel takes: ms_per_step (CUDA events over the timed region, above) x the kernel's share of
        the step.  The share comes from per-node CUDA events of a separate, instrumented pass over the same graph
        (compile(f, true) -> get_performance_data()); that pass serialises the nodes, so only the ratio is taken from it."""
        ng = self.ng
        exe = self.backend.compile(self.model.build(ng, self.batch, fused=True)[0], perf=True)
        passes = 5
        for _ in range(passes):
            exe.call([self.t_out], [self.t_in], validate=False)
        self.torch.cuda.synchronize()
        rows = exe.performance_data()
        contr_us = sum(us for n, us, c in rows if n.startswith("QuantizedConvolution") or n.startswith("QuantizedDot")) / passes
        total_us = sum(us for n, us, c in rows) / passes
        share = contr_us / total_us
        kernel_us = per_step_ms * 1e3 * share
        ops = 2.0 * self.model.macs_per_image() * self.batch
        achieved = ops / (kernel_us * 1e-6) / 1e12
        peak, peak_source = int8_peak(peaks, probe)
        top = sorted(((us / passes, n) for n, us, c in rows), reverse=True)[:6]
        if os.environ.get("B200_BENCH_NODE_TABLE"):  # per-node table for the profile notes
            with open(os.environ["B200_BENCH_NODE_TABLE"], "w") as f:
                for n, us, c in rows:
                    f.write("%10.1f us  %s\n" % (us / passes, n))
        # the same launches against their own rooflines: a layer can go no faster than its ops at the tensor peak or its
        # bytes at the HBM peak, whichever is longer; most 1x1 layers are on the HBM side
        work = self.model.layer_work()
        assert abs(sum(m for _, m, _, _ in work) - self.model.macs_per_image()) < 1
        floor_us = sum(max(2.0 * m * self.batch / (peak * 1e12), (by * self.batch + wt) / (peaks["hbm_gbs"] * 1e9)) * 1e6
                       for _, m, by, wt in work)
        # dram__bytes_read.sum + dram__bytes_write.sum of the 54 contraction launches of one batch-128 step (one ncu capture,
        # summarised in profiles/resnet50_b128_launch_list.txt), averaged per launch and scaled by the batch
        traffic = (1976.9e6 + 350.8e6) / 54 * (self.batch / 128.0)
        return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s", "frac": achieved / peak,
                "ops_per_step": ops, "kernel_us_per_step": kernel_us, "kernel_share_of_step": share,
                "kernel_share_source": "per-node CUDA events, instrumented pass: %.1f of %.1f us" % (contr_us, total_us),
                "traffic": traffic, "traffic_source": "profiles/resnet50_b128_launch_list.txt (ncu dram bytes of the 54 contraction "
                                                      "launches of a batch-128 step / 54, scaled by batch/128)",
                "per_layer_floor_us": floor_us, "frac_of_per_layer_floor": floor_us / kernel_us,
                "kernel": "qcontract_kernel (53 convolutions + dot)",
                "peak_source": peak_source, "peak_i8_measured": probe, "peak_2x_bf16_burst": 2.0 * peaks["bf16_tflops"],
                "slowest_nodes_us_instrumented": [[round(u, 1), n] for u, n in top]}

    def extra_cpu_baselines(self):
        """The north star asks for nGraph's DNNL CPU backend beside the number; that backend cannot be built offline, so the
        oneDNN int8 primitives inside PyTorch run the same network on the same host cores as a labelled proxy."""
        try:
            import torch
            from ngraph_b200.harness.resnet50_int8 import OneDnnProxy
            threads = os.cpu_count() or 1
            torch.set_num_threads(threads)
            rate = OneDnnProxy(self.model).images_per_second(batch=32, seconds=8.0)
            return {"cpu_baseline_onednn_proxy": {
                "value": rate, "unit": "img/s", "cores": threads, "kind": "proxy",
                "sample": "the same int8 ResNet-50 through torch.ops.quantized (oneDNN %s engine), batch 32, 8 s; stands in for nGraph's "
                          "CPU backend (DNNL), which needs downloaded dependencies to build" % torch.backends.quantized.engine}}
        except Exception as e:  # a baseline that cannot run is reported, never fatal
            return {"cpu_baseline_onednn_proxy": {"unavailable": str(e)[:200]}}

    def check_and_cpu_baseline(self, skip_cpu):
        """INTERPRETER on an image strip: timing for cpu_baseline and the parity check of the B200 output"""
        if skip_cpu:
            return None, None
        from ngraph_b200.harness.resnet50_int8 import synthetic_images
        ng, model = self.ng, self.model
        rates, procs, sample, (ph, pw), first = cpu_reference_rate(model, budget_s=20.0)
        rate = rates[0]
        x = synthetic_images(1, 77, 224)[:, :, :ph, :pw]  # the patch the workers ran, through the plugin
        fn, _ = model.build(ng, 1, fused=True, image_hw=(ph, pw))
        got = self.backend.compile(fn).run(x)[0]
        # every logit of the patch, bit for bit (the float tail of the graph is one Dequantize: a single IEEE multiply)
        ok = bool(np.array_equal(np.asarray(first["logit_bits"], np.uint32), got.view(np.uint32).ravel()))
        return {"value": rate, "unit": "img/s", "cores": procs, "kind": "reference", "sample": sample}, ok


class BertEncoder:
    """The int8 BERT-base-shaped encoder (12 layers, hidden 768, 12 heads, FFN 3072, seq 384, batch 64) as an nGraph Function through the plugin.  The int8 dots are the
    QuantizedDotBias layers; everything between them (dynamic activation scales, attention products, softmax, LayerNorm,
    GELU) is f32 glue that keeps the reference kernels' arithmetic."""
    name, metric, unit = "bert", "int8 BERT-base-shaped encoder inference throughput", "tokens/s"
    dtype, bound = "i8*i8->i32 dots, f32 glue", "tensor"
    dims = dict(layers=12, hidden=768, heads=12, ffn=3072, seq=384, vocab=30522)
    cpu_kind = "reference"

    def __init__(self, batch=64):
        self.batch = batch

    def describe(self, world=1):
        d = self.dims
        return {"workload": "int8 BERT-base-shaped encoder, nGraph Function through the B200 backend plugin: %d layers, hidden %d, "
                            "%d heads, FFN %d, seq %d; QKV/out/FFN = QuantizedDotBias with dynamic per-tensor i8 activation scales"
                            % (d["layers"], d["hidden"], d["heads"], d["ffn"], d["seq"]),
                "batch_per_gpu": self.batch, "global_batch": self.batch * world, "input": "i32 token ids and segment ids [B*S]",
                "weights": "random N(0, 0.02), per-output-channel i8", "parallelism": "batch-sharded replicas, no collective",
                "l2": "per-layer activations (75 MB x several) > 126 MB L2"}

    def host_inputs(self, seed):
        rng = np.random.default_rng(seed)
        m = self.batch * self.dims["seq"]
        self.ids = rng.integers(0, self.dims["vocab"], m).astype(np.int32)
        self.seg = (rng.random(m) < 0.5).astype(np.int32)

    def setup(self, torch, rank, local_rank, world):
        from ngraph_b200 import ngraph_api as ng
        self.torch, self.ng = torch, ng
        ng.load_b200()
        self.host_inputs(1 + rank)
        m, hidden = self.batch * self.dims["seq"], self.dims["hidden"]
        stream = torch.cuda.current_stream().cuda_stream
        self.backend = ng.Backend("B200:%d,stream=%d" % (local_rank, stream))
        self.fn = ng.bert_encoder(seed=1, batch=self.batch, **self.dims)
        self.exe = self.backend.compile(self.fn)
        self.dev = [torch.from_numpy(self.ids).cuda(), torch.from_numpy(self.seg).cuda()]
        self.out = torch.empty((m, hidden), dtype=torch.float32, device="cuda")
        self.t_in = [self.backend.create_tensor(np.int32, (m,), t.data_ptr()) for t in self.dev]
        self.t_out = self.backend.create_tensor(np.float32, (m, hidden), self.out.data_ptr())
        self.pin_in = [torch.from_numpy(self.ids).pin_memory(), torch.from_numpy(self.seg).pin_memory()]
        self.pin_out = torch.empty((m, hidden), dtype=torch.float32).pin_memory()

    def units_per_step(self):
        return float(self.batch * self.dims["seq"])

    def step(self):
        self.exe.call([self.t_out], self.t_in, validate=False)

    def step_e2e(self):
        for t, h in zip(self.t_in, self.pin_in):
            t.write_ptr(h.data_ptr(), h.numel() * 4)
        self.exe.call([self.t_out], self.t_in, validate=False)
        self.t_out.read_ptr(self.pin_out.data_ptr(), self.pin_out.numel() * 4)

    def io_bytes(self):
        return sum(h.numel() * 4 for h in self.pin_in), self.pin_out.numel() * 4

    def int8_ops_per_step(self):
        d = self.dims
        return 2.0 * (4 * d["hidden"] ** 2 + 2 * d["hidden"] * d["ffn"]) * d["layers"] * self.batch * d["seq"]

    def roofline(self, peaks, per_step_ms, probe):
        """the int8 dots against the tensor peak: their share of the step from per-node CUDA events of an instrumented pass,
        applied to the timed step; the f32 glue is listed beside them because it is most of the step"""
        exe = self.backend.compile(self.fn, perf=True)
        passes = 3
        for _ in range(passes):
            exe.call([self.t_out], self.t_in, validate=False)
        self.torch.cuda.synchronize()
        rows = exe.performance_data()
        by_op = {}
        for n, us, c in rows:
            by_op[n.split(":")[0]] = by_op.get(n.split(":")[0], 0.0) + us / passes
        total_us = sum(by_op.values())
        share = by_op.get("QuantizedDotBias", 0.0) / total_us
        dots_us = per_step_ms * 1e3 * share
        peak, peak_source = int8_peak(peaks, probe)
        achieved = self.int8_ops_per_step() / (dots_us * 1e-6) / 1e12
        top = sorted(((round(v, 1), k) for k, v in by_op.items()), reverse=True)[:8]
        return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s", "frac": achieved / peak, "traffic": None,
                "kernel": "qcontract_kernel (72 QuantizedDotBias layers)", "kernel_us_per_step": dots_us, "kernel_share_of_step": share,
                "kernel_share_source": "per-node CUDA events, instrumented pass", "glue_share_of_step": 1.0 - share,
                "op_types_us_per_step_instrumented": top, "peak_source": peak_source, "peak_i8_measured": probe}

    def cpu_sample(self):
        """nGraph's INTERPRETER on ONE layer of the same width over one short sequence, scaled to the depth of the model"""
        from ngraph_b200 import ngraph_api as ng
        from oracle import interpreter
        d = dict(self.dims, layers=1, seq=8)
        fn = ng.bert_encoder(seed=1, batch=1, decomposed=True, **d)
        rng = np.random.default_rng(3)
        self.sample_inputs = [rng.integers(0, d["vocab"], 8).astype(np.int32), (rng.random(8) < 0.5).astype(np.int32)]
        exe = interpreter.backend().compile(fn)
        t = time.time()
        self.sample_output = exe.run(*self.sample_inputs)[0]
        dt = time.time() - t
        rate = 8.0 / (dt * self.dims["layers"])
        return rate, ("INTERPRETER, 1 thread: one encoder layer (hidden %d, FFN %d) on 8 tokens in %.1f s, scaled to %d layers"
                      % (d["hidden"], d["ffn"], dt, self.dims["layers"]))

    def check_and_cpu_baseline(self, skip_cpu):
        if skip_cpu:
            return None, None
        rate, sample = self.cpu_sample()
        d = dict(self.dims, layers=1, seq=8)
        got = self.backend.compile(self.ng.bert_encoder(seed=1, batch=1, **d)).run(*self.sample_inputs)[0]
        err = float(np.max(np.abs(got - self.sample_output)) / max(1e-30, float(np.max(np.abs(self.sample_output)))))
        return {"value": rate, "unit": self.unit, "cores": 1, "kind": "reference", "sample": sample}, bool(err <= 1e-5)


class MicroWorkload:
    """single-kernel workloads called through the C ABI (ngraph_b200.ops)"""
    bound = "tensor"

    light = False  # True: device buffers only (no pinned host mirrors for the end-to-end loop)

    def setup(self, torch, rank, local_rank, world):
        from ngraph_b200 import ops
        self.torch, self.ops = torch, ops
        self.alloc(1 + rank)

    def roofline(self, peaks, per_step_ms, probe):
        alg = self.alg_per_launch()
        if self.bound == "hbm":
            achieved, peak, unit, src = alg / (per_step_ms / 1e3) / 1e9, peaks["hbm_gbs"], "GB/s", peaks["source"] + ": device copy"
        else:
            achieved, unit = alg / (per_step_ms / 1e3) / 1e12, "TOP/s"
            peak, src = int8_peak(peaks, probe)
        return {"bound": self.bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak, "traffic": None,
                "peak_source": src}

    def check_and_cpu_baseline(self, skip_cpu):
        ok = self.check()
        if skip_cpu:
            return None, ok
        v, sample = self.cpu_sample()
        return {"value": v, "unit": self.unit, "cores": 1, "kind": "port", "sample": sample}, ok


class QConvLayer(MicroWorkload):
    name, metric, unit, dtype = "qconv", "QuantizedConvolutionBias+Relu int8 throughput", "TOPS", "u8*i8->i32"

    def __init__(self, batch=32):
        # the 3x3 64 -> 64 channel layer on 56x56 images by default; B200_BENCH_CONV="C,K,R,HW[,sum]" times another ResNet layer shape (stride 1,
        # same padding); a fifth field 1 adds a u8 residual input (QuantizedConvolutionBiasAdd)
        f = [int(v) for v in os.environ.get("B200_BENCH_CONV", "64,64,3,56").split(",")]
        c, k, r, hw = f[:4]
        self.with_sum = len(f) > 4 and f[4] != 0
        self.B, self.C, self.H, self.W, self.K, self.R = batch, c, hw, hw, k, r

    def describe(self, world=1):
        return {"workload": "QuantizedConvolutionBias%s+Relu u8[%d,%d,%d,%d]*i8[%d,%d,%d,%d] s1 same-pad, per-channel scales, "
                            "i32 bias -> u8" % ("Add (u8 residual)" if self.with_sum else "", self.B, self.C, self.H, self.W, self.K,
                                                self.C, self.R, self.R),
                "layout": "channels-last on device",
                "l2": "input %.1f MB + output %.1f MB per step, rotated over %d buffers (> 126 MB L2)"
                      % (self.B * self.C * self.H * self.W / 1e6, self.B * self.K * self.H * self.W / 1e6, self.nbufs())}

    def nbufs(self):
        per = self.B * (self.C + self.K * (2 if self.with_sum else 1)) * self.H * self.W
        return max(2, min(24, int(300e6 // per) + 1))

    def host_inputs(self, seed):
        rng = np.random.default_rng(seed)
        d = {"data": rng.integers(0, 256, size=(self.B, self.H, self.W, self.C), dtype=np.uint8),
             "filt": rng.integers(-127, 128, size=(self.K, self.R, self.R, self.C)).astype(np.int8),
             "bias": rng.integers(-1000, 1001, size=self.K).astype(np.int32)}
        sf = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), size=self.K)).astype(np.float32)
        d["scale"] = (np.float32(0.02) * sf / np.float32(0.05)).astype(np.float32)
        d["sum"] = rng.integers(0, 256, size=(self.B, self.H, self.W, self.K), dtype=np.uint8) if self.with_sum else None
        self.h = d
        return d

    def alloc(self, seed):
        torch, ops = self.torch, self.ops
        h = self.host_inputs(seed)
        self.nbuf = self.nbufs()
        self.data = [torch.from_numpy(h["data"]).cuda() for _ in range(self.nbuf)]
        self.out = [torch.empty((self.B, self.H, self.W, self.K), dtype=torch.uint8, device="cuda") for _ in range(self.nbuf)]
        self.filt, self.bias, self.scale = (torch.from_numpy(h[k]).cuda() for k in ("filt", "bias", "scale"))
        self.sum = [torch.from_numpy(h["sum"]).cuda() for _ in range(self.nbuf)] if self.with_sum else None
        self.sum_scale = torch.full((1,), 0.37, device="cuda") if self.with_sum else None
        pad = self.R // 2
        self.cp = ops.conv_params((self.B, self.H, self.W, self.C), (self.K, self.R, self.R, self.C), (1, 1), (pad, pad))
        if not self.light:
            self.pin_in = torch.from_numpy(h["data"]).pin_memory()
            self.pin_out = torch.empty((self.B, self.H, self.W, self.K), dtype=torch.uint8).pin_memory()
        self.i = 0

    def units_per_step(self):
        return 2.0 * self.B * self.H * self.W * self.K * self.C * self.R * self.R / 1e12

    def alg_per_launch(self):
        return self.units_per_step() * 1e12

    def _launch(self, i):
        self.ops.qconv(self.data[i], self.filt, self.scale, self.torch.uint8, self.cp, bias=self.bias, relu=True, out=self.out[i],
                       sum_in=self.sum[i] if self.with_sum else None, sum_scale=self.sum_scale)

    def step(self):
        i = self.i = (self.i + 1) % self.nbuf
        self._launch(i)

    def step_e2e(self):
        i = self.i = (self.i + 1) % self.nbuf
        self.data[i].copy_(self.pin_in, non_blocking=True)
        self._launch(i)
        self.pin_out.copy_(self.out[i], non_blocking=True)

    def io_bytes(self):
        return self.pin_in.numel(), self.pin_out.numel()

    def _oracle(self, nimg):
        from oracle import ref
        pad = self.R // 2
        cs = ref.conv_shape((nimg, self.C, self.H, self.W), (self.K, self.C, self.R, self.R), (1, 1), (pad, pad))
        nchw = np.ascontiguousarray(self.h["data"][:nimg].transpose(0, 3, 1, 2))
        kcrs = np.ascontiguousarray(self.h["filt"].transpose(0, 3, 1, 2))
        if self.with_sum:
            return ref.qconv_fused(nchw, kcrs, self.h["bias"], self.h["scale"], cs, np.uint8, relu=True,
                                   sum_in=np.ascontiguousarray(self.h["sum"][:nimg].transpose(0, 3, 1, 2)), sum_scale=np.float32(0.37))
        return ref.qconv_fused(nchw, kcrs, self.h["bias"], self.h["scale"], cs, np.uint8, relu=True)

    def check(self):
        got = self.out[self.i][:2].cpu().numpy().transpose(0, 3, 1, 2)
        return bool(np.array_equal(got, self._oracle(2)))

    def cpu_sample(self):
        t, reps = time.time(), 0
        while time.time() - t < 10.0:
            self._oracle(2)
            reps += 1
        dt = time.time() - t
        return reps * 2.0 * 2 * self.H * self.W * self.K * self.C * self.R * self.R / 1e12 / dt, "C port of the reference arithmetic, 2 images of the batch, %d passes, %.1f s" % (reps, dt)


class QDotLayer(MicroWorkload):
    name, metric, unit, dtype = "qdot", "QuantizedDotBias+Relu int8 throughput", "TOPS", "u8*i8->i32"

    def __init__(self, m=32768, nk=1024):
        self.M, self.N, self.K = m, nk, nk

    def host_inputs(self, seed):
        from oracle import ref
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((4096, self.K)).astype(np.float32)
        self.h_a = ref.quantize(x[:4096], np.float32(0.02), np.uint8(0))
        self.h_a = np.tile(self.h_a, ((self.M + 4095) // 4096, 1))[:self.M]
        self.h_w = rng.integers(-127, 128, size=(self.N, self.K)).astype(np.int8)
        bias_f = (rng.standard_normal(self.N) * 0.1).astype(np.float32)
        self.h_bias = ref.quantize(bias_f, np.float32(0.02) * np.float32(0.01), np.int32(0))
        self.h_scale = np.array([np.float32(0.02) * np.float32(0.01) / np.float32(0.05)], np.float32)

    def alloc(self, seed):
        torch = self.torch
        self.host_inputs(seed)
        self.nbuf = 8
        self.a = [torch.from_numpy(self.h_a).cuda() for _ in range(self.nbuf)]
        self.out = [torch.empty((self.M, self.N), dtype=torch.uint8, device="cuda") for _ in range(self.nbuf)]
        self.w, self.bias, self.scale = (torch.from_numpy(v).cuda() for v in (self.h_w, self.h_bias, self.h_scale))
        if not self.light:
            self.pin_in = torch.from_numpy(self.h_a).pin_memory()
            self.pin_out = torch.empty((self.M, self.N), dtype=torch.uint8).pin_memory()
        self.i = 0
        # A launch of the small problems (M = 256 is 0.5 GOP) is shorter than the host needs to issue it,
        # so those are timed as a CUDA graph of back-to-back launches, replayed once per step.
        self.graph, self.per_step = None, 1
        if self.M <= 8192:
            self.per_step = 64
            for _ in range(3):
                self._launch()
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                for _ in range(self.per_step):
                    self._launch()

    def describe(self, world=1):
        d = {"workload": "QuantizedDotBias+Relu u8[%d,%d] x i8[%d,%d], i32 bias, scale 0.004 -> u8" % (self.M, self.K, self.K, self.N),
             "l2": "rotated over 8 input/output buffers"}
        if self.M <= 8192:
            d["launches"] = "one step = a CUDA graph of 64 back-to-back launches"
        return d

    def units_per_step(self):
        return self.per_step * 2.0 * self.M * self.N * self.K / 1e12

    def alg_per_launch(self):
        return self.units_per_step() * 1e12

    def launches_per_step(self):
        return self.per_step

    def _launch(self):
        i = self.i = (self.i + 1) % self.nbuf
        self.ops.qgemm(self.a[i], self.w, self.scale, self.torch.uint8, bias=self.bias, relu=True, out=self.out[i])

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self._launch()

    def step_e2e(self):
        i = self.i = (self.i + 1) % self.nbuf
        self.a[i].copy_(self.pin_in, non_blocking=True)
        self.ops.qgemm(self.a[i], self.w, self.scale, self.torch.uint8, bias=self.bias, relu=True, out=self.out[i])
        self.pin_out.copy_(self.out[i], non_blocking=True)

    def e2e_units_per_step(self):
        return 2.0 * self.M * self.N * self.K / 1e12

    def io_bytes(self):
        return self.pin_in.numel(), self.pin_out.numel()

    def check(self):
        from oracle import ref
        exp = ref.qgemm_fused(self.h_a[:512], self.h_w, self.h_bias, self.h_scale, np.uint8, relu=True)
        return bool(np.array_equal(self.out[self.i][:512].cpu().numpy(), exp))

    def cpu_sample(self):
        from oracle import ref
        t, reps, rows = time.time(), 0, 1024
        while time.time() - t < 10.0:
            ref.qgemm_fused(self.h_a[:rows], self.h_w, self.h_bias, self.h_scale, np.uint8, relu=True)
            reps += 1
        dt = time.time() - t
        return reps * 2.0 * rows * self.N * self.K / 1e12 / dt, "C port of the reference arithmetic, %d rows, %d passes, %.1f s" % (rows, reps, dt)


class QuantizeSweepPoint(MicroWorkload):
    name, metric, unit, dtype = "quantize", "Quantize f32->u8 bandwidth", "GB/s", "f32->u8"
    bound = "hbm"

    def __init__(self, batch=64, dequantize=False):
        self.shape = (batch, 64, 256, 256)
        self.dequantize = dequantize
        if dequantize:
            self.metric, self.dtype = "Dequantize u8->f32 bandwidth", "u8->f32"

    def describe(self, world=1):
        n = int(np.prod(self.shape))
        what = "Dequantize u8%s -> f32" if self.dequantize else "Quantize f32%s -> u8"
        return {"workload": (what + " per-tensor scale 0.05 zp 128%s") % (list(self.shape), "" if self.dequantize else " RNE"),
                "l2": "f32 side %.0f MB per step (> 126 MB L2)" % (n * 4 / 1e6) if n * 4 > 126e6 else
                      "f32 side %.0f MB per step: fits the 126 MB L2, so the timed loop alternates between buffers that together exceed it" % (n * 4 / 1e6)}

    def host_inputs(self, seed):
        self.h_x = np.random.default_rng(seed).standard_normal(1 << 24).astype(np.float32)

    def alloc(self, seed):
        torch = self.torch
        self.host_inputs(seed)
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        n = int(np.prod(self.shape))
        self.nbuf = max(1, int(300e6 // (n * 5)) + 1) if n * 4 <= 126e6 else 1  # small tensors: rotate so that L2 does not serve them
        self.x = [torch.randn(self.shape, device="cuda", generator=g) for _ in range(self.nbuf)]
        self.y = [torch.empty(self.shape, dtype=torch.uint8, device="cuda") for _ in range(self.nbuf)]
        self.s = torch.full((), 0.05, device="cuda")
        self.z = torch.full((), 128, dtype=torch.uint8, device="cuda")
        self.i = 0
        if self.dequantize:
            for x, y in zip(self.x, self.y):
                self.ops.quantize(x, self.s, self.z, (), 4, out=y)
        if not self.light:
            self.pin_in = torch.empty(self.shape, dtype=torch.float32).pin_memory()
            self.pin_in.copy_(self.x[0])
            self.pin_out = torch.empty(self.shape, dtype=torch.uint8).pin_memory()

    def units_per_step(self):
        return 5.0 * self.x[0].numel() / 1e9

    def alg_per_launch(self):
        return 5.0 * self.x[0].numel()

    def step(self):
        i = self.i = (self.i + 1) % self.nbuf
        if self.dequantize:
            self.ops.dequantize(self.y[i], self.s, self.z, (), out=self.x[i])
        else:
            self.ops.quantize(self.x[i], self.s, self.z, (), 4, out=self.y[i])

    def step_e2e(self):
        self.x[0].copy_(self.pin_in, non_blocking=True)
        self.ops.quantize(self.x[0], self.s, self.z, (), 4, out=self.y[0])
        self.pin_out.copy_(self.y[0], non_blocking=True)

    def io_bytes(self):
        return self.pin_in.numel() * 4, self.pin_out.numel()

    def check(self):
        from oracle import ref
        n = 1 << 20
        i = self.i
        if self.dequantize:
            exp = ref.dequantize(self.y[i].view(-1)[:n].cpu().numpy(), np.float32(0.05), np.uint8(128))
            return bool(np.array_equal(self.x[i].view(-1)[:n].cpu().numpy().view(np.uint32), exp.view(np.uint32)))
        exp = ref.quantize(self.x[i].view(-1)[:n].cpu().numpy(), np.float32(0.05), np.uint8(128))
        return bool(np.array_equal(self.y[i].view(-1)[:n].cpu().numpy(), exp))

    def cpu_sample(self):
        from oracle import ref
        t, reps = time.time(), 0
        while time.time() - t < 10.0:
            ref.quantize(self.h_x, np.float32(0.05), np.uint8(128))
            reps += 1
        dt = time.time() - t
        return reps * 5.0 * self.h_x.size / 1e9 / dt, "C port of the reference arithmetic, %d elements, %d passes, %.1f s" % (self.h_x.size, reps, dt)


def per_config_block(torch, peaks, probe, steps=20):
    """The other workloads the baseline names, each timed for a moment through the C ABI on this GPU (device-resident
    inputs, CUDA events, parity against the oracle on a sample): so that one default run records a roofline fraction for
    every one of them, not only for the headline network."""
    cases = [("QuantizedDotBias+Relu M=256 (CUDA graph of 64 launches)", QDotLayer(256)),
             ("QuantizedDotBias+Relu M=4096", QDotLayer(4096)),
             ("QuantizedDotBias+Relu M=32768", QDotLayer(32768)),
             ("QuantizedConvolutionBias+Relu 3x3 C=K=64 56x56 batch 32", QConvLayer(32)),
             ("QuantizedConvolutionBias+Relu 3x3 C=K=64 56x56 batch 128", QConvLayer(128)),
             ("Quantize f32->u8 RNE 67 MB", QuantizeSweepPoint(4)), ("Quantize f32->u8 RNE 268 MB", QuantizeSweepPoint(16)),
             ("Quantize f32->u8 RNE 1074 MB", QuantizeSweepPoint(64)),
             ("Dequantize u8->f32 67 MB", QuantizeSweepPoint(4, True)), ("Dequantize u8->f32 268 MB", QuantizeSweepPoint(16, True)),
             ("Dequantize u8->f32 1074 MB", QuantizeSweepPoint(64, True))]
    out = []
    for name, wl in cases:
        try:
            wl.light = True
            wl.setup(torch, 0, torch.cuda.current_device(), 1)
            for _ in range(5):
                wl.step()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                wl.step()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            r = wl.roofline(peaks, ms, probe)
            launches = wl.launches_per_step() if hasattr(wl, "launches_per_step") else 1
            out.append({"workload": name, "us_per_launch": ms * 1e3 / launches, "achieved": r["achieved"], "unit": r["unit"],
                        "peak": r["peak"], "frac": r["frac"], "bound": r["bound"], "parity_vs_oracle": wl.check()})
        except Exception as e:  # one case that cannot run must not lose the headline line
            out.append({"workload": name, "error": str(e)[:160]})
        del wl
        torch.cuda.empty_cache()
    return out


WORKLOADS = {"resnet50": ResNet50, "qconv": QConvLayer, "qdot": QDotLayer, "quantize": QuantizeSweepPoint, "bert": BertEncoder}


def run_reference(args, wl, rank):
    """The reference arm: nGraph's own CPU arithmetic for the path on the host cores, rank 0 only."""
    if rank != 0:
        return
    total = args.steps + args.warmup
    if isinstance(wl, ResNet50):
        model = wl.build_model()
        budget = min(12.0, 120.0 / max(total, 1))  # seconds per step: the whole arm stays within a few minutes
        rates, procs, sample, _, _ = cpu_reference_rate(model, budget, reps=total)
        value, cores, kind = float(np.mean(rates[args.warmup:])), procs, "reference"
    else:
        wl.host_inputs(1)
        value, sample = wl.cpu_sample()
        cores, kind = 1, getattr(wl, "cpu_kind", "port")
    line = {"impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.describe(args.gpus),
            "cpu_baseline": {"value": value, "unit": wl.unit, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    if len(sys.argv) >= 5 and sys.argv[1] == "--cpu-worker":
        cpu_worker(sys.argv[2], sys.argv[3], int(sys.argv[4]))
        return
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="resnet50", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch (images / rows); for small profiler captures")
    ap.add_argument("--nk", type=int, default=0, help="qdot: reduction length and output width (default 1024 x 1024); with --batch "
                    "for a square GEMM")
    ap.add_argument("--pipeline", type=int, default=2, choices=[1, 2, 3, 4], help="resnet50: batches in flight per GPU (2 = two "
                    "executables on two streams, steps alternate; 1 = one executable on one stream)")
    ap.add_argument("--no-per-config", action="store_true", help="skip the short per-workload block of the default run")
    ap.add_argument("--no-peak-probe", action="store_true", help="skip the in-run int8 GEMM peak measurement (profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload == "qdot" and args.nk:
        wl = QDotLayer(args.batch or 32768, args.nk)
    else:
        wl = WORKLOADS[args.workload](args.batch) if args.batch else WORKLOADS[args.workload]()
    if isinstance(wl, ResNet50):
        wl.pipeline = args.pipeline

    if args.impl == "reference":
        run_reference(args, wl, rank)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        sys.exit("bench.py needs a CUDA device: the B200 path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        # NCCL prints its version banner on stdout at the first collective: keep stdout for the one JSON line
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            dist.all_reduce(torch.zeros(1, device="cuda"))
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    from ngraph_b200 import lib

    wl.setup(torch, rank, local_rank, world)
    peaks = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        wl.step()
    if hasattr(wl, "finish"):
        wl.finish()
    barrier()
    lib.device_status()

    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    lib.LIB.b200_reset_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.time()
    ev0.record()
    if hasattr(wl, "begin"):
        wl.begin()
    for _ in range(args.steps):
        wl.step()
    if hasattr(wl, "finish"):
        wl.finish()
    ev1.record()
    barrier()
    t1 = time.time()
    launches = lib.launch_count()
    if hasattr(wl, "launches_per_step") and wl.launches_per_step() > 1:
        launches = args.steps * wl.launches_per_step()  # replayed from a CUDA graph: the host-side counter does not see them
    ms = ev0.elapsed_time(ev1)

    # the same steps without the pipelining (one executable, one stream), for comparison
    ms_single = None
    if isinstance(wl, ResNet50) and wl.pipeline > 1:
        depth = wl.pipeline
        wl.pipeline = 1
        for _ in range(3):
            wl.step()
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            wl.step()
        wl.finish()
        s1.record()
        barrier()
        ms_single = s0.elapsed_time(s1)
        wl.pipeline = depth

    # end to end: pinned host -> device, kernels, device -> pinned host, every step
    for _ in range(2):
        wl.step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        wl.step_e2e()
    if hasattr(wl, "finish"):
        wl.finish()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    clocks = sampler.stop(t0, time.time())  # both timed regions (device-resident and end-to-end)
    lib.device_status()

    # the floor under the end-to-end number: this rank's pinned host -> device copy of one step's input alone, while every
    # other rank does the same (the ranks share the host's memory and PCIe fabric)
    h2d_floor_gbs = None
    h2d_bytes = wl.io_bytes()[0]
    if h2d_bytes >= (1 << 20):
        src = torch.empty(h2d_bytes, dtype=torch.uint8).pin_memory()
        dst = torch.empty(h2d_bytes, dtype=torch.uint8, device="cuda")
        dst.copy_(src, non_blocking=True)
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(10):
            dst.copy_(src, non_blocking=True)
        c1.record()
        barrier()
        h2d_floor_gbs = h2d_bytes * 10 / (c0.elapsed_time(c1) * 1e-3) / 1e9
        del src, dst

    t = torch.tensor([ms, ms_e2e, -(h2d_floor_gbs or 0.0), ms_single or 0.0], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    ms_single = float(t[3]) if ms_single else None
    h2d_floor_gbs = -float(t[2]) if h2d_floor_gbs else None  # the slowest rank's copy rate

    if rank == 0:
        per_step = ms / args.steps
        value = wl.units_per_step() * world / (per_step / 1e3)
        e2e_units = wl.e2e_units_per_step() if hasattr(wl, "e2e_units_per_step") else wl.units_per_step()
        e2e_value = e2e_units * world / (ms_e2e / args.steps / 1e3)
        h2d, d2h = wl.io_bytes()
        e2e = {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": ms_e2e / args.steps}
        if h2d_floor_gbs:
            # what the host -> device copy alone allows (slowest rank, all ranks copying at once) against what was reached
            floor_ms = h2d / (h2d_floor_gbs * 1e9) * 1e3
            e2e.update({"h2d_floor_gbs": h2d_floor_gbs, "h2d_floor_ms_per_step": floor_ms,
                        "frac_of_h2d_floor": floor_ms / (ms_e2e / args.steps)})
        probe = {"n": 0} if args.no_peak_probe or wl.bound != "tensor" else measure_int8_peak(torch)
        line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.describe(world),
                "gpu_launches": launches, "clocks": clocks, "e2e": e2e, "roofline": wl.roofline(peaks, per_step, probe)}
        if ms_single:
            line["single_stream"] = {"ms_per_step": ms_single / args.steps, "value": wl.units_per_step() * world / (ms_single / args.steps / 1e3),
                                     "unit": wl.unit, "note": "one executable on one stream (pipeline depth 1), same steps"}
        if isinstance(wl, ResNet50) and world == 1 and not args.no_per_config:
            line["per_config"] = per_config_block(torch, peaks, probe)
        cpu, ok = wl.check_and_cpu_baseline(args.no_cpu_baseline or world > 1)
        line["parity_vs_oracle"] = ok
        if cpu is not None:
            line["cpu_baseline"] = cpu
            extra = wl.extra_cpu_baselines() if hasattr(wl, "extra_cpu_baselines") else None
            if extra:
                line.update(extra)
            # the end-to-end figure over each host baseline of this run (vs_baseline stays null: no published number
            # exists for this metric)
            for key in ("cpu_baseline", "cpu_baseline_onednn_proxy"):
                base = line.get(key)
                if isinstance(base, dict) and base.get("value") and base.get("unit") == e2e.get("unit"):
                    base["e2e_over_this_baseline"] = e2e["value"] / base["value"]
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
