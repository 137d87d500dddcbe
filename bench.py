#!/usr/bin/env python3
"""Benchmark of the B200 quantized-inference path (and, with --impl reference, of nGraph's own CPU
reference kernels on the host cores).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl b200|reference]

One JSON line on stdout (rank 0).  Workloads (synthetic, seeded; shapes from the baseline configs):
    qconv     QuantizedConvolutionBias+Relu layer, u8 [B,64,56,56] * i8 [64,64,3,3], per-channel scales
    qdot      QuantizedDotBias+Relu layer, u8 [M,1024] x i8 [1024,1024]
    quantize  Quantize f32 -> u8, per-tensor, [B,64,256,256]
A step is one pass of the hot path over one batch.  `value` is timed with CUDA events with the
inputs resident in HBM; `e2e` includes the pinned-host -> device copy of the step's input and the
device -> host copy of its result, through the same C-ABI calls.
"""
import argparse
import json
import os
import subprocess
import sys
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
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
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


# ------------------------------------------------------------------------------------------ workloads
class QConvLayer:
    """BASELINE config: single QuantizedConvolutionBias+Relu layer (u8 NHWC on device)."""
    name, metric, unit, dtype = "qconv", "QuantizedConvolutionBias+Relu int8 throughput", "TOPS", "u8*i8->i32"
    bound = "tensor"

    def __init__(self, batch=32):
        self.B, self.C, self.H, self.W, self.K = batch, 64, 56, 56, 64

    def describe(self):
        return {"workload": "QuantizedConvolutionBias+Relu u8[%d,64,56,56]*i8[64,64,3,3] s1 p1, per-channel scales, "
                            "i32 bias -> u8" % self.B, "layout": "channels-last on device",
                "l2": "input+output 2x%.1f MB per step, rotated over 24 buffers (> 126 MB L2)" % (self.B * 64 * 3136 / 1e6)}

    def host_inputs(self, seed):
        rng = np.random.default_rng(seed)
        d = {"data": rng.integers(0, 256, size=(self.B, self.H, self.W, self.C), dtype=np.uint8),
             "filt": rng.integers(-127, 128, size=(self.K, 3, 3, self.C)).astype(np.int8),
             "bias": rng.integers(-1000, 1001, size=self.K).astype(np.int32)}
        sf = np.exp(rng.uniform(np.log(1e-3), np.log(1e-2), size=self.K)).astype(np.float32)
        d["scale"] = (np.float32(0.02) * sf / np.float32(0.05)).astype(np.float32)
        return d

    def setup(self, torch, ops, seed):
        self.torch, self.ops = torch, ops
        h = self.host_inputs(seed)
        self.h = h
        self.nbuf = 24
        self.data = [torch.from_numpy(h["data"]).cuda() for _ in range(self.nbuf)]
        self.out = [torch.empty((self.B, 56, 56, self.K), dtype=torch.uint8, device="cuda") for _ in range(self.nbuf)]
        self.filt, self.bias, self.scale = (torch.from_numpy(h[k]).cuda() for k in ("filt", "bias", "scale"))
        self.cp = ops.conv_params((self.B, 56, 56, 64), (64, 3, 3, 64), (1, 1), (1, 1))
        self.pin_in = torch.from_numpy(h["data"]).pin_memory()
        self.pin_out = torch.empty((self.B, 56, 56, self.K), dtype=torch.uint8).pin_memory()
        self.i = 0

    def units_per_step(self):  # tera-ops per step
        return 2.0 * self.B * 56 * 56 * self.K * self.C * 9 / 1e12

    def alg_per_launch(self):
        return self.units_per_step() * 1e12  # ops of the one launch

    def step(self):
        i = self.i = (self.i + 1) % self.nbuf
        self.ops.qconv(self.data[i], self.filt, self.scale, self.torch.uint8, self.cp, bias=self.bias, relu=True, out=self.out[i])

    def step_e2e(self):
        i = self.i = (self.i + 1) % self.nbuf
        self.data[i].copy_(self.pin_in, non_blocking=True)
        self.ops.qconv(self.data[i], self.filt, self.scale, self.torch.uint8, self.cp, bias=self.bias, relu=True, out=self.out[i])
        self.pin_out.copy_(self.out[i], non_blocking=True)

    def io_bytes(self):
        return self.pin_in.numel(), self.pin_out.numel()

    def check(self):
        from oracle import ref
        cs = ref.conv_shape((2, 64, 56, 56), (64, 64, 3, 3), (1, 1), (1, 1))
        nchw = np.ascontiguousarray(self.h["data"][:2].transpose(0, 3, 1, 2))
        kcrs = np.ascontiguousarray(self.h["filt"].transpose(0, 3, 1, 2))
        exp = ref.qconv_fused(nchw, kcrs, self.h["bias"], self.h["scale"], cs, np.uint8, relu=True)
        got = self.out[self.i][:2].cpu().numpy().transpose(0, 3, 1, 2)
        return bool(np.array_equal(got, exp))

    def cpu_sample(self):
        from oracle import ref
        nimg = 2
        cs = ref.conv_shape((nimg, 64, 56, 56), (64, 64, 3, 3), (1, 1), (1, 1))
        nchw = np.ascontiguousarray(self.h["data"][:nimg].transpose(0, 3, 1, 2))
        kcrs = np.ascontiguousarray(self.h["filt"].transpose(0, 3, 1, 2))
        t = time.time()
        reps = 0
        while time.time() - t < 10.0:
            ref.qconv_fused(nchw, kcrs, self.h["bias"], self.h["scale"], cs, np.uint8, relu=True)
            reps += 1
        dt = time.time() - t
        return reps * 2.0 * nimg * 56 * 56 * 64 * 64 * 9 / 1e12 / dt, "%d images of the batch, %d passes, %.1f s" % (nimg, reps, dt)


class QDotLayer:
    """BASELINE config: QuantizedDotBias+Relu, X u8 [M,1024], W i8 [1024,1024], bias, requantise to u8."""
    name, metric, unit, dtype = "qdot", "QuantizedDotBias+Relu int8 throughput", "TOPS", "u8*i8->i32"
    bound = "tensor"

    def __init__(self, m=32768):
        self.M, self.N, self.K = m, 1024, 1024

    def describe(self):
        return {"workload": "QuantizedDotBias+Relu u8[%d,1024] x i8[1024,1024], i32 bias, scale 0.004 -> u8" % self.M,
                "l2": "rotated over 8 input/output buffers"}

    def host_inputs(self, seed):
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((4096, self.K)).astype(np.float32)
        from oracle import ref
        self.h_a = ref.quantize(x[:4096], np.float32(0.02), np.uint8(0))
        self.h_a = np.tile(self.h_a, ((self.M + 4095) // 4096, 1))[:self.M]
        self.h_w = rng.integers(-127, 128, size=(self.N, self.K)).astype(np.int8)
        bias_f = (rng.standard_normal(self.N) * 0.1).astype(np.float32)
        self.h_bias = ref.quantize(bias_f, np.float32(0.02) * np.float32(0.01), np.int32(0))
        self.h_scale = np.array([np.float32(0.02) * np.float32(0.01) / np.float32(0.05)], np.float32)

    def setup(self, torch, ops, seed):
        self.torch, self.ops = torch, ops
        self.host_inputs(seed)
        self.nbuf = 8
        self.a = [torch.from_numpy(self.h_a).cuda() for _ in range(self.nbuf)]
        self.out = [torch.empty((self.M, self.N), dtype=torch.uint8, device="cuda") for _ in range(self.nbuf)]
        self.w, self.bias, self.scale = (torch.from_numpy(v).cuda() for v in (self.h_w, self.h_bias, self.h_scale))
        self.pin_in = torch.from_numpy(self.h_a).pin_memory()
        self.pin_out = torch.empty((self.M, self.N), dtype=torch.uint8).pin_memory()
        self.i = 0

    def units_per_step(self):
        return 2.0 * self.M * self.N * self.K / 1e12

    def alg_per_launch(self):
        return self.units_per_step() * 1e12

    def step(self):
        i = self.i = (self.i + 1) % self.nbuf
        self.ops.qgemm(self.a[i], self.w, self.scale, self.torch.uint8, bias=self.bias, relu=True, out=self.out[i])

    def step_e2e(self):
        i = self.i = (self.i + 1) % self.nbuf
        self.a[i].copy_(self.pin_in, non_blocking=True)
        self.ops.qgemm(self.a[i], self.w, self.scale, self.torch.uint8, bias=self.bias, relu=True, out=self.out[i])
        self.pin_out.copy_(self.out[i], non_blocking=True)

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
        return reps * 2.0 * rows * self.N * self.K / 1e12 / dt, "%d rows of the batch, %d passes, %.1f s" % (rows, reps, dt)


class QuantizeSweepPoint:
    """BASELINE config: Quantize f32 -> u8 (zero point 128, scale 0.05, ROUND_NEAREST_TOWARD_EVEN), [B,64,256,256]."""
    name, metric, unit, dtype = "quantize", "Quantize f32->u8 bandwidth", "GB/s", "f32->u8"
    bound = "hbm"

    def __init__(self, batch=64):
        self.shape = (batch, 64, 256, 256)

    def describe(self):
        n = int(np.prod(self.shape))
        return {"workload": "Quantize f32%s -> u8 per-tensor scale 0.05 zp 128 RNE" % (list(self.shape),),
                "l2": "input %.0f MB per step (> 126 MB L2)" % (n * 4 / 1e6)}

    def host_inputs(self, seed):
        self.h_x = np.random.default_rng(seed).standard_normal(1 << 24).astype(np.float32)

    def setup(self, torch, ops, seed):
        self.torch, self.ops = torch, ops
        self.host_inputs(seed)
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        self.x = torch.randn(self.shape, device="cuda", generator=g)
        self.y = torch.empty(self.shape, dtype=torch.uint8, device="cuda")
        self.s = torch.full((), 0.05, device="cuda")
        self.z = torch.full((), 128, dtype=torch.uint8, device="cuda")
        self.pin_in = torch.empty(self.shape, dtype=torch.float32).pin_memory()
        self.pin_in.copy_(self.x)
        self.pin_out = torch.empty(self.shape, dtype=torch.uint8).pin_memory()

    def units_per_step(self):  # GB per step (5 bytes per element)
        return 5.0 * self.x.numel() / 1e9

    def alg_per_launch(self):
        return 5.0 * self.x.numel()

    def step(self):
        self.ops.quantize(self.x, self.s, self.z, (), 4, out=self.y)

    def step_e2e(self):
        self.x.copy_(self.pin_in, non_blocking=True)
        self.ops.quantize(self.x, self.s, self.z, (), 4, out=self.y)
        self.pin_out.copy_(self.y, non_blocking=True)

    def io_bytes(self):
        return self.pin_in.numel() * 4, self.pin_out.numel()

    def check(self):
        from oracle import ref
        n = 1 << 20
        exp = ref.quantize(self.x.view(-1)[:n].cpu().numpy(), np.float32(0.05), np.uint8(128))
        return bool(np.array_equal(self.y.view(-1)[:n].cpu().numpy(), exp))

    def cpu_sample(self):
        from oracle import ref
        n = 1 << 24
        x = self.h_x
        t, reps = time.time(), 0
        while time.time() - t < 10.0:
            ref.quantize(x, np.float32(0.05), np.uint8(128))
            reps += 1
        dt = time.time() - t
        return reps * 5.0 * n / 1e9 / dt, "%d elements, %d passes, %.1f s" % (n, reps, dt)


WORKLOADS = {"qconv": QConvLayer, "qdot": QDotLayer, "quantize": QuantizeSweepPoint}


def run_reference(args, wl, rank):
    """The reference arm: nGraph's reference arithmetic on the host cores (bounded sample per step)."""
    if rank != 0:
        return
    h = wl.host_inputs(1)
    if h is not None:
        wl.h = h
    value, sample = wl.cpu_sample()
    line = {"impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.describe(),
            "cpu_baseline": {"value": value, "unit": wl.unit, "cores": 1, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="qconv", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch (images / rows); for small profiler captures")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    wl = WORKLOADS[args.workload](args.batch) if args.batch else WORKLOADS[args.workload]()

    if args.impl == "reference":
        run_reference(args, wl, rank)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        sys.exit("bench.py needs a CUDA device: the B200 path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from ngraph_b200 import lib, ops

    wl.setup(torch, ops, seed=1 + rank)
    peaks = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        wl.step()
    barrier()
    lib.device_status()
    ok = wl.check()

    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    lib.LIB.b200_reset_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.time()
    ev0.record()
    for _ in range(args.steps):
        wl.step()
    ev1.record()
    barrier()
    t1 = time.time()
    launches = lib.launch_count()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop(t0, t1)

    # end to end: pinned host -> device, kernels, device -> pinned host, every step
    for _ in range(2):
        wl.step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        wl.step_e2e()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    lib.device_status()

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])

    if rank == 0:
        per_step = ms / args.steps
        value = wl.units_per_step() * world / (per_step / 1e3)
        e2e_value = wl.units_per_step() * world / (ms_e2e / args.steps / 1e3)
        h2d, d2h = wl.io_bytes()
        if wl.bound == "hbm":
            achieved, peak, runit = wl.alg_per_launch() / (per_step / 1e3) / 1e9, peaks["hbm_gbs"], "GB/s"
        else:
            achieved, peak, runit = wl.alg_per_launch() / (per_step / 1e3) / 1e12, 2.0 * peaks["bf16_tflops"], "TOP/s"
        line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.describe(),
                "parity_vs_oracle": ok, "gpu_launches": launches, "clocks": clocks,
                "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                "roofline": {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": runit, "frac": achieved / peak,
                             "traffic": None,
                             "peak_source": peaks["source"] + (" (int8 peak taken as 2 x measured bf16 burst)" if wl.bound == "tensor" else "")}}
        if not args.no_cpu_baseline:
            v, sample = wl.cpu_sample()
            line["cpu_baseline"] = {"value": v, "unit": wl.unit, "cores": 1, "kind": "port", "sample": sample}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
