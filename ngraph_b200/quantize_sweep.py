"""Quantize / Dequantize bandwidth sweep on one GPU (the Quantize / Dequantize bandwidth workload): x f32 ~ N(0,1) of shape [N,64,H,W] from 1 MB to
4 GB of f32, element types u8 (zero point 128) and i8 (zero point 0), one scale per tensor (0.05) or per channel
(axes = {1}, log-uniform in [1e-3, 1e-1]), every RoundMode, and Dequantize of the produced tensors.

    python -m ngraph_b200.quantize_sweep [--max-mb 4096] [--out table.txt]

The last column is a plain device copy of the same f32 tensor timed the same way (8 bytes per element): the bandwidth a
single launch of that size can reach.  Each figure is algorithmic bytes (5 per element: 4 + 1) over the mean device time of `--iters` launches, timed one by one
with CUDA events on the launching stream; before every timed launch a 512 MB buffer is rewritten so that neither the
input nor a previous output is still in the 126 MB L2.  The kernels are called through the C ABI (ngraph_b200.ops)."""
import argparse
import sys

import numpy as np
import torch

from . import ops

ROUND_MODES = ["NEAREST_TOWARD_INFINITY", "NEAREST_TOWARD_ZERO", "NEAREST_UPWARD", "NEAREST_DOWNWARD", "NEAREST_TOWARD_EVEN",
               "TOWARD_INFINITY", "TOWARD_ZERO", "UP", "DOWN"]  # op::v0::Quantize::RoundMode, in declaration order

# [N, 64, H, W] for 1, 4, 16, 64, 256, 1024, 4096 MB of f32
SHAPES = {1: (1, 64, 64, 64), 4: (4, 64, 64, 64), 16: (16, 64, 64, 64), 64: (64, 64, 64, 64), 256: (64, 64, 128, 128),
          1024: (64, 64, 256, 256), 4096: (256, 64, 256, 256)}


def timed(fn, flush, iters):
    """mean milliseconds of fn() over `iters` launches, each after an L2 flush that is outside the timed span"""
    for _ in range(3):
        fn()
    total = 0.0
    for _ in range(iters):
        flush.add_(1.0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def sweep(max_mb=4096, iters=10, out=print):
    dev = torch.device("cuda")
    flush = torch.zeros(128 * 1024 * 1024, dtype=torch.float32, device=dev)  # 512 MB
    gen = torch.Generator(device=dev).manual_seed(1)
    rng = np.random.default_rng(1)
    per_axis = torch.from_numpy(np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), 64)).astype(np.float32)).to(dev)
    scalar = torch.full((), 0.05, device=dev)
    zps = {"u8": torch.full((), 128, dtype=torch.uint8, device=dev), "i8": torch.zeros((), dtype=torch.int8, device=dev)}
    zps_axis = {"u8": torch.full((64,), 128, dtype=torch.uint8, device=dev), "i8": torch.zeros(64, dtype=torch.int8, device=dev)}
    rows = []
    out("%-8s %-22s %-4s %-10s %12s %12s %12s" % ("f32 MB", "shape", "type", "scale", "Quantize", "Dequantize", "f32 copy"))
    for mb, shape in SHAPES.items():
        if mb > max_mb:
            continue
        x = torch.randn(shape, generator=gen, device=dev)
        n = x.numel()
        # the same launch-by-launch timing of a plain device copy of the tensor (8 bytes per element): what the memory
        # system gives a single launch of this size
        spare = torch.empty_like(x)
        g_copy = 8.0 * n / timed(lambda: spare.copy_(x), flush, iters) / 1e6
        del spare
        for ty in ("u8", "i8"):
            for what, scale, zp, axes in (("per-tensor", scalar, zps[ty], ()), ("per-axis", per_axis, zps_axis[ty], (1,))):
                q = torch.empty(shape, dtype=zp.dtype, device=dev)
                back = torch.empty(shape, dtype=torch.float32, device=dev)
                t_q = timed(lambda: ops.quantize(x, scale, zp, axes=axes, round_mode=4, out=q), flush, iters)
                t_d = timed(lambda: ops.dequantize(q, scale, zp, axes=axes, out=back), flush, iters)
                gq, gd = 5.0 * n / t_q / 1e6, 5.0 * n / t_d / 1e6
                rows.append((mb, ty, what, "RNE", gq, gd))
                out("%-8d %-22s %-4s %-10s %7.0f GB/s %7.0f GB/s %7.0f GB/s" % (mb, list(shape), ty, what, gq, gd, g_copy))
                del q, back
        del x
    mb = min(1024, max(m for m in SHAPES if m <= max_mb))
    x = torch.randn(SHAPES[mb], generator=gen, device=dev)
    q = torch.empty(SHAPES[mb], dtype=torch.uint8, device=dev)
    out("")
    out("Quantize f32 -> u8, per-tensor scale, %d MB, every RoundMode:" % mb)
    for mode, name in enumerate(ROUND_MODES):
        t = timed(lambda: ops.quantize(x, scalar, zps["u8"], round_mode=mode, out=q), flush, iters)
        g = 5.0 * x.numel() / t / 1e6
        rows.append((mb, "u8", "per-tensor", name, g, None))
        out("  ROUND_%-24s %7.0f GB/s" % (name, g))
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--max-mb", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        sys.exit("quantize_sweep needs a CUDA device")
    lines = []

    def emit(s):
        print(s, flush=True)
        lines.append(s)

    sweep(a.max_mb, a.iters, emit)
    if a.out:
        with open(a.out, "w") as f:
            f.write("\n".join(lines) + "\n")


if __name__ == "__main__":
    main()
