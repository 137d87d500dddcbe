"""Parity of the CUDA Quantize/Dequantize kernels (through the C ABI) with
(1) the committed golden fixtures (reference tests + INTERPRETER outputs) and
(2) the CPU oracle on seeded inputs: all nine round modes, u8/i8/i32, per-tensor / per-axis /
multi-axis, ragged sizes, tie-heavy data.  Integer outputs bit-exact; Dequantize f32 bit-exact."""
import numpy as np
import pytest
import torch

from oracle import ref
from tests.fixtures import NP, blob, interpreter_cases, reference_tests

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from ngraph_b200 import ops as o
    return o


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_reference_test_vectors(ops):
    n = 0
    for case in reference_tests(("Quantize", "Dequantize")):
        if "f64" in (case["input_type"], case["output_type"]):
            continue
        shape, ss = case["shape"], case["scale_shape"]
        if case["op"] == "Quantize":
            qt = NP[case["output_type"]]
            got = ops.quantize(dev(np.array(case["x"], np.float32).reshape(shape)),
                               dev(np.array(case["scale"], np.float32).reshape(ss)),
                               dev(np.array(case["zero_point"], qt).reshape(ss)), case["axes"], case["round_mode"])
            np.testing.assert_array_equal(got.cpu().numpy().ravel(), np.array(case["expected"], qt), err_msg=case["name"])
        else:
            qt = NP[case["input_type"]]
            got = ops.dequantize(dev(np.array(case["x"], qt).reshape(shape)),
                                 dev(np.array(case["scale"], np.float32).reshape(ss)),
                                 dev(np.array(case["zero_point"], qt).reshape(ss)), case["axes"])
            np.testing.assert_array_equal(got.cpu().numpy().ravel(), np.array(case["expected"], np.float32),
                                          err_msg=case["name"])
        n += 1
    assert n >= 20


def test_interpreter_fixtures(ops):
    for case in interpreter_cases(("Quantize", "Dequantize")):
        i = {k: blob(v) for k, v in case["inputs"].items()}
        exp = blob(case["outputs"]["y"])
        if case["op"] == "Quantize":
            got = ops.quantize(dev(i["x"]), dev(i["scale"]), dev(i["zero_point"]), case["attrs"]["axes"],
                               case["attrs"]["round_mode"]).cpu().numpy()
            np.testing.assert_array_equal(got, exp, err_msg=case["name"])
        else:
            got = ops.dequantize(dev(i["x"]), dev(i["scale"]), dev(i["zero_point"]), case["attrs"]["axes"]).cpu().numpy()
            np.testing.assert_array_equal(got.view(np.uint32), exp.view(np.uint32), err_msg=case["name"])


def seeded_input(rng, shape, scale, axes):
    """N(0,1)-like data scaled into the quantised range, with exact and near ties mixed in."""
    x = rng.standard_normal(shape).astype(np.float32)
    bshape = [shape[d] if d in axes else 1 for d in range(len(shape))]
    s = scale.reshape(bshape) if axes else scale.reshape([1] * len(shape))
    k = rng.integers(-140, 141, size=shape).astype(np.float32)
    kind = rng.integers(0, 4, size=shape)
    ties = ((k + np.float32(0.5)) * s).astype(np.float32)
    near = np.nextafter(ties, np.float32(np.inf) * np.where(rng.integers(0, 2, size=shape) == 0, -1, 1)).astype(np.float32)
    wide = (x * np.float32(60) * s).astype(np.float32)
    return np.where(kind == 0, ties, np.where(kind == 1, near, np.where(kind == 2, wide, x))).astype(np.float32)


SHAPES = [
    ((3, 64, 17, 33), ()),        # per tensor, ragged total (not a multiple of 4... 17*33 odd)
    ((2, 64, 32, 32), (1,)),      # per channel, vector path (inner 1024)
    ((2, 64, 7, 7), (1,)),        # per channel, inner 49 -> generic path
    ((5, 6, 7, 8), (0, 2)),       # two non-adjacent axes -> generic path
    ((4, 8, 4100), (0, 1)),       # adjacent axes -> rows path with a ragged chunk tail
    ((1000003,), ()),             # prime length, per tensor
    ((6, 5), (1,)),               # innermost axis
]


@pytest.mark.parametrize("mode", range(9))
@pytest.mark.parametrize("qname", ["u8", "i8", "i32"])
def test_quantize_vs_oracle(ops, mode, qname):
    qt = NP[qname]
    for si, (shape, axes) in enumerate(SHAPES):
        rng = np.random.default_rng(1234 + 97 * mode + si)
        ss = tuple(shape[a] for a in axes)
        scale = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=ss)).astype(np.float32)
        if not axes:
            scale = np.float32(0.05) * np.ones((), np.float32)
        zp = {"u8": rng.integers(120, 136, size=ss), "i8": rng.integers(-8, 8, size=ss),
              "i32": rng.integers(-1000, 1000, size=ss)}[qname].astype(qt)
        x = seeded_input(rng, shape, scale, axes)
        exp = ref.quantize(x, scale, zp, axes, mode)
        got = ops.quantize(dev(x), dev(scale), dev(zp), axes, mode).cpu().numpy()
        np.testing.assert_array_equal(got, exp, err_msg="shape %s axes %s" % (shape, axes))


@pytest.mark.parametrize("qname", ["u8", "i8", "i32"])
def test_dequantize_vs_oracle(ops, qname):
    qt = NP[qname]
    info = np.iinfo(qt)
    for si, (shape, axes) in enumerate(SHAPES):
        rng = np.random.default_rng(4321 + si)
        ss = tuple(shape[a] for a in axes)
        scale = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=ss)).astype(np.float32)
        lo, hi = max(info.min, -100000), min(info.max, 100000)
        zp = rng.integers(lo // 2, hi // 2, size=ss).astype(qt)
        x = rng.integers(lo, hi + 1, size=shape).astype(qt)
        exp = ref.dequantize(x, scale, zp, axes)
        got = ops.dequantize(dev(x), dev(scale), dev(zp), axes).cpu().numpy()
        np.testing.assert_array_equal(got.view(np.uint32), exp.view(np.uint32), err_msg="shape %s axes %s" % (shape, axes))


def test_special_values(ops):
    x = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e30, -1e30, 3.4e38, 1e-45, -1e-45, 127.5, -128.5], np.float32)
    for qname in ("u8", "i8"):
        zp = np.zeros((), NP[qname])
        for mode in range(9):
            exp = ref.quantize(x, np.float32(1.0), zp, (), mode)
            got = ops.quantize(dev(x), dev(np.float32(1.0) * np.ones((), np.float32)), dev(zp), (), mode).cpu().numpy()
            np.testing.assert_array_equal(got, exp)


def test_empty_and_errors(ops):
    from ngraph_b200.lib import B200Error
    e = ops.quantize(torch.empty((0, 4), device="cuda"), torch.ones((), device="cuda"),
                     torch.zeros((), dtype=torch.uint8, device="cuda"))
    assert e.shape == (0, 4)
    with pytest.raises(B200Error):
        ops.quantize(torch.ones((4,), device="cuda"), torch.ones((), device="cuda"),
                     torch.zeros((), dtype=torch.uint8, device="cuda"), round_mode=12)


def test_roundtrip_property_full_size(ops):
    """Size-independent property on a full-size tensor (256 MB f32): for u8 zp 128 scale 0.05,
    dequantize(quantize(x)) differs from clamp(x) by at most scale/2, and quantize is idempotent on it."""
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    x = torch.randn((64, 64, 128, 128), device="cuda", generator=g)
    s = torch.full((), 0.05, device="cuda")
    zp = torch.full((), 128, dtype=torch.uint8, device="cuda")
    q = ops.quantize(x, s, zp)
    d = ops.dequantize(q, s, zp)
    clamped = torch.clamp(x, -128 * 0.05, 127 * 0.05)
    assert float((d - clamped).abs().max()) <= 0.025 + 1e-6
    q2 = ops.quantize(d, s, zp)
    assert torch.equal(q, q2)
    # a strided sample of the big tensor against the oracle, bit-exact
    idx = torch.arange(0, x.numel(), 4099, device="cuda")
    exp = ref.quantize(x.view(-1)[idx].cpu().numpy(), np.float32(0.05), np.uint8(128))
    np.testing.assert_array_equal(q.view(-1)[idx].cpu().numpy(), exp)


def test_fast_division_is_exact_for_every_float(ops):
    """The strength-reduced division of the RNE 8-bit kernel against the plain IEEE division, over ALL
    2^32 float bit patterns, for the benchmark's scales (0.05 and log-uniform per-channel values) and a
    few awkward ones.  Any difference in any output byte fails."""
    from ngraph_b200 import lib
    rng = np.random.default_rng(99)
    scales = [0.05, 1.0, 3.0, 0.1, 1e-3, 7.0 / 255.0, 0.02, 1.9999999, 1.0000001]
    scales += list(np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=7)))
    chunk = 1 << 28
    base = torch.arange(chunk, dtype=torch.int64, device="cuda")
    for qdt, zpv in ((torch.uint8, 128), (torch.int8, 0)):
        zp = torch.full((), zpv, dtype=qdt, device="cuda")
        for sv in scales:
            s = torch.full((), float(np.float32(sv)), device="cuda")
            for c in range(16):
                x = (base + c * chunk).to(torch.int32).view(torch.float32) if c < 8 else \
                    (base + c * chunk - (1 << 32)).to(torch.int32).view(torch.float32)
                fast = ops.quantize(x, s, zp)
                old = lib.LIB.b200_set_fast_division(0)
                try:
                    exact = ops.quantize(x, s, zp)
                finally:
                    lib.LIB.b200_set_fast_division(old)
                assert torch.equal(fast, exact), "scale %r chunk %d: %d bytes differ" % (sv, c, int((fast != exact).sum()))


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 5, 6, 7, 8])
def test_fast_division_is_exact_for_every_float_in_the_other_round_modes(ops, mode):
    """The directed and half-away modes see the last bit of the quotient (ceil / floor of it), so their strength-reduced
    division must return the correctly rounded x / s itself: all 2^32 bit patterns, device against device."""
    from ngraph_b200 import lib
    chunk = 1 << 28
    base = torch.arange(chunk, dtype=torch.int64, device="cuda")
    for qdt, zpv in ((torch.uint8, 128), (torch.int8, 0)):
        zp = torch.full((), zpv, dtype=qdt, device="cuda")
        # 1.5e6 / 3e-9 / 2^40: scales for which the quotient of small inputs underflows (the directed modes then depend on
        # whether the IEEE quotient is zero or the smallest denormal)
        for sv in (0.05, 3.0, 7.0 / 255.0, 1.0000001, 0.0137, 1.5e6, 3e-9, 1.0995116e12):
            s = torch.full((), float(np.float32(sv)), device="cuda")
            for c in range(16):
                x = (base + c * chunk).to(torch.int32).view(torch.float32) if c < 8 else \
                    (base + c * chunk - (1 << 32)).to(torch.int32).view(torch.float32)
                fast = ops.quantize(x, s, zp, round_mode=mode)
                old = lib.LIB.b200_set_fast_division(0)
                try:
                    exact = ops.quantize(x, s, zp, round_mode=mode)
                finally:
                    lib.LIB.b200_set_fast_division(old)
                assert torch.equal(fast, exact), "mode %d scale %r chunk %d: %d bytes differ" % (mode, sv, c, int((fast != exact).sum()))


@pytest.mark.gpu
def test_bandwidth_sweep_tool_runs():
    """python -m ngraph_b200.quantize_sweep (the bandwidth sweep table) on its two smallest sizes"""
    from ngraph_b200 import quantize_sweep
    lines = []
    rows = quantize_sweep.sweep(max_mb=4, iters=2, out=lines.append)
    assert len(rows) == 2 * 2 * 2 + 9 and all(r[4] > 0 for r in rows)
    assert any("ROUND_DOWN" in l for l in lines)
