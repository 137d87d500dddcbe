"""The f32 glue kernels through the C ABI against numpy restatements of nGraph's reference kernels
(runtime/reference/{sum,max,broadcast,reshape,batch_mat_mul,gather}.hpp and the elementwise headers): bit-exact, except
exp / erf, which are held to one unit in the last place of the float result."""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

OPS = dict(add=0, sub=1, mul=2, div=3, max=4, min=5, abs=6, neg=7, sqrt=8, exp=9, erf=10, relu=11)


@pytest.fixture(scope="module")
def L():
    from ngraph_b200 import lib
    return lib


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def i64(v):
    return (ctypes.c_int64 * max(len(v), 1))(*[int(x) for x in v])


def stream():
    return torch.cuda.current_stream().cuda_stream


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_elementwise_is_ieee_exact(L):
    rng = np.random.default_rng(1)
    a = (rng.standard_normal(100003) * 10 ** rng.uniform(-6, 6, 100003)).astype(np.float32)
    b = (rng.standard_normal(100003) * 10 ** rng.uniform(-6, 6, 100003)).astype(np.float32)
    a[:4] = [0.0, -0.0, np.inf, np.nan]
    ad, bd, out = dev(a), dev(b), torch.empty(a.size, device="cuda")
    with np.errstate(all="ignore"):
        want = dict(add=a + b, sub=a - b, mul=a * b, div=a / b, max=np.where(a > b, a, b), min=np.where(a < b, a, b))
        for name, exp in want.items():
            L.check(L.LIB.b200_f32_binary(OPS[name], ad.data_ptr(), bd.data_ptr(), out.data_ptr(), a.size, stream()), name)
            got = out.cpu().numpy()
            ok = (bits(got) == bits(exp)) | (np.isnan(got) & np.isnan(exp))  # NaN payloads are not part of the contract
            assert ok.all(), name
        want = dict(abs=np.abs(a), neg=-a, sqrt=np.sqrt(a), relu=np.where(a > 0, a, np.float32(0)))
        for name, exp in want.items():
            L.check(L.LIB.b200_f32_unary(OPS[name], ad.data_ptr(), out.data_ptr(), a.size, stream()), name)
            got = out.cpu().numpy()
            ok = (bits(got) == bits(exp)) | (np.isnan(got) & np.isnan(exp))
            assert ok.all(), name


@pytest.mark.parametrize("rows,period", [(37, 768), (50, 6), (1000, 1), (3, 5)])
def test_binary_with_a_repeating_operand(L, rows, period):
    """out[i] = a[i] op v[i % period]: what the op computes on a Broadcast of v along new leading axes"""
    rng = np.random.default_rng(9)
    a = rng.standard_normal((rows, period)).astype(np.float32)
    v = rng.standard_normal(period).astype(np.float32)
    ad, vd, out = dev(a), dev(v), torch.empty(a.size, device="cuda")
    fns = dict(add=np.add, sub=np.subtract, mul=np.multiply, div=np.divide, max=np.maximum, min=np.minimum)
    for name, fn in fns.items():
        for v_left in (0, 1):
            L.check(L.LIB.b200_f32_binary_periodic(OPS[name], ad.data_ptr(), vd.data_ptr(), out.data_ptr(), a.size, period, v_left,
                                                   stream()), name)
            want = fn(v[None, :], a) if v_left else fn(a, v[None, :])
            np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(want.astype(np.float32)).ravel(), err_msg="%s %d" % (name, v_left))


def test_exp_and_erf_within_one_ulp(L):
    x = np.linspace(-20, 20, 200001).astype(np.float32)
    xd, out = dev(x), torch.empty(x.size, device="cuda")
    for name, fn in (("exp", math.exp), ("erf", math.erf)):
        L.check(L.LIB.b200_f32_unary(OPS[name], xd.data_ptr(), out.data_ptr(), x.size, stream()), name)
        exact = np.array([fn(float(v)) for v in x], np.float64)
        got = out.cpu().numpy().astype(np.float64)
        ulp = np.spacing(np.abs(exact).astype(np.float32)).astype(np.float64)
        assert (np.abs(got - exact) <= ulp).all(), name


def kahan_sum_rows(x):
    """reference::sum over the last axis: sequential, compensated, in float32"""
    z = np.zeros(x.shape[:-1], np.float32)
    c = np.zeros(x.shape[:-1], np.float32)
    for k in range(x.shape[-1]):
        v = x[..., k]
        y = (v - c).astype(np.float32)
        t = (z + y).astype(np.float32)
        c = ((t - z).astype(np.float32) - y).astype(np.float32)
        z = t
    return z


@pytest.mark.parametrize("shape,axes", [((37, 768), (1,)), ((6, 5, 384), (2,)), ((9, 33, 7), (0, 2)), ((50000,), (0,)), ((4, 3), ()),
                                        ((300, 1000), (0, 1)), ((200, 768), (1,)), ((70, 3, 33), (2,)), ((64, 1535), (1,))])
def test_sum_and_max_follow_the_reference_order(L, shape, axes):
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(shape) * 100).astype(np.float32)
    keep = [i for i in range(len(shape)) if i not in axes]
    moved = np.transpose(x, keep + list(axes)).reshape([shape[i] for i in keep] + [-1])  # reduced axes last, row-major order
    want_sum = kahan_sum_rows(moved) if axes else x.copy()
    want_max = moved.max(axis=-1) if axes else x.copy()
    xd = dev(x)
    out = torch.empty(max(want_sum.size, 1), device="cuda")
    want_min = moved.min(axis=-1) if axes else x.copy()
    want_max_abs = np.abs(moved).max(axis=-1) if axes else np.abs(x)
    for op, want in ((0, want_sum), (1, want_max), (2, want_min), (3, want_max_abs)):
        L.check(L.LIB.b200_reduce_f32(op, xd.data_ptr(), out.data_ptr(), i64(shape), len(shape), i64(axes), len(axes), stream()), "reduce")
        np.testing.assert_array_equal(bits(out.cpu().numpy()[:want.size]), bits(want).ravel())


@pytest.mark.parametrize("rows,n", [(100, 384), (65, 33), (3, 1535), (40, 1), (1000, 64)])
def test_softmax_rows_equals_the_five_steps(L, rows, n):
    """the fused last-axis Softmax against Max, Subtract, Exp, Sum, Divide run one after another (softmax.hpp)"""
    rng = np.random.default_rng(6)
    x = (rng.standard_normal((rows, n)) * 4).astype(np.float32)
    x[0, 0] = np.inf if n > 1 else 1.0  # a row whose sum is not finite
    xd = dev(x)
    shape, last = i64([rows, n]), i64([1])
    small = torch.empty(rows, device="cuda")
    wide, e, want, got = (torch.empty((rows, n), device="cuda") for _ in range(4))
    S = stream()
    P = lambda t: t.data_ptr()
    L.check(L.LIB.b200_reduce_f32(1, P(xd), P(small), shape, 2, last, 1, S), "max")
    L.check(L.LIB.b200_broadcast_b32(P(small), P(wide), shape, 2, last, 1, S), "broadcast")
    L.check(L.LIB.b200_f32_binary(OPS["sub"], P(xd), P(wide), P(e), x.size, S), "sub")
    L.check(L.LIB.b200_f32_unary(OPS["exp"], P(e), P(e), x.size, S), "exp")
    L.check(L.LIB.b200_reduce_f32(0, P(e), P(small), shape, 2, last, 1, S), "sum")
    L.check(L.LIB.b200_broadcast_b32(P(small), P(wide), shape, 2, last, 1, S), "broadcast")
    L.check(L.LIB.b200_f32_binary(OPS["div"], P(e), P(wide), P(want), x.size, S), "div")
    L.check(L.LIB.b200_softmax_rows_f32(P(xd), P(got), rows, n, S), "softmax")
    w, g = want.cpu().numpy(), got.cpu().numpy()
    np.testing.assert_array_equal(np.isnan(w), np.isnan(g))
    np.testing.assert_array_equal(bits(np.nan_to_num(g)), bits(np.nan_to_num(w)))
    assert abs(float(g[1:].sum()) - (rows - 1)) < 1e-3 * rows
    # and against the CPU restatement of reference::softmax (oracle/glue.py, pinned against INTERPRETER): exp is the one
    # step whose last bit may differ between the device's routine and the host's, so a row may carry a one-ulp difference
    # into its sum: held to two units in the last place, and to identity on all but a small share of the elements
    from oracle import glue
    with np.errstate(all="ignore"):
        o = glue.softmax(x[1:])
    np.testing.assert_allclose(g[1:], o, rtol=2.4e-7, atol=0)
    assert (bits(g[1:]) != bits(o)).mean() < 0.02


@pytest.mark.parametrize("rows,n", [(100, 768), (33, 65), (5, 1535), (64, 1)])
def test_layer_norm_rows_follows_the_decomposition(L, rows, n):
    """op::v0::LayerNorm's decomposition (layer_norm.cpp:68-150, reduce_ops.cpp:68-127) step by step in float32"""
    rng = np.random.default_rng(7)
    f = np.float32
    x = (rng.standard_normal((rows, n)) * 3 + 1).astype(f)
    gamma, beta = rng.standard_normal(n).astype(f), rng.standard_normal(n).astype(f)
    eps, count = f(1e-5), f(n)
    mean = (kahan_sum_rows(x) / count).astype(f)
    d = (x - mean[:, None]).astype(f)
    var = (kahan_sum_rows((d * d).astype(f)) / count).astype(f)
    sd = np.sqrt((var + eps).astype(f)).astype(f)
    want = (((d / sd[:, None]).astype(f) * gamma).astype(f) + beta).astype(f)
    xd, gd, bd = dev(x), dev(gamma), dev(beta)
    out = torch.empty((rows, n), device="cuda")
    L.check(L.LIB.b200_layer_norm_rows_f32(xd.data_ptr(), gd.data_ptr(), bd.data_ptr(), out.data_ptr(), rows, n, ctypes.c_float(1e-5),
                                           stream()), "layer_norm")
    np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(want))
    from oracle import glue  # the CPU restatement pinned against INTERPRETER (tests/test_oracle_glue.py): bit for bit
    np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(glue.layer_norm(x, gamma, beta, 1e-5)))


def test_gelu_equals_its_decomposition_on_the_device(L):
    """(0.5 * x) * (1 + erf(x / sqrt 2)) of gelu.cpp:46-60 against the same five elementwise kernels run one by one"""
    x = np.concatenate([np.linspace(-9, 9, 100001), [0.0, -0.0, np.inf, -np.inf]]).astype(np.float32)
    n = x.size
    xd = dev(x)
    c = {k: dev(np.full(n, v, np.float32)) for k, v in (("half", 0.5), ("one", 1.0), ("sqrt2", np.float32(math.sqrt(2.0))))}
    q, e, t, h, want, got = (torch.empty(n, device="cuda") for _ in range(6))
    S, P = stream(), lambda a: a.data_ptr()
    L.check(L.LIB.b200_f32_binary(OPS["div"], P(xd), P(c["sqrt2"]), P(q), n, S), "div")
    L.check(L.LIB.b200_f32_unary(OPS["erf"], P(q), P(e), n, S), "erf")
    L.check(L.LIB.b200_f32_binary(OPS["add"], P(c["one"]), P(e), P(t), n, S), "add")
    L.check(L.LIB.b200_f32_binary(OPS["mul"], P(c["half"]), P(xd), P(h), n, S), "mul")
    L.check(L.LIB.b200_f32_binary(OPS["mul"], P(h), P(t), P(want), n, S), "mul")
    L.check(L.LIB.b200_gelu_f32(P(xd), P(got), n, S), "gelu")
    w, g = want.cpu().numpy(), got.cpu().numpy()
    np.testing.assert_array_equal(np.isnan(w), np.isnan(g))
    np.testing.assert_array_equal(bits(np.nan_to_num(g)), bits(np.nan_to_num(w)))
    # against the CPU restatement of the reference's Gelu (oracle/glue.py, pinned against INTERPRETER): erf is computed in
    # double and rounded on both sides, so the results agree except where the two double routines round differently
    from oracle import glue
    fin = np.isfinite(x)
    o = glue.gelu(x[fin])
    np.testing.assert_allclose(g[fin], o, rtol=2.4e-7, atol=1e-9)
    assert (bits(g[fin]) != bits(o)).mean() < 0.01


def test_row_kernels_with_the_producer_op_folded_in(L):
    """Softmax(x * scalar) and LayerNorm(x + y) from one kernel each equal the elementwise kernel followed by the plain row kernel"""
    rng = np.random.default_rng(11)
    rows, n = 70, 384
    x, y = (rng.standard_normal((rows, n)) * 3).astype(np.float32), rng.standard_normal((rows, n)).astype(np.float32)
    gamma, beta = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    xd, yd, gd, bd = dev(x), dev(y), dev(gamma), dev(beta)
    f = dev(np.float32([0.125]))
    tmp, want, got = (torch.empty((rows, n), device="cuda") for _ in range(3))
    S, P = stream(), lambda a: a.data_ptr()
    L.check(L.LIB.b200_f32_binary_periodic(OPS["mul"], P(xd), P(f), P(tmp), x.size, 1, 0, S), "mul")
    L.check(L.LIB.b200_softmax_rows_f32(P(tmp), P(want), rows, n, S), "softmax")
    L.check(L.LIB.b200_softmax_rows_scaled_f32(P(xd), P(f), P(got), rows, n, S), "softmax scaled")
    np.testing.assert_array_equal(bits(got.cpu().numpy()), bits(want.cpu().numpy()))
    L.check(L.LIB.b200_f32_binary(OPS["add"], P(xd), P(yd), P(tmp), x.size, S), "add")
    L.check(L.LIB.b200_layer_norm_rows_f32(P(tmp), P(gd), P(bd), P(want), rows, n, ctypes.c_float(1e-5), S), "ln")
    L.check(L.LIB.b200_layer_norm_rows_sum_f32(P(xd), P(yd), P(gd), P(bd), P(got), rows, n, ctypes.c_float(1e-5), S), "ln sum")
    np.testing.assert_array_equal(bits(got.cpu().numpy()), bits(want.cpu().numpy()))


def test_broadcast_and_permute(L):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 7)).astype(np.float32)
    out = torch.empty((3, 5, 4, 7), device="cuda")
    xd = dev(x)
    L.check(L.LIB.b200_broadcast_b32(xd.data_ptr(), out.data_ptr(), i64(out.shape), 4, i64([0, 2]), 2, stream()), "broadcast")
    np.testing.assert_array_equal(out.cpu().numpy(), np.broadcast_to(x[None, :, None, :], (3, 5, 4, 7)))
    s = torch.empty(6, device="cuda")
    one = dev(np.float32([2.5]))
    L.check(L.LIB.b200_broadcast_b32(one.data_ptr(), s.data_ptr(), i64([6]), 1, i64([0]), 1, stream()), "broadcast")
    assert (s.cpu().numpy() == 2.5).all()
    for shape in ((2, 3, 4, 5), (3, 16, 5, 8)):  # last axis 8: four neighbours move together when it stays last
        y = rng.standard_normal(shape).astype(np.float32)
        yd = dev(y)
        for order in ((0, 2, 1, 3), (0, 2, 3, 1), (3, 2, 1, 0), (1, 0, 2, 3)):
            o = torch.empty(y.size, device="cuda")
            L.check(L.LIB.b200_permute_b32(yd.data_ptr(), o.data_ptr(), i64(y.shape), 4, i64(order), stream()), "permute")
            np.testing.assert_array_equal(o.cpu().numpy(), np.transpose(y, order).ravel())
    x8 = rng.standard_normal((5, 8)).astype(np.float32)
    x8d, out8 = dev(x8), torch.empty((3, 5, 4, 8), device="cuda")
    L.check(L.LIB.b200_broadcast_b32(x8d.data_ptr(), out8.data_ptr(), i64(out8.shape), 4, i64([0, 2]), 2, stream()), "broadcast")
    np.testing.assert_array_equal(out8.cpu().numpy(), np.broadcast_to(x8[None, :, None, :], (3, 5, 4, 8)))
    col = rng.standard_normal(6).astype(np.float32)  # a new LAST axis: every output row repeats one value
    cold, outc = dev(col), torch.empty((6, 8), device="cuda")
    L.check(L.LIB.b200_broadcast_b32(cold.data_ptr(), outc.data_ptr(), i64([6, 8]), 2, i64([1]), 1, stream()), "broadcast")
    np.testing.assert_array_equal(outc.cpu().numpy(), np.broadcast_to(col[:, None], (6, 8)))


@pytest.mark.parametrize("batch,m,k,n", [(3, 17, 96, 21), (2, 130, 70, 200), (2, 100, 33, 64), (1, 384, 64, 384), (5, 64, 16, 48), (1, 140, 300, 130)])
def test_bmm_accumulates_in_double_in_order(L, batch, m, k, n):
    """small products run one thread per 4 x 4 outputs, large ones through shared-memory panels: the same bits either way"""
    rng = np.random.default_rng(4)
    a = (rng.standard_normal((batch, m, k)) * 50).astype(np.float32)
    b = (rng.standard_normal((batch, k, n)) * 50).astype(np.float32)
    acc = np.zeros((batch, m, n), np.float64)
    for kk in range(k):
        acc += a[:, :, kk, None].astype(np.float64) * b[:, kk, None, :].astype(np.float64)
    out = torch.empty((batch, m, n), device="cuda")
    ad, bd = dev(a), dev(b)  # kept alive until the result has been read
    L.check(L.LIB.b200_bmm_f32(ad.data_ptr(), bd.data_ptr(), out.data_ptr(), batch, m, k, n, stream()), "bmm")
    np.testing.assert_array_equal(bits(out.cpu().numpy()), bits(acc.astype(np.float32)))


def test_gather_rows(L):
    rng = np.random.default_rng(5)
    table = rng.standard_normal((50, 24)).astype(np.float32)
    for dt, code in ((np.int32, 2), (np.int64, 4)):
        idx = rng.integers(0, 50, 77).astype(dt)
        out = torch.empty((77, 24), device="cuda")
        td, idxd = dev(table), dev(idx)
        L.check(L.LIB.b200_gather_rows_b32(td.data_ptr(), 50, 24, idxd.data_ptr(), code, 77, out.data_ptr(), stream()), "gather")
        np.testing.assert_array_equal(out.cpu().numpy(), table[idx])
