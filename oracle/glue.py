"""TEST INFRASTRUCTURE ONLY (checker, never the product path): numpy restatements of the f32 reference kernels that the
float islands of quantized graphs use, each step rounded to float32 the way the reference's C++ loops round it.
Pinned against nGraph's INTERPRETER in tests/test_oracle_glue.py.

  kahan_sum        runtime/reference/sum.hpp:56-90     compensated sum over the last axis, elements in order
  softmax          runtime/reference/softmax.hpp       max, x - max, exp, sum (Kahan), divide
  layer_norm       op/layer_norm.cpp:68-150 + builder/reduce_ops.cpp:68-127 (mean, variance), last axis, scale and bias
  gelu             op/gelu.cpp:46-60                   (0.5 * x) * (1 + erf(x / sqrt(2)))
  batch_mat_mul    runtime/reference/dot.hpp:108-160   products summed over k in order; accumulated in double here
                                                       (the reference accumulates f32 dots in the element type)
  avg_pool         runtime/reference/avg_pool.hpp:160-236  window walked in (h, w) order over the padded image, sum kept in
                                                       the element type (f32: sequential float adds; u8 / i8: wraps), then
                                                       sum / count (one-byte types: nearbyint of the float quotient)
"""
import math

import numpy as np

F = np.float32


def kahan_sum(x):
    """reference::sum over the last axis: sequential, compensated, in float32 (non-finite terms are added plainly)"""
    x = np.asarray(x, F)
    z = np.zeros(x.shape[:-1], F)
    c = np.zeros(x.shape[:-1], F)
    for k in range(x.shape[-1]):
        v = x[..., k]
        ok = np.isfinite(v) & np.isfinite(z)
        with np.errstate(invalid="ignore", over="ignore"):
            y = (v - c).astype(F)
            t = (z + y).astype(F)
            c = np.where(ok, ((t - z).astype(F) - y).astype(F), c)
            z = np.where(ok, t, (z + v).astype(F))
    return z


def softmax(x):
    """over the last axis"""
    x = np.asarray(x, F)
    m = x.max(axis=-1, keepdims=True)
    e = np.exp((x - m).astype(F).astype(np.float64)).astype(F)  # std::exp on float: the correctly rounded value in all but rare cases
    return (e / kahan_sum(e)[..., None]).astype(F)


def layer_norm(x, gamma, beta, epsilon=1e-5):
    """over the last axis; every operation of the decomposition rounded separately"""
    x, gamma, beta = np.asarray(x, F), np.asarray(gamma, F), np.asarray(beta, F)
    n, eps = F(x.shape[-1]), F(epsilon)
    mean = (kahan_sum(x) / n).astype(F)
    d = (x - mean[..., None]).astype(F)
    var = (kahan_sum((d * d).astype(F)) / n).astype(F)
    sd = np.sqrt((var + eps).astype(F)).astype(F)
    return (((d / sd[..., None]).astype(F) * gamma).astype(F) + beta).astype(F)


def gelu(x):
    x = np.asarray(x, F)
    q = (x / F(math.sqrt(2.0))).astype(F)
    e = np.vectorize(math.erf, otypes=[np.float64])(q.astype(np.float64)).astype(F)
    return ((F(0.5) * x).astype(F) * (F(1.0) + e).astype(F)).astype(F)


def batch_mat_mul(a, b):
    """a [B, M, K] x b [B, K, N]"""
    a, b = np.asarray(a, F), np.asarray(b, F)
    acc = np.zeros((a.shape[0], a.shape[1], b.shape[2]), np.float64)
    for k in range(a.shape[2]):
        acc += a[:, :, k, None].astype(np.float64) * b[:, k, None, :].astype(np.float64)
    return acc.astype(F)


def avg_pool(x, window, stride=(1, 1), pad_below=(0, 0), pad_above=None, include_padding=False, out_hw=None):
    """x [N, C, H, W], f32 / u8 / i8.  out_hw: the op's output extent when it differs from the floor formula (ceil mode);
    window positions beyond the padded image are then not counted (the reference itself refuses such windows)."""
    x = np.asarray(x)
    pad_above = pad_below if pad_above is None else pad_above
    n, c, h, w = x.shape
    if out_hw is None:
        out_hw = tuple((x.shape[2 + i] + pad_below[i] + pad_above[i] - window[i]) // stride[i] + 1 for i in (0, 1))
    out = np.empty((n, c) + tuple(out_hw), x.dtype)
    for p in range(out_hw[0]):
        for q in range(out_hw[1]):
            acc = np.zeros((n, c), x.dtype)
            count = 0
            for r in range(window[0]):
                hh = p * stride[0] - pad_below[0] + r
                if hh >= h + pad_above[0]:
                    break
                for s_ in range(window[1]):
                    ww = q * stride[1] - pad_below[1] + s_
                    if ww >= w + pad_above[1]:
                        break
                    inside = 0 <= hh < h and 0 <= ww < w
                    if inside or include_padding:
                        if inside:
                            with np.errstate(over="ignore"):
                                acc = (acc + x[:, :, hh, ww]).astype(x.dtype)  # the running sum has the element type
                        count += 1
            if x.dtype == np.float32:
                out[:, :, p, q] = (acc / F(count)).astype(F)
            else:
                out[:, :, p, q] = np.rint((acc.astype(F) / F(count)).astype(F)).astype(x.dtype)
    return out
